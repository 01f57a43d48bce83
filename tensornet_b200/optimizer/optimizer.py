"""``tn.optimizer.Optimizer``: the dense-side optimizer shell.

Like the reference's Keras shell (tensornet/optimizer/optimizer.py:26-82) it owns a dense
table: the first step gathers every dense parameter (sorted by name) into the flat table,
and each later step is a single fused update over that array.  ``PCGrad`` projects
conflicting per-task gradients before the update (tensornet/optimizer/optimizer.py:85-150).
"""
from __future__ import annotations

import random
from typing import Iterable, Sequence, Tuple

import torch

from .. import core


class Optimizer:
    def __init__(self, dense_opt, name: str = "TensornetOptimizer"):
        self.dense_opt = dense_opt
        self.name = name
        self.dense_table_handle = core.create_dense_table(dense_opt)
        self.table = core.dense_table(self.dense_table_handle)
        self.learning_rate = core.get_opt_learning_rate(dense_opt)
        self.iterations = 0

    # ------------------------------------------------------------------
    def attach(self, named_params: Iterable[Tuple[str, torch.Tensor]]):
        """Move the given parameters into the flat dense table (idempotent)."""
        if not self.table.initialized:
            named = [(n, p) for n, p in named_params if p.requires_grad]
            self.table.init(named)
            core.barrier()

    def _lr(self) -> float:
        return self.dense_opt.current_lr(self.iterations)

    def step(self, peers_past_backward: bool = False):
        """One fused dense update: mean gradient over ranks -> optimizer on the owned chunk ->
        new weights visible on every rank; gradients are re-zeroed.  ``peers_past_backward``: see
        :meth:`tensornet_b200.ops.dense_table.DenseTable.step`."""
        self.table.set_lr(self._lr())
        self.table.step(peers_past_backward)
        self.iterations += 1

    def apply_gradients(self, grads_and_vars=None):
        self.step()

    def zero_grad(self):
        if self.table.initialized:
            self.table.G.zero_()

    def get_config(self) -> dict:
        """Name and the dense optimizer's hyper-parameters (optimizer.py:80-82)."""
        return {"name": self.name, "dense_opt": self.dense_opt.get_config()}

    def save_dense_table(self, filepath: str):
        return core.save_dense_table(self.dense_table_handle, filepath)

    def load_dense_table(self, filepath: str):
        return core.load_dense_table(self.dense_table_handle, filepath)


class PCGrad(Optimizer):
    """Gradient surgery for multi-task losses: every task gradient is projected onto the normal
    plane of each other task gradient it conflicts with (negative inner product), in random
    order, and the projected gradients are summed."""

    def project(self, task_grads: Sequence[torch.Tensor]) -> torch.Tensor:
        """``task_grads``: one flat gradient per task over the same parameters."""
        out = []
        n = len(task_grads)
        for i in range(n):
            g = task_grads[i].clone()
            order = list(range(n))
            random.shuffle(order)
            for j in order:
                if j == i:
                    continue
                gj = task_grads[j]
                dot = torch.dot(g, gj)
                if dot < 0:
                    g -= dot / gj.dot(gj).clamp_min(1e-30) * gj
            out.append(g)
        return torch.stack(out).sum(dim=0)

    def compute_gradients(self, loss: Sequence[torch.Tensor], var_list=None, tape=None, grad_loss=None) -> torch.Tensor:
        """One backward pass per task loss over the attached dense parameters, then the projection; the result is
        left in the flat gradient that ``step()`` applies and is returned (optimizer.py:91-130 in the reference, whose
        ``var_list`` / ``tape`` / ``grad_loss`` arguments have no meaning here and are accepted for the call's shape)."""
        G = self.table.G
        grads = []
        for k, task_loss in enumerate(loss):
            G.zero_()
            task_loss.backward(retain_graph=k < len(loss) - 1)
            grads.append(G.clone())
        G.copy_(self.project(grads))
        return G

    def step_multi(self, losses: Sequence[torch.Tensor]):
        """Backward every task loss separately, project, write the result into the flat gradient, step."""
        self.compute_gradients(losses)
        self.step()

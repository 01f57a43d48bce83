"""The dense parameter table: all dense parameters of a model as one flat fp32 array.

Mirrors the reference's DenseTable (core/ps/table/dense_table.cc:37-87): variables are laid
out in name order, the array is cut into ``ceil(total/world)`` contiguous chunks and rank r
owns chunk r together with its optimizer state.  On GPUs the array, its gradient and a bf16
shadow live in symmetric memory so the fused dense kernel can reduce-scatter the gradient,
update the owned chunk and all-gather the new weights in one launch; model parameters are
re-pointed to views of the flat array, so there is no copy-back step
(core/kernels/dense_table_ops.cc:199-244 in the reference).
"""
from __future__ import annotations

import weakref
from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

from .. import _build
from .._opentelemetry import phase
from ..core.config import config
from ..core.optimizers import KIND_ADAGRAD, KIND_ADAM, OptimizerBase
from ..core.runtime import runtime
from ..parallel.symm import SymmArena

ALIGN = 8  # elements; keeps every parameter's bf16 shadow 16-byte aligned for TMA

#: every live dense table of this process (``core.recover`` resets the exchange state of all of them)
live_tables: "weakref.WeakSet[DenseTable]" = weakref.WeakSet()


class DenseTable:
    def __init__(self, opt: OptimizerBase):
        if opt.kind not in (KIND_ADAM, KIND_ADAGRAD):
            raise ValueError("dense parameters support Adam and AdaGrad (the reference's dense Ftrl is an empty stub, "
                             "core/ps/optimizer/ftrl_kernel.cc:24-32)")
        self.opt = opt
        self.initialized = False
        self.grad_pre_reduced = False      # CPU ranks: the next step finds the mean gradient in G already
        self.step_count = 0
        self.names: List[str] = []
        self.offsets: List[int] = []
        self.sizes: List[int] = []
        self.total = 0
        live_tables.add(self)

    # ------------------------------------------------------------------
    def init(self, named_params: Sequence[Tuple[str, torch.Tensor]]):
        rt = runtime()
        named = sorted(named_params, key=lambda kv: kv[0])   # tensornet/optimizer/optimizer.py:57-58
        self.names = [n for n, _ in named]
        self.params = [p for _, p in named]
        off = 0
        for p in self.params:
            self.offsets.append(off)
            self.sizes.append(p.numel())
            off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        self.total = sum(self.sizes)
        W = rt.world
        self.chunk = ((off + W - 1) // W + 3) // 4 * 4
        self.n = self.chunk * W
        dev = rt.device
        self.world, self.rank = W, rt.rank
        if rt.on_gpu:
            self.arena = SymmArena([("W", (self.n,), torch.float32), ("G", (self.n,), torch.float32),
                                    ("Wb", (self.n,), torch.bfloat16), ("sig", (4 * 8,), torch.int64)])
            self.W, self.G, self.Wb = self.arena.tensor("W"), self.arena.tensor("G"), self.arena.tensor("Wb")
        else:
            self.W = torch.zeros(self.n)
            self.G = torch.zeros(self.n)
            self.Wb = None
        with torch.no_grad():
            for p, o, s in zip(self.params, self.offsets, self.sizes):
                self.W[o:o + s].copy_(p.detach().reshape(-1).to(dev))
            if W > 1:   # one set of initial values for the whole job
                dist.broadcast(self.W, src=0, group=rt.device_group if rt.on_gpu else rt.host_group)
            if self.Wb is not None:
                self.Wb.copy_(self.W)
        for p, o, s in zip(self.params, self.offsets, self.sizes):
            p.data = self.W[o:o + s].view(p.shape)
            p.grad = self.G[o:o + s].view(p.shape)
            if self.Wb is not None:
                p._tn_bf16 = self.Wb[o:o + s].view(p.shape)
        n_state = self.chunk if (rt.on_gpu and W > 1) else self.n
        self.state_lo = self.rank * self.chunk if (rt.on_gpu and W > 1) else 0
        self.s0 = torch.zeros(n_state, device=dev)
        self.s1 = torch.zeros(n_state, device=dev)
        self.s2 = torch.zeros(n_state, device=dev) if self.opt.kind == KIND_ADAGRAD else None
        if self.opt.kind == KIND_ADAGRAD:
            self.s1.fill_(float(self.opt.initial_g2sum))
        self.lr = self.opt.current_lr(0)
        self.state = torch.tensor([1.0, 1.0, self.lr, 0.0], dtype=torch.float32, device=dev)
        if rt.on_gpu:
            want_mc = (W >= 4) if int(config.use_multimem) < 0 else bool(int(config.use_multimem))
            use_mc = want_mc and W > 1 and self.arena.buf.mc_ptr != 0
            d = dict(kind=0 if self.opt.kind == KIND_ADAM else 1,
                     beta1=float(getattr(self.opt, "beta1", 0.9)), beta2=float(getattr(self.opt, "beta2", 0.999)),
                     eps=float(self.opt.epsilon), grad_decay=float(getattr(self.opt, "grad_decay_rate", 1.0)),
                     mom_decay=float(getattr(self.opt, "mom_decay_rate", 1.0)), state=self.state, n=self.n,
                     chunk=self.chunk if W > 1 else self.n, world=W, rank=self.rank, grad_scale=1.0 / W,
                     W=self.arena.ptrs("W"), G=self.arena.ptrs("G"), Wb=self.arena.ptrs("Wb"), sig=self.arena.ptrs("sig"),
                     W_mc=self.arena.mc("W") if use_mc else 0, G_mc=self.arena.mc("G") if use_mc else 0,
                     Wb_mc=self.arena.mc("Wb") if use_mc else 0, s0=self.s0, s1=self.s1, s2=self.s2,
                     epoch=torch.zeros(1, dtype=torch.int64, device=dev), bar=torch.zeros(4, dtype=torch.int32, device=dev),
                     status=rt.status, wait_ns=rt.wait_ns)
            self.uses_multimem = bool(use_mc)
            self._ctx_args = d
            self.ctx = _build.cuda_ext().DenseCtx(d)
        self.initialized = True
        rt.barrier()

    # ------------------------------------------------------------------
    def enable_gate(self):
        """Drop the closing cross-GPU barrier of the dense step: every owner instead publishes a "my chunk is
        written" flag on every GPU, and the returned gate ``(flags, epoch, world, wait_ns)`` makes the first GEMM
        that reads the weights wait for those flags (``ops.functional.mlp(..., gate=...)``).  Only valid when that
        GEMM really is the first reader of any dense parameter in a step.  Returns None with one GPU."""
        rt = runtime()
        if not (rt.on_gpu and self.world > 1 and self.initialized):
            return None
        self.ctx.set_gated(True)
        flags = self.arena.tensor("sig")[2 * 8: 2 * 8 + self.world]
        return (flags, self._ctx_args["epoch"], self.world, int(rt.wait_ns))

    def limit_grid(self, max_ctas: int):
        """Cap the multi-GPU dense kernel's grid so that it can share the GPU with a kernel on another stream."""
        if runtime().on_gpu and self.initialized:
            self.ctx.set_max_ctas(int(max_ctas))

    def limit_grid_to_sms(self, n_sms: int):
        """Cap the multi-GPU dense kernel's grid at what ``n_sms`` SMs hold, so that all of it is resident beside a
        kernel that leaves that many SMs free."""
        if runtime().on_gpu and self.initialized:
            self.ctx.set_max_ctas(int(n_sms) * int(_build.cuda_ext().dense_ctas_per_sm()))

    def set_lr(self, lr: float):
        if lr != self.lr:
            self.lr = float(lr)
            self.state[2] = self.lr

    def step(self, peers_past_backward: bool = False):
        """Average the gradient over ranks, update the owned chunk, publish the new weights, zero the gradient.
        ``peers_past_backward``: a kernel launched earlier on this stream in this step has already waited for every
        peer to finish its backward pass (the multi-GPU sparse push has), so the kernel skips its opening barrier."""
        rt = runtime()
        self.step_count += 1
        if rt.on_gpu:
            with phase("tn.dense_step"):
                self.ctx.step(bool(peers_past_backward and self.world > 1))
            return
        with torch.no_grad():
            reduced, self.grad_pre_reduced = self.grad_pre_reduced, False
            if self.world > 1 and not reduced:        # (a caller that exchanged the gradient itself left the mean in G)
                dist.all_reduce(self.G, group=rt.host_group)
                self.G.div_(self.world)
            g, w = self.G, self.W
            o = self.opt
            if all(t.is_contiguous() and t.dtype == torch.float32 for t in (g, w, self.s0, self.s1)):
                # one native pass over the flat arrays instead of a dozen tensor-op passes
                import numpy as np
                alpha = 0.0
                if o.kind == KIND_ADAM:
                    self.state[0] *= o.beta1
                    self.state[1] *= o.beta2
                    alpha = float(self.lr * torch.sqrt(1 - self.state[1]) / (1 - self.state[0]))
                s2 = self.s2.numpy() if self.s2 is not None else np.zeros(0, np.float32)
                _build.cpu_ext().dense_step(int(o.kind), w.detach().numpy().reshape(-1), g.numpy().reshape(-1), self.s0.numpy(),
                                            self.s1.numpy(), s2, float(self.lr), alpha, float(getattr(o, "beta1", 0.0)),
                                            float(getattr(o, "beta2", 0.0)), float(o.epsilon),
                                            float(getattr(o, "grad_decay_rate", 1.0)), float(getattr(o, "mom_decay_rate", 1.0)))
                return
            if o.kind == KIND_ADAM:   # core/ps/optimizer/adam_kernel.cc:46-55
                self.state[0] *= o.beta1
                self.state[1] *= o.beta2
                alpha = self.lr * torch.sqrt(1 - self.state[1]) / (1 - self.state[0])
                self.s0 += (g - self.s0) * (1 - o.beta1)
                self.s1 += (g * g - self.s1) * (1 - o.beta2)
                w -= self.s0 * alpha / (self.s1.sqrt() + o.epsilon)
            else:                      # core/ps/optimizer/ada_grad_kernel.cc:42-48
                self.s0.mul_(o.grad_decay_rate).add_(1.0)
                self.s1.mul_(o.grad_decay_rate).add_(g * g)
                self.s2 += (g - self.s2) * (1 - o.mom_decay_rate)
                w -= self.lr * self.s2 / (self.s1.sqrt() / self.s0.sqrt() + o.epsilon)
            g.zero_()

    def reset_exchange(self, epoch: int):
        """After a device error: clear the barrier / flag words, drop the partial gradient and restart the step
        counter the flags are compared with at ``epoch`` (the same on every rank).  Part of
        :func:`tensornet_b200.core.recover`."""
        if not (runtime().on_gpu and self.initialized):
            return
        self._ctx_args["epoch"].fill_(int(epoch))
        self._ctx_args["bar"].zero_()
        self.arena.tensor("sig").zero_()
        self.state[3] = 0.0
        self.G.zero_()

    def exchange_epoch(self) -> int:
        return int(self._ctx_args["epoch"].item()) if (runtime().on_gpu and self.initialized) else 0

    def refresh_shadow(self):
        """Re-derive the bf16 shadow after the fp32 master was written from outside the optimizer."""
        if self.Wb is not None:
            with torch.no_grad():
                self.Wb.copy_(self.W)

    # ------------------------------------------------------------------ checkpoint helpers
    def owned_range(self) -> Tuple[int, int]:
        lo = self.rank * self.chunk
        return lo, min(self.n, lo + self.chunk)

    def owned_state(self):
        """(w, s0, s1, s2, beta1_power, beta2_power) of the chunk this rank owns, on the host."""
        lo, hi = self.owned_range()
        a, b = lo - self.state_lo, hi - self.state_lo
        st = self.state.tolist()
        s2 = self.s2[a:b].cpu() if self.s2 is not None else None
        return self.W[lo:hi].float().cpu(), self.s0[a:b].cpu(), self.s1[a:b].cpu(), s2, st[0], st[1]

    def load_owned_state(self, w, s0, s1, s2, b1p, b2p):
        rt = runtime()
        lo, hi = self.owned_range()
        a, b = lo - self.state_lo, hi - self.state_lo
        dev = self.W.device
        with torch.no_grad():
            self.s0[a:b].copy_(s0.to(dev))
            self.s1[a:b].copy_(s1.to(dev))
            if self.s2 is not None and s2 is not None:
                self.s2[a:b].copy_(s2.to(dev))
            self.state[0] = b1p
            self.state[1] = b2p
            full = torch.zeros_like(self.W)
            full[lo:hi].copy_(w.to(dev))
            if self.world > 1:
                dist.all_reduce(full, group=rt.device_group if rt.on_gpu else rt.host_group)
            self.W.copy_(full)
            if self.Wb is not None:
                self.Wb.copy_(self.W)
        rt.barrier()

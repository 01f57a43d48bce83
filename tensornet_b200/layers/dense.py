"""Dense building blocks that run on the tcgen05 GEMM family.

The reference builds its towers from Keras ``Dense`` layers, ``FMLayer`` and ``DeepCrossLayer``
(examples/models/deepfm.py:37-57, examples/common/layers.py:21-103).  Here activations travel
between layers as bf16 matrices padded to a multiple of 8 columns whose first pad column is
the constant 1, so every layer is one GEMM with the bias folded into the weight matrix.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch
from torch import nn

from ..ops import functional as F


def _glorot_aug(n_out: int, n_in: int) -> torch.Tensor:
    """[n_out, pad8(n_in + 1)]: glorot-uniform weights, zero bias column, zero padding."""
    w = torch.zeros(n_out, F.pad8(n_in + 1))
    limit = math.sqrt(6.0 / (n_in + n_out))
    w[:, :n_in].uniform_(-limit, limit)
    return w


class MLP(nn.Module):
    """``in_dim -> hidden_units[0] -> ...`` with ReLU after every layer (optionally not the last).
    Input and output are padded bf16 operands (see :func:`tensornet_b200.ops.functional.concat_cast`)."""

    def __init__(self, in_dim: int, hidden_units: Sequence[int], relu_last: bool = True):
        super().__init__()
        self.in_dim = int(in_dim)
        self.hidden_units = [int(h) for h in hidden_units]
        self.relu_last = relu_last
        dims = [self.in_dim] + self.hidden_units
        self.weights = nn.ParameterList([nn.Parameter(_glorot_aug(dims[i + 1], dims[i])) for i in range(len(self.hidden_units))])
        # set by Model.compile on multi-GPU runs when this tower is the first reader of the dense weights in a step:
        # its first GEMM then waits for the optimizer's all-gather instead of the optimizer kernel waiting for everyone
        self.weight_gate = None

    @property
    def out_dim(self) -> int:
        return self.hidden_units[-1]

    def forward(self, x: torch.Tensor, grad_premasked: bool = False) -> torch.Tensor:
        return F.mlp(x, list(self.weights), self.in_dim, self.relu_last, grad_premasked, gate=self.weight_gate)

    def weight(self, i: int) -> torch.Tensor:
        dims = [self.in_dim] + self.hidden_units
        return self.weights[i][:, : dims[i]]

    def bias(self, i: int) -> torch.Tensor:
        dims = [self.in_dim] + self.hidden_units
        return self.weights[i][:, dims[i]]


class DenseHead(nn.Module):
    """``Dense(1)`` on a padded bf16 operand: returns fp32 logits ``[B, 1]``."""

    def __init__(self, in_dim: int):
        super().__init__()
        self.in_dim = int(in_dim)
        w = torch.zeros(in_dim + 1)
        limit = math.sqrt(6.0 / (in_dim + 1))
        w[:in_dim].uniform_(-limit, limit)
        self.weight = nn.Parameter(w)

    def forward(self, z: torch.Tensor) -> torch.Tensor:
        return F.head(z, self.weight)


class FMLayer(nn.Module):
    """Second-order factorisation-machine term without linear part and bias.
    Input ``[B, fields, dim]`` (or ``[B, fields*dim]`` with ``fields`` given), output ``[B, 1]``."""

    def __init__(self, fields: int = 0, dim: int = 0):
        super().__init__()
        self.fields, self.dim = fields, dim

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() == 3:
            return F.fm(x.reshape(x.shape[0], -1), x.shape[1], x.shape[2])
        if x.dim() != 2 or not self.fields:
            raise ValueError("Unexpected inputs dimensions %d, expect to be 3 dimensions" % x.dim())
        return F.fm(x, self.fields, self.dim)


class DeepCrossLayer(nn.Module):
    """DCN-v1 cross network: ``x_{l+1} = x_0 * (x_l . w_l) + b_l + x_l`` (rank-1 cross)."""

    def __init__(self, input_dim: int, num_layer: int = 3):
        super().__init__()
        self.num_layer = num_layer
        limit = math.sqrt(6.0 / (input_dim + 1))
        self.W = nn.ParameterList([nn.Parameter(torch.empty(input_dim, 1).uniform_(-limit, limit)) for _ in range(num_layer)])
        self.bias = nn.ParameterList([nn.Parameter(torch.zeros(input_dim)) for _ in range(num_layer)])

    def forward(self, inputs: torch.Tensor) -> torch.Tensor:
        cross = inputs
        for w, b in zip(self.W, self.bias):
            cross = F.cross_v1(inputs, cross, w, b)
        return cross

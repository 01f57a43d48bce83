"""Deep & Cross networks.

``DeepCross`` is the reference's example (examples/models/deep_cross.py): DCN-v1 rank-1 cross layers
next to a ReLU MLP.  ``DCNv2`` is the full-matrix variant ``x_{l+1} = x0 * (W_l x_l + b_l) + x_l``
whose cross layers are tcgen05 GEMMs with the Hadamard-residual fused into the epilogue.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch
from torch import nn

from .. import core, feature_column as fc
from ..layers import DeepCrossLayer, DenseHead, EmbeddingFeatures, MLP
from ..model import Model
from ..ops import functional as F


class DeepCrossSubModel(nn.Module):
    def __init__(self, in_dim: int, hidden_units: Sequence[int], num_cross: int = 3):
        super().__init__()
        self.in_dim = in_dim
        self.cross = DeepCrossLayer(in_dim, num_cross)
        self.mlp = MLP(in_dim, hidden_units)
        self.head = DenseHead(self.mlp.out_dim + in_dim)

    def forward(self, x: torch.Tensor):
        cross = self.cross(x)
        h = self.mlp(F.concat_cast([x], ones=True))
        z = F.concat_cast([h, cross], ones=True, widths=[self.mlp.out_dim, None])
        return self.head(z)


class CrossV2(nn.Module):
    """Stack of DCN-v2 cross layers on a padded bf16 operand ``[B, pad8(D + 1)]``."""

    def __init__(self, dim: int, num_layer: int = 3):
        super().__init__()
        self.dim, self.num_layer = dim, num_layer
        limit = math.sqrt(6.0 / (2 * dim))
        self.weights = nn.ParameterList()
        for _ in range(num_layer):
            w = torch.zeros(dim, F.pad8(dim + 1))
            w[:, :dim].uniform_(-limit, limit)
            self.weights.append(nn.Parameter(w))

    def forward(self, x0: torch.Tensor) -> torch.Tensor:
        return F.cross_v2(x0, list(self.weights), self.dim)


class DCNv2SubModel(nn.Module):
    def __init__(self, in_dim: int, hidden_units: Sequence[int], num_cross: int = 3):
        super().__init__()
        self.in_dim = in_dim
        self.cross = CrossV2(in_dim, num_cross)
        self.mlp = MLP(in_dim, hidden_units)
        self.head = DenseHead(self.mlp.out_dim)

    def forward(self, x):
        """``x``: the input matrix, or its column blocks (embeddings, dense features): the blocks go straight into
        the padded bf16 operand, without an fp32 concatenation in between (a 210 MB copy each way at width 6413)."""
        x0 = F.concat_cast(list(x) if isinstance(x, (list, tuple)) else [x], ones=True)
        xc = self.cross(x0)          # stacked structure: cross network feeds the deep network
        h = self.mlp(xc)
        return self.head(h)


class _CrossModel(Model):
    def __init__(self, sub_cls, features: Sequence[str], dnn_hidden_units, embedding_dim, dense_dim, dense_key, sparse_opt,
                 bucket_size, target_columns, combiner, num_cross, table_rows):
        super().__init__(name="full_model")
        sparse_opt = sparse_opt or core.AdaGrad(learning_rate=0.01, initial_g2sum=0.1, initial_scale=0.1)
        cols = [fc.embedding_column(fc.category_column(key=s, bucket_size=bucket_size), embedding_dim, combiner) for s in features]
        self.dense_key, self.dense_dim = dense_key, dense_dim
        self.deep_emb = EmbeddingFeatures(cols, sparse_opt, name="deep_input", is_concat=True, target_columns=target_columns,
                                          rows=table_rows)
        self.sub_model = sub_cls(len(features) * self.deep_emb.out_dim + dense_dim, dnn_hidden_units, num_cross)

    def forward(self, features):
        x = self.deep_emb(features)
        if self.dense_dim:
            dense = features[self.dense_key].to(x.device, non_blocking=True).float()
            if x.is_cuda and isinstance(self.sub_model, DCNv2SubModel):
                return self.sub_model([x, dense])
            x = torch.cat([x, dense], dim=1)
        return self.sub_model(x)


class DeepCross(_CrossModel):
    def __init__(self, features, dnn_hidden_units=(128, 128), embedding_dim=8, dense_dim=0, dense_key="dense", sparse_opt=None,
                 bucket_size=1024, target_columns=None, combiner="mean", num_cross=3, table_rows=None):
        super().__init__(DeepCrossSubModel, features, dnn_hidden_units, embedding_dim, dense_dim, dense_key, sparse_opt, bucket_size,
                         target_columns, combiner, num_cross, table_rows)


class DCNv2(_CrossModel):
    def __init__(self, features, dnn_hidden_units=(1024, 512, 256), embedding_dim=64, dense_dim=13, dense_key="dense",
                 sparse_opt=None, bucket_size=1024, target_columns=None, combiner="sum", num_cross=3, table_rows=None):
        super().__init__(DCNv2SubModel, features, dnn_hidden_units, embedding_dim, dense_dim, dense_key, sparse_opt, bucket_size,
                         target_columns, combiner, num_cross, table_rows)

"""Wide & Deep (examples/models/wide_deep.py in the reference): dim-1 "wide" embeddings concatenated
with a ReLU MLP over the deep embeddings (plus optional dense features), normalised by a
synchronised TNBatchNormalization, then ``Dense(1)``."""
from __future__ import annotations

from typing import Optional, Sequence

import torch
from torch import nn

from .. import core, feature_column as fc
from ..layers import DenseHead, EmbeddingFeatures, MLP, TNBatchNormalization
from ..model import Model
from ..ops import functional as F


class WideDeepSubModel(nn.Module):
    def __init__(self, n_linear: int, deep_in: int, dense_dim: int, hidden_units: Sequence[int], use_bn: bool = True):
        super().__init__()
        self.n_linear, self.deep_in, self.dense_dim = n_linear, deep_in, dense_dim
        self.mlp = MLP(deep_in + dense_dim, hidden_units)
        width = self.mlp.out_dim + n_linear
        self.bn = TNBatchNormalization(width, synchronized=True, sync_freq=4, max_count=1000000, name="both_bn") if use_bn else None
        self.head = DenseHead(width)

    def forward(self, linear_emb, deep_emb, dense=None):
        x0 = F.concat_cast([deep_emb] + ([dense.float()] if self.dense_dim else []), ones=True)
        h = self.mlp(x0)
        if self.bn is None:
            z = F.concat_cast([h, linear_emb], ones=True, widths=[self.mlp.out_dim, None])
        else:
            both = torch.cat([h[:, : self.mlp.out_dim].float(), linear_emb], dim=1)
            z = F.concat_cast([self.bn(both)], ones=True)
        return self.head(z)


class WideDeep(Model):
    def __init__(self, linear_features: Sequence[str], dnn_features: Sequence[str], dnn_hidden_units: Sequence[int] = (128, 128),
                 embedding_dim: int = 8, dense_dim: int = 0, dense_key: str = "dense", sparse_opt=None, bucket_size: int = 1024,
                 target_columns: Optional[Sequence[str]] = None, combiner: str = "mean", use_bn: bool = True,
                 table_rows: Optional[int] = None):
        super().__init__(name="full_model")
        sparse_opt = sparse_opt or core.AdaGrad(learning_rate=0.01, initial_g2sum=0.1, initial_scale=0.1)
        cols = {s: fc.category_column(key=s, bucket_size=bucket_size) for s in dict.fromkeys(list(linear_features) + list(dnn_features))}
        self.dense_key, self.dense_dim = dense_key, dense_dim
        self.linear_emb = EmbeddingFeatures([fc.embedding_column(cols[s], 1, combiner) for s in linear_features], sparse_opt,
                                            name="linear_input", is_concat=True, target_columns=target_columns, rows=table_rows)
        self.deep_emb = EmbeddingFeatures([fc.embedding_column(cols[s], embedding_dim, combiner) for s in dnn_features], sparse_opt,
                                          name="deep_input", is_concat=True, target_columns=target_columns, rows=table_rows)
        self.sub_model = WideDeepSubModel(len(linear_features) * self.linear_emb.out_dim, len(dnn_features) * self.deep_emb.out_dim,
                                          dense_dim, dnn_hidden_units, use_bn)

    def forward(self, features):
        lin = self.linear_emb(features)
        deep = self.deep_emb(features)
        dense = features[self.dense_key].to(deep.device, non_blocking=True) if self.dense_dim else None
        return self.sub_model(lin, deep, dense)

"""DeepFM (examples/models/deepfm.py in the reference): a linear term over dim-1 embeddings,
a second-order FM term and a ReLU MLP over the concatenated deep embeddings (plus optional
dense features), joined by a final ``Dense(1)``.

As in the reference the model is split into an embedding part (``emb_model``: the two
EmbeddingFeatures layers) and a pure dense ``sub_model`` (what gets exported for serving).
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
from torch import nn

from .. import core, feature_column as fc
from ..layers import DenseHead, EmbeddingFeatures, MLP
from ..model import Model
from ..ops import functional as F


class DeepFMSubModel(nn.Module):
    """Dense part: inputs are the pooled embeddings, output is the logit."""

    def __init__(self, n_linear: int, n_fields: int, emb_dim: int, dense_dim: int, hidden_units: Sequence[int]):
        super().__init__()
        self.n_linear, self.n_fields, self.emb_dim, self.dense_dim = n_linear, n_fields, emb_dim, dense_dim
        self.mlp = MLP(n_fields * emb_dim + dense_dim, hidden_units)
        self.head = DenseHead(self.mlp.out_dim + n_linear + 1)

    def forward(self, linear_emb: Optional[torch.Tensor], deep_emb: torch.Tensor, dense: Optional[torch.Tensor] = None):
        fm = F.fm(deep_emb, self.n_fields, self.emb_dim)
        pieces = [deep_emb] + ([dense.float()] if self.dense_dim else [])
        x0 = F.concat_cast(pieces, ones=True)
        h = self.mlp(x0)
        tail = [h] + ([linear_emb] if self.n_linear else []) + [fm]
        z = F.concat_cast(tail, ones=True, widths=[self.mlp.out_dim] + [None] * (len(tail) - 1))
        return self.head(z)


class DeepFM(Model):
    def __init__(self, linear_features: Sequence[str], dnn_features: Sequence[str], dnn_hidden_units: Sequence[int] = (128, 128),
                 embedding_dim: int = 8, dense_dim: int = 0, dense_key: str = "dense", sparse_opt=None, linear_sparse_opt=None,
                 bucket_size: int = 1024, target_columns: Optional[Sequence[str]] = None, combiner: str = "mean",
                 table_rows: Optional[int] = None, share_linear_table: bool = False):
        super().__init__(name="full_model")
        sparse_opt = sparse_opt or core.AdaGrad(learning_rate=0.01, initial_g2sum=0.1, initial_scale=0.1)
        linear_sparse_opt = linear_sparse_opt or sparse_opt
        cols = {s: fc.category_column(key=s, bucket_size=bucket_size) for s in dict.fromkeys(list(linear_features) + list(dnn_features))}
        self.dense_key, self.dense_dim = dense_key, dense_dim
        self.linear_emb = None
        # One table for both parts: a slot's linear weight is stored as an extra column of its embedding row, so
        # the batch is deduplicated, pulled and pushed once.  Exact for element-wise sparse optimizers (Adam, Ftrl);
        # AdaGrad keeps one accumulator per row and therefore needs separate tables.
        self.share_linear_table = bool(share_linear_table and linear_features and list(linear_features) == list(dnn_features)
                                       and sparse_opt.kind != 0 and not target_columns)
        self.emb_dim = embedding_dim
        if self.share_linear_table:
            self.deep_emb = EmbeddingFeatures([fc.embedding_column(cols[s], embedding_dim + 4, combiner) for s in dnn_features],
                                              sparse_opt, name="deep_input", is_concat=True, rows=table_rows)
            self.sub_model = DeepFMSubModel(len(linear_features), len(dnn_features), embedding_dim, dense_dim, dnn_hidden_units)
            return
        if linear_features:
            self.linear_emb = EmbeddingFeatures([fc.embedding_column(cols[s], 1, combiner) for s in linear_features],
                                                linear_sparse_opt, name="linear_input", is_concat=True,
                                                target_columns=target_columns, rows=table_rows)
        self.deep_emb = EmbeddingFeatures([fc.embedding_column(cols[s], embedding_dim, combiner) for s in dnn_features],
                                          sparse_opt, name="deep_input", is_concat=True, target_columns=target_columns,
                                          rows=table_rows)
        n_lin = len(linear_features) * (self.linear_emb.out_dim if self.linear_emb else 0)
        self.sub_model = DeepFMSubModel(n_lin, len(dnn_features), self.deep_emb.out_dim, dense_dim, dnn_hidden_units)

    def first_dense_tower(self):
        """The embedding pooling, FM term and input assembly read no dense parameter: the MLP is the first reader."""
        return self.sub_model.mlp

    def fused_train_loss(self, features, labels, sums):
        """Training loss through the fused DeepFM kernels (gather + FM + operand build in one kernel; head, loss and
        head backward in one kernel).  Returns None when the inputs do not qualify (ragged slots, CVM columns,
        CPU); the caller then uses the generic path."""
        if not core.runtime().on_gpu or (self.linear_emb is None and not self.share_linear_table):
            return None
        mlp = self.sub_model.mlp
        dq = self.emb_dim // 4
        if self.emb_dim % 4 or dq & (dq - 1) or dq > 32 or F.pad8(mlp.out_dim + 1) > 512 or self.sub_model.n_linear > 32:
            return None
        got = self.deep_emb.fused_single_hot_inputs(features, True)
        if got is None:
            return None
        ids, B = got
        dense = features[self.dense_key].to(ids.device, non_blocking=True) if self.dense_dim else None
        if self.share_linear_table:
            x0, fm, lin = F.deepfm_input(self.deep_emb._anchor, self.deep_emb.link, ids, B, len(self.deep_emb._keys), dense, True,
                                         self.emb_dim, self.emb_dim)
        else:
            lin = self.linear_emb(features, training=True)
            x0, fm, _ = F.deepfm_input(self.deep_emb._anchor, self.deep_emb.link, ids, B, len(self.deep_emb._keys), dense, True)
        h = mlp(x0, grad_premasked=True)
        loss, _ = F.deepfm_head_loss(h, lin, fm, self.sub_model.head.weight, labels.to(ids.device, non_blocking=True), sums,
                                     mlp.out_dim)
        return loss

    def forward(self, features):
        if self.share_linear_table:
            both = self.deep_emb(features)
            both = both.view(both.shape[0], -1, self.emb_dim + 4)
            lin = both[:, :, self.emb_dim].contiguous()
            deep = both[:, :, : self.emb_dim].reshape(both.shape[0], -1)
            dense = features[self.dense_key].to(deep.device, non_blocking=True) if self.dense_dim else None
            return self.sub_model(lin, deep, dense)
        lin = self.linear_emb(features) if self.linear_emb is not None else None
        deep = self.deep_emb(features)
        dense = None
        if self.dense_dim:
            dense = features[self.dense_key].to(deep.device, non_blocking=True)
        return self.sub_model(lin, deep, dense)

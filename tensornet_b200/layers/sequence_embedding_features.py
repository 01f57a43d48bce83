"""``SequenceEmbeddingFeatures`` (tensornet/layers/sequence_embedding_features.py:35-234): like
EmbeddingFeatures but the ids of a slot form an ordered sequence that is NOT pooled: the layer
returns ``([B, T, sum of dims], sequence_length)``.  ``need_stop_gradient`` skips the sparse push."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch
from torch import nn

from .. import core
from ..feature_column import EmbeddingColumn
from ..ops.embedding import pull_sequence


class SequenceEmbeddingFeatures(nn.Module):
    def __init__(self, feature_columns: Sequence[EmbeddingColumn], sparse_opt, trainable: bool = True, name: Optional[str] = None,
                 is_concat: bool = False, embedding_share: Optional[str] = None, need_stop_gradient: bool = False,
                 max_length: int = 0, rows: Optional[int] = None):
        super().__init__()
        assert len(feature_columns) != 0, "feature_columns must not empty"
        dim = feature_columns[0].dimension
        for c in feature_columns:
            assert c.dimension == dim, "currently we only support feature_columns with same dimension"
        self.layer_name = name or ""
        self._sparse_opt = sparse_opt
        self.is_concat = is_concat
        self.trainable = trainable
        self._feature_columns = list(feature_columns)
        self._keys = [c.categorical_column.name for c in feature_columns]
        self._need_stop_gradient = need_stop_gradient
        self.embedding_share = embedding_share
        self.dim = dim
        self.max_length = max_length or max(getattr(c.categorical_column, "max_length", 0) for c in feature_columns)
        self.sparse_table_handle = core.create_sparse_table(sparse_opt, self.layer_name, dim, False, embedding_share or "", rows=rows)
        self.table = core.sparse_table(self.sparse_table_handle)
        # one exchange context per column: every column is pulled (and pushed) on its own
        self.links = [self.table.link(c.categorical_column.bucket_size) for c in feature_columns]
        self._anchor = torch.zeros(1, requires_grad=True, device=core.runtime().device)
        self._pending = []

    def filter_not_used_features(self, features: Dict) -> Dict:
        """The entries of ``features`` that this layer's columns read (sequence_embedding_features.py:147-152)."""
        return {k: features[k] for k in self._keys}

    def get_sparse_pulling_feature(self, features: Dict) -> Dict:
        """The id features whose signs this layer looks up (sequence_embedding_features.py:154-162)."""
        return {k: v for k, v in features.items() if k in self._keys}

    def get_config(self) -> Dict:
        return {"name": self.layer_name, "trainable": self.trainable, "is_concat": self.is_concat,
                "embedding_share": self.embedding_share, "need_stop_gradient": self._need_stop_gradient,
                "max_length": self.max_length, "feature_columns": [c.get_config() for c in self._feature_columns],
                "sparse_opt": self._sparse_opt.get_config()}

    @classmethod
    def from_config(cls, config: Dict, sparse_opt=None):
        from ..core.optimizers import optimizer_from_config
        from ..feature_column import EmbeddingColumn
        cfg = dict(config)
        cols = [EmbeddingColumn.from_config(c) for c in cfg.pop("feature_columns")]
        opt = sparse_opt or optimizer_from_config(cfg.pop("sparse_opt"))
        cfg.pop("sparse_opt", None)
        return cls(cols, opt, **cfg)

    def forward(self, features: Dict, training: Optional[bool] = None):
        if not isinstance(features, dict):
            raise ValueError("We expected a dictionary here. Instead we got: ", features)
        training = self.training if training is None else bool(training)
        dev = core.runtime().device
        self.table.set_training(training)
        outs, lengths = [], None
        self._pending = []
        for key, link in zip(self._keys, self.links):
            f = features[key]
            if torch.is_tensor(f):          # [B, T] dense block of ids: every position valid
                B, T0 = f.shape
                values = f.reshape(-1).to(dev).long()
                offsets = torch.arange(0, B * T0 + 1, T0, device=dev, dtype=torch.int32)
            else:
                values, offsets = f[0].to(dev).long(), f[1].to(dev).int()
                B = offsets.numel() - 1
            T = self.max_length or int((offsets[1:] - offsets[:-1]).max().item())
            count = training and self.trainable and not self._need_stop_gradient
            out, ln = pull_sequence(self._anchor, link, values, offsets, B, T, None, count)
            if self._need_stop_gradient:
                out = out.detach()
            if count:
                self._pending.append(link)
            outs.append(out)
            lengths = ln if lengths is None else lengths
        return torch.cat(outs, dim=-1), lengths

    def backwards(self, grads_and_vars=None):
        if self._need_stop_gradient:
            return
        for link in self._pending:
            link.push()
        self._pending = []

    def save_sparse_table(self, filepath, mode="txt"):
        return core.save_sparse_table(self.sparse_table_handle, filepath, mode)

    def load_sparse_table(self, filepath, mode="txt"):
        return core.load_sparse_table(self.sparse_table_handle, filepath, mode)

    def show_decay(self, delta_days=0):
        return core.show_decay(self.sparse_table_handle, delta_days)

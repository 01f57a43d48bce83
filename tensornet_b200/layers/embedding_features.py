"""``tn.layers.EmbeddingFeatures``: the first layer of every model.

Creates one sparse table for the layer (or shares one through ``embedding_share``), and on
every call dedups the batch's signs, pulls their rows from the owning shards into the small
per-batch matrix and pools them per example - the reference's EmbeddingFeatures /
StateManagerImpl (tensornet/layers/embedding_features.py:36-177,180-406).  ``backwards()``
pushes the gradient of that per-batch matrix to the owners, where the sparse optimizer runs.

With ``target_columns`` the table counts show / click per sign and every embedding gets two
extra, gradient-free columns ``show`` and ``ln(click+1) - ln(show+1)`` (the CVM plug-in,
embedding_features.py:288-295, core/ps/optimizer/ada_grad_kernel.cc:121-128).
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch
from torch import nn

from .. import core
from ..data.features import PACKED_KEY, gather_columns
from ..feature_column import EmbeddingColumn
from ..ops.embedding import pull_pool


class EmbeddingFeatures(nn.Module):
    def __init__(self, feature_columns: Sequence[EmbeddingColumn], sparse_opt, trainable: bool = True,
                 name: Optional[str] = None, is_concat: bool = False, target_columns: Optional[Sequence[str]] = None,
                 embedding_share: Optional[str] = None, rows: Optional[int] = None):
        super().__init__()
        assert len(feature_columns) != 0, "feature_columns must not empty"
        dim = feature_columns[0].dimension
        combiner = feature_columns[0].combiner
        for c in feature_columns:
            if not isinstance(c, EmbeddingColumn):
                raise ValueError(f"Items of feature_columns must be a {EmbeddingColumn}. Given: {c}")
            assert c.dimension == dim, "currently we only support feature_columns with same dimension in EmbeddingFeatures"
            assert c.combiner == combiner, "all columns of one EmbeddingFeatures layer must use the same combiner"
        if target_columns and len(target_columns) > 1:
            raise ValueError(f"For now cvm plugin only support one column, Given: {target_columns}")
        self.layer_name = name or ""
        self.trainable = trainable
        self.is_concat = is_concat
        self._sparse_opt = sparse_opt
        self._feature_columns = list(feature_columns)
        self._target_columns = list(target_columns) if target_columns else None
        self._keys = [c.categorical_column.name for c in feature_columns]
        self.dim = dim
        self.combiner = combiner
        self.use_cvm = bool(target_columns)
        self.embedding_share = embedding_share
        self.sparse_table_handle = core.create_sparse_table(sparse_opt, self.layer_name, dim, self.use_cvm,
                                                            embedding_share or "", rows=rows)
        self.table = core.sparse_table(self.sparse_table_handle)
        max_unique = sum(c.categorical_column.bucket_size for c in feature_columns)
        self.link = self.table.link(max_unique)
        self.out_dim = dim + (2 if self.use_cvm else 0)
        self._anchor = torch.zeros(1, requires_grad=True, device=core.runtime().device)
        self._pending_push = False
        self._args_cache = None

    # --------------------------------------------------------------------------------
    @property
    def feature_columns(self):
        return self._feature_columns

    def filter_not_used_features(self, features: Dict) -> Dict:
        """The entries of ``features`` that this layer's columns read (embedding_features.py:314-319)."""
        return {k: features[k] for k in self._keys}

    def get_sparse_pulling_feature(self, features: Dict):
        """``(pulled, targets)``: the id features of ``features`` split into those whose signs are looked up and the
        target columns that only feed the show / click counters (embedding_features.py:321-334)."""
        pulled, targets = {}, {}
        for k, v in features.items():
            if self._target_columns and k in self._target_columns:
                targets[k] = v
            elif k in self._keys:
                pulled[k] = v
        return pulled, targets

    def get_config(self) -> Dict:
        """Constructor arguments as plain data (embedding_features.py:369-379); ``from_config`` builds the layer again."""
        return {"name": self.layer_name, "trainable": self.trainable, "is_concat": self.is_concat,
                "target_columns": self._target_columns, "embedding_share": self.embedding_share,
                "feature_columns": [c.get_config() for c in self._feature_columns], "sparse_opt": self._sparse_opt.get_config()}

    @classmethod
    def from_config(cls, config: Dict, sparse_opt=None):
        """``sparse_opt`` overrides the optimizer described in ``config`` (a learning-rate schedule is not part of a
        configuration)."""
        from ..core.optimizers import optimizer_from_config
        from ..feature_column import EmbeddingColumn
        cfg = dict(config)
        cols = [EmbeddingColumn.from_config(c) for c in cfg.pop("feature_columns")]
        opt = sparse_opt or optimizer_from_config(cfg.pop("sparse_opt"))
        cfg.pop("sparse_opt", None)
        return cls(cols, opt, **cfg)

    def _pull_args(self, features: Dict, training: bool):
        """What this layer's pull needs from a batch: ``(ids, offsets, B, labels, label_mod, count)``.  A model that
        runs several layers' pulls with shared round trips asks for them first; the ``forward`` of the same batch
        then finds them here (once) instead of gathering the columns again."""
        c, self._args_cache = self._args_cache, None
        if c is not None and c[0] is features and c[1] == training:
            return c[2]
        dev = core.runtime().device
        ids, offsets, B = gather_columns(features, self._keys, dev)
        S = len(self._keys)
        labels, label_mod = None, 0
        if self._target_columns:
            y = features[self._target_columns[0]].to(dev, non_blocking=True).reshape(-1).float()
            if offsets is None:
                labels, label_mod = y, B
            else:
                lens = (offsets[1:] - offsets[:-1]).long()
                labels = torch.repeat_interleave(y.repeat(S), lens, output_size=int(ids.numel()))
        return ids, offsets, B, labels, label_mod, training and self.trainable

    def stash_pull_args(self, features: Dict, training: bool):
        args = self._pull_args(features, training)
        self._args_cache = (features, training, args)
        return args

    def forward(self, features: Dict, training: Optional[bool] = None):
        if not isinstance(features, dict):
            raise ValueError("We expected a dictionary here. Instead we got: ", features)
        training = self.training if training is None else bool(training)
        self.table.set_training(training)
        ids, offsets, B, labels, label_mod, count = self._pull_args(features, training)
        S = len(self._keys)
        out = pull_pool(self._anchor, self.link, ids, offsets, B, S, self.combiner, labels, label_mod, count)
        self._pending_push = count
        if self.is_concat:
            return out
        pd = self.out_dim
        return [out[:, s * pd:(s + 1) * pd] for s in range(S)]

    def fused_single_hot_inputs(self, features: Dict, training: bool):
        """(ids, B) when this layer's slots are all single-hot and carry no CVM columns, else None.
        Used by model-specific fused kernels that consume the pulled rows directly."""
        if self.use_cvm or self.dim % 4 != 0:
            return None
        dev = core.runtime().device
        ids, offsets, B = gather_columns(features, self._keys, dev)
        if offsets is not None:
            return None
        self.table.set_training(training)
        self._pending_push = training and self.trainable
        return ids, B

    def ids_pulled_for(self, features: Dict):
        """The id tensor this layer's next training pull will receive for ``features``, when that is known ahead
        without any work: the packed single-hot ids of exactly this layer's slots, already on the device (the
        tensor the pull gets is then a view of it, same address).  None otherwise, and for layers whose table
        serves several links (their pulls share one step counter)."""
        rt = core.runtime()
        if not (rt.on_gpu and self.trainable and isinstance(features, dict)) or not hasattr(self.link, "prefetch"):
            return None
        if len(getattr(self.table, "links", ())) != 1:
            return None
        packed = features.get(PACKED_KEY)
        if packed is None or list(packed.keys) != list(self._keys) or packed.ids is None or not packed.ids.is_cuda:
            return None
        return packed.ids.reshape(-1)

    def backwards(self, grads_and_vars=None):
        """Push this step's sparse gradients to the owning shards and apply the sparse optimizer."""
        if self._pending_push:
            self.link.push()
            self._pending_push = False

    # --------------------------------------------------------------------------------
    def save_sparse_table(self, filepath: str, mode: str = "txt"):
        return core.save_sparse_table(self.sparse_table_handle, filepath, mode)

    def load_sparse_table(self, filepath: str, mode: str = "txt"):
        return core.load_sparse_table(self.sparse_table_handle, filepath, mode)

    def show_decay(self, delta_days: int = 0):
        return core.show_decay(self.sparse_table_handle, delta_days)

"""Input containers for categorical features.

A model input is a dict ``{slot name: feature}`` where a feature is
* an int64 tensor ``[B]`` / ``[B, 1]``   one sign per example,
* an int64 tensor ``[B, L]``            exactly L signs per example,
* a :class:`Ragged` ``(values, offsets)``  a variable number of signs per example
  (the SparseTensor inputs of the reference, tensornet/layers/embedding_features.py:252-284).

:class:`PackedFeatures` carries several slots in one buffer so a batch costs one host->device
copy instead of one per slot; layers pick the slots they need out of it.
"""
from __future__ import annotations

from typing import Dict, List, NamedTuple, Optional, Sequence, Tuple

import torch


class Ragged(NamedTuple):
    values: torch.Tensor   # int64 [nnz]
    offsets: torch.Tensor  # int32/int64 [B + 1]


class PackedFeatures:
    """Slots ``keys`` stored together.  Single-hot: ``ids [S, B]``.  Ragged: ``values [nnz]`` with
    ``offsets [S*B + 1]`` where bag ``s*B + b`` belongs to slot s, example b."""

    def __init__(self, keys: Sequence[str], ids: Optional[torch.Tensor] = None, values: Optional[torch.Tensor] = None,
                 offsets: Optional[torch.Tensor] = None, batch_size: Optional[int] = None):
        self.keys = [str(k) for k in keys]
        self.ids, self.values, self.offsets = ids, values, offsets
        if ids is not None:
            assert ids.dim() == 2 and ids.shape[0] == len(self.keys)
            self.batch_size = int(ids.shape[1])
        else:
            assert values is not None and offsets is not None and batch_size is not None
            self.batch_size = int(batch_size)

    def to(self, device, non_blocking: bool = True) -> "PackedFeatures":
        mv = lambda t: None if t is None else t.to(device, non_blocking=non_blocking)
        return PackedFeatures(self.keys, mv(self.ids), mv(self.values), mv(self.offsets), self.batch_size)

    def pin_memory(self) -> "PackedFeatures":
        pm = lambda t: None if t is None else t.pin_memory()
        return PackedFeatures(self.keys, pm(self.ids), pm(self.values), pm(self.offsets), self.batch_size)


PACKED_KEY = "__packed__"


def batch_size_of(feature) -> int:
    if isinstance(feature, Ragged) or (isinstance(feature, (tuple, list)) and len(feature) == 2):
        return int(feature[1].numel()) - 1
    return int(feature.shape[0])


def gather_columns(features: Dict, keys: List[str], device) -> Tuple[torch.Tensor, Optional[torch.Tensor], int]:
    """Collect the slots ``keys`` as ``(ids, offsets, B)`` in the column-after-column layout the
    pull kernel expects; ``offsets`` is None when every bag holds exactly one id."""
    packed = features.get(PACKED_KEY) if isinstance(features, dict) else None
    if packed is not None and packed.keys == keys:
        if packed.ids is not None:
            return packed.ids.to(device, non_blocking=True).reshape(-1), None, packed.batch_size
        return (packed.values.to(device, non_blocking=True), packed.offsets.to(device, non_blocking=True).int(),
                packed.batch_size)
    if packed is not None and packed.ids is not None and all(k in packed.keys for k in keys):
        idx = [packed.keys.index(k) for k in keys]
        ids = packed.ids.to(device, non_blocking=True)
        return ids[idx].reshape(-1).contiguous(), None, packed.batch_size
    cols = [features[k] for k in keys]
    single = all(torch.is_tensor(c) and (c.dim() == 1 or (c.dim() == 2 and c.shape[1] == 1)) for c in cols)
    B = batch_size_of(cols[0])
    if single:
        ids = torch.stack([c.reshape(-1).to(device, non_blocking=True).long() for c in cols]).reshape(-1)
        return ids, None, B
    vals, offs, base = [], [], 0
    for c in cols:
        if torch.is_tensor(c):
            c = c.to(device, non_blocking=True).long()
            c2 = c.reshape(B, -1)
            L = c2.shape[1]
            v = c2.reshape(-1)
            o = torch.arange(0, B * L + 1, L, device=device, dtype=torch.int64)
        else:
            v = c[0].to(device, non_blocking=True).long().reshape(-1)
            o = c[1].to(device, non_blocking=True).long().reshape(-1)
        vals.append(v)
        offs.append(o[:-1] + base)
        base += int(v.numel())
    offs.append(torch.tensor([base], device=device, dtype=torch.int64))
    return torch.cat(vals), torch.cat(offs).int(), B

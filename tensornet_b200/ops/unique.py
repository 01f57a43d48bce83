"""``unique_assign``: GPU dedup of a batch's signs with virtual-index assignment and show / click
counting (stand-alone form of the first phase of the fused pull kernel)."""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from .. import _build
from ..core.runtime import runtime


class UniqueAssign:
    """Re-usable dedup context for up to ``max_unique`` distinct signs per call."""

    def __init__(self, max_unique: int):
        rt = runtime()
        self.max_unique = int(max_unique)
        self.on_gpu = rt.on_gpu
        if self.on_gpu:
            cap2 = 1 << max(1, (2 * self.max_unique + 16 - 1).bit_length())
            d = rt.device
            self.dd_keys = torch.full((cap2,), -1, dtype=torch.int64, device=d)
            self.dd_vals = torch.zeros(cap2, dtype=torch.int32, device=d)
            self.count = torch.zeros(1, dtype=torch.int32, device=d)

    def __call__(self, ids: torch.Tensor, labels: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, ...]:
        """Returns ``(uniq int64 [max_unique], inverse int32 [n], show fp32 [max_unique], click fp32 [max_unique], count int32 [1])``;
        entries of ``uniq`` / ``show`` / ``click`` past ``count`` are unspecified / zero."""
        ids = ids.reshape(-1).contiguous()
        if not self.on_gpu:
            u, inv, show, click = _build.cpu_ext().unique_first_occurrence(
                ids.cpu().numpy(), None if labels is None else labels.reshape(-1).float().cpu().numpy())
            return (torch.from_numpy(u.view(np.int64)), torch.from_numpy(inv), torch.from_numpy(show), torch.from_numpy(click),
                    torch.tensor([len(u)], dtype=torch.int32))
        rt = runtime()
        d = ids.device
        uniq = torch.empty(self.max_unique, dtype=torch.int64, device=d)
        inverse = torch.empty(ids.numel(), dtype=torch.int32, device=d)
        show = torch.zeros(self.max_unique, dtype=torch.float32, device=d)
        click = torch.zeros(self.max_unique, dtype=torch.float32, device=d)
        self.count.zero_()
        _build.cuda_ext().unique_assign(ids, None if labels is None else labels.reshape(-1).float().contiguous(), self.dd_keys,
                                        self.dd_vals, uniq, inverse, show, click, self.count, rt.status)
        return uniq, inverse, show, click, self.count

"""Input helpers: day-partitioned file listing and end-of-input load balancing.

``list_files`` mirrors tensornet/data/dataset.py:29-51 (one glob per day directory, error when
nothing matches).  ``BalanceDataset`` covers the purpose of the reference's BalanceDataset op
(core/kernels/data/balance_dataset_ops.cc:198-311): ranks whose input runs dry must not leave
the others waiting inside a collective step.  In a synchronous job that means every rank has
to take the same number of steps; a rank that exhausts its input receives batches from a rank
that still has some, exchanged on the host over the control-plane process group.
"""
from __future__ import annotations

import glob
import os
from typing import Iterable, Iterator, List, Sequence

import torch

from ..core.runtime import runtime

_balance_epoch = 0


def list_files(datapath: str, days: Sequence[str], match_pattern: str) -> List[str]:
    patterns = [os.path.join(datapath, str(day), match_pattern) for day in days]
    files: List[str] = []
    for p in patterns:
        files.extend(sorted(glob.glob(p)))
    if not files:
        raise FileNotFoundError("No files matched pattern: " + ", ".join(patterns))
    return files


def reset_balance_dataset():
    """Start a new balancing epoch (called by PsWeightCheckpoint before train / predict)."""
    global _balance_epoch
    _balance_epoch += 1


class BalanceDataset:
    """Wrap an iterable of batches so that all ranks yield the same number of batches.

    Each round every rank tells the others whether it still has a batch.  While at least one rank
    has data, ranks without data are handed a batch by the lowest-ranked donor that has more than
    it needs for itself (donors read one batch ahead, up to ``buffer_size`` batches)."""

    def __init__(self, input_dataset: Iterable, buffer_size: int = 100):
        self._input = input_dataset
        self.buffer_size = buffer_size

    def __iter__(self) -> Iterator:
        rt = runtime()
        it = iter(self._input)
        if rt.world == 1:
            yield from it
            return
        buf: List = []
        exhausted = False

        def refill():
            nonlocal exhausted
            while not exhausted and len(buf) < 2:
                try:
                    buf.append(next(it))
                except StopIteration:
                    exhausted = True

        while True:
            refill()
            have = rt.all_gather_object(len(buf))
            if sum(have) == 0:
                return
            needy = [r for r, h in enumerate(have) if h == 0]
            donors = [r for r, h in enumerate(have) if h >= 2]
            gifts = {}
            for n, d in zip(needy, donors):
                gifts[n] = d
            # every rank takes part in every exchange so the object collectives stay matched
            mine = None
            for n, d in sorted(gifts.items()):
                payload = buf.pop() if rt.rank == d else None
                got = rt.broadcast_object(payload, src=d)
                if rt.rank == n:
                    mine = got
            if have[rt.rank] > 0:
                yield buf.pop(0)
            elif mine is not None:
                yield mine
            elif len(needy) > len(donors):
                # not enough spare batches this round: everyone stops together
                if all(h <= 1 for h in have) and any(h == 0 for h in have):
                    return

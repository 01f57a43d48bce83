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
from typing import Iterable, Iterator, List, Optional, Sequence

from ..core.runtime import runtime

_balance_epoch = 0


def list_files(datapath: str, days: Sequence[str], match_pattern: str) -> List[str]:
    """Files ``datapath/<day>/<match_pattern>`` of the given days, sorted within a day.  ``datapath`` may carry a URL
    scheme (``hdfs://...``): the day directories are then listed through the remote file-system layer and the
    names come back as URLs, which :class:`TFRecordDataset` fetches as it reads."""
    from ..utils.checkpoint import _fs_for, is_remote
    patterns = [os.path.join(datapath, str(day), match_pattern) for day in days]
    files: List[str] = []
    if is_remote(datapath):
        import fnmatch
        for day in days:
            url = datapath.rstrip("/") + "/" + str(day)
            fs, rpath = _fs_for(url)
            if not fs.exists(rpath):
                continue
            names = sorted(os.path.basename(str(e).rstrip("/")) for e in fs.ls(rpath, detail=False))
            files.extend(url + "/" + n for n in names if fnmatch.fnmatch(n, match_pattern))
    else:
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

    One round = one synchronous step.  Every rank reports how many batches it holds (each reads ahead up to
    ``min(buffer_size, max(world, 16))`` batches, so a single rank that still has input can feed all the others,
    and while every rank holds several batches one exchange covers several rounds).  While
    the ranks hold at least ``world`` batches between them, every rank without one is handed a batch by the
    rank with the most to spare, and every rank yields exactly one batch.  When fewer than ``world`` batches
    are left all ranks stop together; at most ``world - 1`` trailing batches of a pass are not used."""

    def __init__(self, input_dataset: Iterable, buffer_size: int = 100):
        self._input = input_dataset
        self.buffer_size = buffer_size

    @staticmethod
    def plan(have: Sequence[int]) -> Optional[List[tuple]]:
        """Gifts ``(receiver, donor)`` for one round given every rank's batch count, or None when the round
        cannot give one batch to every rank.  Pure and deterministic: all ranks compute the same plan."""
        world = len(have)
        if sum(have) < world:
            return None
        spare = {r: h - 1 for r, h in enumerate(have) if h >= 2}
        gifts = []
        for n in (r for r, h in enumerate(have) if h == 0):
            d = max(spare, key=lambda r: (spare[r], -r))
            gifts.append((n, d))
            spare[d] -= 1
            if spare[d] == 0:
                del spare[d]
        return gifts

    def __iter__(self) -> Iterator:
        rt = runtime()
        it = iter(self._input)
        if rt.world == 1:
            yield from it
            return
        buf: List = []
        exhausted = False
        # read-ahead: enough for one rank to feed all others, and enough that ranks with plenty of input can agree
        # on several rounds per exchange
        ahead = max(2, min(int(self.buffer_size), max(rt.world, 16)))

        def refill():
            nonlocal exhausted
            while not exhausted and len(buf) < ahead:
                try:
                    buf.append(next(it))
                except StopIteration:
                    exhausted = True

        while True:
            refill()
            have = rt.all_gather_object(len(buf))
            if min(have) >= 2:
                # every rank can serve the next rounds from its own buffer: no exchange until the poorest rank is
                # down to its last batch (all ranks derive the same number from the same counts)
                for _ in range(min(have) - 1):
                    yield buf.pop(0)
                continue
            gifts = self.plan(have)
            if gifts is None:
                return
            # every rank takes part in every exchange so the object collectives stay matched
            mine = None
            for n, d in gifts:
                payload = buf.pop() if rt.rank == d else None
                got = rt.broadcast_object(payload, src=d)
                if rt.rank == n:
                    mine = got
            yield buf.pop(0) if have[rt.rank] > 0 else mine

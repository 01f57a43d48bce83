"""``tn.distribute.PsStrategy`` (tensornet/distribute/ps_strategy.py:23-58).  Constructing it
initialises the runtime; ``scope()`` exists for source compatibility with code written against
the reference and does nothing else."""
from __future__ import annotations

import contextlib

from .. import core


class PsStrategy:
    def __init__(self):
        core.init()

    @contextlib.contextmanager
    def scope(self):
        yield self

    @property
    def should_checkpoint(self) -> bool:
        return core.self_shard_id() == 0

    @property
    def num_replicas_in_sync(self) -> int:
        return core.shard_num()


__all__ = ["PsStrategy"]

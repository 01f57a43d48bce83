"""Checkpoint helpers and the structured step log."""


def __getattr__(name):
    # resolved on first use: the step log imports the callback base class, which imports the core package
    if name in ("StepLog", "merge_rank_records"):
        from . import steplog

        return getattr(steplog, name)
    raise AttributeError(name)

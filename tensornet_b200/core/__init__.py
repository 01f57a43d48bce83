"""``tn.core``: the control API of the runtime.

Same twenty entry points as the reference's pybind module
(core/main/py_wrapper.cc:61-263, re-exported by tensornet/core/__init__.py:15-34), backed by
GPU-resident tables when a CUDA device is present and by the plain C++ tables otherwise.
Table handles are small integers handed out in creation order; every rank builds the same
model, so handles agree across ranks (core/ps/table/sparse_table.cc:151-158).
"""
from __future__ import annotations

from typing import Dict, List

from .config import Config, config
from .optimizers import AdaGrad, Adam, Ftrl, OptimizerBase
from .runtime import DeviceError, runtime

_sparse_tables: List[object] = []
_sparse_groups: Dict[str, int] = {}
_dense_tables: List[object] = []
_bn_tables: List[object] = []


def init() -> bool:
    """Bind this process to its GPU (or the CPU path) and set up the process groups."""
    return runtime().init()


def shutdown():
    """Tear down process groups and forget all tables (used by tests)."""
    _sparse_tables.clear()
    _sparse_groups.clear()
    _dense_tables.clear()
    _bn_tables.clear()
    runtime().shutdown()


def get_opt_learning_rate(opt: OptimizerBase):
    return opt.schedule if opt.schedule is not None else opt.learning_rate


def set_sparse_init_mode(opt: OptimizerBase, is_training: bool):
    """Rows created while ``is_training`` is false start at zero instead of the random initial value
    (core/main/py_wrapper.cc: ``set_sparse_init_mode``); applies to every table that uses ``opt``."""
    opt.sparse_zero_init = not is_training
    for t in _sparse_tables:
        if t.opt is opt:
            t.refresh_opt()


# ----------------------------------------------------------------------------- sparse
def create_sparse_table(opt: OptimizerBase, name: str, dimension: int, use_cvm: bool = False,
                        embedding_group: str = "", rows: int = None) -> int:
    """Create (or, with a non-empty ``embedding_group`` seen before, share) a sparse table."""
    rt = runtime()
    if embedding_group:
        if embedding_group in _sparse_groups:
            h = _sparse_groups[embedding_group]
            t = _sparse_tables[h]
            assert t.dim == dimension, "tables of one embedding_group must share the dimension"
            return h
    if rt.on_gpu:
        from ..ops.sparse_table_gpu import GpuSparseTable

        table = GpuSparseTable(opt, dimension, use_cvm, name=name, rows=rows)
    else:
        from ..ops.sparse_table_cpu import CpuSparseTable

        table = CpuSparseTable(opt, dimension, use_cvm, name=name)
    _sparse_tables.append(table)
    h = len(_sparse_tables) - 1
    table.handle = h
    if embedding_group:
        _sparse_groups[embedding_group] = h
    return h


def sparse_table(handle: int):
    return _sparse_tables[handle]


def save_sparse_table(handle: int, path: str, mode: str = "txt"):
    from ..utils import checkpoint

    checkpoint.save_sparse_table(_sparse_tables[handle], path, mode)


def load_sparse_table(handle: int, path: str, mode: str = "txt"):
    from ..utils import checkpoint

    checkpoint.load_sparse_table(_sparse_tables[handle], path, mode)


def show_decay(handle: int, delta_days: int):
    _sparse_tables[handle].show_decay(delta_days)


# ----------------------------------------------------------------------------- dense
def create_dense_table(opt: OptimizerBase) -> int:
    from ..ops.dense_table import DenseTable

    t = DenseTable(opt)
    t.handle = len(_dense_tables)
    _dense_tables.append(t)
    return t.handle


def dense_table(handle: int):
    return _dense_tables[handle]


def save_dense_table(handle: int, path: str):
    from ..utils import checkpoint

    checkpoint.save_dense_table(_dense_tables[handle], path)


def load_dense_table(handle: int, path: str):
    from ..utils import checkpoint

    checkpoint.load_dense_table(_dense_tables[handle], path)


# ----------------------------------------------------------------------------- batch norm
def create_bn_table(name: str, bn_size: int, sync: bool, moment: float, max_count: int, use_pctr_dnn_bn: bool = False) -> int:
    from ..ops.bn_table import BnTable, GpuBnTable

    cls = GpuBnTable if runtime().on_gpu else BnTable
    t = cls(name, bn_size, sync, moment, max_count, use_pctr_dnn_bn)
    t.handle = len(_bn_tables)
    _bn_tables.append(t)
    return t.handle


def bn_table(handle: int):
    return _bn_tables[handle]


def save_bn_table(handle: int, path: str):
    from ..utils import checkpoint

    checkpoint.save_bn_table(_bn_tables[handle], path)


def load_bn_table(handle: int, path: str):
    from ..utils import checkpoint

    checkpoint.load_bn_table(_bn_tables[handle], path)


# ----------------------------------------------------------------------------- cluster
def shard_num() -> int:
    return runtime().world


def self_shard_id() -> int:
    return runtime().rank


def barrier():
    runtime().barrier()


def recover() -> int:
    """Collective: make the exchange state usable again after a ``DeviceError``.

    A kernel that reports an error (a wait on a peer that ran out, a full table, an overflowing segment) stops
    where it is, and from then on every fused kernel of the process returns at once, so no step is half-applied
    on top of it; peers that were waiting for this GPU give up after their own wait budget and fail the same way.
    Once every rank has caught its ``DeviceError`` they all call ``recover()``: it waits for the others on the
    host, clears the per-step scratch, counters, barrier and flag words of every sparse link and dense table,
    moves every step counter that flags are compared with to one value agreed between the ranks (beyond anything
    a stale flag can hold), clears the status words and lines the ranks up again.  Rows already in the tables are
    kept; the step that failed is lost.  Returns the agreed counter value.  The reference's answer to the same
    situation is three retries and ``abort()`` (core/ps/ps_remote_server.cc:48-83)."""
    import torch

    rt = runtime()
    if not rt.on_gpu:
        rt.failed = False
        rt.barrier()
        return 0
    from ..ops import dense_table as _dt, sparse_table_gpu as _st

    rt.barrier()                       # includes a device synchronise: nothing of the failed step is still running
    sparse, dense = list(_st.live_tables), list(_dt.live_tables)
    mine = 0
    for t in sparse:
        mine = max(mine, int(t.epoch.item()))
    for t in dense:
        mine = max(mine, t.exchange_epoch())
    for t in _bn_tables:
        if getattr(t, "_epoch", None) is not None:
            mine = max(mine, int(t._epoch.item()))
    agreed = max(rt.all_gather_object(mine)) + 2
    for t in sparse:
        t.epoch.fill_(agreed)
        for lk in t.links:
            lk.reset_exchange()
    for t in dense:
        t.reset_exchange(agreed)
    for t in _bn_tables:
        if getattr(t, "_epoch", None) is not None:
            t._epoch.fill_(agreed)
            t._arena.tensor("sig").zero_()
    rt.status.zero_()
    torch.cuda.synchronize()
    rt.failed = False
    rt.barrier()
    return agreed


def reset_balance_dataset():
    from ..data import dataset

    dataset.reset_balance_dataset()


__all__ = [
    "init", "shutdown", "AdaGrad", "Adam", "Ftrl", "get_opt_learning_rate", "set_sparse_init_mode",
    "create_sparse_table", "create_dense_table", "create_bn_table", "save_sparse_table", "load_sparse_table",
    "save_dense_table", "load_dense_table", "save_bn_table", "load_bn_table", "shard_num", "self_shard_id",
    "barrier", "recover", "reset_balance_dataset", "show_decay", "config", "Config", "DeviceError", "runtime",
    "sparse_table", "dense_table", "bn_table",
]

"""Checkpoint I/O in the reference's on-disk layout (core/ps/table/sparse_table.cc:85-137,
core/ps/table/dense_table.cc:103-157, core/ps/table/bn_table.cc:171-214):

    <cp_dir>/sparse_table/<layer name | handle>/rank_<r>/block_<0..7>.gz      (txt)
                                                        /block_<0..7>_bin.gz  (bin)
    <cp_dir>/dense_table/<handle>/<r>
    <cp_dir>/bn_table/<handle>

A row lives in ``rank_(sign % world)`` and ``block_(((sign >> 32) | (sign << 32)) % 8)``.  Unlike the
reference, loading accepts a checkpoint written by a different number of ranks: every rank then
reads all ``rank_*`` directories and keeps the signs it owns (the reference needs an offline
Spark job for that, tensornet_tools/python/resize_sparse.py:35-54).
"""
from __future__ import annotations

import os
import re
from typing import List

import numpy as np
import torch

from .. import _build
from ..core.optimizers import KIND_ADAGRAD, KIND_ADAM, KIND_FTRL
from ..core.config import config
from ..core.runtime import runtime


def _table_dirname(table) -> str:
    return table.name if getattr(table, "name", "") else str(getattr(table, "handle", 0))


def _evict_args(opt):
    if opt.kind == KIND_ADAGRAD:
        return True, float(opt.show_threshold), int(opt.no_show_days), int(opt.elimination_logic)
    if opt.kind == KIND_FTRL:
        return True, float(opt.show_threshold), 0, 0
    return False, 0.0, 0, 0


def save_sparse_table(table, path: str, mode: str = "txt") -> int:
    rt = runtime()
    ext = _build.cpu_ext()
    d = os.path.join(path, "sparse_table", _table_dirname(table), f"rank_{rt.rank}")
    ev = _evict_args(table.opt)
    if hasattr(table, "export_chunks"):
        # GPU shard: filtered and grouped by block on the device, streamed through one pinned buffer
        w = ext.SparseDirWriter(d, mode, table.kind, table.dim, table.use_cvm, *ev)
        for signs, rows, offsets in table.export_chunks(config.checkpoint_chunk_rows, ev):
            w.append_grouped(signs, rows, offsets)
        return int(w.close())
    signs, rows = table.dump()
    return ext.write_sparse_dir(d, mode, table.kind, table.dim, table.use_cvm, np.ascontiguousarray(signs, dtype=np.uint64),
                                np.ascontiguousarray(rows, dtype=np.float32), *ev)


def _rank_dirs(base: str) -> List[str]:
    if not os.path.isdir(base):
        return []
    out = [d for d in os.listdir(base) if re.fullmatch(r"rank_\d+", d)]
    return sorted(out, key=lambda s: int(s.split("_")[1]))


def load_sparse_table(table, path: str, mode: str = "txt") -> int:
    rt = runtime()
    ext = _build.cpu_ext()
    base = os.path.join(path, "sparse_table", _table_dirname(table))
    dirs = _rank_dirs(base)
    if not dirs:
        raise FileNotFoundError(f"no sparse table checkpoint under {base}")
    same_world = len(dirs) == rt.world
    total = 0
    for d in ([f"rank_{rt.rank}"] if same_world else dirs):
        signs, rows = ext.read_sparse_dir(os.path.join(base, d), table.kind, table.dim, table.use_cvm)
        if not same_world and rt.world > 1:
            keep = (signs % np.uint64(rt.world)) == np.uint64(rt.rank)
            signs, rows = signs[keep], rows[keep]
        elif not same_world:
            pass
        if len(signs):
            table.load_rows(signs, rows)
            total += len(signs)
    return total


# ------------------------------------------------------------------------------------------------
def save_dense_table(dtable, path: str, handle: int = None):
    rt = runtime()
    ext = _build.cpu_ext()
    h = dtable.handle if handle is None else handle
    w, s0, s1, s2, b1p, b2p = dtable.owned_state()
    kind = KIND_ADAM if dtable.opt.kind == KIND_ADAM else KIND_ADAGRAD
    ext.write_dense_file(os.path.join(path, "dense_table", str(h), str(rt.rank)), int(dtable.n), rt.world, kind,
                         w.numpy(), s0.numpy(), s1.numpy(), None if s2 is None else s2.numpy(), float(b1p), float(b2p))


def load_dense_table(dtable, path: str, handle: int = None):
    """Reads every shard file present, so a checkpoint written by another world size can be loaded
    (the reference refuses a different rank count, core/ps/table/dense_table.cc:142)."""
    rt = runtime()
    ext = _build.cpu_ext()
    h = dtable.handle if handle is None else handle
    base = os.path.join(path, "dense_table", str(h))
    files = sorted((f for f in os.listdir(base) if f.isdigit()), key=int)
    kind = KIND_ADAM if dtable.opt.kind == KIND_ADAM else KIND_ADAGRAD
    parts = [ext.read_dense_file(os.path.join(base, f), kind) for f in files]
    if parts[0]["rank_num"] != len(files):
        raise RuntimeError(f"dense checkpoint incomplete: rank_num {parts[0]['rank_num']} but {len(files)} shard files")
    cat = lambda k: np.concatenate([p[k] for p in parts]) if len(parts[0][k]) else None
    w, s0, s1, s2 = cat("w"), cat("s0"), cat("s1"), cat("s2")
    if len(w) < dtable.n:
        pad = dtable.n - len(w)
        w, s0, s1 = (np.concatenate([x, np.zeros(pad, np.float32)]) for x in (w, s0, s1))
        if s2 is not None:
            s2 = np.concatenate([s2, np.zeros(pad, np.float32)])
    lo, hi = dtable.owned_range()
    tt = lambda x: None if x is None else torch.from_numpy(np.ascontiguousarray(x[lo:hi]))
    dtable.load_owned_state(tt(w), tt(s0), tt(s1), tt(s2), parts[0]["beta1_power"], parts[0]["beta2_power"])


# ------------------------------------------------------------------------------------------------
def save_bn_table(bn, path: str):
    ext = _build.cpu_ext()
    s, q, c = bn.totals()
    ext.write_bn_file(os.path.join(path, "bn_table", str(bn.handle)), bool(bn.use_pctr_dnn_bn), s, q, c)


def load_bn_table(bn, path: str):
    ext = _build.cpu_ext()
    pctr, s, q, c = ext.read_bn_file(os.path.join(path, "bn_table", str(bn.handle)))
    if bool(pctr) != bool(bn.use_pctr_dnn_bn):
        raise RuntimeError(f"bn calculate logic should be same, before use pctrdnn is {pctr}")
    bn.set_totals(s, q, c)

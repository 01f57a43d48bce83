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

Both directions are streamed.  A shard is written piece by piece from one pinned staging buffer
and read back block file by block file in pieces of ``config.checkpoint_load_chunk_rows`` rows (up to
eight files in flight, like the reference's eight loader threads,
core/ps/optimizer/optimizer_kernel.h:488-538), so the host holds a few pieces at a time however
large the shard is.  Paths with a URL scheme (``hdfs://``, ``s3://`` ...) are served through
``fsspec`` when it is installed: such a checkpoint is staged file by file through a local
scratch directory (the reference reaches them through TensorFlow's file-system layer,
core/utility/file_io.cc:47-50,132).
"""
from __future__ import annotations

import os
import re
import shutil
import tempfile
from concurrent.futures import ThreadPoolExecutor
from typing import Callable, Iterator, List, Optional, Tuple

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
    view = LocalView(path)
    d = os.path.join(view.local, "sparse_table", _table_dirname(table), f"rank_{rt.rank}")
    ev = _evict_args(table.opt)
    if hasattr(table, "export_chunks"):
        # GPU shard: filtered and grouped by block on the device, streamed through one pinned buffer
        w = ext.SparseDirWriter(d, mode, table.kind, table.dim, table.use_cvm, *ev)
        for signs, rows, offsets in table.export_chunks(config.checkpoint_chunk_rows, ev):
            w.append_grouped(signs, rows, offsets)
        n = int(w.close())
    else:
        signs, rows = table.dump()
        n = ext.write_sparse_dir(d, mode, table.kind, table.dim, table.use_cvm, np.ascontiguousarray(signs, dtype=np.uint64),
                                 np.ascontiguousarray(rows, dtype=np.float32), *ev)
    view.publish()
    return n


def _rank_dirs(base: str) -> List[str]:
    if not os.path.isdir(base):
        return []
    out = [d for d in os.listdir(base) if re.fullmatch(r"rank_\d+", d)]
    return sorted(out, key=lambda s: int(s.split("_")[1]))


# ------------------------------------------------------------------------------------------------
# remote file systems
# ------------------------------------------------------------------------------------------------
def is_remote(path: str) -> bool:
    return bool(re.match(r"^[a-zA-Z][a-zA-Z0-9+.-]*://", path)) and not path.startswith("file://")


_remote_fs: Optional[Callable] = None      # tests (and sites with their own client) may install a factory here


def set_remote_fs(factory: Optional[Callable]):
    """``factory(url) -> (fs, path)`` where ``fs`` offers ``ls / get / put / makedirs / exists`` in the fsspec
    sense.  None restores the default (``fsspec.core.url_to_fs``)."""
    global _remote_fs
    _remote_fs = factory


def _fs_for(url: str):
    if _remote_fs is not None:
        return _remote_fs(url)
    try:
        import fsspec
    except ImportError as e:      # pragma: no cover - depends on the installation
        raise RuntimeError(f"{url}: remote checkpoint paths need the fsspec package (or set_remote_fs)") from e
    return fsspec.core.url_to_fs(url)


class LocalView:
    """A local directory standing in for ``path``.  Local paths are used as they are.  A remote path gets a
    scratch directory: ``fetch(rel)`` brings one file or directory over before it is read, ``publish()`` uploads
    what was written and removes the scratch copy."""

    def __init__(self, path: str):
        self.path, self.remote = path, is_remote(path)
        if self.remote:
            self.fs, self.rpath = _fs_for(path)
            self.local = tempfile.mkdtemp(prefix="tn_ckpt_")
        else:
            self.local = path[7:] if path.startswith("file://") else path

    def fetch(self, rel: str) -> str:
        dst = os.path.join(self.local, rel)
        if self.remote and not os.path.exists(dst):
            src = self.rpath.rstrip("/") + "/" + rel
            if self.fs.exists(src):
                os.makedirs(os.path.dirname(dst) or ".", exist_ok=True)
                self.fs.get(src, dst, recursive=True)
        return dst

    def listdir(self, rel: str) -> List[str]:
        if not self.remote:
            d = os.path.join(self.local, rel)
            return sorted(os.listdir(d)) if os.path.isdir(d) else []
        src = self.rpath.rstrip("/") + "/" + rel
        if not self.fs.exists(src):
            return []
        return sorted(os.path.basename(str(e).rstrip("/")) for e in self.fs.ls(src, detail=False))

    def drop(self, rel: str):
        """Forget the scratch copy of one fetched entry (bounds local disk use while streaming a large table)."""
        if self.remote:
            p = os.path.join(self.local, rel)
            if os.path.isdir(p):
                shutil.rmtree(p, ignore_errors=True)
            elif os.path.exists(p):
                os.remove(p)

    def publish(self):
        if self.remote:
            self.fs.makedirs(self.rpath, exist_ok=True)
            for name in os.listdir(self.local):
                self.fs.put(os.path.join(self.local, name), self.rpath.rstrip("/") + "/" + name, recursive=True)
            shutil.rmtree(self.local, ignore_errors=True)

    def close(self):
        if self.remote:
            shutil.rmtree(self.local, ignore_errors=True)


# ------------------------------------------------------------------------------------------------
# streamed reading
# ------------------------------------------------------------------------------------------------
def iter_rank_dir(rank_dir: str, kind: int, dim: int, use_cvm: bool, chunk_rows: Optional[int] = None,
                  files_in_flight: int = 8) -> Iterator[Tuple[np.ndarray, np.ndarray]]:
    """Yield ``(signs uint64 [m], rows float32 [m, row_floats])`` pieces of every block file of one rank directory.
    Up to ``files_in_flight`` files are decompressed and parsed side by side (native code, the GIL is released);
    at most that many pieces of ``chunk_rows`` rows exist at a time."""
    ext = _build.cpu_ext()
    chunk_rows = int(chunk_rows or config.checkpoint_load_chunk_rows)
    files = ext.list_block_files(rank_dir)
    if not files:
        return
    readers = [ext.SparseBlockReader(os.path.join(rank_dir, f), kind, dim, use_cvm) for f in files]
    with ThreadPoolExecutor(max_workers=max(1, min(files_in_flight, len(readers)))) as pool:
        live = list(readers)
        while live:
            futures = [(r, pool.submit(r.next, chunk_rows)) for r in live]
            live = []
            for r, fut in futures:
                signs, rows = fut.result()
                if len(signs):
                    live.append(r)
                    yield signs, rows


def load_sparse_table(table, path: str, mode: str = "txt") -> int:
    rt = runtime()
    view = LocalView(path)
    rel = os.path.join("sparse_table", _table_dirname(table))
    dirs = [d for d in view.listdir(rel) if re.fullmatch(r"rank_\d+", d)]
    dirs.sort(key=lambda s: int(s.split("_")[1]))
    if not dirs:
        view.close()
        raise FileNotFoundError(f"no sparse table checkpoint under {os.path.join(path, rel)}")
    same_world = len(dirs) == rt.world
    total = 0
    try:
        for d in ([f"rank_{rt.rank}"] if same_world else dirs):
            local = view.fetch(os.path.join(rel, d))
            for signs, rows in iter_rank_dir(local, table.kind, table.dim, table.use_cvm):
                if not same_world and rt.world > 1:
                    keep = (signs % np.uint64(rt.world)) == np.uint64(rt.rank)
                    signs, rows = signs[keep], rows[keep]
                if len(signs):
                    table.load_rows(signs, rows)
                    total += len(signs)
            view.drop(os.path.join(rel, d))
    finally:
        view.close()
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

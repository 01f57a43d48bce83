"""Checkpoint tools: what the reference ships as Spark jobs (tensornet_tools/python/{merge_sparse,
resize_sparse,resize_dense,merge_extra_embedding}.py) as plain functions and a CLI.

Every sparse tool streams: block files are read in pieces (``checkpoint.iter_rank_dir``) and written through
``SparseDirWriter`` objects that keep their eight block files open, so a table far larger than host memory goes
through with a few pieces in memory.  The reference used Spark for these because its dictionaries "may approach
TB" (doc/tutorial/05-export-sparse-feature-embedding.ipynb:156).
"""
from __future__ import annotations

import gzip
import os
import re
from typing import Dict, Iterator, Optional, Tuple

import numpy as np

from .. import _build
from ..utils.checkpoint import iter_rank_dir

KINDS = {"AdaGrad": 0, "Adam": 1, "Ftrl": 2}


def _rank_dirs(table_dir: str):
    ds = [d for d in os.listdir(table_dir) if re.fullmatch(r"rank_\d+", d)]
    return sorted(ds, key=lambda s: int(s.split("_")[1]))


def _sniff(table_dir: str) -> Tuple[str, int]:
    """Optimizer name and dim of a table checkpoint (from the first text block, or given by the caller for bin)."""
    for r in _rank_dirs(table_dir):
        for f in sorted(os.listdir(os.path.join(table_dir, r))):
            if f.endswith(".gz") and "_bin" not in f:
                with gzip.open(os.path.join(table_dir, r, f), "rt") as fh:
                    l1, l2 = fh.readline(), fh.readline()
                if l1.startswith("opt_name:"):
                    return l1.strip().split(":")[1], int(l2.strip().split(":")[1])
    raise ValueError("cannot infer optimizer/dim (binary checkpoint): pass opt_name= and dim=")


def iter_sparse_table(table_dir: str, opt_name: Optional[str] = None, dim: Optional[int] = None, use_cvm: bool = False,
                      chunk_rows: Optional[int] = None) -> Iterator[Tuple[np.ndarray, np.ndarray]]:
    """Pieces ``(signs uint64 [m], rows float32 [m, row_floats])`` of a table checkpoint, all rank directories in turn."""
    if opt_name is None or dim is None:
        opt_name, dim = _sniff(table_dir)
    for r in _rank_dirs(table_dir):
        yield from iter_rank_dir(os.path.join(table_dir, r), KINDS[opt_name], dim, use_cvm, chunk_rows)


def read_sparse_table(table_dir: str, opt_name: Optional[str] = None, dim: Optional[int] = None, use_cvm: bool = False):
    """All rows of a table checkpoint at once: (signs uint64 [n], rows float32 [n, row_floats], opt_name, dim).
    For inspection and tests; the tools below never hold a whole table."""
    ext = _build.cpu_ext()
    if opt_name is None or dim is None:
        opt_name, dim = _sniff(table_dir)
    signs, rows = [], []
    for s, x in iter_sparse_table(table_dir, opt_name, dim, use_cvm):
        signs.append(s)
        rows.append(x)
    rf = ext.row_floats(KINDS[opt_name], dim)
    return (np.concatenate(signs) if signs else np.zeros(0, np.uint64),
            np.concatenate(rows) if rows else np.zeros((0, rf), np.float32), opt_name, dim)


def merge_sparse(table_dir: str, out_file: str, opt_name: Optional[str] = None, dim: Optional[int] = None,
                 use_cvm: bool = False, brackets: bool = False, compress: bool = False) -> int:
    """Write ``sign \\t w0 \\t ... \\t w{dim-1}`` per line (optionally wrapped in ``[`` ``]`` columns): the embedding
    dictionary the serving side loads (tensornet_tools/python/merge_sparse.py:34-41, utils.py:309-316)."""
    if opt_name is None or dim is None:
        opt_name, dim = _sniff(table_dir)
    opener = gzip.open if compress else open
    os.makedirs(os.path.dirname(os.path.abspath(out_file)), exist_ok=True)
    n = 0
    with opener(out_file, "wt") as f:
        for signs, rows in iter_sparse_table(table_dir, opt_name, dim, use_cvm):
            lines = []
            for s, r in zip(signs.tolist(), rows[:, :dim]):
                w = "\t".join("%g" % x for x in r)
                lines.append(f"{s}\t[\t{w}\t]\n" if brackets else f"{s}\t{w}\n")
            f.write("".join(lines))
            n += len(signs)
    return n


def _writers(out_dir: str, world: int, mode: str, kind: int, dim: int, use_cvm: bool):
    ext = _build.cpu_ext()
    return [ext.SparseDirWriter(os.path.join(out_dir, f"rank_{r}"), mode, kind, dim, use_cvm, False, 0.0, 0, 0) for r in range(world)]


def _route(writers, signs: np.ndarray, rows: np.ndarray):
    world = len(writers)
    owner = (signs % np.uint64(world)).astype(np.int64)
    for r in range(world):
        m = owner == r
        if m.any():
            writers[r].append(np.ascontiguousarray(signs[m]), np.ascontiguousarray(rows[m]))


def resize_sparse(table_dir: str, out_dir: str, new_world: int, mode: str = "txt", opt_name: Optional[str] = None,
                  dim: Optional[int] = None, use_cvm: bool = False) -> int:
    """Re-partition rows by ``sign % new_world`` into ``out_dir/rank_<r>/block_*``
    (tensornet_tools/python/resize_sparse.py:35-54)."""
    if opt_name is None or dim is None:
        opt_name, dim = _sniff(table_dir)
    writers = _writers(out_dir, new_world, mode, KINDS[opt_name], dim, use_cvm)
    n = 0
    for signs, rows in iter_sparse_table(table_dir, opt_name, dim, use_cvm):
        _route(writers, signs, rows)
        n += len(signs)
    for w in writers:
        w.close()
    return n


def resize_dense(table_dir: str, out_dir: str, new_world: int, opt_name: str = "Adam") -> int:
    """Concatenate the shard files ``0..N-1`` and cut them again into ``ceil(total/new_world)`` chunks
    (tensornet_tools/python/resize_dense.py:32-47).  Dense arrays are small next to the sparse tables."""
    ext = _build.cpu_ext()
    kind = 1 if opt_name == "Adam" else 0
    files = sorted((f for f in os.listdir(table_dir) if f.isdigit()), key=int)
    parts = [ext.read_dense_file(os.path.join(table_dir, f), kind) for f in files]
    cat = lambda k: np.concatenate([p[k] for p in parts])
    w, s0, s1 = cat("w"), cat("s0"), cat("s1")
    s2 = cat("s2") if len(parts[0]["s2"]) else None
    total = len(w)
    chunk = (total + new_world - 1) // new_world
    for r in range(new_world):
        lo, hi = r * chunk, min(total, (r + 1) * chunk)
        ext.write_dense_file(os.path.join(out_dir, str(r)), int(parts[0]["total_elements"]), new_world, kind, w[lo:hi], s0[lo:hi],
                             s1[lo:hi], None if s2 is None else s2[lo:hi], float(parts[0]["beta1_power"]),
                             float(parts[0]["beta2_power"]))
    return total


def merge_extra_embedding(table_dir: str, out_dir: str, sign_map: Dict[int, int], mode: str = "txt",
                          opt_name: Optional[str] = None, dim: Optional[int] = None, use_cvm: bool = False) -> int:
    """For every ``old -> new`` pair whose old sign exists (and whose new sign does not), add a row for the new sign
    with the old row's contents; the table keeps its rank count (tensornet_tools/python/merge_extra_embedding.py:39-83).

    Two streamed passes over the table: the first copies every row through and collects the rows of the old signs
    named in ``sign_map`` plus which of the new signs already exist; the second pass is only over those collected
    rows.  Memory is bounded by the size of ``sign_map``, not by the table."""
    if opt_name is None or dim is None:
        opt_name, dim = _sniff(table_dir)
    world = len(_rank_dirs(table_dir))
    writers = _writers(out_dir, world, mode, KINDS[opt_name], dim, use_cvm)
    olds = np.array(sorted(int(k) for k in sign_map), dtype=np.uint64)
    news = np.array(sorted(int(v) for v in sign_map.values()), dtype=np.uint64)
    found: Dict[int, np.ndarray] = {}
    new_present = set()
    for signs, rows in iter_sparse_table(table_dir, opt_name, dim, use_cvm):
        _route(writers, signs, rows)
        if len(olds):
            hit = np.isin(signs, olds)
            for s, r in zip(signs[hit].tolist(), rows[hit]):
                found[int(s)] = r.copy()
            new_present.update(signs[np.isin(signs, news)].tolist())
    add_s, add_r = [], []
    for old, new in sign_map.items():
        r = found.get(int(old))
        if r is not None and int(new) not in new_present and int(new) not in add_s:
            add_s.append(int(new))
            add_r.append(r)
    if add_s:
        _route(writers, np.array(add_s, dtype=np.uint64), np.stack(add_r))
    for w in writers:
        w.close()
    return len(add_s)

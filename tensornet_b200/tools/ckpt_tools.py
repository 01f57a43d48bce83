from __future__ import annotations

import gzip
import os
import re
from typing import Dict, Iterable, Optional, Tuple

import numpy as np

from .. import _build

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


def read_sparse_table(table_dir: str, opt_name: Optional[str] = None, dim: Optional[int] = None, use_cvm: bool = False):
    """All rows of a table checkpoint: (signs uint64 [n], rows float32 [n, row_floats], opt_name, dim)."""
    ext = _build.cpu_ext()
    if opt_name is None or dim is None:
        opt_name, dim = _sniff(table_dir)
    kind = KINDS[opt_name]
    signs, rows = [], []
    for r in _rank_dirs(table_dir):
        s, x = ext.read_sparse_dir(os.path.join(table_dir, r), kind, dim, use_cvm)
        signs.append(s)
        rows.append(x)
    rf = ext.row_floats(kind, dim)
    return (np.concatenate(signs) if signs else np.zeros(0, np.uint64),
            np.concatenate(rows) if rows else np.zeros((0, rf), np.float32), opt_name, dim)


def merge_sparse(table_dir: str, out_file: str, opt_name: Optional[str] = None, dim: Optional[int] = None,
                 use_cvm: bool = False, brackets: bool = False, compress: bool = False) -> int:
    """Write ``sign \\t w0 \\t ... \\t w{dim-1}`` per line (optionally wrapped in ``[`` ``]`` columns)."""
    signs, rows, opt_name, dim = read_sparse_table(table_dir, opt_name, dim, use_cvm)
    opener = gzip.open if compress else open
    os.makedirs(os.path.dirname(os.path.abspath(out_file)), exist_ok=True)
    with opener(out_file, "wt") as f:
        for s, r in zip(signs.tolist(), rows[:, :dim]):
            w = "\t".join("%g" % x for x in r)
            f.write(f"{s}\t[\t{w}\t]\n" if brackets else f"{s}\t{w}\n")
    return len(signs)


def resize_sparse(table_dir: str, out_dir: str, new_world: int, mode: str = "txt", opt_name: Optional[str] = None,
                  dim: Optional[int] = None, use_cvm: bool = False) -> int:
    """Re-partition rows by ``sign % new_world`` into ``out_dir/rank_<r>/block_*``."""
    ext = _build.cpu_ext()
    signs, rows, opt_name, dim = read_sparse_table(table_dir, opt_name, dim, use_cvm)
    kind = KINDS[opt_name]
    owner = (signs % np.uint64(new_world)).astype(np.int64)
    for r in range(new_world):
        m = owner == r
        ext.write_sparse_dir(os.path.join(out_dir, f"rank_{r}"), mode, kind, dim, use_cvm, np.ascontiguousarray(signs[m]),
                             np.ascontiguousarray(rows[m]), False, 0.0, 0, 0)
    return len(signs)


def resize_dense(table_dir: str, out_dir: str, new_world: int, opt_name: str = "Adam") -> int:
    """Concatenate the shard files ``0..N-1`` and cut them again into ``ceil(total/new_world)`` chunks."""
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
    """For every ``old -> new`` pair whose old sign exists, add a row for the new sign with the old row's
    contents; the table keeps its rank count."""
    ext = _build.cpu_ext()
    signs, rows, opt_name, dim = read_sparse_table(table_dir, opt_name, dim, use_cvm)
    world = len(_rank_dirs(table_dir))
    index = {int(s): i for i, s in enumerate(signs.tolist())}
    add_s, add_r = [], []
    for old, new in sign_map.items():
        i = index.get(int(old))
        if i is not None and int(new) not in index:
            add_s.append(int(new))
            add_r.append(rows[i])
    if add_s:
        signs = np.concatenate([signs, np.array(add_s, dtype=np.uint64)])
        rows = np.concatenate([rows, np.stack(add_r)])
    owner = (signs % np.uint64(world)).astype(np.int64)
    for r in range(world):
        m = owner == r
        ext.write_sparse_dir(os.path.join(out_dir, f"rank_{r}"), mode, KINDS[opt_name], dim, use_cvm,
                             np.ascontiguousarray(signs[m]), np.ascontiguousarray(rows[m]), False, 0.0, 0, 0)
    return len(add_s)

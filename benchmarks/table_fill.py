"""Fill one GPU shard of a hashed embedding table with N distinct signs (default 1e8, dim 8, AdaGrad rows), then look
every sign up again: insert and lookup rates, key-array load factor, device memory held.

    python benchmarks/table_fill.py --rows 100000000 --dim 8

The signs are generated on the device in pieces of 4 M (a 64-bit mixing function of a counter, so they are distinct
and spread over the whole key space); nothing of size N ever lives on the host.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

import tensornet_b200 as tn
from tensornet_b200.ops.sparse_table_gpu import GpuSparseTable


def signs(lo: int, n: int, dev) -> torch.Tensor:
    """Distinct pseudo-random int64 signs for the counters lo .. lo+n-1 (odd multiplier = bijection on 2^64)."""
    x = torch.arange(lo + 1, lo + n + 1, dtype=torch.int64, device=dev)
    return x * -7046029254386353131         # 0x9E3779B97F4A7C15 as a signed 64-bit value: odd, so distinct counters stay distinct


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=100_000_000)
    ap.add_argument("--dim", type=int, default=8)
    ap.add_argument("--piece", type=int, default=4 << 20)
    a = ap.parse_args()
    tn.core.init()
    rt = tn.core.runtime()
    dev = rt.device
    torch.cuda.reset_peak_memory_stats()
    t = GpuSparseTable(tn.core.AdaGrad(learning_rate=0.01), a.dim, rows=a.rows + 1024)
    idx = torch.empty(a.piece, dtype=torch.int32, device=dev)
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    torch.cuda.synchronize()
    e0.record()
    for lo in range(0, a.rows, a.piece):
        n = min(a.piece, a.rows - lo)
        t.ext.table_insert_keys(t.table_dict(), signs(lo, n, dev), idx[:n], rt.status)
    e1.record()
    found = 0
    for lo in range(0, a.rows, a.piece):
        n = min(a.piece, a.rows - lo)
        found += int((t.lookup_rows(signs(lo, n, dev)) >= 0).sum())
    e2.record()
    torch.cuda.synchronize()
    rt.check_status()
    ins_ms, look_ms = e0.elapsed_time(e1), e1.elapsed_time(e2)
    print(json.dumps({"rows": a.rows, "dim": a.dim, "n_rows_in_table": t.n_rows, "all_found": found == a.rows,
                      "insert_Mkeys_per_s": a.rows / ins_ms / 1e3, "lookup_Mkeys_per_s": a.rows / look_ms / 1e3,
                      "key_array_load_factor": a.rows / t.keys.numel(),
                      "device_GB": torch.cuda.max_memory_allocated() / 1e9}), flush=True)
    tn.core.shutdown()


if __name__ == "__main__":
    main()

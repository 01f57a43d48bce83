"""Sparse pull / push micro-benchmark: hashed fp32 tables, uint64 ids Zipf(s=1.05) over 2^40, AdaGrad.

Reports, per embedding dim and batch size, the device time of the fused pull and push kernels,
the bytes they move (ids out + rows back; gradient records out + row read-modify-write) and the
achieved GB/s, against the same exchange done with library calls only (torch.unique +
all_to_all_single + index ops) and against the roofline (HBM copy bandwidth on one GPU, NVLink
per-direction bandwidth across GPUs).  Multi-GPU numbers are the max over ranks.

    python benchmarks/sparse_microbench.py --dims 8 64 128 --ids 65536 1048576 --rows 20000000
    torchrun --nproc-per-node 8 benchmarks/sparse_microbench.py ...
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np
import torch
import torch.distributed as dist

import tensornet_b200 as tn


def zipf_ids(n, rng, s=1.05, N=float(2 ** 40)):
    u = rng.random(n)
    x = np.floor(((N ** (1 - s) - 1) * u + 1) ** (1 / (1 - s))).astype(np.uint64)
    x ^= x >> np.uint64(33); x *= np.uint64(0xff51afd7ed558ccd); x ^= x >> np.uint64(33)
    return torch.from_numpy(x.view(np.int64))


def time_us(fn, iters, rt):
    rt.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k in range(iters):
        fn(k)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], dtype=torch.float64)
    if rt.world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=rt.host_group)
    return float(t)


def nccl_baseline_pull(ids, table_rows, dim, rt):
    """Library-only pull: unique, bucket by owner, all_to_all ids, gather rows, all_to_all rows back."""
    W = rt.world
    u, inv = torch.unique(ids, return_inverse=True)
    if W == 1:
        return table_rows[(u % table_rows.shape[0])][inv]
    owner = (u.view(torch.int64) % W + W) % W
    order = torch.argsort(owner)
    counts = torch.bincount(owner, minlength=W)
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts, group=rt.device_group)
    sc, rc = counts.tolist(), recv_counts.tolist()
    recv_ids = torch.empty(sum(rc), dtype=torch.int64, device=ids.device)
    dist.all_to_all_single(recv_ids, u[order], rc, sc, group=rt.device_group)
    rows = table_rows[recv_ids % table_rows.shape[0]]
    back = torch.empty(u.numel(), dim, device=ids.device)
    dist.all_to_all_single(back, rows, sc, rc, group=rt.device_group)
    out = torch.empty_like(back)
    out[order] = back
    return out[inv]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dims", type=int, nargs="+", default=[8, 64, 128])
    ap.add_argument("--ids", type=int, nargs="+", default=[65536, 1048576])
    ap.add_argument("--rows", type=int, default=20_000_000, help="row capacity per GPU")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--pool", type=int, default=4)
    a = ap.parse_args()
    tn.core.init()
    rt = tn.core.runtime()
    from tensornet_b200.ops.sparse_table_gpu import GpuSparseTable
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm = peaks.get("hbm_gbs", 6650.0)
    link = 770.0
    rng = np.random.default_rng(100 + rt.rank)
    results = []
    for dim in a.dims:
        for n in a.ids:
            t = GpuSparseTable(tn.core.AdaGrad(learning_rate=0.01, initial_g2sum=0.1, initial_scale=0.1), dim, rows=a.rows)
            lk = t.link(n)
            batches = [zipf_ids(n, rng).to(rt.device) for _ in range(a.pool)]
            for b in batches + batches:                         # populate, then steady state
                lk.pull(b, training=True); lk.gU[:, :dim] += 1e-3; lk.push()
            torch.cuda.synchronize(); rt.check_status()
            uniq = []
            def pull(k):
                lk.pull(batches[k % a.pool], training=True)
            def pull_push(k):
                lk.pull(batches[k % a.pool], training=True); lk.push()
            t_pull = time_us(pull, a.iters, rt)
            for _ in range(1):
                lk.push()
            t_both = time_us(pull_push, a.iters, rt)
            t_push = t_both - t_pull
            nu = float(sum(lk.unique_counts()))
            W = rt.world
            remote = (W - 1) / W
            row_b, rec_b = 4 * t.ustride, 4 * t.gstride
            pull_bytes = n * 8 + nu * (8 + row_b) + nu * row_b       # read ids, write staged ids, read rows, write rows
            push_bytes = nu * rec_b + nu * 2 * 4 * t.stride            # read records, read + write the stored rows
            pull_link = nu * remote * (8 + row_b)
            push_link = nu * remote * rec_b
            dense_rows = torch.randn(1 << 20, dim, device=rt.device)
            t_base = time_us(lambda k: nccl_baseline_pull(batches[k % a.pool], dense_rows, dim, rt), max(2, a.iters // 2), rt)
            floor_pull = max(pull_bytes / (hbm * 1e3), pull_link / (link * 1e3))      # us
            floor_push = max(push_bytes / (hbm * 1e3), push_link / (link * 1e3))
            r = dict(dim=dim, ids_per_gpu=n, unique=nu, world=W, pull_us=t_pull, push_us=t_push,
                     pull_GBps=pull_bytes / t_pull / 1e3, push_GBps=push_bytes / t_push / 1e3,
                     pull_roofline_frac=floor_pull / t_pull, push_roofline_frac=floor_push / t_push,
                     library_pull_us=t_base, speedup_vs_library_pull=t_base / t_pull, phases_us=lk.pull_phase_us(),
                     roofline="of measured HBM copy bandwidth" if "hbm_gbs" in peaks else "of fallback 6.65 TB/s")
            results.append(r)
            if rt.rank == 0:
                print(json.dumps(r), flush=True)
            del t, lk, batches
            torch.cuda.empty_cache()
    tn.core.shutdown()


if __name__ == "__main__":
    main()

"""Sparse pull / push micro-benchmark: hashed fp32 tables, uint64 ids Zipf(s=1.05) over 2^40, AdaGrad.

The tables hold ``--rows`` rows across the job (1e8 by default, every GPU its ``sign % world`` share), filled before
anything is timed; ids are Zipf ranks folded onto that universe, so the timed steps run against a full table with
no inserts.  Per embedding dim and batch size the script reports the device time of the fused pull and push
kernels, the bytes they move and the achieved GB/s, against

* the same exchange written with library calls only (``library_*``): ``torch.unique`` + NCCL ``all_to_all_single``
  + a sorted key array with ``searchsorted`` + index ops for the pull; ``all_to_all_single`` + ``unique`` +
  ``index_add_`` + an AdaGrad update in torch ops for the push; timed after two warm-up calls;
* the roofline: the slower of (bytes through HBM / measured HBM copy bandwidth) and (bytes that must cross NVLink /
  the SM-issued peer-store bandwidth measured by ``p2p_microbench.py``, 690 GB/s per direction per GPU).

Multi-GPU numbers are device times, max over ranks.

    python benchmarks/sparse_microbench.py --dims 8 64 128 --ids 65536 1048576 4194304
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/sparse_microbench.py ...
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

import tensornet_b200 as tn

LINK_GBS = 690.0          # SM-issued peer stores, per direction per GPU (profiles/peer_copy_link_probe_2gpu.md)
_ODD = -7046029254386353131


def sign_of(x):
    """Sign of universe rank ``x`` (int64 tensor): an odd multiplier is a bijection on 2^64."""
    return (x + (1 << 42)) * _ODD


def zipf_ids(n, gen, universe, dev):
    u = torch.rand(n, generator=gen, device=dev, dtype=torch.float64)
    x = torch.floor((1.0 - 0.75 * u) ** -20.0).to(torch.int64).clamp_(1, 1 << 40)      # Zipf(1.05) over [1, 2^40]
    folded = (((x * _ODD) >> 20) & ((1 << 40) - 1)) % universe + 1
    return sign_of(torch.where(x > universe, folded, x))


def time_us(fn, iters, rt, warm=2):
    for k in range(warm):
        fn(k)
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


def time_pair_us(first, second, iters, rt, warm=2):
    """Device time of ``first(k)`` and of ``second(k)`` run back to back, each from its own event pair (max over ranks)."""
    for k in range(warm):
        first(k)
        second(k)
    rt.barrier()
    torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(iters)]
    for k in range(iters):
        ev[k][0].record()
        first(k)
        ev[k][1].record()
        second(k)
        ev[k][2].record()
    torch.cuda.synchronize()
    a = sorted(e[0].elapsed_time(e[1]) * 1e3 for e in ev)[iters // 2]
    b = sorted(e[1].elapsed_time(e[2]) * 1e3 for e in ev)[iters // 2]
    t = torch.tensor([a, b], dtype=torch.float64)
    if rt.world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=rt.host_group)
    return float(t[0]), float(t[1])


class LibraryTable:
    """The same sharded table from library calls: sorted keys + searchsorted, rows in a dense tensor, AdaGrad in torch ops."""

    def __init__(self, universe, dim, rt, lr=0.01, g2=0.1):
        self.rt, self.dim, self.lr = rt, dim, lr
        W, R, dev = rt.world, rt.rank, rt.device
        keys = []
        step = 1 << 24
        for lo in range(0, universe, step):
            s = sign_of(torch.arange(lo + 1, min(universe, lo + step) + 1, device=dev, dtype=torch.int64))
            keys.append(s[self.owner(s) == R] if W > 1 else s)
        self.keys = torch.sort(torch.cat(keys)).values
        n = self.keys.numel()
        self.w = torch.randn((n, dim), device=dev) * 0.01
        self.g2 = torch.full((n,), g2, device=dev)
        self.show = torch.zeros(n, device=dev)

    def owner(self, s):
        return ((s >> 7) & 0xFFFFFFFF) % self.rt.world

    def a2a(self, x, sc, rc):
        out = x.new_empty((int(sum(rc)),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x, output_split_sizes=rc, input_split_sizes=sc, group=self.rt.device_group)
        return out

    def pull(self, ids):
        W = self.rt.world
        uniq, inv = torch.unique(ids, return_inverse=True)
        if W > 1:
            own = self.owner(uniq)
            order = torch.argsort(own)
            counts = torch.bincount(own, minlength=W)
            rcounts = torch.empty_like(counts)
            dist.all_to_all_single(rcounts, counts, group=self.rt.device_group)
            self.sc, self.rc = counts.tolist(), rcounts.tolist()
            req = self.a2a(uniq[order], self.sc, self.rc)
        else:
            order, req = None, uniq
        self.rows_idx = torch.searchsorted(self.keys, req).clamp_(max=self.keys.numel() - 1)
        vals = self.w[self.rows_idx]
        if W > 1:
            back = self.a2a(vals, self.rc, self.sc)
            U = torch.empty_like(back)
            U[order] = back
        else:
            U = vals
        self.order, self.inv = order, inv
        return U

    def push(self, gU):
        """gU: gradient per unique sign of the last pull."""
        g = gU
        if self.rt.world > 1:
            g = self.a2a(gU[self.order].contiguous(), self.sc, self.rc)
        ur, uinv = torch.unique(self.rows_idx, return_inverse=True)
        gs = torch.zeros((ur.numel(), self.dim), device=g.device).index_add_(0, uinv, g)
        cnt = torch.zeros(ur.numel(), device=g.device).index_add_(0, uinv, torch.ones_like(uinv, dtype=torch.float32))
        g2 = self.g2[ur] + (gs * gs).sum(1) / self.dim
        self.g2[ur] = g2
        self.show[ur] += cnt
        self.w[ur] -= self.lr * gs / (1e-8 + g2.sqrt()).unsqueeze(1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dims", type=int, nargs="+", default=[8, 64, 128])
    ap.add_argument("--ids", type=int, nargs="+", default=[65536, 1048576, 4194304], help="ids per GPU per step")
    ap.add_argument("--rows", type=int, default=100_000_000, help="rows of the table across the whole job")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--pool", type=int, default=4)
    ap.add_argument("--no-library", action="store_true")
    a = ap.parse_args()
    tn.core.init()
    rt = tn.core.runtime()
    dev = rt.device
    W = rt.world
    from tensornet_b200.ops.sparse_table_gpu import GpuSparseTable
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm = peaks.get("hbm_gbs", 6650.0)
    universe = a.rows
    for dim in a.dims:
        t = GpuSparseTable(tn.core.AdaGrad(learning_rate=0.01, initial_g2sum=0.1, initial_scale=0.1), dim,
                           rows=int(universe / W * 1.2) + (1 << 16))
        lib = None
        for n in a.ids:
            lk = t.link(n)
            if t.n_rows == 0:
                # fill: every GPU pulls its stride of the universe in pieces the link can take
                piece = min(n, 1 << 20)
                n_pieces = (universe + piece - 1) // piece
                for k in range((n_pieces + W - 1) // W):
                    c = min(k * W + rt.rank, n_pieces - 1)
                    x = (torch.arange(c * piece, (c + 1) * piece, device=dev, dtype=torch.int64) + 1).clamp_(max=universe)
                    lk.pull(sign_of(x), training=False)
                torch.cuda.synchronize()
                rt.check_status()
                rt.barrier()
            gen = torch.Generator(device=dev).manual_seed(100 + rt.rank)
            batches = [zipf_ids(n, gen, universe, dev) for _ in range(a.pool)]

            def pull(k):
                lk.pull(batches[k % a.pool], training=True)

            def pull_push(k):
                lk.pull(batches[k % a.pool], training=True)
                lk.push()

            for k in range(a.pool):
                pull_push(k)
                lk.gU[:, :dim] += 1e-3
            torch.cuda.synchronize()
            rt.check_status()
            t_pull, t_push = time_pair_us(pull, lambda k: lk.push(), a.iters, rt)      # medians, each from its own events
            nu = float(sum(lk.unique_counts()))
            remote = (W - 1) / W
            row_b, rec_b = 4 * t.ustride, 4 * t.gstride
            pull_bytes = n * 8 + nu * (8 + row_b) + nu * row_b       # read ids, write staged ids, read rows, write rows
            push_bytes = nu * rec_b + nu * 2 * 4 * t.stride            # read records, read + write the stored rows
            pull_link = nu * remote * (8 + row_b)
            push_link = nu * remote * rec_b
            floor_pull = max(pull_bytes / (hbm * 1e3), pull_link / (LINK_GBS * 1e3))      # us
            floor_push = max(push_bytes / (hbm * 1e3), push_link / (LINK_GBS * 1e3))
            r = dict(dim=dim, ids_per_gpu=n, unique=nu, world=W, table_rows_job=int(sum(rt.all_gather_object(t.n_rows))),
                     pull_us=t_pull, push_us=t_push, pull_GBps=pull_bytes / t_pull / 1e3, push_GBps=push_bytes / t_push / 1e3,
                     pull_link_GBps=pull_link / t_pull / 1e3, push_link_GBps=push_link / t_push / 1e3,
                     pull_roofline_frac=floor_pull / t_pull, push_roofline_frac=floor_push / t_push,
                     phases_us=[round(x, 1) for x in lk.pull_phase_us()],
                     roofline=("of measured HBM copy bandwidth" if "hbm_gbs" in peaks else "of fallback 6.65 TB/s") +
                              f" and {LINK_GBS:.0f} GB/s SM-issued peer stores")
            if not a.no_library:
                if lib is None:
                    lib = LibraryTable(universe, dim, rt)
                state = {}

                def lib_pull(k):
                    state["U"] = lib.pull(batches[k % a.pool])

                def lib_push(k):
                    lib.push(torch.full_like(state["U"], 1e-3))

                tl_pull, tl_push = time_pair_us(lib_pull, lib_push, max(5, a.iters // 2), rt)      # medians, each from its own events
                r.update(library_pull_us=tl_pull, library_push_us=tl_push, speedup_vs_library_pull=tl_pull / t_pull,
                         speedup_vs_library_push=tl_push / t_push)
            if rt.rank == 0:
                print(json.dumps(r), flush=True)
            t.links.remove(lk)
            del lk, batches
            torch.cuda.empty_cache()
        del t, lib
        torch.cuda.empty_cache()
    tn.core.shutdown()


if __name__ == "__main__":
    main()

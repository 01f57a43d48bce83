"""Dense path micro-benchmark: fused (barrier + in-switch reduce-scatter + Adam + all-gather, one kernel) against
the same step built from library collectives (NCCL reduce_scatter_tensor + torch Adam ops + all_gather_into_tensor).
Device-timed, max over ranks.  Roofline: the fused step moves 4P*(W-1)/W bytes in and (4+2)P*(W-1)/W bytes out
per GPU over NVLink (P = parameter count); at one GPU it is the HBM-bound Adam sweep (34 B per element).

    torchrun --nproc-per-node 4 benchmarks/dense_microbench.py --params 500000 130000000
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
from tensornet_b200.ops.dense_table import DenseTable


def timed(fn, iters, rt):
    for _ in range(3):
        fn()
    rt.barrier(); torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record(); torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], dtype=torch.float64)
    if rt.world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=rt.host_group)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=int, nargs="+", default=[500_000, 130_000_000])
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    tn.core.init()
    rt = tn.core.runtime()
    W, dev = rt.world, rt.device
    for P in a.params:
        p = torch.nn.Parameter(torch.randn(P, device=dev))
        dt = DenseTable(tn.core.Adam(learning_rate=1e-3)); dt.init([("p", p)])
        def fused():
            dt.step()
        t_fused = timed(fused, a.iters, rt)
        # library baseline on plain tensors
        n = dt.n
        g = torch.randn(n, device=dev); w = torch.randn(n, device=dev)
        chunk = n // W
        gs = torch.empty(chunk, device=dev); m = torch.zeros(chunk, device=dev); v = torch.zeros(chunk, device=dev)
        wb = torch.empty(n, dtype=torch.bfloat16, device=dev)
        def library():
            if W > 1:
                dist.reduce_scatter_tensor(gs, g, op=dist.ReduceOp.AVG, group=rt.device_group)
            else:
                gs.copy_(g)
            ws = w[rt.rank * chunk:(rt.rank + 1) * chunk]
            m.lerp_(gs, 0.1)
            v.mul_(0.999).addcmul_(gs, gs, value=0.001)
            ws.addcdiv_(m, v.sqrt().add_(1e-8), value=-1e-3)
            if W > 1:
                dist.all_gather_into_tensor(w, ws.clone(), group=rt.device_group)
            wb.copy_(w)
            g.zero_()
        t_lib = timed(library, a.iters, rt)
        link_bytes = (4 + 4 + 2) * n * (W - 1) / W
        floor = max(link_bytes / 770e3, 34.0 * n / W / 6464.6e3) if W > 1 else 34.0 * n / 6464.6e3     # us
        if rt.rank == 0:
            print(json.dumps({"params": P, "world": W, "fused_us": t_fused, "library_us": t_lib, "speedup": t_lib / t_fused,
                              "roofline_us": floor, "fraction_of_roofline": floor / t_fused, "multimem": bool(dt.uses_multimem)}), flush=True)
        del dt, p, g, w
        torch.cuda.empty_cache()
    tn.core.shutdown()


if __name__ == "__main__":
    main()

"""Multi-hot DLRM / DCN-v2 training benchmark: 100 categorical slots with bag length Poisson(5) (min 1) and sum
pooling, uint64 ids Zipf(1.05) over 2^40, embedding dim 64 with sparse FTRL, 13 dense features, 3 DCN-v2 cross
layers on the 6413-wide concat (tcgen05 GEMMs with the Hadamard-residual epilogue), bf16 MLP 1024-512-256-1,
8192 examples per GPU.  The tables are filled with the whole sign universe (``--universe`` signs across the job,
``--universe 1000000000`` is the named configuration: 1.25e8 FTRL rows of 784 bytes per GPU on eight GPUs) before
anything is timed, and Zipf ranks beyond a slot's share of the universe are folded onto it, so the timed steps run
against full tables.  Ragged inputs run eagerly (no CUDA graph).  Prints one JSON line on rank 0.

    python benchmarks/dcn_bench.py --steps 10
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/dcn_bench.py --steps 10 --universe 1000000000
    TN_FORCE_CPU=1 python benchmarks/dcn_bench.py --steps 2 --warmup 1 --batch 512 --universe 200000     # CPU baseline (wall clock)
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


_ODD = np.uint64(0x9E3779B97F4A7C15)      # odd: x -> x * _ODD is a bijection on 2^64


def slot_signs(x, slot):
    """Sign of rank ``x`` of slot ``slot`` (uint64 arrays): distinct per (slot, rank)."""
    return (x + ((slot + np.uint64(1)) << np.uint64(42))) * _ODD


def make_batch(rng, B, S, mean_len, n_dense, ranks_per_slot):
    lens = np.maximum(rng.poisson(mean_len, (S, B)), 1)
    offs = np.concatenate([[0], np.cumsum(lens.reshape(-1))]).astype(np.int32)
    n = int(offs[-1])
    s, N = 1.05, float(2 ** 40)
    x = np.floor(((N ** (1 - s) - 1) * rng.random(n) + 1) ** (1 / (1 - s))).astype(np.uint64)
    R = np.uint64(ranks_per_slot)
    folded = (((x * _ODD) >> np.uint64(20)) & np.uint64((1 << 40) - 1)) % R + np.uint64(1)
    x = np.where(x > R, folded, x)
    slot = np.repeat(np.arange(S, dtype=np.uint64), lens.sum(axis=1))
    h = slot_signs(x, slot)
    pin = (lambda t: t.pin_memory()) if torch.cuda.is_available() and tn.core.runtime().on_gpu else (lambda t: t)
    return (pin(torch.from_numpy(h.view(np.int64))), pin(torch.from_numpy(offs)),
            pin(torch.from_numpy(np.log1p(rng.exponential(1.0, (B, n_dense))).astype(np.float32))),
            pin(torch.from_numpy((rng.random(B) < 0.25).astype(np.float32))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8192)
    ap.add_argument("--slots", type=int, default=100)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--universe", type=int, default=0, help="distinct signs across the job (default: 24 M per GPU)")
    ap.add_argument("--pool", type=int, default=4)
    a = ap.parse_args()
    tn.core.init()
    rt = tn.core.runtime()

    def sync():
        if rt.on_gpu:
            torch.cuda.synchronize()

    universe = a.universe or 24_000_000 * rt.world
    ranks_per_slot = max(1, universe // a.slots)
    a.rows = int(ranks_per_slot * a.slots / rt.world * 1.1) + (1 << 16)      # this GPU's share of the universe plus head-room
    tn.core.config.table_grow_at = 0.0                                       # sized for the universe: nothing to grow into
    slots = [str(i) for i in range(a.slots)]
    torch.manual_seed(0)
    max_ids = int(a.batch * a.slots * 5 * 1.3)
    model = tn.models.DCNv2(slots, dnn_hidden_units=(1024, 512, 256), embedding_dim=a.dim, dense_dim=13,
                            sparse_opt=tn.core.Ftrl(learning_rate=0.05, lambda1=1e-4, lambda2=1e-3, initial_scale=0.05),
                            bucket_size=max_ids // a.slots, combiner="sum", num_cross=3, table_rows=a.rows)
    model.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=1e-3)), cuda_graph=False)
    # fill: every GPU pulls its stride of the universe through the layer's own link, in pieces of one batch's capacity
    import time
    t_fill = time.time()
    link = model.deep_emb.link
    piece = min(max_ids, 4 << 20)
    per_slot_pieces = (ranks_per_slot + piece - 1) // piece
    jobs = [(s_, c) for s_ in range(a.slots) for c in range(per_slot_pieces)]
    for k in range((len(jobs) + rt.world - 1) // rt.world):
        s_, c = jobs[min(k * rt.world + rt.rank, len(jobs) - 1)]
        x = (torch.arange(c * piece, (c + 1) * piece, device=rt.device, dtype=torch.int64) + 1).clamp_(max=ranks_per_slot)
        link.pull((x + ((s_ + 1) << 42)) * -7046029254386353131, training=False)
    sync(); rt.check_status(); rt.barrier()
    rows_here = link.table.n_rows
    rows_all = sum(rt.all_gather_object(rows_here))
    t_fill = time.time() - t_fill
    rng = np.random.default_rng(10 + rt.rank)
    data = [make_batch(rng, a.batch, a.slots, 5, 13, ranks_per_slot) for _ in range(a.pool)]

    def step(k):
        v, o, d, y = data[k % a.pool]
        f = {tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, values=v, offsets=o, batch_size=a.batch), "dense": d}
        return model.train_on_batch(f, y)

    for k in range(a.warmup):
        step(k)
    sync(); rt.check_status(); rt.barrier()
    if rt.on_gpu:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for k in range(a.steps):
            loss = step(k)
        e1.record(); sync(); rt.barrier(); rt.check_status()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64)
    else:                      # TN_FORCE_CPU=1: the same steps on the CPU path, wall clock (the CPU baseline of this config)
        t0 = time.perf_counter()
        for k in range(a.steps):
            loss = step(k)
        rt.barrier()
        t = torch.tensor([(time.perf_counter() - t0) * 1e3], dtype=torch.float64)
    if rt.world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=rt.host_group)
    ms = float(t) / a.steps
    D = a.slots * a.dim + 13
    flops = 2.0 * a.batch * ((D + 1) * D * 3 * 4 + 3 * ((D + 1) * 1024 + 1025 * 512 + 513 * 256))
    if rt.rank == 0:
        print(json.dumps({"metric": "train examples/sec (DCN-v2 multi-hot, device-timed incl. H2D, max over ranks)",
                          "value": a.batch * rt.world / ms * 1e3, "ms_per_step": ms, "n_gpus": rt.world, "loss": float(loss),
                          "dense_tflops_per_gpu": flops / ms / 1e9, "ids_per_gpu_per_step": int(data[0][0].numel()),
                          "config": {"slots": a.slots, "dim": a.dim, "cross_width": D, "batch_per_gpu": a.batch, "table_rows_resident": rows_all,
                                     "table_rows_this_gpu": rows_here, "table_GB_this_gpu": rows_here * getattr(link.table, "stride", 0) * 4 / 1e9, "device": str(rt.device),
                                     "table_fill_seconds": t_fill, "gate_first_gemm": bool(tn.core.config.gate_first_gemm)}}),
              flush=True)
    tn.core.shutdown()


if __name__ == "__main__":
    main()

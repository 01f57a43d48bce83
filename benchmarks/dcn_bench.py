"""Multi-hot DLRM / DCN-v2 training benchmark: 100 categorical slots with bag length Poisson(5) (min 1) and sum
pooling, uint64 ids Zipf(1.05) over 2^40, embedding dim 64 with sparse FTRL, 13 dense features, 3 DCN-v2 cross
layers on the 6413-wide concat (tcgen05 GEMMs with the Hadamard-residual epilogue), bf16 MLP 1024-512-256-1,
8192 examples per GPU.  Ragged inputs run eagerly (no CUDA graph).  Prints one JSON line on rank 0.

    python benchmarks/dcn_bench.py --steps 10
    torchrun --nproc-per-node 8 benchmarks/dcn_bench.py --steps 10
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


def make_batch(rng, B, S, mean_len, n_dense):
    lens = np.maximum(rng.poisson(mean_len, (S, B)), 1)
    offs = np.concatenate([[0], np.cumsum(lens.reshape(-1))]).astype(np.int32)
    n = int(offs[-1])
    s, N = 1.05, float(2 ** 40)
    x = np.floor(((N ** (1 - s) - 1) * rng.random(n) + 1) ** (1 / (1 - s))).astype(np.uint64)
    slot = np.repeat(np.arange(S, dtype=np.uint64), lens.sum(axis=1))
    h = x ^ ((slot + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15))
    h ^= h >> np.uint64(33); h *= np.uint64(0xff51afd7ed558ccd); h ^= h >> np.uint64(33)
    return (torch.from_numpy(h.view(np.int64)).pin_memory(), torch.from_numpy(offs).pin_memory(),
            torch.from_numpy(np.log1p(rng.exponential(1.0, (B, n_dense))).astype(np.float32)).pin_memory(),
            torch.from_numpy((rng.random(B) < 0.25).astype(np.float32)).pin_memory())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8192)
    ap.add_argument("--slots", type=int, default=100)
    ap.add_argument("--dim", type=int, default=64)
    ap.add_argument("--rows", type=int, default=24_000_000)
    ap.add_argument("--pool", type=int, default=4)
    a = ap.parse_args()
    tn.core.init()
    rt = tn.core.runtime()
    slots = [str(i) for i in range(a.slots)]
    torch.manual_seed(0)
    max_ids = int(a.batch * a.slots * 5 * 1.3)
    model = tn.models.DCNv2(slots, dnn_hidden_units=(1024, 512, 256), embedding_dim=a.dim, dense_dim=13,
                            sparse_opt=tn.core.Ftrl(learning_rate=0.05, lambda1=1e-4, lambda2=1e-3, initial_scale=0.05),
                            bucket_size=max_ids // a.slots, combiner="sum", num_cross=3, table_rows=a.rows)
    model.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=1e-3)), cuda_graph=False)
    rng = np.random.default_rng(10 + rt.rank)
    data = [make_batch(rng, a.batch, a.slots, 5, 13) for _ in range(a.pool)]

    def step(k):
        v, o, d, y = data[k % a.pool]
        f = {tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, values=v, offsets=o, batch_size=a.batch), "dense": d}
        return model.train_on_batch(f, y)

    for k in range(a.warmup):
        step(k)
    torch.cuda.synchronize(); rt.check_status(); rt.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k in range(a.steps):
        loss = step(k)
    e1.record(); torch.cuda.synchronize(); rt.barrier(); rt.check_status()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64)
    if rt.world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=rt.host_group)
    ms = float(t) / a.steps
    D = a.slots * a.dim + 13
    flops = 2.0 * a.batch * ((D + 1) * D * 3 * 4 + 3 * ((D + 1) * 1024 + 1025 * 512 + 513 * 256))
    if rt.rank == 0:
        print(json.dumps({"metric": "train examples/sec (DCN-v2 multi-hot, device-timed incl. H2D, max over ranks)",
                          "value": a.batch * rt.world / ms * 1e3, "ms_per_step": ms, "n_gpus": rt.world, "loss": float(loss),
                          "dense_tflops_per_gpu": flops / ms / 1e9, "ids_per_gpu_per_step": int(data[0][0].numel()),
                          "config": {"slots": a.slots, "dim": a.dim, "cross_width": D, "batch_per_gpu": a.batch, "table_rows_per_gpu": a.rows}}),
              flush=True)
    tn.core.shutdown()


if __name__ == "__main__":
    main()

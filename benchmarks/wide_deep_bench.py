"""Wide&Deep in the configuration of the reference's quick-start tutorial, the only training throughput it
publishes (doc/tutorial/01-begin-with-wide-deep.ipynb:446: 8 ms per step of 32 examples, ~4 000 examples/s on one CPU
host): 4 categorical slots (slots 1-3 one id, slot 4 three ids), embedding dim 1 (wide) + 8 (deep), MLP 512-256-256,
synchronised batch norm, AdaGrad(lr 0.01, g2sum 0.1, scale 0.1) for the tables, Adam for the dense part, batch 32
(examples/common/config.py:19-39).  ``--batch`` scales the batch; the step runs from one CUDA graph.

    python benchmarks/wide_deep_bench.py                 # the tutorial's batch 32
    python benchmarks/wide_deep_bench.py --batch 8192
    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/wide_deep_bench.py --batch 8192

Times K steps with CUDA events after W warm-up steps (max over ranks) and prints one JSON line; ``e2e`` includes the
host-to-device copy of each batch from pinned memory and the read-back of the loss.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np
import torch
import torch.distributed as dist

import tensornet_b200 as tn

REFERENCE_EXAMPLES_PER_S = 4000.0     # doc/tutorial/01-begin-with-wide-deep.ipynb:446 (750 steps of 32 in 6 s)


def make_batch(rng, B):
    """Slots 1-3 single id, slot 4 three ids, pools of hashed signs as in examples/gen_example_data.py."""
    pool = 100_000
    lens = np.concatenate([np.ones((3, B), np.int64), np.full((1, B), 3, np.int64)])
    offs = np.concatenate([[0], np.cumsum(lens.reshape(-1))]).astype(np.int32)
    n = int(offs[-1])
    slot = np.repeat(np.arange(4, dtype=np.uint64), lens.sum(axis=1))
    x = rng.integers(0, pool, n, dtype=np.int64).astype(np.uint64) ^ ((slot + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15))
    x ^= x >> np.uint64(33); x *= np.uint64(0xff51afd7ed558ccd); x ^= x >> np.uint64(33)
    pin = (lambda t: t.pin_memory()) if torch.cuda.is_available() else (lambda t: t)
    return (pin(torch.from_numpy(x.view(np.int64))), pin(torch.from_numpy(offs)),
            pin(torch.from_numpy((rng.random(B) < 0.25).astype(np.float32))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    a = ap.parse_args()
    tn.core.init()
    rt = tn.core.runtime()
    slots = ["1", "2", "3", "4"]
    torch.manual_seed(0)
    model = tn.models.WideDeep(slots, slots, dnn_hidden_units=(512, 256, 256), embedding_dim=8,
                               sparse_opt=tn.core.AdaGrad(learning_rate=0.01, initial_g2sum=0.1, initial_scale=0.1),
                               bucket_size=max(1024, 8 * a.batch), table_rows=1 << 20)
    model.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=1e-3)))
    rng = np.random.default_rng(3 + rt.rank)
    data = [make_batch(rng, a.batch) for _ in range(8)]

    def step(k):
        ids, offs, y = data[k % len(data)]
        f = {tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, values=ids, offsets=offs, batch_size=a.batch)}
        return model.train_on_batch(f, y)

    for k in range(a.warmup):
        step(k)
    gpu = rt.on_gpu
    if gpu:
        torch.cuda.synchronize()
    rt.barrier()
    if gpu:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    for k in range(a.steps):
        loss = step(k)
    if gpu:
        e1.record()
        torch.cuda.synchronize()
    last = float(loss)
    wall = time.perf_counter() - t0
    dev_ms = e0.elapsed_time(e1) / a.steps if gpu else wall * 1e3 / a.steps
    ms = torch.tensor([dev_ms, wall * 1e3 / a.steps], dtype=torch.float64)
    if rt.world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=rt.host_group)
    rt.check_status()
    if rt.rank == 0:
        eps = a.batch * rt.world / (float(ms[0]) / 1e3)
        print(json.dumps({"metric": "train examples/sec (Wide&Deep, reference tutorial config)", "value": eps, "unit": "examples/s",
                          "n_gpus": rt.world, "batch_per_gpu": a.batch, "ms_per_step": float(ms[0]), "ms_per_step_wall": float(ms[1]),
                          "vs_reference_published": eps / REFERENCE_EXAMPLES_PER_S, "last_loss": last,
                          "config": {"slots": 4, "ids_per_example": 6, "emb": "1 + 8", "mlp": "512-256-256", "bn": "synchronised",
                                     "sparse_opt": "AdaGrad", "dense_opt": "Adam", "data": "synthetic"}}), flush=True)
    rt.barrier()
    tn.core.shutdown()


if __name__ == "__main__":
    main()

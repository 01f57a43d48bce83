"""Serving benchmark: 200 single-hot slots, embedding dim 32 looked up in an exported dictionary,
bf16 MLP 6400->1024->512->256->1, request batches of 512 with ids Zipf(1.1) over 2^40.
Reports p50 / p99 latency (host wall clock per request batch incl. H2D of the ids and D2H of the
probabilities) and request batches / s.

    python benchmarks/serving_bench.py --requests 500
    TN_FORCE_CPU=1 python benchmarks/serving_bench.py --requests 40          # CPU baseline: dictionary lookup + fp32 towers on the host
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/serving_bench.py --sharded     # dictionary sharded over the GPUs

With ``--sharded`` every rank serves its own request batches while the lookups cross NVLink inside the fused pull
kernel (read-only); the reported rate is the sum over ranks and the latencies are those of the slowest rank.
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

import tensornet_b200 as tn
from tensornet_b200.layers import DenseHead, MLP
from tensornet_b200.serving import EmbeddingDictionary, InferenceEngine, ShardedInferenceEngine


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--slots", type=int, default=200)
    ap.add_argument("--dim", type=int, default=32)
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--dict-rows", type=int, default=5_000_000)
    ap.add_argument("--requests", type=int, default=300)
    ap.add_argument("--sharded", action="store_true", help="shard the dictionary over all ranks (sign %% world)")
    a = ap.parse_args()
    tn.core.init()
    rt = tn.core.runtime()
    rng = np.random.default_rng(0)
    signs = np.unique(rng.integers(1, 2 ** 40, a.dict_rows, dtype=np.int64).astype(np.uint64))
    weights = rng.standard_normal((len(signs), a.dim)).astype(np.float32) * 0.05
    torch.manual_seed(0)
    mlp = MLP(a.slots * a.dim, [1024, 512, 256]).to(rt.device)
    head = DenseHead(256).to(rt.device)
    if a.sharded:
        eng = ShardedInferenceEngine.from_dictionary(signs, weights, mlp, head, a.slots, a.slots * a.batch)
        rng = np.random.default_rng(100 + rt.rank)           # every rank serves its own requests
    else:
        eng = InferenceEngine(EmbeddingDictionary(signs, weights), mlp, head, a.slots)
    s = 1.1
    def req():
        u = rng.random((a.slots, a.batch))
        x = np.floor(((float(2 ** 40) ** (1 - s) - 1) * u + 1) ** (1 / (1 - s))).astype(np.int64)
        pick = signs[(x % len(signs))].view(np.int64)          # most requests hit the dictionary
        t = torch.from_numpy(np.where(rng.random((a.slots, a.batch)) < 0.9, pick, x))
        return t.pin_memory() if rt.on_gpu else t          # TN_FORCE_CPU=1: the same requests through the CPU path (the baseline)
    reqs = [req() for _ in range(16)]
    for r in reqs[:4]:
        eng.infer(r).cpu()
    lat = []
    t_all = time.perf_counter()
    for k in range(a.requests):
        t0 = time.perf_counter()
        p = eng.infer(reqs[k % len(reqs)]).cpu()
        lat.append((time.perf_counter() - t0) * 1e3)
    total = time.perf_counter() - t_all
    lat = np.array(lat)
    rate = a.requests / total
    if rt.world > 1:
        stats = rt.all_gather_object((float(np.percentile(lat, 50)), float(np.percentile(lat, 99)), rate))
        if rt.rank == 0:
            print(json.dumps({"metric": "sharded serving latency, batch %d x %d slots per rank" % (a.batch, a.slots), "world": rt.world,
                              "p50_ms": max(x[0] for x in stats), "p99_ms": max(x[1] for x in stats),
                              "request_batches_per_s": sum(x[2] for x in stats), "examples_per_s": sum(x[2] for x in stats) * a.batch,
                              "dict_rows": int(len(signs))}), flush=True)
        rt.barrier()
        tn.core.shutdown()
        return
    print(json.dumps({"metric": "serving latency, batch %d x %d slots" % (a.batch, a.slots), "p50_ms": float(np.percentile(lat, 50)),
                      "p99_ms": float(np.percentile(lat, 99)), "request_batches_per_s": a.requests / total,
                      "examples_per_s": a.requests * a.batch / total, "dict_rows": int(len(signs)), "device": str(rt.device),
                      "mean_prob": float(p.mean())}), flush=True)
    tn.core.shutdown()


if __name__ == "__main__":
    main()

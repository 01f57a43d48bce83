"""Serving demo (the role of examples/online_serving/main.cc in the reference): load the sparse dictionary
exported from a checkpoint and the dense sub-model saved by examples/main.py, then score request batches.
Unlike the reference demo, whose lookup returns random vectors, the ids are looked up in the real dictionary.

    python examples/main.py --data /tmp/tn_example_data --model-dir /tmp/tn_model --model deepfm --hidden 64 32
    python examples/online_serving.py --model-dir /tmp/tn_model --hidden 64 32
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

import tensornet_b200 as tn
from tensornet_b200.serving import EmbeddingDictionary, InferenceEngine, export_sparse_dictionary


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model-dir", default="/tmp/tn_model")
    ap.add_argument("--slots", type=int, default=4)
    ap.add_argument("--emb-dim", type=int, default=8)
    ap.add_argument("--hidden", type=int, nargs="+", default=[512, 256, 256])
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--requests", type=int, default=100)
    ap.add_argument("--export-tower", default="", help="also write the dense tower to this file for examples/native_serving/serve.cpp")
    a = ap.parse_args()
    tn.core.init()
    rt = tn.core.runtime()
    dt = tn.model.read_last_train_dt(a.model_dir)
    cp = os.path.join(a.model_dir, dt) if dt else a.model_dir
    dict_file = os.path.join(a.model_dir, "deep_input.dict.txt")
    n = export_sparse_dictionary(cp, "deep_input", dict_file)
    d = EmbeddingDictionary.from_file(dict_file, dim=a.emb_dim)
    # the dense tower of the trained model (MLP part of the sub-model; the demo scores with the deep tower only)
    mlp = tn.layers.MLP(a.slots * a.emb_dim, a.hidden).to(rt.device)
    head = tn.layers.DenseHead(a.hidden[-1]).to(rt.device)
    sd = torch.load(os.path.join(a.model_dir, "sub_model.pt"), map_location="cpu")
    with torch.no_grad():
        for k, v in sd.items():
            if k.startswith("mlp.weights.") and v.shape == mlp.weights[int(k.split(".")[-1])].shape:
                mlp.weights[int(k.split(".")[-1])].copy_(v)
    if a.export_tower:
        tn.serving.export_tower(mlp, head, a.export_tower)
    eng = InferenceEngine(d, mlp, head, a.slots, combiner="mean")
    g = torch.Generator().manual_seed(0)
    signs = torch.from_numpy(d.signs.view("int64")) if not rt.on_gpu else d.row_keys[: d.n].cpu()
    lat = []
    for _ in range(a.requests):
        ids = signs[torch.randint(0, max(d.n, 1), (a.slots, a.batch), generator=g)]
        t0 = time.perf_counter()
        p = eng.infer(ids).cpu()
        lat.append((time.perf_counter() - t0) * 1e3)
    lat.sort()
    print(json.dumps({"dictionary_rows": n, "requests": a.requests, "batch": a.batch, "p50_ms": lat[len(lat) // 2],
                      "p99_ms": lat[int(len(lat) * 0.99) - 1], "mean_probability": float(p.mean())}))
    tn.core.shutdown()


if __name__ == "__main__":
    main()

"""Synthetic click data (the role of examples/gen_example_data.py in the reference): a few files per
day, ``slots`` categorical features drawn from small id pools so ids repeat, one multi-valued slot,
a slot that is missing for negative examples, dense features and a label correlated with the ids.

Files are ``torch.save``d dicts of tensors: {"ids": {slot: (values, offsets)}, "dense": [N, D], "label": [N]}.
"""
from __future__ import annotations

import argparse
import os

import torch


def make_file(path: str, n: int, slots, dense_dim: int, seed: int, pool: int = 1000):
    g = torch.Generator().manual_seed(seed)
    label = (torch.rand(n, generator=g) < 0.3)
    ids = {}
    for k, s in enumerate(slots):
        base = torch.randint(0, pool, (n,), generator=g)
        # make the label learnable: positives prefer even ids in the first slot
        if k == 0:
            base = torch.where(label, base - base % 2, base | 1)
        sign = (base.long() * 2654435761 + (k + 1) * 0x9E3779B97F4A7C15 % (1 << 62)) & ((1 << 62) - 1)
        if k == len(slots) - 1:      # last slot: three ids for positives, none for negatives (missing feature)
            lens = torch.where(label, torch.tensor(3), torch.tensor(0))
            offsets = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
            vals = torch.randint(0, pool, (int(offsets[-1]),), generator=g).long() * 40503 + 77
            ids[s] = (vals, offsets)
        else:
            ids[s] = (sign, torch.arange(n + 1))
    dense = torch.randn(n, dense_dim, generator=g)
    os.makedirs(os.path.dirname(path), exist_ok=True)
    torch.save({"ids": ids, "dense": dense, "label": label.float()}, path)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="/tmp/tn_example_data")
    ap.add_argument("--days", nargs="+", default=["2020-05-10", "2020-05-11"])
    ap.add_argument("--files-per-day", type=int, default=4)
    ap.add_argument("--examples-per-file", type=int, default=12000)
    ap.add_argument("--slots", type=int, default=4)
    ap.add_argument("--dense-dim", type=int, default=0)
    a = ap.parse_args()
    slots = [str(i + 1) for i in range(a.slots)]
    for d, day in enumerate(a.days):
        for f in range(a.files_per_day):
            make_file(os.path.join(a.out, day, f"part-{f:05d}.pt"), a.examples_per_file, slots, a.dense_dim, d * 100 + f)
    print("wrote", a.out)


if __name__ == "__main__":
    main()

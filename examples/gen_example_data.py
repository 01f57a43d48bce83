"""Synthetic click data (the role of examples/gen_example_data.py in the reference): a few files per
day, ``slots`` categorical features drawn from small id pools so ids repeat, one multi-valued slot,
a slot that is missing for negative examples, dense features and a label correlated with the ids.

Files are ``torch.save``d dicts of tensors: {"ids": {slot: (values, offsets)}, "dense": [N, D], "label": [N]}, or with
``--format tfrecord`` TFRecord files of ``tf.train.Example`` records named ``tf-part.NNNNN`` with the features the
reference's generator writes: int64 ``label``, bytes ``uniq_id``, one int64 list per slot (absent where the slot is
missing) and, when asked for, a float list ``dense``.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def make_file(path: str, n: int, slots, dense_dim: int, seed: int, pool: int = 1000, fmt: str = "pt"):
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
    if fmt == "pt":
        torch.save({"ids": ids, "dense": dense, "label": label.float()}, path)
        return
    import tensornet_b200 as tn
    cols = {s: (v.numpy(), o.numpy()) for s, (v, o) in ids.items()}
    with tn.data.TFRecordWriter(path) as w:
        for i in range(n):
            ints = {"label": [int(label[i])]}
            for s, (v, o) in cols.items():
                if o[i + 1] > o[i]:
                    ints[s] = v[o[i]:o[i + 1]]
            floats = {"dense": dense[i].numpy()} if dense_dim else {}
            w.write(tn.data.encode_example(ints, floats, {"uniq_id": b"%08d" % i}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="/tmp/tn_example_data")
    ap.add_argument("--days", nargs="+", default=["2020-05-10", "2020-05-11"])
    ap.add_argument("--files-per-day", type=int, default=4)
    ap.add_argument("--examples-per-file", type=int, default=12000)
    ap.add_argument("--slots", type=int, default=4)
    ap.add_argument("--dense-dim", type=int, default=0)
    ap.add_argument("--format", default="pt", choices=["pt", "tfrecord"])
    a = ap.parse_args()
    slots = [str(i + 1) for i in range(a.slots)]
    for d, day in enumerate(a.days):
        for f in range(a.files_per_day):
            name = f"part-{f:05d}.pt" if a.format == "pt" else f"tf-part.{f:05d}"
            make_file(os.path.join(a.out, day, name), a.examples_per_file, slots, a.dense_dim, d * 100 + f, fmt=a.format)
    print("wrote", a.out)


if __name__ == "__main__":
    main()

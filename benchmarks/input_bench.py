"""Throughput of the native TFRecord reader (``tn.data.TFRecordDataset``) on records of the headline model's shape:
26 int64 slots with one id each, a float list of 13 dense values and an int64 label (about 640 bytes per record).

    python benchmarks/input_bench.py --records 200000 --workers 1 2 4 8

Writes ``--files`` TFRecord files under ``--dir`` once (kept between runs), then reads them with each worker count and
prints one JSON line per run: records / s, MB / s of file data and batches / s at ``--batch``.  Then the same pass is
written once as a batch cache (``tn.data.write_batch_cache``) and read back (``tn.data.BatchCacheDataset``): no
parsing, one contiguous read per batch.  Host-only: no GPU is touched; page-locked output buffers are off so that
the figures are the readers' own.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np

import tensornet_b200 as tn


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dir", default="/tmp/tn_input_bench")
    ap.add_argument("--records", type=int, default=200000)
    ap.add_argument("--files", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8192)
    ap.add_argument("--workers", type=int, nargs="+", default=[1, 2, 4, 8])
    ap.add_argument("--gzip", action="store_true")
    ap.add_argument("--repeat", type=int, default=3, help="passes per setting; the best one is reported")
    a = ap.parse_args()

    slots = [str(i) for i in range(1, 27)]
    per_file = a.records // a.files
    os.makedirs(a.dir, exist_ok=True)
    files = [os.path.join(a.dir, f"tf-part.{k:05d}" + (".gz" if a.gzip else "")) for k in range(a.files)]
    rng = np.random.default_rng(0)
    for p in files:
        if os.path.exists(p):
            continue
        ids = rng.integers(1, 2 ** 62, size=(per_file, 26))
        dense = rng.standard_normal((per_file, 13)).astype(np.float32)
        with tn.data.TFRecordWriter(p, gzip=a.gzip) as w:
            for i in range(per_file):
                ints = {s: ids[i, j:j + 1] for j, s in enumerate(slots)}
                ints["label"] = [i & 1]
                w.write(tn.data.encode_example(ints, {"dense": dense[i]}))
    size = sum(os.path.getsize(p) for p in files)

    for nw in a.workers:
        for single_hot in (False, True):
            best = None
            for _ in range(a.repeat):
                ds = tn.data.TFRecordDataset(files, a.batch, slots, dense_keys={"dense": 13}, num_workers=nw, single_hot=single_hot,
                                             packed=True, pin_memory=False)
                t0 = time.perf_counter()
                n = nb = 0
                for _, y in ds:
                    n += int(y.numel())
                    nb += 1
                dt = time.perf_counter() - t0
                best = dt if best is None else min(best, dt)
            print(json.dumps({"workers": nw, "single_hot": single_hot, "gzip": a.gzip, "records": n,
                              "records_per_s": round(n / best), "file_mb_per_s": round(size / best / 1e6, 1),
                              "batches_per_s": round(nb / best, 1), "host_cores": os.cpu_count()}), flush=True)

    cache = os.path.join(a.dir, "pass.tnbc")
    if not os.path.exists(cache):
        src = tn.data.TFRecordDataset(files, a.batch, slots, dense_keys={"dense": 13}, num_workers=max(a.workers), single_hot=True,
                                      packed=True, pin_memory=False)
        tn.data.write_batch_cache(cache, src, slots, dense_name="dense")
    best = None
    for _ in range(a.repeat):
        t0 = time.perf_counter()
        n = nb = 0
        for _, y in tn.data.BatchCacheDataset(cache, pin_memory=False):
            n += int(y.numel())
            nb += 1
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    print(json.dumps({"reader": "batch_cache", "records": n, "records_per_s": round(n / best),
                      "file_mb_per_s": round(os.path.getsize(cache) / best / 1e6, 1), "batches_per_s": round(nb / best, 1),
                      "host_cores": os.cpu_count()}), flush=True)


if __name__ == "__main__":
    main()

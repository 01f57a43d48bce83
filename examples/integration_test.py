"""End-to-end check of the example (the role of examples/integration-test.py in the reference): rank 0 writes the
synthetic days that are missing and removes an old model directory, then every rank runs the training driver; at the
end rank 0 checks what the run must leave behind.

    python examples/integration_test.py --data /tmp/tn_it_data --model-dir /tmp/tn_it_model
    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 examples/integration_test.py ...   # same flags as main.py

The other ranks cannot run ahead of rank 0's preparation: the first thing the driver does is the rendezvous of the
process group, which completes only when rank 0 joins it.
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import gen_example_data  # noqa: E402
import main as driver  # noqa: E402


def prepare(argv):
    ap = argparse.ArgumentParser(add_help=False)
    ap.add_argument("--data", default="/tmp/tn_example_data")
    ap.add_argument("--model-dir", default="/tmp/tn_model")
    ap.add_argument("--days", nargs="+", default=["2020-05-10", "2020-05-11"])
    ap.add_argument("--slots", type=int, default=4)
    ap.add_argument("--dense-dim", type=int, default=0)
    ap.add_argument("--files-per-day", type=int, default=4)
    ap.add_argument("--examples-per-file", type=int, default=12000)
    ap.add_argument("--format", default="pt", choices=["pt", "tfrecord"], help="input files: torch-saved tensors or TFRecord")
    a, rest = ap.parse_known_args(argv)
    if int(os.environ.get("RANK", "0")) == 0:
        slots = [str(i + 1) for i in range(a.slots)]
        for d, day in enumerate(a.days):
            if not os.path.isdir(os.path.join(a.data, day)):
                for f in range(a.files_per_day):
                    name = f"part-{f:05d}.pt" if a.format == "pt" else f"tf-part.{f:05d}"
                    gen_example_data.make_file(os.path.join(a.data, day, name), a.examples_per_file, slots, a.dense_dim,
                                               d * 100 + f, fmt=a.format)
        shutil.rmtree(a.model_dir, ignore_errors=True)
    # what the driver understands: everything but the generator-only flags
    fwd = ["--data", a.data, "--model-dir", a.model_dir, "--days", *a.days, "--slots", str(a.slots),
           "--dense-dim", str(a.dense_dim)] + rest
    return a, fwd


def check(a):
    import tensornet_b200 as tn
    last = tn.model.read_last_train_dt(a.model_dir)
    assert last == a.days[-1], f"done-file names {last!r}, expected {a.days[-1]!r}"
    for day in a.days:
        d = os.path.join(a.model_dir, day)
        assert os.path.isdir(os.path.join(d, "sparse_table")), f"no sparse tables under {d}"
        assert os.path.isdir(os.path.join(d, "dense_table")), f"no dense table under {d}"
    assert os.path.isfile(os.path.join(a.model_dir, "sub_model.pt")), "dense sub-model was not exported"
    print("integration test passed", flush=True)


if __name__ == "__main__":
    args, forwarded = prepare(sys.argv[1:])
    sys.argv = [sys.argv[0]] + forwarded
    driver.main()
    if int(os.environ.get("RANK", "0")) == 0:
        check(args)

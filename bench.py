"""Headline benchmark: DeepFM training throughput (examples/s) on N B200 GPUs of one node.

Config (the reference's DeepFM example, examples/models/deepfm.py, at the size named for this
build): 26 single-hot categorical slots, uint64 ids Zipf(s=1.05) over 2^40 hashed per slot,
13 dense fp32 features log1p(Exp(1)), labels Bernoulli(0.25); deep embeddings dim 16 with
sparse Adam state, dim-1 linear embeddings, second-order FM term, bf16 MLP
429->400->400->400->1 (ReLU) with fp32 master weights and dense Adam; batch 8192 per GPU.
Data is synthetic and weights are random-init.

    python bench.py --gpus 1 --steps 50 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 50 --warmup 5

Prints ONE JSON line on rank 0.  ``value`` is the device-timed aggregate over all GPUs with the
inputs already resident on the device; ``e2e`` is the same step driven through the public
``Model.train_on_batch`` API with, every step, the host->device copy of that step's inputs from
pinned memory and a device->host read of the loss.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REFERENCE_EXAMPLES_PER_S = 4000.0   # the only published training throughput: Wide&Deep, 8 ms/step at batch 32 on one CPU host


def reference_arm(args):
    """The unmodified reference needs TensorFlow 2.8 (CPU), OpenMPI and brpc; report honestly."""
    why = None
    ref_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref")
    try:
        sys.path.insert(0, ref_dir)
        import tensorflow  # noqa: F401
        import tensornet  # noqa: F401
        why = "reference imported but no driver for it is wired up"
    except Exception as e:  # pragma: no cover - depends on the box
        why = f"reference not runnable here: {type(e).__name__}: {str(e)[:120]} (needs tensorflow-cpu 2.8, OpenMPI, brpc; none installable offline)"
    finally:
        if ref_dir in sys.path:
            sys.path.remove(ref_dir)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def _start_nvml(self) -> bool:
        """Read-only NVML polling every ~4 ms from a thread (the timed region of a short run lasts milliseconds)."""
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu)
            smax = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
        except Exception:
            return False
        bits = [("hw_slowdown", getattr(pynvml, "nvmlClocksThrottleReasonHwSlowdown", 0x8)),
                ("hw_thermal_slowdown", getattr(pynvml, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40)),
                ("sw_thermal_slowdown", getattr(pynvml, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20)),
                ("sw_power_cap", getattr(pynvml, "nvmlClocksThrottleReasonSwPowerCap", 0x4))]
        self._stop = False

        def poll():
            while not self._stop:
                try:
                    sm = float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                    mask = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                    act = ["Active" if mask & b else "Not Active" for _, b in bits]
                    self.rows.append((time.time(), ",".join([str(self.gpu), str(sm), str(smax), "0", "x"] + act)))
                except Exception:
                    pass
                time.sleep(0.004)

        self.thread = threading.Thread(target=poll, daemon=True)
        self.thread.start()
        self.nvml = True
        return True

    def start(self):
        self.nvml = False
        if self._start_nvml():
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float):
        if getattr(self, "nvml", False):
            self._stop = True
            self.thread.join(timeout=1)
        elif self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        else:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.rows:
            if t < t0 - 0.05 or t > t1 + 0.05:
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples inside the timed region"], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons), "samples": len(sm)}


def make_batches(n_batches, B, n_slots, n_dense, seed):
    """Synthetic batches in pinned host memory."""
    import numpy as np
    import torch
    import tensornet_b200 as tn

    rng = np.random.default_rng(seed)
    s, N = 1.05, float(2 ** 40)
    out = []
    for _ in range(n_batches):
        u = rng.random((n_slots, B))
        x = np.floor(((N ** (1 - s) - 1) * u + 1) ** (1 / (1 - s))).astype(np.uint64)      # Zipf(s) over [1, 2^40]
        slot = (np.arange(n_slots, dtype=np.uint64)[:, None] + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15)
        h = x ^ slot
        h ^= h >> np.uint64(33); h *= np.uint64(0xff51afd7ed558ccd); h ^= h >> np.uint64(33)
        h *= np.uint64(0xc4ceb9fe1a85ec53); h ^= h >> np.uint64(33)
        ids = torch.from_numpy(h.view(np.int64)).pin_memory()
        dense = torch.from_numpy(np.log1p(rng.exponential(1.0, (B, n_dense))).astype(np.float32)).pin_memory()
        label = torch.from_numpy((rng.random(B) < 0.25).astype(np.float32)).pin_memory()
        out.append((ids, dense, label))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8192, help="examples per GPU per step")
    ap.add_argument("--pool", type=int, default=16, help="distinct synthetic batches cycled through")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--separate-tables", action="store_true", help="keep the dim-1 linear weights in a table of their own")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)

    import torch
    import tensornet_b200 as tn

    if args.gpus > 1 and "RANK" not in os.environ:
        raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    tn.core.init()
    rt = tn.core.runtime()
    assert rt.on_gpu, "bench.py needs a CUDA device"
    assert rt.world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE is {rt.world}"
    from tensornet_b200 import _build
    ext = _build.cuda_ext()

    n_slots, n_dense, emb_dim, B = 26, 13, 16, args.batch
    slots = [str(i) for i in range(1, n_slots + 1)]
    total_steps = 2 * (args.warmup + args.steps) + 8
    # rows per GPU: every step can add at most n_slots * B * world / world new signs per shard
    rows = min(1 << 27, max(1 << 20, int(n_slots * B * total_steps * 1.3)))
    torch.manual_seed(1234)
    model = tn.models.DeepFM(slots, slots, dnn_hidden_units=(400, 400, 400), embedding_dim=emb_dim, dense_dim=n_dense,
                             sparse_opt=tn.core.Adam(learning_rate=1e-3, initial_scale=0.1), bucket_size=B,
                             table_rows=rows, share_linear_table=not args.separate_tables)
    model.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=1e-3)), loss="binary_crossentropy",
                  cuda_graph=not args.no_graph)

    host = make_batches(args.pool, B, n_slots, n_dense, seed=1000 + rt.rank)
    dev = [(i.to(rt.device), d.to(rt.device), l.to(rt.device)) for i, d, l in host]

    def feats(ids, dense):
        return {tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, ids=ids), "dense": dense}

    # ---------------- warm-up (eager steps, graph capture, a few replays) ----------------
    for k in range(args.warmup + 4):
        i, d, l = dev[k % args.pool]
        model.train_on_batch(feats(i, d), l)
    # the end-to-end path (Model.fit: prefetch stream, pinned loss buffers) gets its warm-up too
    model.fit(((feats(*host[k % args.pool][:2]), host[k % args.pool][2]) for k in range(4)), epochs=1, prefetch=True, record_step_loss=True)
    torch.cuda.synchronize()
    rt.check_status()
    if model._graph is not None:
        per_step_launches = model._launches_per_step
    else:
        c0 = ext.launch_count()
        i, d, l = dev[0]
        model.train_on_batch(feats(i, d), l)
        per_step_launches = ext.launch_count() - c0
    torch.cuda.synchronize()

    # ---------------- timed region 1: device-resident inputs -----------------------------
    sampler = ClockSampler(rt.device.index or 0)
    sampler.start()
    time.sleep(0.3)
    rt.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    e0.record()
    for k in range(args.steps):
        i, d, l = dev[k % args.pool]
        model.train_on_batch(feats(i, d), l)
    e1.record()
    torch.cuda.synchronize()
    t1 = time.time()
    rt.barrier()
    clocks = sampler.stop(t0, t1)
    ms = e0.elapsed_time(e1)
    rt.check_status()

    # ---------------- timed region 2: end to end through the public API ------------------
    rt.barrier()
    torch.cuda.synchronize()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()

    def host_batches():
        for k in range(args.steps):
            i, d, l = host[k % args.pool]                   # pinned host tensors: every step's inputs are copied H2D
            yield feats(i, d), l

    # Model.fit copies batch k+1 to the device while step k runs and reads every step's loss back to the host
    # (history["step_loss"]: one 4-byte D2H copy per step, collected one step later)
    hist = model.fit(host_batches(), epochs=1, prefetch=True, record_step_loss=True)
    assert len(hist["step_loss"]) == args.steps, "every step's loss must reach the host"
    last = hist["step_loss"][-1]
    f1.record()
    torch.cuda.synchronize()
    rt.barrier()
    ms_e2e = f0.elapsed_time(f1)
    rt.check_status()

    t = torch.tensor([ms, ms_e2e], dtype=torch.float64)
    if rt.world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=rt.host_group)
    ms, ms_e2e = float(t[0]), float(t[1])
    G = B * rt.world
    value = G * args.steps / (ms / 1e3)
    e2e = G * args.steps / (ms_e2e / 1e3)
    h2d = host[0][0].numel() * 8 + host[0][1].numel() * 4 + host[0][2].numel() * 4
    if rt.rank == 0:
        print(json.dumps({
            "metric": "train examples/sec (DeepFM, device-timed, max over ranks)",
            "value": value, "unit": "examples/s", "n_gpus": rt.world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / REFERENCE_EXAMPLES_PER_S,
            "baseline_note": "the only training throughput the reference publishes: Wide&Deep, batch 32, one CPU host, ~4000 examples/s (doc/tutorial/01-begin-with-wide-deep.ipynb:446)",
            "dtype": "bf16", "data": "synthetic",
            "config": {"model": "DeepFM 26 slots x dim16 (+dim1 linear), FM, MLP 429-400-400-400-1, sparse Adam, dense Adam",
                       "global_batch": G, "seq_len": 1, "parallelism": f"dp{rt.world}+row-sharded embedding tables",
                       "l2": f"inputs cycle through {args.pool} distinct batches; touched table rows exceed L2",
                       "cuda_graph": model._graph is not None, "linear_weights": "stored in the embedding rows (one table)" if model.share_linear_table else "separate dim-1 table", "last_loss": last,
                       "dense_multimem": bool(getattr(model.optimizer.table, "uses_multimem", False))},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "examples/s", "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": int(per_step_launches) * args.steps,
            "gpu_launches_per_step": int(per_step_launches),
        }), flush=True)
    tn.core.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())

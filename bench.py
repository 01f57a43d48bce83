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

Before anything is timed every GPU's shard of the embedding table is filled with its part of a
universe of ~1e8 signs (the 1e8/26 most popular ranks of every slot); ids are drawn Zipf(1.05)
over 2^40 and ranks beyond the universe are folded onto it, so training runs in the steady
state of a long job: every step is fresh ids against a table of ~1e8 rows.

Prints ONE JSON line on rank 0.  The block of ``--steps`` steps is repeated back to back until at
least a second has been timed; ``value`` is the aggregate over all GPUs from the MEDIAN block
(device-timed with CUDA events, each block the max over ranks, inputs already resident on the
device); ``e2e`` is the same measurement through ``Model.fit`` with, every step, the
host->device copy of that step's inputs from pinned memory and a device->host read of the loss.
``context`` holds two more arms for orientation only: the same step written with library calls
(torch.unique, NCCL all-to-all, index ops, torch matmul) and on the CPU path of this package.
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


N_SLOTS, N_DENSE, EMB_DIM = 26, 13, 16
UNIVERSE = 100_000_000                      # distinct signs of the job (all slots together)
ZIPF_S, ZIPF_N = 1.05, float(2 ** 40)
_ODD = -7046029254386353131                 # 0x9E3779B97F4A7C15 as int64: odd, so x -> x * _ODD is a bijection on 2^64


def slot_signs(x, slot):
    """Sign of rank ``x`` (int64 tensor, 1 <= x < 2^41) in slot ``slot`` (int64 tensor or int): distinct per (slot, rank)."""
    return (x + ((slot + 1) << 42)) * _ODD


def zipf_batch(gen, B, ranks_per_slot, dev):
    """ids [N_SLOTS, B] int64: per slot a Zipf(1.05) rank over [1, 2^40]; ranks beyond the universe are folded onto
    it uniformly (a long tail of cold signs); then hashed per slot."""
    import torch

    u = torch.rand((N_SLOTS, B), generator=gen, device=dev, dtype=torch.float64)
    x = torch.floor(((ZIPF_N ** (1 - ZIPF_S) - 1) * u + 1) ** (1 / (1 - ZIPF_S))).to(torch.int64).clamp_(1, 1 << 40)
    folded = (((x * _ODD) >> 20) & ((1 << 40) - 1)) % ranks_per_slot + 1
    x = torch.where(x > ranks_per_slot, folded, x)
    slot = torch.arange(N_SLOTS, device=dev, dtype=torch.int64)[:, None]
    return slot_signs(x, slot)


def make_batches(n_batches, B, ranks_per_slot, dev, seed):
    """Synthetic batches, generated on the device: (ids [26, B], dense [B, 13], labels [B])."""
    import torch

    gen = torch.Generator(device=dev).manual_seed(seed)
    out = []
    for _ in range(n_batches):
        ids = zipf_batch(gen, B, ranks_per_slot, dev)
        dense = torch.log1p(torch.empty((B, N_DENSE), device=dev).exponential_(1.0, generator=gen))
        label = (torch.rand(B, generator=gen, device=dev) < 0.25).float()
        out.append((ids, dense, label))
    return out


def universe_chunks(B, ranks_per_slot, rank, world, dev):
    """This rank's share of the universe as [26, B] id blocks (the same number of blocks on every rank)."""
    import torch

    n_chunks = (ranks_per_slot + B - 1) // B
    per_rank = (n_chunks + world - 1) // world
    slot = torch.arange(N_SLOTS, device=dev, dtype=torch.int64)[:, None]
    for k in range(per_rank):
        c = min(k * world + rank, n_chunks - 1)
        x = (torch.arange(c * B, (c + 1) * B, device=dev, dtype=torch.int64) + 1).clamp_(max=ranks_per_slot)
        yield slot_signs(x[None, :].expand(N_SLOTS, B), slot).contiguous()


def block_times(events):
    return [events[i].elapsed_time(events[i + 1]) for i in range(len(events) - 1)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8192, help="examples per GPU per step")
    ap.add_argument("--pool", type=int, default=64, help="distinct synthetic batches drawn before timing (>= warmup + steps)")
    ap.add_argument("--universe", type=int, default=UNIVERSE, help="distinct signs of the job; the tables hold them all")
    ap.add_argument("--min-seconds", type=float, default=1.0, help="repeat the block of --steps steps until this much is timed")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-context", action="store_true", help="skip the library-only and CPU context arms")
    ap.add_argument("--separate-tables", action="store_true", help="keep the dim-1 linear weights in a table of their own")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)
    K = args.steps

    import torch
    import torch.distributed as dist
    import tensornet_b200 as tn

    if args.gpus > 1 and "RANK" not in os.environ:
        raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    tn.core.init()
    # every rank draws batches of one shape at every step, so the captured steps may start the next batch's pull
    # (dedup + id dispatch) ahead on several GPUs too; one GPU does so by default
    tn.core.config.pull_front_ahead = 1
    rt = tn.core.runtime()
    assert rt.on_gpu, "bench.py needs a CUDA device"
    assert rt.world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE is {rt.world}"
    from tensornet_b200 import _build
    ext = _build.cuda_ext()
    dev = rt.device

    B = args.batch
    slots = [str(i) for i in range(1, N_SLOTS + 1)]
    ranks_per_slot = max(B, (args.universe + N_SLOTS - 1) // N_SLOTS)
    universe = ranks_per_slot * N_SLOTS
    rows = int(universe / rt.world * 1.25) + (1 << 16)          # slab of one shard: its part of the universe at 80 % fill
    torch.manual_seed(1234)
    model = tn.models.DeepFM(slots, slots, dnn_hidden_units=(400, 400, 400), embedding_dim=EMB_DIM, dense_dim=N_DENSE,
                             sparse_opt=tn.core.Adam(learning_rate=1e-3, initial_scale=0.1), bucket_size=B,
                             table_rows=rows, share_linear_table=not args.separate_tables)
    model.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=1e-3)), loss="binary_crossentropy",
                  cuda_graph=not args.no_graph)

    # ---------------- fill the tables: every sign of the universe gets its row ------------
    t_fill = time.time()
    layers = [model.deep_emb] + ([model.linear_emb] if model.linear_emb is not None else [])
    for ids in universe_chunks(B, ranks_per_slot, rt.rank, rt.world, dev):
        for layer in layers:
            layer.link.pull(ids.reshape(-1), training=False)
    torch.cuda.synchronize()
    rt.check_status()
    rt.barrier()
    table = model.deep_emb.table
    rows_here = table.n_rows
    rows_all = sum(rt.all_gather_object(rows_here))
    t_fill = time.time() - t_fill

    pool = max(args.pool, args.warmup + K)
    drawn = make_batches(pool, B, ranks_per_slot, dev, seed=1000 + rt.rank)
    # Ids and dense features cycle with different periods (pool, pool-3); the labels come from a pool of their own with
    # a prime number of batches (32 KB each), so that no (ids, labels) pairing returns within a run: with only a few
    # dozen label batches a one-GPU run sees each pairing twice and the embeddings of rare ids learn the random labels
    # by heart, which says nothing about speed but makes the reported loss meaningless.
    per = (pool, max(pool - 3, 1))
    n_lab = 4099
    lab_gen = torch.Generator(device=dev).manual_seed(77 + rt.rank)
    label_pool = (torch.rand((n_lab, B), generator=lab_gen, device=dev) < 0.25).float()
    host_drawn = [tuple(t.cpu().pin_memory() for t in b[:2]) for b in drawn]
    host_labels = label_pool.cpu().pin_memory()

    def dev_batch(k):
        return drawn[k % per[0]][0], drawn[k % per[1]][1], label_pool[k % n_lab]

    def host_batch(k):
        return host_drawn[k % per[0]][0], host_drawn[k % per[1]][1], host_labels[k % n_lab]

    def feats(ids, dense):
        return {tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, ids=ids), "dense": dense}

    # ---------------- warm-up (eager steps, graph capture, a few replays) ----------------
    def dev_step(k):
        # the step on batch k; naming batch k+1 lets the captured step start that batch's dedup and id dispatch ahead
        i, d, l = dev_batch(k)
        i2, d2, l2 = dev_batch(k + 1)
        return model.train_on_batch(feats(i, d), l, next_batch=(feats(i2, d2), l2))

    for k in range(args.warmup + 4):
        dev_step(k)
    # the end-to-end path (Model.fit: overlapped input copies, pinned loss buffers) gets its warm-up too
    model.fit(((feats(*host_batch(k)[:2]), host_batch(k)[2]) for k in range(args.warmup)), epochs=1, record_step_loss=True)
    torch.cuda.synchronize()
    rt.check_status()
    graphed = model._graph is not None
    if graphed:
        per_step_launches = model._launches_per_step
    else:
        c0 = ext.launch_count()
        dev_step(0)
        per_step_launches = ext.launch_count() - c0
    torch.cuda.synchronize()

    def agree_max(x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64)
        if rt.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=rt.host_group)
        return float(t[0])

    def max_over_ranks(v):
        t = torch.tensor(v, dtype=torch.float64)
        if rt.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=rt.host_group)
        return t.tolist()

    step_no = [args.warmup + 4]

    def device_block():
        for _ in range(K):
            dev_step(step_no[0])
            step_no[0] += 1

    # calibration block (also warm-up): how many blocks make up the minimum timed duration
    rt.barrier()
    torch.cuda.synchronize()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    device_block()
    c1.record()
    torch.cuda.synchronize()
    repeats = int(min(5000, max(3, agree_max(args.min_seconds * 1e3 / max(c0.elapsed_time(c1), 1e-3)) + 1)))

    # ---------------- timed region 1: device-resident inputs -----------------------------
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    time.sleep(0.3)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(repeats + 1)]
    rt.barrier()
    torch.cuda.synchronize()
    t0 = time.time()
    ev[0].record()
    for r in range(repeats):
        device_block()
        ev[r + 1].record()
    torch.cuda.synchronize()
    t1 = time.time()
    rt.barrier()
    clocks = sampler.stop(t0, t1)
    blocks = max_over_ranks(block_times(ev))
    rt.check_status()

    # ---------------- timed region 2: end to end through the public API ------------------
    class BlockMarks(tn.callbacks.Callback):
        """An event every K steps of the pass."""

        def __init__(self):
            self.events = []

        def on_train_batch_end(self, step, logs=None):
            if (step + 1) % K == 0:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                self.events.append(e)

    def host_stream():
        for k in range(repeats * K):
            i, d, l = host_batch(k)                         # pinned host tensors: every step's inputs are copied H2D
            yield feats(i, d), l

    marks = BlockMarks()
    rt.barrier()
    torch.cuda.synchronize()
    f0 = torch.cuda.Event(enable_timing=True)
    f0.record()
    # Model.fit copies the inputs of step k+1 to the device while step k runs and reads every step's loss back to the
    # host (history["step_loss"]: one 4-byte D2H copy per step, collected one step later)
    hist = model.fit(host_stream(), epochs=1, callbacks=[marks], record_step_loss=True)
    torch.cuda.synchronize()
    rt.barrier()
    assert len(hist["step_loss"]) == repeats * K, "every step's loss must reach the host"
    last = hist["step_loss"][-1]
    e2e_blocks = max_over_ranks(block_times([f0] + marks.events))
    rt.check_status()

    G = B * rt.world
    med, e2e_med = statistics.median(blocks), statistics.median(e2e_blocks)
    value = G * K / (med / 1e3)
    e2e = G * K / (e2e_med / 1e3)
    h2d = sum(t.numel() * t.element_size() for t in host_batch(0))

    # ---------------- context arms (not the reference; for orientation) -------------------
    context = {}
    if not args.no_context:
        sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "benchmarks"))
        try:
            import deepfm_context_arms as arms
            context["library_only_path"] = arms.library_arm(
                rt, drawn, lambda: universe_chunks(B, ranks_per_slot, 0, 1, dev), steps=K, warmup=args.warmup, emb_dim=EMB_DIM)
        except Exception as e:  # pragma: no cover - orientation only, never fails the bench
            context["library_only_path"] = {"error": f"{type(e).__name__}: {str(e)[:160]}"}
        rt.barrier()
        if rt.rank == 0:
            try:
                context["cpu_path_of_this_package"] = arms.cpu_arm(B)
            except Exception as e:  # pragma: no cover
                context["cpu_path_of_this_package"] = {"error": f"{type(e).__name__}: {str(e)[:160]}"}
        rt.barrier()

    if rt.rank == 0:
        print(json.dumps({
            "metric": "train examples/sec (DeepFM, device-timed, max over ranks)",
            "value": value, "unit": "examples/s", "n_gpus": rt.world, "steps": K, "warmup": args.warmup,
            "ms_per_step": med / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / REFERENCE_EXAMPLES_PER_S,
            "baseline_note": "the only training throughput the reference publishes: Wide&Deep, batch 32, one CPU host, ~4000 examples/s (doc/tutorial/01-begin-with-wide-deep.ipynb:446)",
            "dtype": "bf16", "data": "synthetic",
            "timing": {"repeats": repeats, "statistic": "median block of `steps` steps, each block the max over ranks",
                       "block_ms_min": min(blocks), "block_ms_median": med, "block_ms_max": max(blocks),
                       "timed_seconds": sum(blocks) / 1e3, "e2e_block_ms_min": min(e2e_blocks), "e2e_block_ms_max": max(e2e_blocks),
                       "e2e_timed_seconds": sum(e2e_blocks) / 1e3},
            "config": {"model": "DeepFM 26 slots x dim16 (+dim1 linear), FM, MLP 429-400-400-400-1, sparse Adam, dense Adam",
                       "global_batch": G, "seq_len": 1, "parallelism": f"dp{rt.world}+row-sharded embedding tables",
                       "ids": f"Zipf(1.05) over 2^40 per slot, ranks beyond the {ranks_per_slot} most popular of a slot folded onto them",
                       "table_rows_resident": rows_all, "table_rows_this_gpu": rows_here,
                       "key_array_load_factor": rows_here / table.keys.numel(), "table_fill_seconds": t_fill,
                       "l2": f"no flush: every step draws fresh ids (pool of {pool} batches) against {rows_here * table.stride * 4 / 1e9:.1f} GB of rows per GPU, far beyond L2",
                       "cuda_graph": graphed, "pull_front_ahead": bool(getattr(model, "_rings", None)), "linear_weights": "stored in the embedding rows (one table)" if model.share_linear_table else "separate dim-1 table", "last_loss": last,
                       "dense_multimem": bool(getattr(model.optimizer.table, "uses_multimem", False))},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "examples/s", "ms_per_step": e2e_med / K, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4},
            "gpu_launches": int(per_step_launches) * K * repeats,
            "gpu_launches_per_step": int(per_step_launches),
            "context": context,
        }), flush=True)
    tn.core.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Two orientation arms for the DeepFM headline benchmark (``bench.py`` prints them under ``context``).

Neither is the reference (which needs TensorFlow 2.8, OpenMPI and brpc).  They answer two narrower questions on
the same box, model, batch and id distribution:

* ``library_arm``  what the same synchronous step costs when every hot path is a library call: ``torch.unique``
  for the dedup, NCCL ``all_to_all_single`` for the id / row / gradient exchanges, a sorted key array with
  ``searchsorted`` plus index ops for the table, autocast ``nn.Linear`` for the towers, fused ``torch.optim.Adam``
  and an NCCL all-reduce for the dense part.  This is the baseline the fused kernels of the package are written
  against.
* ``cpu_arm``      the package's own CPU path (the plain C++ restatement of the reference's parameter-server
  algorithms, driven by the same model code) on the host cores, one process.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import time


def library_arm(rt, dev_batches, universe_blocks, steps: int, warmup: int, emb_dim: int = 16, hidden=(400, 400, 400),
                lr: float = 1e-3):
    """Examples/s of the library-only DeepFM step on ``rt.world`` GPUs (device-timed, max over ranks).

    ``dev_batches``: list of (ids [S, B] int64, dense [B, Dd], labels [B]) on the device.
    ``universe_blocks``: callable yielding int64 tensors that together hold every sign of the job once."""
    import torch
    import torch.distributed as dist
    from torch import nn

    W, R, dev = rt.world, rt.rank, rt.device
    S, B = dev_batches[0][0].shape
    Dd = dev_batches[0][1].shape[1]
    D = emb_dim + 1                                   # 16 embedding columns + the slot's linear weight

    def owner_of(x):
        return ((x >> 7) & 0xFFFFFFFF) % W

    mine = []
    for blk in universe_blocks():
        flat = blk.reshape(-1)
        mine.append(flat[owner_of(flat) == R] if W > 1 else flat)
    keys = torch.unique(torch.cat(mine))               # sorted, distinct
    del mine
    n = keys.numel()
    gen = torch.Generator(device=dev).manual_seed(7 + R)
    w = torch.randn((n, D), device=dev, generator=gen) * 0.01
    m = torch.zeros_like(w)
    v = torch.zeros_like(w)

    torch.manual_seed(99)
    dims = [S * emb_dim + Dd] + list(hidden)
    mlp = nn.Sequential(*[x for i in range(len(hidden)) for x in (nn.Linear(dims[i], dims[i + 1]), nn.ReLU())]).to(dev)
    head = nn.Linear(hidden[-1] + S + 1, 1).to(dev)
    params = list(mlp.parameters()) + list(head.parameters())
    opt = torch.optim.Adam(params, lr=lr, fused=True)
    group = rt.device_group

    def a2a(x, send_counts, recv_counts):
        out = x.new_empty((int(sum(recv_counts)),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x, output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
        return out

    def step(batch):
        ids, dense, y = batch
        uniq, inv = torch.unique(ids.reshape(-1), return_inverse=True)
        if W > 1:
            own = owner_of(uniq)
            order = torch.argsort(own)
            send_ids = uniq[order]
            send_counts = torch.bincount(own, minlength=W)
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts, group=group)
            sc, rc = send_counts.tolist(), recv_counts.tolist()
            req = a2a(send_ids, sc, rc)
        else:
            req = uniq
        rows = torch.searchsorted(keys, req).clamp_(max=n - 1)
        vals = w[rows]
        if W > 1:
            back = a2a(vals, rc, sc)
            U = torch.empty_like(back)
            U[order] = back
        else:
            U = vals
        U.requires_grad_(True)
        e = U[inv].view(S, B, D).permute(1, 0, 2)
        deep, lin = e[..., :emb_dim], e[..., emb_dim]
        fm = 0.5 * (deep.sum(1).pow(2) - deep.pow(2).sum(1)).sum(-1, keepdim=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            h = mlp(torch.cat([deep.reshape(B, -1), dense], dim=1))
        logit = head(torch.cat([h.float(), lin, fm], dim=1)).view(-1)
        loss = torch.nn.functional.binary_cross_entropy_with_logits(logit, y)
        opt.zero_grad(set_to_none=False)
        loss.backward()
        g = U.grad
        if W > 1:
            g = a2a(g[order].contiguous(), sc, rc)
        ur, uinv = torch.unique(rows, return_inverse=True)
        gs = torch.zeros((ur.numel(), D), device=dev).index_add_(0, uinv, g)
        mm = 0.9 * m[ur] + 0.1 * gs
        vv = 0.999 * v[ur] + 0.001 * gs * gs
        m[ur] = mm
        v[ur] = vv
        w[ur] -= lr * mm / (1e-8 + vv.sqrt())
        if W > 1:
            flat = torch.cat([p.grad.reshape(-1) for p in params])
            dist.all_reduce(flat, group=group)
            flat /= W
            off = 0
            for p in params:
                p.grad.copy_(flat[off:off + p.numel()].view_as(p))
                off += p.numel()
        opt.step()
        return loss

    for k in range(warmup):
        step(dev_batches[k % len(dev_batches)])
    torch.cuda.synchronize()
    rt.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k in range(steps):
        loss = step(dev_batches[(warmup + k) % len(dev_batches)])
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64)
    if W > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX, group=rt.host_group)
    ms = float(ms[0])
    out = {"what": "same DeepFM step from library calls only: torch.unique, NCCL all_to_all_single, searchsorted + index ops, "
                   "autocast nn.Linear, fused torch Adam, NCCL all-reduce; not the reference",
           "examples_per_s": B * W * steps / (ms / 1e3), "ms_per_step": ms / steps, "steps": steps, "warmup": warmup,
           "table_rows_this_gpu": int(n), "last_loss": float(loss)}
    del w, m, v, keys
    torch.cuda.empty_cache()
    return out


_CPU_SCRIPT = r"""
import json, sys, time, torch
import tensornet_b200 as tn
B, S, Dd = int(sys.argv[1]), 26, 13
tn.core.init()
slots = [str(i) for i in range(1, S + 1)]
torch.manual_seed(0)
m = tn.models.DeepFM(slots, slots, dnn_hidden_units=(400, 400, 400), embedding_dim=16, dense_dim=Dd,
                     sparse_opt=tn.core.Adam(learning_rate=1e-3, initial_scale=0.1), bucket_size=B, share_linear_table=True)
m.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=1e-3)))
g = torch.Generator().manual_seed(1)
def batch():
    u = torch.rand((S, B), generator=g, dtype=torch.float64)
    x = torch.floor((1 - 0.75 * u) ** -20.0).to(torch.int64).clamp_(1, 1 << 40)
    x = torch.where(x > 3846154, x % 3846154 + 1, x)
    ids = (x + ((torch.arange(S)[:, None] + 1) << 42)) * -7046029254386353131
    f = {tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, ids=ids), "dense": torch.log1p(torch.empty(B, Dd).exponential_(1.0, generator=g))}
    return f, (torch.rand(B, generator=g) < 0.25).float()
data = [batch() for _ in range(4)]
for k in range(2):
    m.train_on_batch(*data[k])
t0 = time.perf_counter()
n = 4
for k in range(n):
    loss = m.train_on_batch(*data[k % 4])
dt = (time.perf_counter() - t0) / n
print(json.dumps({"ms_per_step": dt * 1e3, "examples_per_s": B / dt, "steps": n, "threads": torch.get_num_threads(), "last_loss": float(loss)}))
"""


def cpu_arm(batch: int, timeout_s: int = 240):
    """Examples/s of the package's CPU path (one process, host cores) on the same model and batch size; wall clock."""
    env = dict(os.environ, TN_FORCE_CPU="1", CUDA_VISIBLE_DEVICES="")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT", "LOCAL_WORLD_SIZE", "GROUP_RANK",
              "TORCHELASTIC_RUN_ID"):
        env.pop(k, None)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    t0 = time.time()
    r = subprocess.run([sys.executable, "-c", _CPU_SCRIPT, str(batch)], env=env, capture_output=True, text=True, timeout=timeout_s)
    if r.returncode != 0:
        return {"error": (r.stderr or r.stdout)[-200:]}
    out = json.loads(r.stdout.strip().splitlines()[-1])
    out["what"] = ("same DeepFM step on this package's CPU path (C++ restatement of the reference's parameter-server algorithms + "
                   "torch CPU towers), one process, wall clock; not the reference")
    out["wall_s"] = time.time() - t0
    return out

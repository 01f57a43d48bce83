"""Small, self-contained launches of the hot kernels, for timing with CUDA events and for capturing
with Nsight Compute (one GPU, a few launches, a few hundred MB on the device).

    python benchmarks/kernel_cases.py gemm_fwd|gemm_dgrad|gemm_wgrad|gemm_big|sparse|deepfm|dense|small_ops  [--iters N]

Each case prints the per-launch device time (CUDA events around N back-to-back launches after warm-up,
inputs larger than L2 for the sparse cases) and the algorithmic bytes / FLOPs so a roofline fraction
can be formed against MEASURED_PEAKS.json.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

import tensornet_b200 as tn
from tensornet_b200 import _build


def timed(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters


def peaks():
    try:
        return json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")))
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm_fwd", "gemm_dgrad", "gemm_wgrad", "gemm_big", "sparse", "sparse_front", "deepfm", "deepfm_head", "mlp_chain", "dense", "small_ops"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--batch", type=int, default=8192)
    a = ap.parse_args()
    tn.core.init()
    rt = tn.core.runtime()
    ext, st, dev = _build.cuda_ext(), rt.status, rt.device
    pk = peaks()
    tag = "of fallback" if pk.get("fallback") else "of measured"
    out = {"case": a.case}
    if a.case == "gemm_big":
        # one DCN-v2 cross layer: [8192, 6416] x [6416, 6416]^T, the three operand layouts, against the library GEMM
        M, N, K = a.batch, 6416, 6416
        A = torch.randn(M, K, device=dev).bfloat16()
        Bw = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        C = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        dW = torch.zeros(N, K, device=dev)
        flops = 2.0 * M * N * K
        res = {}
        res["fwd_kk"] = timed(lambda: ext.gemm(A, Bw, C, M, N, K, K, K, N, False, False, False, False, None, None, None, None, 0, -1, N, 1, 0, st), a.iters)
        res["fwd_kk_two_accumulators"] = timed(lambda: ext.gemm(A, Bw, C, M, N, K, K, K, N, False, False, False, False, None, None, None, None, 0, -1, N, 1, 256, st, m_halves=2), a.iters)
        res["dgrad_k_mn"] = timed(lambda: ext.gemm(A, Bw, C, M, K, N, K, K, N, False, True, False, False, None, None, None, None, 0, -1, K, 1, 0, st), a.iters)
        res["wgrad_mn_mn"] = timed(lambda: ext.gemm(C, A, dW, N, K, M, N, K, K, True, True, True, False, None, None, None, None, 0, -1, K, 0, 0, st), a.iters)
        res["library_matmul"] = timed(lambda: torch.matmul(A, Bw.t(), out=C), a.iters)
        out.update(shape=[M, N, K], us=res, tflops={k: flops / v / 1e6 for k, v in res.items()},
                   frac_of_bf16_sustained={k: flops / v / 1e6 / pk.get("bf16_tflops_sustained", pk["bf16_tflops"]) for k, v in res.items()}, peak=tag)
    elif a.case.startswith("gemm"):
        M, N, K = a.batch, 400, 430
        A = torch.randn(M, 432, device=dev).bfloat16()
        Bw = (torch.randn(N, 432, device=dev) * 0.1).bfloat16()
        C = torch.empty(M, 408, dtype=torch.bfloat16, device=dev)
        dX = torch.empty(M, 432, dtype=torch.bfloat16, device=dev)
        dW = torch.zeros(N, 432, device=dev)
        fns = {"gemm_fwd": lambda: ext.gemm(A, Bw, C, M, N, K, 432, 432, 408, False, False, False, True, None, None, None, None, 0, N, 408, 1, 0, st),
               "gemm_dgrad": lambda: ext.gemm(C, Bw, dX, M, 432, N, 408, 432, 432, False, True, False, False, None, A, None, None, 432, -1, 432, 1, 0, st),
               "gemm_wgrad": lambda: ext.gemm(C, A, dW, N, K, M, 408, 432, 432, True, True, True, False, None, None, None, None, 0, -1, K, 0, 0, st)}
        us = timed(fns[a.case], a.iters)
        flops = 2.0 * M * N * K
        out.update(us=us, tflops=flops / us / 1e6, frac_of_bf16_peak=flops / us / 1e6 / pk["bf16_tflops"], peak=tag,
                   shape=[M, N, K], min_bytes=(M * 432 + N * 432 + M * 408) * 2, hbm_floor_us=(M * 432 + N * 432 + M * 408) * 2 / pk["hbm_gbs"] / 1e3)
    elif a.case == "sparse":
        import bench
        from tensornet_b200.ops.sparse_table_gpu import GpuSparseTable
        B, S, dim = a.batch, 26, 20
        data = [b[0].reshape(-1) for b in bench.make_batches(8, B, 3846154, dev, 5)]
        t = GpuSparseTable(tn.core.Adam(learning_rate=1e-3, initial_scale=0.1), dim, rows=1 << 22)
        lk = t.link(B * S)
        for ids in data + data:
            lk.pull(ids, training=True); lk.push()
        k = [0]
        def pull():
            lk.pull(data[k[0] % 8], training=True); k[0] += 1
        def both():
            lk.pull(data[k[0] % 8], training=True); lk.push(); k[0] += 1
        tp = timed(pull, a.iters)
        lk.push()
        tb = timed(both, a.iters)
        nu = lk.unique_counts()[0]
        pull_bytes = B * S * 8 + nu * (8 + 2 * 4 * t.ustride)
        push_bytes = nu * 4 * t.gstride + nu * 2 * 4 * t.stride
        out.update(pull_us=tp, push_us=tb - tp, unique=nu, ids=B * S, phases_us=lk.pull_phase_us(), pull_GBps=pull_bytes / tp / 1e3,
                   push_GBps=push_bytes / (tb - tp) / 1e3, pull_frac_of_hbm=pull_bytes / tp / 1e3 / pk["hbm_gbs"],
                   push_frac_of_hbm=push_bytes / (tb - tp) / 1e3 / pk["hbm_gbs"], peak=tag)
    elif a.case == "small_ops":
        # the remaining hand-written kernels against the library op a PyTorch user would reach for
        import torch.nn.functional as TF
        from tensornet_b200.ops import functional as F
        from tensornet_b200.ops.unique import UniqueAssign
        import bench
        B, S, D = a.batch, 26, 16
        ids = bench.make_batches(1, B, S, 13, 3)[0][0].to(dev).reshape(-1)
        ua = UniqueAssign(B * S)
        res = {"unique_assign_us": timed(lambda: ua(ids), a.iters),
               "torch_unique_us": timed(lambda: torch.unique(ids, return_inverse=True, return_counts=True), a.iters)}
        # bag pooling: 100 slots x Poisson(5) ids per bag, dim 64, sum
        nb = B * 20
        lens = torch.poisson(torch.full((nb,), 5.0)).clamp(min=1).long()
        offs = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).to(dev)
        nnz = int(offs[-1])
        U = torch.randn(200_000, 64, device=dev)
        inv = torch.randint(0, 200_000, (nnz,), device=dev, dtype=torch.int32)
        pooled = torch.empty(B, 20 * 64, device=dev)
        offs32 = offs.int()
        res["pool_fwd_us"] = timed(lambda: ext.pool_fwd(U, 64, inv, offs32, B, 20, 64, 0, pooled, 20 * 64), a.iters)
        inv64 = inv.long()
        res["torch_embedding_bag_us"] = timed(lambda: TF.embedding_bag(inv64, U, offs[:-1], mode="sum"), a.iters)
        gU = torch.zeros(200_000, 64, device=dev)
        gout = torch.randn(B, 20 * 64, device=dev)
        res["pool_bwd_us"] = timed(lambda: ext.pool_bwd(gU, 64, inv, offs32, B, 20, 64, 64, 0, gout, 20 * 64), a.iters)
        bag = torch.repeat_interleave(torch.arange(nb, device=dev), lens.to(dev))
        gflat = gout.view(B, 20, 64).permute(1, 0, 2).reshape(nb, 64)
        res["torch_index_add_us"] = timed(lambda: gU.index_add_(0, inv64, gflat[bag]), a.iters)
        # FM second-order term and BCE
        E = torch.randn(B, S * D, device=dev)
        res["fm_fwd_us"] = timed(lambda: F.fm(E, S, D), a.iters)
        def torch_fm():
            x = E.view(B, S, D); s_ = x.sum(1)
            return 0.5 * (s_ * s_ - (x * x).sum(1)).sum(1, keepdim=True)
        res["torch_fm_us"] = timed(torch_fm, a.iters)
        logit, y = torch.randn(B, 1, device=dev), (torch.rand(B, device=dev) < 0.3).float()
        res["bce_us"] = timed(lambda: F.bce_with_logits(logit, y), a.iters)
        res["torch_bce_us"] = timed(lambda: (TF.binary_cross_entropy_with_logits(logit.view(-1), y), torch.sigmoid(logit)), a.iters)
        out.update({k: round(v, 2) for k, v in res.items()}, nnz=nnz, ids=int(ids.numel()))
    elif a.case == "deepfm_head":
        # Dense(1) over [h | linear | fm | 1] + loss + the head's whole backward, alone
        from tensornet_b200.ops import functional as F
        B, NH, NL = a.batch, 400, 26
        h = torch.randn(B, 408, device=dev).relu().bfloat16()
        lin, fm = torch.randn(B, NL, device=dev) * 0.1, torch.randn(B, device=dev) * 0.1
        w = torch.nn.Parameter(torch.randn(NH + NL + 2, device=dev) * 0.05)
        y = (torch.rand(B, device=dev) < 0.25).float()
        sums = torch.zeros(4, device=dev)
        us = timed(lambda: F.deepfm_head_loss(h, lin, fm, w, y, sums, NH), a.iters)
        nbytes = B * 408 * 2 * 2 + B * NL * 4 * 2 + B * 12
        out.update(us=us, min_bytes=nbytes, GBps=nbytes / us / 1e3, frac_of_hbm=nbytes / us / 1e3 / pk["hbm_gbs"], peak=tag)
    elif a.case == "mlp_chain":
        # the DeepFM tower 429-400-400-400 as one kernel per direction against the three GEMM launches it replaces
        from tensornet_b200.layers import MLP
        from tensornet_b200.ops import functional as F
        B = a.batch
        mlp = MLP(429, (400, 400, 400)).to(dev)
        x = F.concat_cast([torch.randn(B, 429, device=dev)], ones=True)
        bws = [w.detach().to(torch.bfloat16) for w in mlp.weights]
        outs = [torch.empty((B, 408), dtype=torch.bfloat16, device=dev) for _ in range(3)]
        g = torch.randn(B, 408, device=dev).to(torch.bfloat16)
        bouts = [torch.empty((B, 408), dtype=torch.bfloat16, device=dev), torch.empty((B, 408), dtype=torch.bfloat16, device=dev),
                 torch.empty((B, 432), dtype=torch.bfloat16, device=dev)]
        fwd = lambda: ext.mlp_chain(False, x, 432, bws, [400] * 3, [430, 401, 401], outs, [1, 1, 1], [], [], st)
        bwd = lambda: ext.mlp_chain(True, g, 408, bws[::-1], [400] * 3, [408, 408, 432], bouts, [], [400, 400, 432], [outs[1], outs[0], None], st)
        def layers_fwd():
            h_ = x
            for l in range(3):
                ext.gemm(h_, bws[l], outs[l], B, 400, (430, 401, 401)[l], int(h_.stride(0)), int(bws[l].stride(0)), 408, False, False, False, True,
                         None, None, None, None, 0, 400, 408, 1, 0, st)
                h_ = outs[l]
        flops = 2.0 * B * 400 * (430 + 401 + 401)
        res = {"chain_fwd": timed(fwd, a.iters), "chain_bwd": timed(bwd, a.iters), "three_gemm_launches_fwd": timed(layers_fwd, a.iters)}
        out.update(us=res, tflops={k: flops / v / 1e6 for k, v in res.items()}, shape=[B, 429, 400, 400, 400])
    elif a.case == "sparse_front":
        # the pull split in two: front (dedup, id dispatch, inverse map; plain kernels that run ahead under the previous
        # step) and the probe-only pull that follows it, on the DeepFM batch
        import bench
        from tensornet_b200.ops.sparse_table_gpu import GpuSparseTable
        B, S, dim = a.batch, 26, 20
        data = [b[0].reshape(-1) for b in bench.make_batches(8, B, 3846154, dev, 5)]
        t = GpuSparseTable(tn.core.Adam(learning_rate=1e-3, initial_scale=0.1), dim, rows=1 << 22)
        lk = t.link(B * S)
        for ids in data + data:
            lk.pull(ids, training=True); lk.push()
        k = [0]
        def front():
            lk.prefetch(data[k[0] % 8])
        def back():
            lk.pull(data[k[0] % 8], training=True); lk.push(); k[0] += 1
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        tf, tb = [], []
        for _ in range(a.iters + 3):
            ev[0].record(); front(); ev[1].record(); back(); ev[2].record()
            torch.cuda.synchronize()
            tf.append(ev[0].elapsed_time(ev[1]) * 1e3); tb.append(ev[1].elapsed_time(ev[2]) * 1e3)
        tf, tb = sorted(tf[3:]), sorted(tb[3:])
        out.update(front_us=tf[len(tf) // 2], probe_only_pull_plus_push_us=tb[len(tb) // 2], phases_us=[round(x, 1) for x in lk.pull_phase_us()])
    elif a.case == "deepfm":
        import bench
        slots = [str(i) for i in range(1, 27)]
        model = tn.models.DeepFM(slots, slots, dnn_hidden_units=(400, 400, 400), embedding_dim=16, dense_dim=13,
                                 sparse_opt=tn.core.Adam(learning_rate=1e-3, initial_scale=0.1), bucket_size=a.batch,
                                 table_rows=1 << 22, share_linear_table=True)
        model.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=1e-3)), cuda_graph=False)
        data = bench.make_batches(4, a.batch, 3846154, dev, 7)
        k = [0]
        def step():
            i, d, l = data[k[0] % 4]; k[0] += 1
            model.train_on_batch({tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, ids=i), "dense": d}, l)
        out.update(step_us_eager=timed(step, a.iters))
    else:
        from tensornet_b200.ops.dense_table import DenseTable
        p = torch.nn.Parameter(torch.randn(64 << 20, device=dev))
        dt = DenseTable(tn.core.Adam(learning_rate=1e-3)); dt.init([("p", p)])
        us = timed(lambda: dt.step(), a.iters)
        nbytes = p.numel() * (4 * 7 + 2)          # read g,w,m,v; write w,m,v,g(zero) ; write bf16
        out.update(us=us, GBps=nbytes / us / 1e3, frac_of_hbm=nbytes / us / 1e3 / pk["hbm_gbs"], peak=tag)
    rt.check_status()
    print(json.dumps(out), flush=True)
    tn.core.shutdown()


if __name__ == "__main__":
    main()

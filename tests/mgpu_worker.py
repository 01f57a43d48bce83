"""Worker of tests/test_gpu_multi.py: trains a small DeepFM on WORLD_SIZE GPUs.  Every rank draws the
same global batches and trains on its own slice, so the run is comparable with a one-GPU run on the
full batch.  Rank 0 prints one JSON line."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

import tensornet_b200 as tn


def main():
    out = sys.argv[1]
    tn.core.init()
    rt = tn.core.runtime()
    torch.manual_seed(0)
    slots = [str(i) for i in range(1, 7)]
    Bg = 1024
    B = Bg // rt.world
    model = tn.models.DeepFM(slots, slots, dnn_hidden_units=(64, 32), embedding_dim=8, dense_dim=5,
                             sparse_opt=tn.core.Adam(learning_rate=5e-3, initial_scale=0.1), bucket_size=Bg, table_rows=1 << 16)
    model.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=5e-3)), cuda_graph=True, graph_warmup=2)
    g = torch.Generator().manual_seed(1)
    data = []
    for _ in range(6):
        ids = torch.randint(0, 3000, (len(slots), Bg), generator=g, dtype=torch.int64) * 2654435761 + 17
        dense = torch.randn(Bg, 5, generator=g)
        label = ((ids[0] % 3 == 0) ^ (torch.rand(Bg, generator=g) < 0.1)).float()
        lo, hi = rt.rank * B, (rt.rank + 1) * B
        data.append(({tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, ids=ids[:, lo:hi].contiguous()), "dense": dense[lo:hi]}, label[lo:hi]))
    losses = []
    # every step names the batch of the following one, as `fit` does: after the warm-up the captured steps run that
    # batch's dedup and id dispatch ahead on a second stream (the last step names a batch that never comes: its
    # front is discarded by whatever touches the tables next)
    tn.core.config.pull_front_ahead = 1      # every rank feeds batches of one shape at every step
    order = [data[k % len(data)] for k in range(5 * len(data) + 1)]
    for k in range(5 * len(data)):
        if True:
            f, y = order[k]
            l = model.train_on_batch(f, y, next_batch=order[k + 1])
            t = l.detach().clone()
            if rt.world > 1:
                torch.distributed.all_reduce(t, group=rt.device_group)
            losses.append(float(t) / rt.world)
    torch.cuda.synchronize()
    rt.check_status()
    # synchronised batch norm: every rank ends with the statistics of all ranks' batches
    bn = tn.layers.TNBatchNormalization(11, name="bn_sync", synchronized=True, sync_freq=2)
    bn.train()
    gb = torch.Generator().manual_seed(7)
    allx = [torch.randn(rt.world * 64, 11, generator=gb) * (k + 1) + k for k in range(4)]
    for xk in allx:
        bn(xk[rt.rank * 64:(rt.rank + 1) * 64].to(rt.device))
    torch.cuda.synchronize()
    rt.check_status()
    cat = torch.cat(allx).double()
    bn_ok = bool(torch.allclose(bn.moving_mean.cpu().double(), cat.mean(0), atol=1e-5)
                 and torch.allclose(bn.moving_variance.cpu().double(), cat.var(0, unbiased=False), rtol=1e-3, atol=1e-3))
    bn_oks = rt.all_gather_object(bn_ok)
    # sharded serving: lookups through the read-only fused pull against a replicated dictionary on the same rank
    import numpy as np
    from tensornet_b200.layers import DenseHead, MLP
    from tensornet_b200.serving import EmbeddingDictionary, InferenceEngine, ShardedInferenceEngine
    rng = np.random.default_rng(5)
    signs = np.unique(rng.integers(1, 2 ** 40, 4000, dtype=np.int64).astype(np.uint64))
    weights = rng.standard_normal((len(signs), 8)).astype(np.float32) * 0.3
    torch.manual_seed(3)
    s_mlp, s_head = MLP(4 * 8, [16]).to(rt.device), DenseHead(16).to(rt.device)
    ref_eng = InferenceEngine(EmbeddingDictionary(signs, weights), s_mlp, s_head, 4)
    sh_eng = ShardedInferenceEngine.from_dictionary(signs, weights, s_mlp, s_head, 4, 4 * 32)
    rq = np.random.default_rng(50 + rt.rank)
    serving_ok = True
    for _ in range(3):
        pick = signs[rq.integers(0, len(signs), (4, 32))].view(np.int64)
        req = torch.from_numpy(np.where(rq.random((4, 32)) < 0.85, pick, rq.integers(2 ** 41, 2 ** 42, (4, 32), dtype=np.int64)))
        serving_ok = serving_ok and bool(torch.allclose(ref_eng.infer(req).cpu(), sh_eng.infer(req).cpu(), atol=2e-3))
    torch.cuda.synchronize()
    rt.check_status()
    serving_oks = rt.all_gather_object(serving_ok)
    # checkpoint round trip across the ranks: save (streamed export per rank), move the weights on, load, same predictions
    ck = out + ".ckpt"
    f0, y0 = data[0]
    _, p_before = model.predict_step((f0, y0))
    p_before = p_before.detach().float().cpu().clone()
    model.save_weights(ck, mode="bin")
    model.train_on_batch(f0, y0)
    _, p_moved = model.predict_step((f0, y0))
    model.is_loaded_from_checkpoint = False
    model.load_weights(ck, mode="bin")
    _, p_after = model.predict_step((f0, y0))
    torch.cuda.synchronize()
    rt.check_status()
    ckpt_ok = bool(torch.allclose(p_after.detach().float().cpu(), p_before, atol=2e-3)) and \
        not bool(torch.allclose(p_moved.detach().float().cpu(), p_before, atol=1e-6))
    ckpt_oks = rt.all_gather_object(ckpt_ok)
    # unequal input: rank 0 holds 9 batches, the others 3; BalanceDataset hands batches over so that every rank takes
    # the same number of steps, the step log aggregates over ranks, the guard words of the shared regions are intact
    from tensornet_b200.parallel.symm import verify_all_arenas
    mine = [data[i % len(data)] for i in range(9 if rt.rank == 0 else 3)]
    log = tn.utils.StepLog(None, every=2)
    steps0 = model.optimizer.iterations
    model.fit(tn.data.BalanceDataset(mine), epochs=1, callbacks=[log], prefetch=False)
    torch.cuda.synchronize()
    rt.check_status()
    verify_all_arenas()
    took = model.optimizer.iterations - steps0
    tooks = rt.all_gather_object(took)
    balance_ok = len(set(tooks)) == 1 and took == (9 + 3 * (rt.world - 1)) // rt.world and len(log.records) >= 1 \
        and all(r["world"] == rt.world and r["examples"] == r["steps"] * Bg for r in log.records)
    balance_oks = rt.all_gather_object(bool(balance_ok))
    rows = [int(m.table.n_rows) for m in (model.linear_emb, model.deep_emb)]
    allrows = rt.all_gather_object(rows)
    w = model.sub_model.head.weight.detach().float().cpu()
    ws = rt.all_gather_object(w)
    if rt.rank == 0:
        same = all(torch.equal(ws[0], x) for x in ws)
        json.dump({"world": rt.world, "losses": losses, "rows": [sum(r[i] for r in allrows) for i in range(2)],
                   "replicas_identical": same, "bn_sync_ok": all(bn_oks), "serving_ok": all(serving_oks), "ckpt_ok": all(ckpt_oks), "balance_ok": all(balance_oks), "balance_steps": tooks, "graph": model._graph is not None,
                   "multimem": bool(getattr(model.optimizer.table, "uses_multimem", False))}, open(out, "w"))
    tn.core.shutdown()


if __name__ == "__main__":
    main()

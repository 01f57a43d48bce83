"""Other model families and the serving engine on the GPU path."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ragged_batches(tn, slots, B, n, seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        feats = {}
        first = None
        for k, s in enumerate(slots):
            lens = torch.randint(1, 4, (B,), generator=g)
            offs = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
            vals = torch.randint(0, 500, (int(offs[-1]),), generator=g, dtype=torch.int64) * 7919 + k * 1000003
            feats[s] = tn.data.Ragged(vals, offs.int())
            if first is None:
                first = vals[offs[:-1]]
        feats["dense"] = torch.randn(B, 3, generator=g)
        y = (first % 2 == 0).float()
        feats["label"] = y
        out.append((feats, y))
    return out


def _train(tn, family):
    torch.manual_seed(0)
    slots = ["a", "b", "c"]
    opt = tn.core.AdaGrad(learning_rate=0.05, initial_g2sum=0.1, initial_scale=0.1)
    kw = dict(dnn_hidden_units=(32, 16), embedding_dim=8, dense_dim=3, sparse_opt=opt, bucket_size=2048, table_rows=1 << 15)
    if family == "wide_deep":
        m = tn.models.WideDeep(slots, slots, target_columns=["label"], combiner="mean", **kw)
    elif family == "deep_cross":
        m = tn.models.DeepCross(slots, combiner="sum", **kw)
    else:
        m = tn.models.DCNv2(slots, combiner="sum", num_cross=2, **kw)
    m.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=5e-3)))
    data = _ragged_batches(tn, slots, 256, 6, seed=2)
    losses = []
    for epoch in range(6):
        for f, y in data:
            losses.append(float(m.train_on_batch(f, y)))
    return losses


@pytest.mark.parametrize("family", ["wide_deep", "deep_cross", "dcn_v2"])
def test_model_families_follow_the_cpu_oracle(tn_gpu, family):
    """Ragged (multi-hot) inputs, AdaGrad tables, every tower type: the GPU run must follow the trajectory of the
    same model on the CPU path (plain C++ tables + PyTorch restatement of the kernels)."""
    tn = tn_gpu
    gpu = _train(tn, family)
    torch.cuda.synchronize()
    tn.core.runtime().check_status()
    try:
        tn.core.shutdown(); tn.core.config.force_cpu = True; tn.core.init()
        cpu = _train(tn, family)
    finally:
        tn.core.shutdown(); tn.core.config.force_cpu = False; tn.core.init()
    assert all(np.isfinite(gpu))
    assert np.mean(gpu[-6:]) < np.mean(gpu[:6])
    # identical arithmetic up to summation order and bf16 rounding: the first steps agree closely, later ones
    # drift apart slowly as the differences feed back through training
    for a, b in zip(gpu[:8], cpu[:8]):
        assert abs(a - b) < 5e-3 * max(1.0, abs(b)), (family, gpu[:8], cpu[:8])
    assert abs(np.mean(gpu[-6:]) - np.mean(cpu[-6:])) < 0.1 * np.mean(cpu[-6:]), (family, gpu[-6:], cpu[-6:])


def test_cross_v2_matches_cpu_restatement(tn_gpu, status_ok):
    from tensornet_b200.models.deep_cross import CrossV2
    from tensornet_b200.ops import functional as F

    dev = tn_gpu.core.runtime().device
    torch.manual_seed(1)
    B, D = 512, 120
    cr = CrossV2(D, 2)
    ref = CrossV2(D, 2)
    ref.load_state_dict(cr.state_dict())
    cr.to(dev)
    x = torch.randn(B, D)
    xin = x.to(dev).requires_grad_(True)
    out = cr(F.concat_cast([xin], ones=True))
    g = torch.randn(B, out.shape[1]).bfloat16()
    g[:, D:] = 0
    out.backward(g.to(dev))
    xr = x.clone().requires_grad_(True)
    outr = ref(F.concat_cast([xr], ones=True))
    outr.backward(g)
    rel = lambda a, b: float((a.float() - b.float()).norm() / (b.float().norm() + 1e-9))
    assert rel(out.cpu()[:, :D], outr[:, :D]) < 2e-2
    assert rel(xin.grad.cpu(), xr.grad) < 3e-2
    for w, wr in zip(cr.weights, ref.weights):
        assert rel(w.grad.cpu()[:, : D + 1], wr.grad[:, : D + 1]) < 3e-2


def test_serving_engine_matches_training_forward(tn_gpu, status_ok):
    tn = tn_gpu
    from tensornet_b200.serving import EmbeddingDictionary, InferenceEngine
    from tensornet_b200.ops import functional as F

    torch.manual_seed(0)
    slots = [str(i) for i in range(6)]
    opt = tn.core.Adam(learning_rate=0.01, initial_scale=0.2)
    cols = [tn.feature_column.embedding_column(tn.feature_column.category_column(s, 512), 8, "mean") for s in slots]
    layer = tn.layers.EmbeddingFeatures(cols, opt, name="srv", is_concat=True, rows=1 << 14)
    ids = torch.randint(0, 300, (6, 256), dtype=torch.int64) * 104729 + 3
    emb = layer({s: ids[i] for i, s in enumerate(slots)}, training=True).detach()
    d = EmbeddingDictionary.from_table(layer.table)
    dev = tn.core.runtime().device
    mlp = tn.layers.MLP(48, [32, 16]).to(dev)
    head = tn.layers.DenseHead(16).to(dev)
    eng = InferenceEngine(d, mlp, head, n_slots=6)
    want = torch.sigmoid(head(mlp(F.concat_cast([emb], ones=True)))).view(-1)
    got1 = eng.infer(ids).clone()
    got2 = eng.infer(ids)                      # second call replays the captured graph
    assert torch.allclose(got1, want, atol=1e-2) and torch.allclose(got2, want, atol=1e-2)
    unseen = eng.infer(ids * 0 + 999999937)    # signs missing from the dictionary contribute zeros
    assert torch.isfinite(unseen).all()


def test_sharded_serving_matches_single_dictionary(tn_gpu, status_ok):
    """The read-only pull (lookup_only) + pooling + towers gives the same probabilities as the single-GPU
    dictionary engine, creates no rows for unknown signs, and replays from its CUDA graph."""
    import numpy as np
    from tensornet_b200.layers import DenseHead, MLP
    from tensornet_b200.serving import EmbeddingDictionary, InferenceEngine, ShardedInferenceEngine

    tn = tn_gpu
    dev = tn.core.runtime().device
    rng = np.random.default_rng(3)
    S, D, B = 6, 8, 64
    signs = np.unique(rng.integers(1, 2 ** 40, 5000, dtype=np.int64).astype(np.uint64))
    weights = rng.standard_normal((len(signs), D)).astype(np.float32) * 0.3
    torch.manual_seed(1)
    mlp = MLP(S * D, [32, 16]).to(dev)
    head = DenseHead(16).to(dev)
    ref = InferenceEngine(EmbeddingDictionary(signs, weights), mlp, head, S, combiner="mean")
    eng = ShardedInferenceEngine.from_dictionary(signs, weights, mlp, head, S, S * B, combiner="mean")
    n0 = eng.table.n_rows
    for k in range(3):
        pick = signs[rng.integers(0, len(signs), (S, B))].view(np.int64)
        unknown = rng.integers(2 ** 41, 2 ** 42, (S, B), dtype=np.int64)
        ids = torch.from_numpy(np.where(rng.random((S, B)) < 0.8, pick, unknown))
        a = ref.infer(ids).cpu()
        b = eng.infer(ids).cpu()
        assert torch.allclose(a, b, atol=2e-3), float((a - b).abs().max())
    assert eng.table.n_rows == n0                      # nothing was inserted
    assert B in eng._graphs

"""End-to-end DeepFM steps on one GPU: eager vs CUDA-graph replay, checkpoint-free sanity."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _make(tn, graph, seed=0, B=512, share=False):
    torch.manual_seed(seed)
    slots = [str(i) for i in range(1, 7)]
    model = tn.models.DeepFM(slots, slots, dnn_hidden_units=(64, 32), embedding_dim=8, dense_dim=5,
                             sparse_opt=tn.core.Adam(learning_rate=5e-3, initial_scale=0.1), bucket_size=B, table_rows=1 << 16,
                             share_linear_table=share)
    model.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=5e-3)), cuda_graph=graph, graph_warmup=2)
    return model, slots


def _batches(tn, slots, B, n, seed=1):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        ids = torch.randint(0, 2000, (len(slots), B), generator=g, dtype=torch.int64) * 2654435761 + 17
        dense = torch.randn(B, 5, generator=g)
        # label depends on the ids so there is something to learn
        label = ((ids[0] % 3 == 0) ^ (torch.rand(B, generator=g) < 0.1)).float()
        out.append(({tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, ids=ids), "dense": dense}, label))
    return out


def test_deepfm_learns_and_graph_matches_eager(tn_gpu):
    tn = tn_gpu
    B = 512
    m1, slots = _make(tn, graph=False)
    m2, _ = _make(tn, graph=True)
    data = _batches(tn, slots, B, 8)
    l1, l2 = [], []
    for epoch in range(6):
        for f, y in data:
            l1.append(float(m1.train_on_batch(f, y)))
            l2.append(float(m2.train_on_batch(f, y)))
    torch.cuda.synchronize()
    tn.core.runtime().check_status()
    assert m2._graph is not None, "the step was not captured"
    assert l1[-1] < 0.75 * l1[0], (l1[0], l1[-1])
    # same seeds, same data: graph replay follows the eager trajectory (atomics reorder sums slightly)
    for a, b in zip(l1, l2):
        assert abs(a - b) < 5e-2 * max(1.0, abs(a)), (a, b)
    y, p = m1.predict_step(data[0])
    assert p.shape[0] == B and float(p.min()) >= 0 and float(p.max()) <= 1
    s = m1.metric_sums()
    assert s["count"] > 0 and 0 < s["ctr"] < 1


@pytest.mark.parametrize("share", [False, True])
def test_fused_deepfm_path_matches_generic_path(tn_gpu, share):
    """The DeepFM-specific fused kernels (gather+FM+operand, head+loss+head backward) against the generic op chain,
    with separate linear / deep tables and with the linear weight stored in the embedding row."""
    tn = tn_gpu
    B = 512
    m1, slots = _make(tn, graph=False, share=share)
    m2, _ = _make(tn, graph=False, share=share)
    assert m2.share_linear_table == share
    m1.use_fused = False
    data = _batches(tn, slots, B, 4, seed=3)
    # same initial dense weights
    m2.load_state_dict(m1.state_dict())
    m2.optimizer.table.refresh_shadow()
    l1, l2 = [], []
    for epoch in range(3):
        for f, y in data:
            l1.append(float(m1.train_on_batch(f, y)))
            l2.append(float(m2.train_on_batch(f, y)))
    torch.cuda.synchronize()
    tn.core.runtime().check_status()
    for a, b in zip(l1, l2):
        assert abs(a - b) < 2e-2 * max(1.0, abs(a)), (l1, l2)
    assert l2[-1] < l2[0]
    s1, s2 = m1.metric_sums(), m2.metric_sums()
    assert abs(s1["ctr"] - s2["ctr"]) < 1e-6 and abs(s1["pctr"] - s2["pctr"]) < 2e-2


def test_ragged_batches_with_repeating_shapes_replay_from_graphs(tn_gpu):
    """Multi-hot (ragged) Wide&Deep batches whose shapes repeat are captured too, one graph per shape; the replayed
    trajectory follows the eager one, and a batch of a new shape simply gets its own graph."""
    import numpy as np
    tn = tn_gpu

    def make(graph):
        torch.manual_seed(4)
        slots = ["1", "2", "3"]
        m = tn.models.WideDeep(slots, slots, dnn_hidden_units=(32, 16), embedding_dim=4, bucket_size=4096, table_rows=1 << 14,
                               use_bn=False)
        m.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=5e-3)), cuda_graph=graph, graph_warmup=2)
        return m, slots

    def batch(rng, B, lens_per_slot):
        lens = np.concatenate([np.full((1, B), n, np.int64) for n in lens_per_slot])
        offs = np.concatenate([[0], np.cumsum(lens.reshape(-1))]).astype(np.int32)
        ids = rng.integers(0, 300, int(offs[-1]), dtype=np.int64) * 2654435761 + 5
        y = (rng.random(B) < 0.3).astype(np.float32)
        return torch.from_numpy(ids), torch.from_numpy(offs), torch.from_numpy(y)

    rng = np.random.default_rng(0)
    shapes = [(64, (1, 2, 3)), (64, (1, 2, 3)), (64, (2, 2, 2)), (64, (2, 2, 3)), (64, (2, 2, 2)), (64, (2, 2, 3))] * 3
    data = [batch(rng, B, lens) for B, lens in shapes]
    m1, slots = make(False)
    m2, _ = make(True)
    l1, l2 = [], []
    for ids, offs, y in data:
        f = {tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, values=ids, offsets=offs, batch_size=64)}
        l1.append(float(m1.train_on_batch(f, y)))
        l2.append(float(m2.train_on_batch(f, y)))
    torch.cuda.synchronize()
    tn.core.runtime().check_status()
    # (1,2,3) and (2,2,2) both have 384 ids: one graph serves both (the offsets are data); (2,2,3) has 448: a second one
    assert len(m2._graphs) == 2, len(m2._graphs)
    for a, b in zip(l1, l2):
        assert abs(a - b) < 5e-2 * max(1.0, abs(a)), (l1, l2)


def test_fit_prefetches_and_reads_every_step_loss(tn_gpu):
    """Model.fit with host batches: the next batch is staged on a copy stream, every step's loss reaches the host
    (one step late), and the trajectory equals train_on_batch on the same data."""
    tn = tn_gpu
    B = 256
    m1, slots = _make(tn, graph=True, B=B)
    m2, _ = _make(tn, graph=True, B=B)
    data = [( {k: (v.pin_memory() if k != tn.data.PACKED_KEY else v.pin_memory()) for k, v in f.items()}, y.pin_memory())
            for f, y in _batches(tn, slots, B, 10)]
    ref = [float(m1.train_on_batch(f, y)) for f, y in data]
    hist = m2.fit(iter(data), epochs=1, prefetch=True, record_step_loss=True)
    torch.cuda.synchronize()
    tn.core.runtime().check_status()
    assert len(hist["step_loss"]) == len(data)
    for a, b in zip(ref, hist["step_loss"]):
        assert abs(a - b) < 5e-2 * max(1.0, abs(a)), (ref, hist["step_loss"])
    assert hist["loss"][-1] == hist["step_loss"][-1]


@pytest.mark.gpu
def test_step_log_windows_on_the_graph_path(tn_gpu, tmp_path):
    """The structured step log closes its windows around graph-replayed steps and reads the table sizes."""
    import json
    tn = tn_gpu
    B = 256
    m, slots = _make(tn, graph=True, B=B)
    data = list(_batches(tn, slots, B, 13))
    path = str(tmp_path / "steps.jsonl")
    log = tn.utils.StepLog(path, every=4)
    m.fit(iter(data), epochs=1, callbacks=[log])
    tn.core.runtime().check_status()
    lines = [json.loads(l) for l in open(path)]
    assert [l["steps"] for l in lines] == [4, 4, 4]
    for l in lines:
        assert l["examples"] == 4 * B and l["examples_per_s"] > 0 and l["loss"] > 0 and l["status"] == "ok"
        for t in l["tables"].values():
            assert t["rows"] > 0 and 0 < t["max_load"] < 1


def test_training_through_table_growth_matches_a_large_table(tn_gpu):
    """A model whose shards start tiny trains from a CUDA graph while the status poll enlarges them (twice) and rows
    are shed once in between; its predictions equal those of the same run on shards that were large from the start."""
    tn = tn_gpu
    slots = [str(i) for i in range(1, 5)]
    B = 32

    def run(rows, grow_at):
        tn.core.config.status_poll_steps = 1
        tn.core.config.table_grow_at = grow_at
        torch.manual_seed(7)
        opt = tn.core.AdaGrad(learning_rate=0.05, initial_g2sum=0.1, initial_scale=0.1, show_threshold=1.5, no_show_days=1000)
        m = tn.models.DeepFM(slots, slots, dnn_hidden_units=(32, 16), embedding_dim=8, sparse_opt=opt, bucket_size=4 * B, table_rows=rows)
        m.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=1e-2)))
        g = torch.Generator().manual_seed(3)
        dropped = 0
        for step in range(90):
            ids = torch.randint(0, 40 * (step + 1), (len(slots), B), generator=g, dtype=torch.int64)
            f = {tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, ids=ids)}
            m.train_on_batch(f, (ids[0] % 3 == 0).float())
            if step == 60:
                torch.cuda.synchronize()
                dropped = m.evict_sparse_rows()
        torch.cuda.synchronize()
        tn.core.runtime().check_status()
        ids = torch.randint(0, 2000, (len(slots), B), generator=g, dtype=torch.int64)
        p = m.predict_on_batch({tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, ids=ids)})
        return p.float().cpu(), m.deep_emb.table.grown, dropped, m._graph is not None

    try:
        p_small, grown, dropped_s, graphed = run(2048, 0.5)
        p_big, grown_big, dropped_b, _ = run(1 << 15, 0.0)
    finally:
        tn.core.config.status_poll_steps = 16
        tn.core.config.table_grow_at = 0.85
    assert graphed and grown >= 2 and grown_big == 0
    assert dropped_s == dropped_b and dropped_s > 0
    assert torch.allclose(p_small, p_big, atol=1e-6), float((p_small - p_big).abs().max())


def test_fit_from_pinned_batches_native_step_path_matches_torch_calls(tn_gpu):
    """`fit` on page-locked host batches: inputs staged and losses read back through the native per-step calls
    against the same run issued with torch stream / event / copy calls; every step's loss reaches the host, and a
    page-locked batch released right after its step is not handed out again before its copy has run."""
    tn = tn_gpu
    B = 512
    runs = []
    for native in (True, False):
        tn.core.config.native_step_path = native
        try:
            m, slots = _make(tn, graph=True, seed=5)
            data = _batches(tn, slots, B, 6, seed=8)

            def stream():
                for epoch in range(5):
                    for f, y in data:
                        # fresh page-locked copies every step, dropped as soon as the step is issued
                        pf = {tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, ids=f[tn.data.PACKED_KEY].ids.clone().pin_memory()),
                              "dense": f["dense"].clone().pin_memory()}
                        yield pf, y.clone().pin_memory()

            hist = m.fit(stream(), epochs=1, record_step_loss=True)
            torch.cuda.synchronize()
            tn.core.runtime().check_status()
            assert m._graph is not None
            assert len(hist["step_loss"]) == 30
            runs.append(hist["step_loss"])
        finally:
            tn.core.config.native_step_path = True
    for a, b in zip(*runs):
        assert abs(a - b) < 5e-2 * max(1.0, abs(a)), (a, b)
    assert runs[0][-1] < runs[0][0]


@pytest.mark.parametrize("share", [False, True])
def test_pull_front_run_ahead_in_the_captured_ring_matches_the_plain_path(tn_gpu, share):
    """`fit` names the following batch, so the captured steps run the next batch's dedup and id dispatch ahead (three
    input sets, cold + warm graphs); the trajectory equals the one without run-ahead, also across an evaluation in the
    middle of training (which discards the pending front) and a second `fit`."""
    tn = tn_gpu
    B = 512
    runs = []
    for ahead in (True, False):
        tn.core.config.pull_front_ahead = 1 if ahead else 0
        try:
            m, slots = _make(tn, graph=True, seed=7, share=share)
            data = _batches(tn, slots, B, 7, seed=9)
            h1 = m.fit(data * 3, epochs=1, record_step_loss=True)
            ev = m.evaluate(data[:2])
            h2 = m.fit(data * 2, epochs=1, record_step_loss=True)
            torch.cuda.synchronize()
            tn.core.runtime().check_status()
            assert bool(m._rings) == ahead, "the ring of captured steps was %sused" % ("not " if ahead else "")
            runs.append((h1["step_loss"] + h2["step_loss"], ev))
        finally:
            tn.core.config.pull_front_ahead = -1
    (la, ea), (lb, eb) = runs
    assert len(la) == len(lb) == 35
    for a, b in zip(la, lb):
        assert abs(a - b) < 5e-2 * max(1.0, abs(a)), (la, lb)
    assert la[-1] < 0.8 * la[0]

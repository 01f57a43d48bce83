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

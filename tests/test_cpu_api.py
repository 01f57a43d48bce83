"""Python surface on the CPU path: feature columns, EmbeddingFeatures (pooling, CVM columns, shared
tables), sequence features, batch-norm table, metrics, done-file helpers, tools, serving."""
import os

import numpy as np
import pytest
import torch

import tensornet_b200 as tn
from tensornet_b200.data import Ragged


@pytest.fixture(autouse=True)
def _cpu_runtime():
    tn.core.shutdown()
    tn.core.config.force_cpu = True
    tn.core.init()
    yield
    tn.core.shutdown()


def _cols(keys, dim, combiner="sum", bucket=64):
    return [tn.feature_column.embedding_column(tn.feature_column.category_column(k, bucket), dim, combiner) for k in keys]


def test_api_surface_names():
    for name in ["init", "AdaGrad", "Adam", "Ftrl", "get_opt_learning_rate", "set_sparse_init_mode", "create_sparse_table",
                 "create_dense_table", "create_bn_table", "save_sparse_table", "load_sparse_table", "save_dense_table",
                 "load_dense_table", "save_bn_table", "load_bn_table", "shard_num", "self_shard_id", "barrier",
                 "reset_balance_dataset", "show_decay"]:
        assert hasattr(tn.core, name), name
    assert tn.feature_column.category_column("a").bucket_size == 1024
    assert tn.core.shard_num() == 1 and tn.core.self_shard_id() == 0
    for name in ["EmbeddingFeatures", "SequenceEmbeddingFeatures", "TNBatchNormalization", "PCTRDNNBatchNormalization",
                 "TNBatchNormalizationBase", "PositionMappingLayer"]:
        assert hasattr(tn.layers, name)
    assert hasattr(tn.model, "Model") and hasattr(tn.model, "PCGradModel") and hasattr(tn.optimizer, "PCGrad")
    assert hasattr(tn.callbacks, "PsWeightCheckpoint") and hasattr(tn.distribute, "PsStrategy")
    assert hasattr(tn.data, "list_files") and hasattr(tn.data, "BalanceDataset") and callable(tn.utils.StepLog)
    assert isinstance(tn.__version__, str) and tn.__version__


def test_embedding_features_pooling_and_push():
    opt = tn.core.AdaGrad(learning_rate=0.1, initial_g2sum=0.1, initial_scale=1.0)
    layer = tn.layers.EmbeddingFeatures(_cols(["a", "b"], 4, "mean"), opt, name="emb", is_concat=False)
    feats = {"a": torch.tensor([11, 12, 11]),
             "b": Ragged(torch.tensor([5, 6, 7, 5]), torch.tensor([0, 2, 2, 4]))}        # bags: [5,6] [] [7,5]
    layer.train()
    out = layer(feats)
    assert len(out) == 2 and out[0].shape == (3, 4)
    w = {s: layer.table.native.pull(np.array([s], np.uint64))[0] for s in (11, 12, 5, 6, 7)}
    assert np.allclose(out[0][0].detach(), w[11]) and np.allclose(out[0][1].detach(), w[12])
    assert np.allclose(out[1][0].detach(), (w[5] + w[6]) / 2) and np.allclose(out[1][1].detach(), 0)
    assert np.allclose(out[1][2].detach(), (w[7] + w[5]) / 2)
    loss = (out[0].sum() + 2 * out[1].sum())
    loss.backward()
    layer.backwards()
    # sign 11 appears twice in column a (grad 1 each), sign 5 twice in column b (grad 2 * 1/2 each)
    g = {11: 2.0, 12: 1.0, 5: 2.0, 6: 1.0, 7: 1.0}
    for s, gv in g.items():
        g2 = 0.1 + gv * gv          # mean over dim of g^2 with all components equal
        want = w[s] - 0.1 * gv / (1e-8 + np.sqrt(g2))
        assert np.allclose(layer.table.native.pull(np.array([s], np.uint64))[0], want, rtol=1e-5), s


def test_cvm_columns_and_shared_table():
    opt = tn.core.AdaGrad(learning_rate=0.1, initial_g2sum=0.1)
    l1 = tn.layers.EmbeddingFeatures(_cols(["a"], 4), opt, name="x", is_concat=True, target_columns=["label"], embedding_share="g")
    l2 = tn.layers.EmbeddingFeatures(_cols(["b"], 4), opt, name="y", is_concat=True, target_columns=["label"], embedding_share="g")
    assert l1.sparse_table_handle == l2.sparse_table_handle
    feats = {"a": torch.tensor([1, 1, 2]), "b": torch.tensor([1, 3, 3]), "label": torch.tensor([1.0, 0.0, 1.0])}
    l1.train()
    o = l1(feats)
    assert o.shape == (3, 6) and float(o[:, 4:].abs().sum()) == 0     # no shows yet
    o.sum().backward()
    l1.backwards()
    o = l1(feats, training=False)
    assert o[0, 4] == 2 and abs(float(o[0, 5]) - (np.log(2) - np.log(3))) < 1e-6     # show 2, click 1 for sign 1
    o2 = l2(feats, training=False)
    assert torch.allclose(o2[0, :4], o[0, :4])                         # same table: sign 1 has one row


def test_sequence_features_and_position_mapping():
    opt = tn.core.Adam(learning_rate=0.01)
    col = tn.feature_column.embedding_column(tn.feature_column.sequence_category_column(tn.feature_column.category_column("s", 64), 3), 4)
    layer = tn.layers.SequenceEmbeddingFeatures([col], opt, name="seq")
    feats = {"s": Ragged(torch.tensor([9, 8, 7, 6, 9]), torch.tensor([0, 4, 4, 5]))}
    layer.train()
    out, lengths = layer(feats)
    assert out.shape == (3, 3, 4) and lengths.tolist() == [3, 0, 1]   # first sequence truncated to max_length 3
    assert torch.allclose(out[0, 0], out[2, 0]) and float(out[1].abs().sum()) == 0
    out.sum().backward()
    layer.backwards()
    pm = tn.layers.PositionMappingLayer([3, 5, 9])
    pm.train()
    assert pm(torch.tensor([5, 9])).tolist() == [[0, 1, 0], [0, 0, 1]]
    pm.eval()
    assert pm(torch.tensor([5, 9])).tolist() == [[1, 0, 0], [1, 0, 0]]
    with pytest.raises(ValueError):
        pm.train()
        pm(torch.tensor([4]))


def test_bn_table_moments_window_and_layer(tmp_path):
    bn = tn.layers.TNBatchNormalization(3, max_count=50)
    bn.train()
    x = torch.randn(40, 3) * 2 + 1
    y = bn(x)
    assert torch.allclose(bn.moving_mean, x.mean(0), atol=1e-5) and torch.allclose(bn.moving_variance, x.var(0, unbiased=False), atol=1e-4)
    assert torch.allclose(y, (x - x.mean(0)) / torch.sqrt(x.var(0, unbiased=False) + 1e-5), atol=1e-4)
    bn(x)                                   # 80 records > max_count: further batches decay instead of adding
    before = bn.table.total_count.copy()
    bn(x)
    assert np.array_equal(bn.table.total_count, before)
    bn.save_bn_table(str(tmp_path))
    mean = bn.moving_mean.clone()
    tn.core.shutdown(); tn.core.config.force_cpu = True; tn.core.init()     # a fresh process builds the same handles
    bn2 = tn.layers.TNBatchNormalization(3, max_count=50)
    bn2.load_bn_table(str(tmp_path))
    assert torch.allclose(bn2.moving_mean, mean)
    pc = tn.layers.PCTRDNNBatchNormalization(3)
    pc.train()
    pc(x)
    assert pc.table.use_pctr_dnn_bn


def test_metrics_and_done_file(tmp_path):
    y = torch.tensor([1.0, 0, 0, 1]); p = torch.tensor([0.9, 0.2, 0.4, 0.7])
    c, pc, co, auc = tn.metric.CTR(), tn.metric.PCTR(), tn.metric.COPC(), tn.metric.AUC()
    for m in (c, pc, co, auc):
        m.update_state(y, p)
    assert c.result() == 0.5 and abs(pc.result() - 0.55) < 1e-6 and abs(co.result() - 2 / 2.2) < 1e-6
    assert auc.result() > 0.99
    assert tn.model.read_last_train_dt(str(tmp_path)) is None
    tn.model.save_done_info(str(tmp_path), "2024-01-02")
    assert tn.model.load_done_info(str(tmp_path)) == {"dt": "2024-01-02"}


def test_tools_merge_resize_and_serving_dictionary(tmp_path):
    from tensornet_b200 import tools
    from tensornet_b200.serving import EmbeddingDictionary, InferenceEngine
    from tensornet_b200.layers import MLP, DenseHead

    opt = tn.core.AdaGrad(learning_rate=0.1, initial_g2sum=0.1)
    layer = tn.layers.EmbeddingFeatures(_cols(["a", "b"], 4, "mean"), opt, name="deep", is_concat=True)
    ids = torch.arange(1, 41).view(2, 20)
    feats = {"a": ids[0], "b": ids[1]}
    emb = layer(feats, training=True).detach()
    cp = str(tmp_path / "cp")
    layer.save_sparse_table(cp, "txt")
    tdir = os.path.join(cp, "sparse_table", "deep")
    out = str(tmp_path / "dict.txt")
    assert tools.merge_sparse(tdir, out) == 40
    d = EmbeddingDictionary.from_file(out)
    assert d.n == 40 and d.dim == 4
    assert np.allclose(d.lookup_cpu(np.array([1, 999], np.uint64))[0], emb[0, :4], rtol=1e-5)
    assert np.all(d.lookup_cpu(np.array([999], np.uint64)) == 0)
    # re-shard 1 -> 3 ranks -> merge again: same dictionary
    assert tools.resize_sparse(tdir, str(tmp_path / "r3"), 3, "bin") == 40
    assert sorted(os.listdir(tmp_path / "r3")) == ["rank_0", "rank_1", "rank_2"]
    s3, r3, name, dim = tools.read_sparse_table(str(tmp_path / "r3"), "AdaGrad", 4)
    assert name == "AdaGrad" and sorted(s3.tolist()) == list(range(1, 41))
    assert tools.merge_extra_embedding(tdir, str(tmp_path / "extra"), {1: 1001, 77: 1002}) == 1
    s4, r4, _, _ = tools.read_sparse_table(str(tmp_path / "extra"))
    assert 1001 in s4.tolist() and np.allclose(r4[s4.tolist().index(1001)], r4[s4.tolist().index(1)])
    # serving: dictionary lookup + towers equals the training-time forward
    torch.manual_seed(0)
    mlp, head = MLP(8, [8, 4]), DenseHead(4)
    eng = InferenceEngine(d, mlp, head, n_slots=2)
    from tensornet_b200.ops import functional as F
    want = torch.sigmoid(head(mlp(F.concat_cast([emb], ones=True)))).view(-1)
    got = eng.infer(ids)
    assert torch.allclose(got, want, atol=2e-2)


def test_pcgrad_projection_and_two_task_model():
    """Conflicting task gradients are projected onto each other's normal plane; agreeing ones are summed untouched
    (tensornet/optimizer/pcgrad.py).  Then one two-task step on the CPU path moves dense and sparse weights."""
    from tensornet_b200.optimizer import PCGrad

    g1 = torch.tensor([1.0, 0.0])
    g2 = torch.tensor([-1.0, 1.0])                      # g1.g2 = -1: conflict
    p1 = g1 - (g1 @ g2) / (g2 @ g2) * g2                # (0.5, 0.5)
    p2 = g2 - (g2 @ g1) / (g1 @ g1) * g1                # (0, 1)
    got = PCGrad.project(None, [g1, g2])
    assert torch.allclose(got, p1 + p2)
    assert torch.allclose(PCGrad.project(None, [g1, torch.tensor([2.0, 1.0])]), torch.tensor([3.0, 1.0]))

    class TwoTask(tn.model.PCGradModel):
        def __init__(self):
            super().__init__()
            self.emb = tn.layers.EmbeddingFeatures(_cols(["a", "b"], 4), tn.core.AdaGrad(learning_rate=0.05), name="emb",
                                                   is_concat=True)
            self.tower = torch.nn.Linear(8, 2)

        def forward(self, features):
            return self.tower(self.emb(features))

    torch.manual_seed(0)
    m = TwoTask()
    m.compile(optimizer=PCGrad(tn.core.Adam(learning_rate=0.01)))
    feats = {"a": torch.tensor([1, 2, 3, 1]), "b": torch.tensor([7, 7, 8, 9])}
    labels = torch.tensor([[1.0, 0.0], [0.0, 0.0], [1.0, 1.0], [0.0, 1.0]])
    l0 = float(m.train_on_batch(feats, labels))
    w0 = m.tower.weight.detach().clone()
    row0 = m.emb.table.native.pull(np.array([1], np.uint64))[0].copy()
    losses = [float(m.train_on_batch(feats, labels)) for _ in range(30)]
    assert losses[-1] < l0
    assert not torch.allclose(m.tower.weight.detach(), w0)
    assert not np.allclose(m.emb.table.native.pull(np.array([1], np.uint64))[0], row0)


def test_dense_learning_rate_schedule_is_evaluated_every_step():
    """``learning_rate`` may be a callable ``step -> float`` (the reference accepts a Keras schedule object,
    core/main/py_wrapper.cc:47-59; tensornet/optimizer/optimizer.py:30-36): with the rate at zero nothing moves, and the
    first non-zero step moves every weight by about that rate (Adam's first update is lr * sign(g))."""
    seen = []

    def sched(step):
        seen.append(step)
        return 0.0 if step < 2 else 0.5

    opt = tn.core.Adam(learning_rate=sched)
    assert tn.core.get_opt_learning_rate(opt) is sched          # handed back as given, like the reference

    class Tiny(tn.model.Model):
        def __init__(self):
            super().__init__()
            self.emb = tn.layers.EmbeddingFeatures(_cols(["a"], 4), tn.core.AdaGrad(learning_rate=0.0), name="e", is_concat=True)
            self.lin = torch.nn.Linear(4, 1)

        def forward(self, features):
            return self.lin(self.emb(features))

    torch.manual_seed(0)
    m = Tiny()
    m.compile(optimizer=tn.optimizer.Optimizer(opt))
    f, y = {"a": torch.tensor([1, 2, 3, 4])}, torch.tensor([1.0, 0.0, 1.0, 0.0])
    m.train_on_batch(f, y)
    w0 = m.lin.weight.detach().clone()
    m.train_on_batch(f, y)
    assert torch.equal(m.lin.weight.detach(), w0)            # steps 0 and 1 ran with rate 0
    m.train_on_batch(f, y)
    moved = (m.lin.weight.detach() - w0).abs()
    assert float(moved.max()) > 0.05 and float(moved.max()) < 0.6
    assert seen[-3:] == [0, 1, 2] or seen[-1] == 2


def test_set_sparse_init_mode_zeroes_new_rows_until_switched_back():
    """core/main/py_wrapper.cc `set_sparse_init_mode`: rows created outside training start at zero."""
    opt = tn.core.AdaGrad(learning_rate=0.1, initial_scale=1.0)
    h = tn.core.create_sparse_table(opt, "t", 4)
    t = tn.core.sparse_table(h)
    a = t.native.pull(np.array([101], np.uint64))[0]
    assert np.abs(a).sum() > 0
    tn.core.set_sparse_init_mode(opt, False)
    assert np.abs(t.native.pull(np.array([202], np.uint64))[0]).sum() == 0
    assert np.allclose(t.native.pull(np.array([101], np.uint64))[0], a)       # existing rows are untouched
    tn.core.set_sparse_init_mode(opt, True)
    assert np.abs(t.native.pull(np.array([303], np.uint64))[0]).sum() > 0


def test_ps_strategy_scope_and_checkpoint_callback_cycle(tmp_path):
    """`PsStrategy().scope()` (tensornet/distribute/ps_strategy.py:23-58) plus the callback cycle of the example driver:
    train a day with PsWeightCheckpoint, then a fresh model under the same strategy resumes from the done-file."""
    strategy = tn.distribute.PsStrategy()
    assert strategy.num_replicas_in_sync == 1 and strategy.should_checkpoint

    def build():
        m = tn.models.WideDeep(["a", "b"], ["a", "b"], dnn_hidden_units=(8,), embedding_dim=4, bucket_size=64)
        m.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=0.01)))
        return m

    g = torch.Generator().manual_seed(0)
    data = []
    for _ in range(6):
        f = {s: torch.randint(1, 30, (16,), generator=g) for s in ("a", "b")}
        data.append((f, (f["a"] % 2 == 0).float()))
    root = str(tmp_path / "model")
    with strategy.scope():
        m = build()
        cb = tn.callbacks.PsWeightCheckpoint(root, need_save_model=True, dt="2020-05-10", delta_days=1, save_mode="bin")
        m.fit(iter(data), epochs=1, callbacks=[cb])
        want = torch.as_tensor(m.predict_on_batch(data[0][0])).reshape(-1).clone()
    assert tn.model.read_last_train_dt(root) == "2020-05-10"
    tn.core.shutdown(); tn.core.config.force_cpu = True
    with tn.distribute.PsStrategy().scope():
        m2 = build()
        cb2 = tn.callbacks.PsWeightCheckpoint(root, need_save_model=False, dt="2020-05-11", save_mode="bin")
        cb2.set_model(m2)
        m2.predict_on_batch(data[0][0])          # creates the dense table the checkpoint is loaded into
        cb2.on_predict_begin()
        got = torch.as_tensor(m2.predict_on_batch(data[0][0])).reshape(-1)
    assert torch.allclose(got, want, atol=1e-5)


def test_cpu_affinity_follows_the_mask_nvml_gives(monkeypatch):
    """The per-GPU CPU binding against a fake NVML: the process keeps the cores NVML names that it is allowed to use,
    and is left alone when there is no overlap or no NVML."""
    import os
    import sys
    import types
    import importlib
    rtmod = importlib.import_module("tensornet_b200.core.runtime")

    allowed = set(range(8))
    calls = []
    monkeypatch.setattr(os, "sched_getaffinity", lambda pid: set(allowed), raising=False)
    monkeypatch.setattr(os, "sched_setaffinity", lambda pid, cpus: calls.append(set(cpus)), raising=False)
    fake = types.SimpleNamespace(nvmlInit=lambda: None, nvmlDeviceGetHandleByIndex=lambda i: ("h", i),
                                 nvmlDeviceGetHandleByUUID=lambda u: (_ for _ in ()).throw(RuntimeError("no such GPU")),
                                 nvmlDeviceGetCpuAffinity=lambda h, n: [0b00111100] + [0] * (n - 1))
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    rtmod._bind_cpus_near(0)
    assert calls == [{2, 3, 4, 5}]
    fake.nvmlDeviceGetCpuAffinity = lambda h, n: [1 << 40] + [0] * (n - 1)      # cores this process may not use
    rtmod._bind_cpus_near(0)
    assert len(calls) == 1
    monkeypatch.setitem(sys.modules, "pynvml", None)                              # import fails: nothing happens
    rtmod._bind_cpus_near(0)
    assert len(calls) == 1


def test_lookahead_pairs_every_batch_with_its_successor():
    from tensornet_b200.model.model import _with_next

    assert list(_with_next(iter([]))) == []
    assert list(_with_next(iter([7]))) == [(7, None)]
    assert list(_with_next(iter("abc"))) == [("a", "b"), ("b", "c"), ("c", None)]
    seen = []

    def gen():
        for k in range(4):
            seen.append(k)
            yield k

    it = _with_next(gen())
    assert next(it) == (0, 1) and seen == [0, 1]          # exactly one batch ahead of the consumer


def test_configuration_and_helper_methods_of_the_reference_surface():
    """get_config / from_config of columns, layers and optimizers, the feature filters of the embedding layers, the
    parse spec of a column and PCGrad.compute_gradients (names of tensornet/layers/embedding_features.py:309-392,
    feature_column/category_column.py:52-58, optimizer/optimizer.py:80-130)."""
    tn.core.init()
    cat = tn.feature_column.category_column("7", bucket_size=64)
    assert cat.parse_example_spec == {"7": ("varlen", "int64")} and cat.parents == ["7"]
    emb = tn.feature_column.embedding_column(cat, 4, "sum")
    again = type(emb).from_config(emb.get_config())
    assert repr(again) == repr(emb)
    seq = tn.feature_column.embedding_column(tn.feature_column.sequence_category_column(tn.feature_column.category_column("s", 32), 5), 4)
    assert type(seq).from_config(seq.get_config()).categorical_column.max_length == 5

    opt = tn.core.AdaGrad(learning_rate=0.05, initial_g2sum=0.2)
    layer = tn.layers.EmbeddingFeatures([emb], opt, name="cfg_layer", is_concat=True, target_columns=["label"])
    cfg = layer.get_config()
    assert cfg["name"] == "cfg_layer" and cfg["sparse_opt"]["name"] == "AdaGrad" and cfg["sparse_opt"]["initial_g2sum"] == 0.2
    cfg["name"] = "cfg_layer_2"
    twin = tn.layers.EmbeddingFeatures.from_config(cfg)
    assert twin.layer_name == "cfg_layer_2" and twin.use_cvm and twin._sparse_opt.initial_g2sum == 0.2
    feats = {"7": torch.tensor([1, 2]), "other": torch.tensor([3, 4]), "label": torch.tensor([1.0, 0.0])}
    assert list(layer.filter_not_used_features(feats)) == ["7"]
    pulled, targets = layer.get_sparse_pulling_feature(feats)
    assert list(pulled) == ["7"] and list(targets) == ["label"]

    slayer = tn.layers.SequenceEmbeddingFeatures([seq], opt, name="cfg_seq")
    scfg = slayer.get_config()
    assert scfg["max_length"] == 5 and list(slayer.get_sparse_pulling_feature({"s": 1, "x": 2})) == ["s"]
    scfg["name"] = "cfg_seq_2"
    assert tn.layers.SequenceEmbeddingFeatures.from_config(scfg).max_length == 5

    bn = tn.layers.TNBatchNormalization(synchronized=True, sync_freq=4, max_count=1000)
    assert bn.get_config()["sync_freq"] == 4 and tn.layers.TNBatchNormalization(**bn.get_config()).max_count == 1000

    dense = tn.optimizer.PCGrad(tn.core.Adam(learning_rate=0.01))
    assert dense.get_config()["dense_opt"]["name"] == "Adam"
    w = torch.nn.Parameter(torch.tensor([1.0, 0.0]))
    dense.attach([("w", w)])
    w = dict(dense.table.named_views())["w"] if hasattr(dense.table, "named_views") else w
    g = dense.compute_gradients([(w * torch.tensor([1.0, 1.0])).sum(), (w * torch.tensor([-1.0, 0.5])).sum()])
    # task gradients (1, 1) and (-1, 0.5) conflict: each loses its component along the other before they are summed
    g1 = torch.tensor([1.0, 1.0]) - (-0.5 / 1.25) * torch.tensor([-1.0, 0.5])
    g2 = torch.tensor([-1.0, 0.5]) - (-0.5 / 2.0) * torch.tensor([1.0, 1.0])
    assert torch.allclose(g[:2].cpu(), g1 + g2, atol=1e-6)

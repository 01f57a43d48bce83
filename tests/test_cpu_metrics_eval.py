"""Compiled metrics are fed during ``fit`` and ``evaluate``; ``predict`` and ``evaluate`` drive the callback hooks; and
the rule that decides when a training step is captured into a CUDA graph keeps several ranks in agreement.
Reference behaviour: tensornet/model/Model.py:79-85,114-115, tensornet/callbacks/callbacks.py:78-91,
examples/main.py:63-74."""
import pytest
import torch

import tensornet_b200 as tn
from tensornet_b200.model.model import graph_decision


@pytest.fixture(autouse=True)
def _cpu_runtime():
    tn.core.shutdown()
    tn.core.config.force_cpu = True
    tn.core.init()
    yield
    tn.core.shutdown()


SLOTS = ["a", "b", "c"]


def _data(n_batches=12, B=64, seed=0):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n_batches):
        f = {s: torch.randint(1, 40, (B,), generator=g) for s in SLOTS}
        out.append((f, ((f["a"] + f["b"]) % 2 == 0).float()))
    return out


def _model(metrics):
    torch.manual_seed(3)
    m = tn.models.WideDeep(SLOTS, SLOTS, dnn_hidden_units=(16, 8), embedding_dim=4, bucket_size=256,
                           sparse_opt=tn.core.AdaGrad(learning_rate=0.1, initial_g2sum=0.1, initial_scale=0.1))
    m.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=0.02)), metrics=metrics)
    return m


def test_fit_feeds_every_compiled_metric_without_per_step_calls():
    data = _data()
    m = _model([tn.metric.AUC(), tn.metric.CTR(), tn.metric.PCTR(), tn.metric.COPC(), "loss"])
    assert m._host_metrics == []          # all five come from the sums the loss keeps
    hist = m.fit(iter(data * 6), epochs=1)
    labels = torch.cat([y for _, y in data * 6])
    assert hist["CTR"][-1] == pytest.approx(float(labels.mean()), rel=1e-6)
    assert 0.0 < hist["PCTR"][-1] < 1.0
    assert hist["COPC"][-1] == pytest.approx(hist["CTR"][-1] / hist["PCTR"][-1], rel=1e-5)
    assert hist["auc"][-1] > 0.6          # the label is a function of the ids: the model learns it
    assert hist["loss"][-1] > 0.0
    # the streamed AUC equals the one computed from all predictions of a pass at once
    res = m.evaluate(iter(data))
    y, p = m.predict(iter(data))
    ref = tn.metric.AUC()
    ref.update_state(y, p)
    assert res["auc"] == pytest.approx(ref.result(), abs=1e-9)
    assert res["CTR"] == pytest.approx(float(y.mean()), rel=1e-6)
    assert res["loss"] == pytest.approx(float(torch.nn.functional.binary_cross_entropy(p.reshape(-1).double(), y.reshape(-1).double())), rel=1e-4)


def test_user_metric_objects_get_update_state_each_step():
    class Acc:
        name = "acc"

        def __init__(self):
            self.hit = self.n = 0

        def reset_state(self):
            self.hit = self.n = 0

        def update_state(self, y, p, sample_weight=None):
            self.hit += int(((p.reshape(-1) > 0.5).float() == y.reshape(-1)).sum())
            self.n += y.numel()

        def result(self):
            return self.hit / max(self.n, 1)

    data = _data(4)
    acc = Acc()
    m = _model([acc, tn.metric.CTR()])
    assert m._host_metrics == [acc]
    hist = m.fit(iter(data * 10), epochs=1)
    assert acc.n == 64 * 40 and 0.0 <= hist["acc"][-1] <= 1.0
    out = m.evaluate(iter(data), return_dict=False)
    assert len(out) == 3 and acc.n == 64 * 4      # evaluate resets metric state first


def test_evaluate_leaves_parameters_alone_and_hooks_fire(tmp_path):
    data = _data(6)
    m = _model([tn.metric.AUC()])
    root = str(tmp_path / "cp")
    m.fit(iter(data), epochs=1, callbacks=[tn.callbacks.PsWeightCheckpoint(root, need_save_model=True, dt="d1", save_mode="bin")])
    before = {k: v.clone() for k, v in m.state_dict().items()}
    want = m.evaluate(iter(data))

    calls = []

    class Spy(tn.callbacks.Callback):
        def on_test_begin(self, logs=None): calls.append("test_begin")
        def on_test_end(self, logs=None): calls.append(("test_end", sorted(logs)))
        def on_predict_begin(self, logs=None): calls.append("predict_begin")
        def on_predict_end(self, logs=None): calls.append("predict_end")

    m.evaluate(iter(data), callbacks=[Spy()])
    m.predict(iter(data), callbacks=[Spy()])
    assert calls == ["test_begin", ("test_end", ["auc", "loss"]), "predict_begin", "predict_end"]
    for k, v in m.state_dict().items():
        assert torch.equal(v, before[k]), k

    # a fresh model restores the checkpoint through the evaluate / predict hooks of PsWeightCheckpoint
    tn.core.shutdown(); tn.core.config.force_cpu = True; tn.core.init()
    m2 = _model([tn.metric.AUC()])
    m2.predict_on_batch(data[0][0])          # builds the dense table the checkpoint is loaded into
    cb = tn.callbacks.PsWeightCheckpoint(root, save_mode="bin")
    got = m2.evaluate(iter(data), callbacks=[cb])
    assert got["auc"] == pytest.approx(want["auc"], abs=1e-6) and got["loss"] == pytest.approx(want["loss"], rel=1e-5)
    tn.core.shutdown(); tn.core.config.force_cpu = True; tn.core.init()
    m3 = _model([])
    m3.predict_on_batch(data[0][0])
    y, p = m3.predict(iter(data), callbacks=[tn.callbacks.PsWeightCheckpoint(root, load_mode="bin")])
    y0, p0 = m.predict(iter(data))
    assert torch.allclose(p, p0, atol=1e-6)


def test_auc_histogram_rides_in_the_sum_buffer():
    from tensornet_b200.ops import functional as F

    g = torch.Generator().manual_seed(1)
    logit, y = torch.randn(500, 1, generator=g) * 2, (torch.rand(500, generator=g) < 0.3).float()
    sums = torch.zeros(4 + 2 * 50)
    F.bce_with_logits(logit, y, sums)
    F.bce_with_logits(logit, y, sums)
    hist = sums[4:].view(torch.int32)
    assert int(hist[:50].sum()) == 2 * int(y.sum()) and int(hist[50:].sum()) == 2 * int((1 - y).sum())
    assert sums[3] == 1000 and sums[1] == pytest.approx(2 * float(y.sum()))


def test_capture_rule_keeps_ranks_in_step():
    # warm-up steps are eager everywhere
    assert graph_decision(8, False, True, 0, 8, 0, 3) == "eager"
    # the first capture happens at the same step on every rank, whatever the shape of that rank's batch
    assert graph_decision(8, False, True, 0, 8, 3, 3) == "capture"
    # a known shape replays; with several ranks no second shape is ever captured (its capture would end in a
    # barrier the other ranks do not enter): a short last batch runs eagerly
    assert graph_decision(8, True, True, 1, 8, 9, 3) == "replay"
    assert graph_decision(8, False, True, 1, 8, 9, 3) == "eager"
    assert graph_decision(2, False, False, 0, 8, 9, 3) == "eager"
    # one rank may capture several shapes, ragged ones up to the cap
    assert graph_decision(1, False, True, 5, 8, 9, 3) == "capture"
    assert graph_decision(1, False, False, 7, 8, 9, 3) == "capture"
    assert graph_decision(1, False, False, 8, 8, 9, 3) == "eager"
    assert graph_decision(1, False, True, 8, 8, 9, 3) == "capture"      # static shapes replace the oldest capture
    # two ranks whose batches differ in size at the capture step still decide alike, step by step
    sizes = {0: [64, 64, 64, 64, 64, 17], 1: [64, 64, 64, 64, 17, 64]}
    trace = {}
    for rank, seq in sizes.items():
        known, eager, out = set(), 0, []
        for b in seq:
            d = graph_decision(2, b in known, True, len(known), 8, eager, 3)
            if d == "eager":
                eager += 1
            if d == "capture":
                known.add(b)
            out.append(d)
        trace[rank] = out
    assert [d == "capture" for d in trace[0]] == [d == "capture" for d in trace[1]]


def test_profile_batches_writes_a_trace(tmp_path):
    data = _data(8)
    m = _model([])
    cb = tn.callbacks.ProfileBatches(str(tmp_path / "prof"), start=2, stop=4)
    m.fit(iter(data), epochs=1, callbacks=[cb])
    import json, os
    assert cb.trace_path and os.path.getsize(cb.trace_path) > 0
    with open(cb.trace_path) as f:
        assert "traceEvents" in json.load(f)


def test_steps_per_epoch_consumes_exactly_that_many_batches_of_a_shared_iterator():
    """`fit` looks one batch ahead; with `steps_per_epoch` the look-ahead must not eat a batch of the next pass."""
    data = _data(n_batches=10)
    taken = []

    def gen():
        for k, b in enumerate(data):
            taken.append(k)
            yield b

    it = gen()
    m = _model([])
    h = m.fit(it, epochs=3, steps_per_epoch=3, record_step_loss=True)
    assert len(h["step_loss"]) == 9
    assert taken == list(range(9))


def test_keras_metric_names_of_the_reference_example():
    """compile(metrics=["acc", "mse", "mae", "mape", AUC, CTR, PCTR, COPC]) as in the reference's examples/main.py."""
    data = _data(4)
    m = _model(["acc", "mse", "mae", "mape", tn.metric.AUC(), tn.metric.CTR(), tn.metric.PCTR(), tn.metric.COPC()])
    assert [x.name for x in m._host_metrics] == ["acc", "mse", "mae", "mape"] and not m._use_graph
    hist = m.fit(iter(data * 5), epochs=1)
    assert set(hist) >= {"loss", "acc", "mse", "mae", "mape", "auc", "CTR", "PCTR", "COPC"}
    # against the definitions, on one batch
    y = torch.tensor([1.0, 0.0, 1.0, 1.0])
    p = torch.tensor([0.9, 0.4, 0.2, 0.6])
    want = {"acc": 0.75, "mse": float(((y - p) ** 2).mean()), "mae": float((y - p).abs().mean()),
            "mape": float((100 * (y - p).abs() / y.abs().clamp(min=1e-7)).mean())}
    for name, v in want.items():
        met = tn.metric.get(name)
        met.update_state(y, p)
        met.update_state(y[:2], p[:2], sample_weight=torch.tensor([0.0, 0.0]))       # weightless examples change nothing
        assert met.name == name and abs(met.result() - v) <= 1e-6 * max(1.0, abs(v))
        met.reset_state()
        assert met.result() == 0.0
    assert tn.metric.get("binary_accuracy").name == "binary_accuracy"
    # the dense part for serving, as sub_model.save(...) in the reference's driver
    import os, tempfile
    with tempfile.TemporaryDirectory() as d:
        path = m.save(os.path.join(d, "saved_model"))
        sd = torch.load(path)
        assert os.path.basename(path) == "sub_model.pt" and set(sd) == set(m.sub_model.state_dict())
    # the calls of the reference's driver: verbose is accepted by fit, predict and evaluate
    y_all, p_all = m.predict(iter(data), verbose=1, callbacks=[])
    assert y_all.shape == p_all.reshape(-1).shape and "loss" in m.evaluate(iter(data), verbose=1)
    with pytest.raises(ValueError):
        tn.metric.get("top_k")

"""Every model family steps on the CPU path (the oracle the GPU tests compare against): losses fall on a fixed batch and
prediction returns one probability per example.  Mirrors the reference's example models
(examples/models/wide_deep.py, examples/models/deepfm.py, examples/models/deep_cross.py)."""
import pytest
import torch

import tensornet_b200 as tn
from tensornet_b200 import models


@pytest.fixture(autouse=True)
def _cpu_runtime():
    tn.core.shutdown()
    tn.core.config.force_cpu = True
    tn.core.init()
    yield
    tn.core.shutdown()


SLOTS = ["s1", "s2", "s3", "s4"]


def _batch(B=64, dense=0, seed=0):
    g = torch.Generator().manual_seed(seed)
    f = {s: torch.randint(1, 50, (B,), generator=g) for s in SLOTS}
    if dense:
        f["dense"] = torch.randn(B, dense, generator=g)
    y = ((f["s1"] + f["s2"]) % 3 == 0).float()
    return f, y


def _build(kind):
    ada = tn.core.AdaGrad(learning_rate=0.05, initial_g2sum=0.1, initial_scale=0.1)
    if kind == "wide_deep":
        return models.WideDeep(SLOTS, SLOTS, dnn_hidden_units=(16, 8), embedding_dim=4, sparse_opt=ada, bucket_size=64), 0
    if kind == "deepfm":
        return models.DeepFM(SLOTS, SLOTS, dnn_hidden_units=(16, 8), embedding_dim=4, sparse_opt=ada, bucket_size=64), 0
    if kind == "deepfm_shared":
        return models.DeepFM(SLOTS, SLOTS, dnn_hidden_units=(16, 8), embedding_dim=4, bucket_size=64, share_linear_table=True,
                             sparse_opt=tn.core.Adam(learning_rate=0.02)), 0
    if kind == "deep_cross":
        return models.DeepCross(SLOTS, dnn_hidden_units=(16, 8), embedding_dim=4, sparse_opt=ada, bucket_size=64, num_cross=2), 0
    if kind == "dcn_v2":
        return models.DCNv2(SLOTS, dnn_hidden_units=(16, 8), embedding_dim=4, dense_dim=3, bucket_size=64, num_cross=2,
                            sparse_opt=tn.core.Ftrl(learning_rate=0.05)), 3
    raise AssertionError(kind)


@pytest.mark.parametrize("kind", ["wide_deep", "deepfm", "deepfm_shared", "deep_cross", "dcn_v2"])
def test_model_family_trains_on_cpu(kind):
    torch.manual_seed(1)
    m, dense = _build(kind)
    m.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=0.01)))
    f, y = _batch(dense=dense)
    first = float(m.train_on_batch(f, y))
    for _ in range(40):
        last = float(m.train_on_batch(f, y))
    assert last < first, (kind, first, last)
    p = m.predict_on_batch(f)
    p = torch.as_tensor(p).reshape(-1)
    assert p.shape[0] == 64 and float(p.min()) >= 0.0 and float(p.max()) <= 1.0


def test_interrupted_save_keeps_previous_done_file(tmp_path):
    """The done-file is written last (tensornet/model/Model.py:165-172): a save that dies between the sparse and the
    dense part leaves `_checkpoint` naming the previous day, and a fresh model resumes from that day."""
    torch.manual_seed(2)
    m, _ = _build("wide_deep")
    m.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=0.01)))
    f, y = _batch()
    for _ in range(3):
        m.train_on_batch(f, y)
    root = str(tmp_path / "model")
    m.save_weights(root, dt="day1", mode="bin")
    want = torch.as_tensor(m.predict_on_batch(f)).reshape(-1).clone()
    for _ in range(3):
        m.train_on_batch(f, y)

    def boom(path):
        raise OSError("disk full")

    real = m.optimizer.save_dense_table
    m.optimizer.save_dense_table = boom
    with pytest.raises(OSError):
        m.save_weights(root, dt="day2", mode="bin")
    m.optimizer.save_dense_table = real
    assert tn.model.read_last_train_dt(root) == "day1"

    tn.core.shutdown(); tn.core.config.force_cpu = True; tn.core.init()
    torch.manual_seed(3)
    m2, _ = _build("wide_deep")
    m2.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=0.01)))
    m2.predict_on_batch(f)                       # builds the dense table
    assert m2.load_weights(root, mode="bin")
    got = torch.as_tensor(m2.predict_on_batch(f)).reshape(-1)
    assert torch.allclose(got, want, atol=1e-5)

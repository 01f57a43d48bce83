"""CPU tables: optimizer math against hand-written formulas of the reference
(core/ps/optimizer/{ada_grad,adam,ftrl}_kernel.cc), dedup, show decay, eviction."""
import math

import numpy as np
import pytest

import tensornet_b200 as tn
from tensornet_b200 import _build
from tensornet_b200.ops.sparse_table_cpu import CpuSparseTable


@pytest.fixture(autouse=True)
def _cpu_runtime(monkeypatch):
    tn.core.shutdown()
    tn.core.config.force_cpu = True
    tn.core.init()
    yield
    tn.core.shutdown()


def test_unique_first_occurrence_counts_show_and_click():
    ext = _build.cpu_ext()
    ids = np.array([7, 3, 7, 9, 3, 7], dtype=np.int64)
    lab = np.array([1, 0, 0, 1, 1, 1], dtype=np.float32)
    u, inv, show, click = ext.unique_first_occurrence(ids, lab)
    assert u.tolist() == [7, 3, 9]              # order of first occurrence (sparse_table_ops.cc:122-131)
    assert inv.tolist() == [0, 1, 0, 2, 1, 0]
    assert show.tolist() == [3, 2, 1]
    assert click.tolist() == [2, 1, 1]


def test_row_init_is_deterministic_normal():
    opt = tn.core.AdaGrad(learning_rate=0.01, initial_g2sum=0.1, initial_scale=0.5)
    t1, t2 = CpuSparseTable(opt, 8), CpuSparseTable(opt, 8)
    signs = np.arange(1, 5001, dtype=np.uint64) * np.uint64(2654435761)
    a = t1.native.pull(signs)
    b = t2.native.pull(signs[::-1].copy())[::-1]
    assert np.array_equal(a, b)                                  # independent of insertion order
    assert abs(a.std() - 0.5 / math.sqrt(8)) < 0.01
    assert abs(a.mean()) < 0.01
    t1.set_training(False)
    z = t1.native.pull(np.array([123456789], dtype=np.uint64))    # inference mode: zero rows
    assert np.all(z == 0)


def test_adagrad_apply_and_cvm_columns():
    opt = tn.core.AdaGrad(learning_rate=0.1, initial_g2sum=0.5, initial_scale=1.0, epsilon=1e-8)
    t = CpuSparseTable(opt, 4, use_cvm=True)
    s = np.array([42], dtype=np.uint64)
    w0 = t.native.pull(s)[0, :4].copy()
    g = np.array([[0.5, -1.0, 2.0, 0.0]], dtype=np.float32)
    t.native.push(s, g, np.array([3.0], np.float32), np.array([1.0], np.float32))
    g2 = 0.5 + float((g ** 2).sum()) / 4
    want = w0 - 0.1 * g[0] / (1e-8 + math.sqrt(g2))
    row = t.native.pull(s)[0]
    assert np.allclose(row[:4], want, rtol=1e-6)
    assert row[4] == 3.0                                                           # show
    assert abs(row[5] - (math.log(2.0) - math.log(4.0))) < 1e-6                   # ln(click+1) - ln(show+1)
    signs, rows = t.dump()
    assert abs(rows[0, 4] - g2) < 1e-6 and rows[0, 5] == 3.0 and rows[0, 6] == 1.0


def test_adam_has_no_bias_correction_and_ftrl_matches_reference_form():
    a = tn.core.Adam(learning_rate=0.01, beta1=0.9, beta2=0.999, epsilon=1e-8)
    t = CpuSparseTable(a, 2)
    s = np.array([5], dtype=np.uint64)
    w0 = t.native.pull(s)[0].copy()
    g = np.array([[1.0, -2.0]], dtype=np.float32)
    t.native.push(s, g, np.ones(1, np.float32), np.zeros(1, np.float32))
    m, v = 0.1 * g[0], 0.001 * g[0] ** 2
    assert np.allclose(t.native.pull(s)[0], w0 - 0.01 * m / (1e-8 + np.sqrt(v)), rtol=1e-5)

    f = tn.core.Ftrl(learning_rate=0.05, beta=1.0, lambda1=0.01, lambda2=1.0, initial_scale=1.0)
    t = CpuSparseTable(f, 2)
    w0 = t.native.pull(s)[0].copy()
    t.native.push(s, g, np.ones(1, np.float32), np.zeros(1, np.float32))
    z = g[0] - 0.05 * (np.sqrt(g[0] ** 2) - 0.0) * w0            # lr multiplies, as written in ftrl_kernel.cc:66
    n = g[0] ** 2
    want = np.where(np.abs(z) <= 0.01, 0.0, -(z - np.sign(z) * 0.01) / ((1.0 + np.sqrt(n)) * 0.05 + 1.0))
    assert np.allclose(t.native.pull(s)[0], want, rtol=1e-5)


def test_show_decay_rules():
    opt = tn.core.AdaGrad(show_decay_rate=0.5)
    t = CpuSparseTable(opt, 2)
    s = np.array([1, 2], dtype=np.uint64)
    t.native.pull(s)
    t.native.push(s, np.zeros((2, 2), np.float32), np.array([4.0, 8.0], np.float32), np.array([2.0, 0.0], np.float32))
    t.show_decay(3)
    _, rows = t.dump()
    rows = rows[np.argsort(_)]
    assert rows[:, 3].tolist() == [2.0, 4.0] and rows[:, 4].tolist() == [1.0, 0.0]
    assert rows[:, 5].view(np.int32).tolist() == [3, 3]            # no_show_days += delta_days


def test_unknown_hyper_parameter_is_rejected():
    with pytest.raises(TypeError):
        tn.core.Adam(learnin_rate=0.1)
    with pytest.raises(ValueError):
        tn.core.AdaGrad(elimination_logic=2)


@pytest.mark.parametrize("kind", ["Adam", "AdaGrad"])
def test_native_dense_step_matches_the_reference_formulas(kind):
    """The one-pass dense optimizer step of the CPU path against the update rules written out in numpy
    (core/ps/optimizer/adam_kernel.cc:46-55, ada_grad_kernel.cc:42-48); the gradient is zeroed on the way."""
    from tensornet_b200 import _build

    ext = _build.cpu_ext()
    rng = np.random.default_rng(4)
    n = 1003
    w = rng.standard_normal(n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    s0 = np.abs(rng.standard_normal(n)).astype(np.float32)
    s1 = np.abs(rng.standard_normal(n)).astype(np.float32) + 0.1
    s2 = rng.standard_normal(n).astype(np.float32)
    lr, b1, b2, eps, gd, md = 0.01, 0.9, 0.999, 1e-8, 0.98, 0.95
    w0, g0, a0, a1, a2 = w.copy(), g.copy(), s0.copy(), s1.copy(), s2.copy()
    if kind == "Adam":
        alpha = lr * np.sqrt(1 - b2 ** 3) / (1 - b1 ** 3)
        ext.dense_step(1, w, g, s0, s1, np.zeros(0, np.float32), lr, alpha, b1, b2, eps, 1.0, 1.0)
        m = a0 + (g0 - a0) * (1 - b1)
        v = a1 + (g0 * g0 - a1) * (1 - b2)
        assert np.allclose(s0, m, rtol=1e-5, atol=1e-6) and np.allclose(s1, v, rtol=1e-5, atol=1e-6)
        assert np.allclose(w, w0 - m * alpha / (np.sqrt(v) + eps), rtol=1e-5, atol=1e-6)
    else:
        ext.dense_step(0, w, g, s0, s1, s2, lr, 0.0, 0.0, 0.0, eps, gd, md)
        c = a0 * gd + 1
        q = a1 * gd + g0 * g0
        m = a2 + (g0 - a2) * (1 - md)
        assert np.allclose(s0, c, rtol=1e-5) and np.allclose(s1, q, rtol=1e-5) and np.allclose(s2, m, rtol=1e-5, atol=1e-6)
        assert np.allclose(w, w0 - lr * m / (np.sqrt(q) / np.sqrt(c) + eps), rtol=1e-5, atol=1e-6)
    assert not g.any()

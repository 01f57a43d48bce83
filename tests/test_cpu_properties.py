"""Property tests (hypothesis) of the dedup / inverse mapping and of the CPU table's invariants.
The reference has no such tests; its dedup is SparsePullVarInfo (core/kernels/sparse_table_ops.cc:113-135)."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

import tensornet_b200 as tn
from tensornet_b200 import _build
from tensornet_b200.ops.sparse_table_cpu import CpuSparseTable

ids_strategy = st.lists(st.integers(min_value=-2**63, max_value=2**63 - 1), min_size=1, max_size=300)
small_ids = st.lists(st.integers(min_value=0, max_value=40), min_size=1, max_size=300)


@pytest.fixture(autouse=True)
def _cpu_runtime():
    tn.core.shutdown()
    tn.core.config.force_cpu = True
    tn.core.init()
    yield
    tn.core.shutdown()


@settings(max_examples=60, deadline=None)
@given(st.one_of(ids_strategy, small_ids), st.randoms(use_true_random=False))
def test_dedup_inverse_roundtrip(ids, rnd):
    ext = _build.cpu_ext()
    x = np.array(ids, dtype=np.int64)
    lab = np.array([rnd.choice([0.0, 1.0]) for _ in ids], dtype=np.float32)
    u, inv, show, click = ext.unique_first_occurrence(x, lab)
    u = np.asarray(u).view(np.uint64) if np.asarray(u).dtype != np.uint64 else np.asarray(u)
    inv = np.asarray(inv)
    assert len(set(u.tolist())) == len(u)                                   # uniques are unique
    assert inv.min() >= 0 and inv.max() == len(u) - 1                        # every unique is referenced
    canon = x.view(np.uint64)
    # reconstruct: every id maps back to its own sign (the all-ones sign is the table's empty marker and is remapped)
    same = u[inv] == canon
    assert np.all(same | (canon == np.uint64(2**64 - 1)))
    assert np.isclose(np.asarray(show).sum(), len(ids))
    assert np.isclose(np.asarray(click).sum(), lab.sum())
    # first-occurrence order: first index of each unique is increasing
    first_pos = [int(np.argmax(inv == k)) for k in range(len(u))]
    assert first_pos == sorted(first_pos)


@settings(max_examples=25, deadline=None)
@given(st.lists(small_ids, min_size=1, max_size=6), st.sampled_from(["adagrad", "adam", "ftrl"]))
def test_table_size_and_pull_stability(batches, kind):
    opt = {"adagrad": tn.core.AdaGrad(learning_rate=0.01), "adam": tn.core.Adam(learning_rate=0.01),
           "ftrl": tn.core.Ftrl(learning_rate=0.01)}[kind]
    t = CpuSparseTable(opt, 4)
    seen = set()
    for b in batches:
        s = np.unique(np.array(b, dtype=np.uint64))
        rows = t.native.pull(s)
        seen.update(s.tolist())
        assert t.native.size() == len(seen)                                  # one row per distinct sign, ever
        again = t.native.pull(s)
        assert np.array_equal(rows, again)                                   # pulling does not mutate
        g = np.zeros((len(s), 4), dtype=np.float32)
        t.native.push(s, g, np.ones(len(s), np.float32), np.zeros(len(s), np.float32))
        assert t.native.size() == len(seen)                                  # pushing never creates rows


@settings(max_examples=12, deadline=None)
@given(st.lists(st.integers(min_value=1, max_value=2**63 - 1), min_size=1, max_size=120, unique=True),
       st.integers(1, 5), st.integers(1, 5), st.sampled_from(["adagrad", "adam", "ftrl"]))
def test_resharding_keeps_every_row_and_routes_by_sign(tmp_path_factory, signs, w1, w2, kind):
    """world w1 -> w2 in binary mode: the same rows come back bit for bit, and every row sits in rank_(sign % w2)
    (what the reference needs an offline Spark job for, tensornet_tools/python/resize_sparse.py:35-54)."""
    import os
    from tensornet_b200 import tools
    from tensornet_b200.utils import checkpoint

    opt = {"adagrad": tn.core.AdaGrad(learning_rate=0.01), "adam": tn.core.Adam(learning_rate=0.01),
           "ftrl": tn.core.Ftrl(learning_rate=0.01)}[kind]
    name = {"adagrad": "AdaGrad", "adam": "Adam", "ftrl": "Ftrl"}[kind]
    t = CpuSparseTable(opt, 4, name="t")
    s = np.array(signs, dtype=np.uint64)
    t.native.pull(s)
    t.native.push(s, np.ones((len(s), 4), np.float32) * 0.5, np.ones(len(s), np.float32), np.zeros(len(s), np.float32))
    root = tmp_path_factory.mktemp("reshard")
    checkpoint.save_sparse_table(t, str(root / "cp"), "bin")
    src = os.path.join(str(root / "cp"), "sparse_table", "t")
    a = tools.resize_sparse(src, str(root / "a"), w1, "bin", name, 4)
    b = tools.resize_sparse(str(root / "a"), str(root / "b"), w2, "bin", name, 4)
    assert a == b == len(s)
    s0, r0, _, _ = tools.read_sparse_table(src, name, 4)
    s2, r2, _, _ = tools.read_sparse_table(str(root / "b"), name, 4)
    o0, o2 = np.argsort(s0), np.argsort(s2)
    assert np.array_equal(s0[o0], s2[o2]) and np.array_equal(r0[o0], r2[o2])
    assert sorted(os.listdir(root / "b")) == [f"rank_{r}" for r in range(w2)]
    ext = _build.cpu_ext()
    kind_id = {"adagrad": 0, "adam": 1, "ftrl": 2}[kind]
    for r in range(w2):
        sr, _ = ext.read_sparse_dir(os.path.join(str(root / "b"), f"rank_{r}"), kind_id, 4, False)
        assert all(int(x) % w2 == r for x in np.asarray(sr).tolist())

"""Stand-alone unique_assign against the CPU first-occurrence dedup."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_unique_assign_matches_cpu(tn_gpu, status_ok):
    from tensornet_b200 import _build
    from tensornet_b200.ops.unique import UniqueAssign

    dev = tn_gpu.core.runtime().device
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 5000, (40000,), generator=g, dtype=torch.int64) * 6364136223846793005 + 1442695040888963407
    labels = (torch.rand(40000, generator=g) < 0.3).float()
    ua = UniqueAssign(8192)
    for _ in range(2):      # the scratch must come back clean
        uniq, inv, show, click, count = ua(ids.to(dev), labels.to(dev))
        n = int(count.item())
        u_ref, inv_ref, show_ref, click_ref = _build.cpu_ext().unique_first_occurrence(ids.numpy(), labels.numpy())
        assert n == len(u_ref)
        u = uniq[:n].cpu().numpy().view(np.uint64)
        assert set(u.tolist()) == set(u_ref.tolist())
        assert np.array_equal(u[inv.cpu().numpy()], ids.numpy().view(np.uint64))
        pos = {int(s): i for i, s in enumerate(u_ref.tolist())}
        perm = np.array([pos[int(s)] for s in u.tolist()])
        assert np.array_equal(show[:n].cpu().numpy(), show_ref[perm])
        assert np.array_equal(click[:n].cpu().numpy(), click_ref[perm])
    assert int((ua.dd_keys != -1).sum()) == 0


def test_unique_assign_properties(tn_gpu, status_ok):
    """Hypothesis-driven: any id list (duplicates inside one warp, extreme bit patterns) dedups to a consistent mapping."""
    from hypothesis import given, settings, strategies as st
    from tensornet_b200.ops.unique import UniqueAssign

    dev = tn_gpu.core.runtime().device
    ua = UniqueAssign(512)
    # -1 (all ones) is the tables' empty marker and is folded onto another sign by design: keep it out of the identity checks
    wide = st.lists(st.integers(min_value=-2**63, max_value=2**63 - 2).filter(lambda v: v != -1), min_size=1, max_size=400)
    hot = st.lists(st.integers(min_value=0, max_value=12), min_size=1, max_size=400)

    @settings(max_examples=40, deadline=None)
    @given(st.one_of(wide, hot))
    def check(ids):
        x = torch.tensor(ids, dtype=torch.int64)
        uniq, inv, show, click, count = ua(x.to(dev), torch.ones(len(ids), device=dev))
        n = int(count.item())
        assert n == len(set(ids))
        u = uniq[:n].cpu()
        assert len(set(u.tolist())) == n
        assert torch.equal(u[inv.cpu().long()], x)
        assert float(show[:n].sum()) == len(ids) and float(click[:n].sum()) == len(ids)
        counts = {k: ids.count(k) for k in set(ids)}
        assert [counts[int(k)] for k in u.tolist()] == show[:n].cpu().int().tolist()

    check()
    assert int((ua.dd_keys != -1).sum()) == 0


def test_table_insert_lookup_properties(tn_gpu, status_ok):
    """Hash-table invariants: one row per distinct sign, lookups agree with inserts, absent signs report -1."""
    from hypothesis import given, settings, strategies as st
    from tensornet_b200.ops.sparse_table_gpu import GpuSparseTable

    t = GpuSparseTable(tn_gpu.core.AdaGrad(learning_rate=0.01), 4, rows=4096)
    dev = t.dev
    seen = {}

    @settings(max_examples=30, deadline=None)
    @given(st.lists(st.integers(min_value=-2**63, max_value=2**63 - 2).filter(lambda v: v != -1), min_size=1, max_size=64, unique=True))
    def check(ids):
        if len(seen) + len(ids) > 3000:
            return
        k = torch.tensor(ids, dtype=torch.int64, device=dev)
        idx = torch.empty(len(ids), dtype=torch.int32, device=dev)
        t.ext.table_insert_keys(t.table_dict(), k, idx, tn_gpu.core.runtime().status)
        got = idx.cpu().tolist()
        for s, r in zip(ids, got):
            assert r >= 0
            assert seen.setdefault(s, r) == r                      # stable row across repeated inserts
        assert t.n_rows == len(seen)
        assert t.lookup_rows(k).cpu().tolist() == got
        absent = torch.tensor([2**63 - 1], dtype=torch.int64, device=dev)
        if 2**63 - 1 not in seen:
            assert t.lookup_rows(absent).item() == -1

    check()
    assert len(set(seen.values())) == len(seen)                    # distinct signs never share a row

"""Fused sparse pull / push on one GPU against a dictionary-based restatement of the reference's
per-sign algorithms (core/ps/optimizer/{ada_grad,adam,ftrl}_kernel.cc)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(tn, opt, dim, use_cvm=False, rows=1 << 14, max_unique=4096):
    from tensornet_b200.ops.sparse_table_gpu import GpuSparseTable

    t = GpuSparseTable(opt, dim, use_cvm, rows=rows)
    return t, t.link(max_unique)


def _host_rows(t):
    keys, rows = t.dump()
    return {int(k): rows[i].copy() for i, k in enumerate(keys)}


@pytest.mark.parametrize("dim", [1, 8, 16, 64, 128])
def test_pull_dedup_and_init(tn_gpu, status_ok, dim):
    tn = tn_gpu
    opt = tn.core.AdaGrad(learning_rate=0.01, initial_g2sum=0.1, initial_scale=0.5)
    t, lk = _mk(tn, opt, dim)
    g = torch.Generator().manual_seed(dim)
    ids = torch.randint(0, 300, (2000,), generator=g, dtype=torch.int64) * 7919 + 11
    ids_d = ids.to(t.dev)
    inv = lk.pull(ids_d, training=True)
    torch.cuda.synchronize()
    tn.core.runtime().check_status()
    n_unique = len(set(ids.tolist()))
    assert lk.unique_counts()[0] == n_unique
    assert t.n_rows == n_unique
    inv_h = inv.cpu().long()
    assert int(inv_h.min()) >= 0
    # same id -> same virtual row, different ids -> different rows
    m = {}
    for i, v in zip(ids.tolist(), inv_h.tolist()):
        assert m.setdefault(i, v) == v
    assert len(set(m.values())) == n_unique
    # pulled rows equal the stored rows; stored rows have the documented initial state
    U = lk.U.cpu()
    rows = _host_rows(t)
    w_all = []
    for i, v in m.items():
        assert np.allclose(U[v, :dim].numpy(), rows[i][:dim])
        assert abs(rows[i][dim] - 0.1) < 1e-7            # g2sum
        assert rows[i][dim + 1] == 0 and rows[i][dim + 2] == 0
        w_all.append(rows[i][:dim])
    w_all = np.concatenate(w_all)
    assert abs(w_all.std() - 0.5 / math.sqrt(dim)) < 0.15 * 0.5 / math.sqrt(dim) + 0.02
    # show counts landed in the gradient record
    shows = lk.cnts.cpu()
    cnt = {}
    for i in ids.tolist():
        cnt[i] = cnt.get(i, 0) + 1
    for i, v in m.items():
        assert shows[v, 0] == cnt[i]
    # a second pull of the same ids finds the same rows (no growth) and the same values
    lk.cnts.zero_()
    inv2 = lk.pull(ids_d, training=False)
    torch.cuda.synchronize()
    assert t.n_rows == n_unique
    U2 = lk.U.cpu()
    assert torch.equal(U2[inv2.cpu().long()], U[inv_h])


def _apply_ref(kind, opt, row, g, show, click, dim):
    row = row.copy()
    if kind == "AdaGrad":
        row[dim + 1] += show
        row[dim + 2] += click
        row[dim] += float((g.astype(np.float64) ** 2).sum() / dim)
        row[:dim] -= opt.learning_rate * g / (opt.epsilon + math.sqrt(row[dim]))
    elif kind == "Adam":
        m, v = row[dim:2 * dim], row[2 * dim:3 * dim]
        m[:] = opt.beta1 * m + (1 - opt.beta1) * g
        v[:] = opt.beta2 * v + (1 - opt.beta2) * g * g
        row[:dim] -= opt.learning_rate * m / (opt.epsilon + np.sqrt(v))
    else:
        w, z, n = row[:dim], row[dim:2 * dim], row[2 * dim:3 * dim]
        g2 = g * g
        z += g - opt.learning_rate * (np.sqrt(n + g2) - np.sqrt(n)) * w
        n += g2
        neww = -1.0 / ((opt.beta + np.sqrt(n)) * opt.learning_rate + opt.lambda2) * np.where(z > 0, z - opt.lambda1, z + opt.lambda1)
        w[:] = np.where(np.abs(z) <= opt.lambda1, 0.0, neww)
    return row


@pytest.mark.parametrize("kind", ["AdaGrad", "Adam", "Ftrl"])
@pytest.mark.parametrize("dim", [8, 16, 64, 128])
def test_push_matches_reference_math(tn_gpu, status_ok, kind, dim):
    tn = tn_gpu
    opt = {"AdaGrad": tn.core.AdaGrad(learning_rate=0.05, initial_g2sum=0.1, initial_scale=0.3),
           "Adam": tn.core.Adam(learning_rate=0.01, initial_scale=0.3),
           "Ftrl": tn.core.Ftrl(learning_rate=0.05, initial_scale=0.3, lambda1=0.001)}[kind]
    t, lk = _mk(tn, opt, dim)
    g = torch.Generator().manual_seed(3)
    ids = (torch.randint(0, 500, (1500,), generator=g, dtype=torch.int64) * 104729 + 5).to(t.dev)
    labels = (torch.rand(1500, generator=g) < 0.3).float().to(t.dev)
    for step in range(3):
        inv = lk.pull(ids, labels=labels, label_mod=0, training=True)
        torch.cuda.synchronize()
        before = _host_rows(t)
        n_u = lk.unique_counts()[0]
        grad = torch.randn(n_u, dim, generator=g)
        lk.gU[:n_u, :dim] = grad.to(t.dev)
        gU = lk.gU.cpu().numpy().copy()
        cn = lk.cnts.cpu().numpy().copy()
        stage = lk.comm["stage_ids"].cpu().numpy().view(np.uint64)
        lk.push()
        torch.cuda.synchronize()
        tn.core.runtime().check_status()
        after = _host_rows(t)
        assert float(lk.gU.abs().sum()) == 0.0 and float(lk.cnts.abs().sum()) == 0.0     # re-zeroed for the next step
        for j in range(n_u):
            key = int(stage[j])
            exp = _apply_ref(kind, opt, before[key], gU[j, :dim], cn[j, 0], cn[j, 1], dim)
            got = after[key]
            nf = dim + 3 if kind == "AdaGrad" else 3 * dim
            assert np.allclose(got[:nf], exp[:nf], rtol=2e-5, atol=1e-6), (kind, step, j)


def test_cvm_columns_and_zero_init(tn_gpu, status_ok):
    tn = tn_gpu
    dim = 8
    opt = tn.core.AdaGrad(learning_rate=0.05, initial_g2sum=0.1)
    t, lk = _mk(tn, opt, dim, use_cvm=True)
    ids = torch.arange(1, 65, dtype=torch.int64).to(t.dev) * 1000003
    labels = torch.ones(64, device=t.dev)
    lk.pull(ids, labels=labels, training=True)
    lk.push()
    inv = lk.pull(ids, labels=labels, training=False)
    torch.cuda.synchronize()
    U = lk.U.cpu()[inv.cpu().long()]
    assert torch.allclose(U[:, dim], torch.ones(64))                        # show
    assert torch.allclose(U[:, dim + 1], torch.zeros(64), atol=1e-6)         # ln(2) - ln(2)
    # unseen signs in inference mode come back as zeros (and are inserted, like the reference)
    t.set_training(False)
    new = torch.arange(1, 9, dtype=torch.int64).to(t.dev) * 7 + 123456789
    inv = lk.pull(new, training=False)
    torch.cuda.synchronize()
    assert float(lk.U[inv.long()].abs().sum()) == 0.0
    assert t.n_rows == 72


def test_table_full_is_reported_not_fatal(tn_gpu):
    tn = tn_gpu
    opt = tn.core.Adam()
    t, lk = _mk(tn, opt, 8, rows=64, max_unique=1024)
    ids = torch.arange(1, 513, dtype=torch.int64).to(t.dev)
    lk.pull(ids, training=False)
    torch.cuda.synchronize()
    with pytest.raises(tn.core.DeviceError) as e:
        tn.core.runtime().check_status()
    assert e.value.code == 3
    assert t.n_rows == 64
    # the context is still usable, and after recover() so is the table: a batch that fits goes through
    assert float(torch.ones(4, device=t.dev).sum()) == 4.0
    tn.core.recover()
    t.clear()                                # the shard is full to the last key slot: start it over
    inv = lk.pull(ids[:32], training=False)
    torch.cuda.synchronize()
    tn.core.runtime().check_status()
    assert int(inv.min()) >= 0 and t.n_rows == 32


@pytest.mark.parametrize("kind,mode", [("adagrad", "txt"), ("adagrad", "bin"), ("adam", "bin"), ("ftrl", "txt")])
def test_streamed_export_matches_dump_and_applies_eviction(tn_gpu, status_ok, tmp_path, kind, mode):
    """A shard saved in small streamed pieces (device-side filter + grouping by block file) reads back as the rows
    of the plain dump minus those the save-time eviction rule drops."""
    from tensornet_b200 import _build
    from tensornet_b200.utils import checkpoint

    tn = tn_gpu
    opt = {"adagrad": tn.core.AdaGrad(learning_rate=0.01, show_threshold=1.5, no_show_days=10),
           "adam": tn.core.Adam(learning_rate=0.01), "ftrl": tn.core.Ftrl(learning_rate=0.01)}[kind]
    dim = 6
    t, lk = _mk(tn, opt, dim, rows=1 << 13, max_unique=8192)
    t.name = f"exp_{kind}_{mode}"
    g = torch.Generator().manual_seed(11)
    ids = (torch.randint(0, 3000, (6000,), generator=g, dtype=torch.int64) * 0x9E3779B97F4A7C15) .to(t.dev)
    lk.pull(ids, labels=torch.ones(6000, device=t.dev), training=True)
    lk.gU.normal_()
    lk.push()
    torch.cuda.synchronize()
    full = _host_rows(t)
    assert len(full) > 1500
    old = tn.core.config.checkpoint_chunk_rows
    tn.core.config.checkpoint_chunk_rows = 700          # several pieces
    try:
        n_written = checkpoint.save_sparse_table(t, str(tmp_path), mode)
    finally:
        tn.core.config.checkpoint_chunk_rows = old
    signs, rows = _build.cpu_ext().read_sparse_dir(str(tmp_path / "sparse_table" / t.name / "rank_0"), t.kind, dim, False)
    if kind == "adagrad":
        keep = {k for k, r in full.items() if not (r[dim + 1] < 1.5)}     # no_show_days is 0 everywhere: only the show rule bites
    else:        # Adam has no rule; Ftrl's show stays 0 (its update only counts delta_show), threshold 0 keeps all
        keep = set(full)
    assert n_written == len(keep) == len(signs)
    assert 0 < len(keep) and (kind != "adagrad" or len(keep) < len(full))
    assert set(int(s) for s in signs) == keep
    for s, r in zip(signs, rows):
        ref = full[int(s)]
        if mode == "bin":
            assert np.array_equal(r[:dim], ref[:dim])
        else:
            assert np.allclose(r[:dim], ref[:dim], rtol=1e-5, atol=1e-6)     # text keeps 6 significant digits


def test_staged_row_return_with_a_48k_tile_buffer(tn_gpu, status_ok):
    """Row width 12 floats (dim 8 + two CVM columns, padded) makes the staged return ask for exactly 48 KiB of dynamic
    shared memory; together with the kernel's static words that needs the large-shared-memory opt-in."""
    tn = tn_gpu
    old = tn.core.config.staged_row_return
    tn.core.config.staged_row_return = 1
    try:
        t, lk = _mk(tn, tn.core.AdaGrad(learning_rate=0.01, initial_scale=0.2), 8, use_cvm=True, rows=1 << 12, max_unique=1024)
        assert lk.ustride == 12
        ids = torch.arange(1, 601, dtype=torch.int64, device=t.dev) * 7919
        inv = lk.pull(ids, training=True)
        torch.cuda.synchronize()
        rows = _host_rows(t)
        U = lk.U.cpu()
        for i in (0, 17, 599):
            assert np.allclose(U[int(inv[i]), :8].numpy(), rows[int(ids[i])][:8])
        lk.push()
    finally:
        tn.core.config.staged_row_return = old


def test_shard_grows_and_compacts_on_the_device(tn_gpu, status_ok):
    """A shard that starts with 256 rows takes 3 000 signs through two enlargements (longer slab, re-filled key array)
    and ends up with the same row for every sign as a shard that was large from the start; dropping half of the rows
    on the device keeps the others findable and frees the slab for new signs."""
    tn = tn_gpu
    opt = tn.core.AdaGrad(learning_rate=0.05, initial_g2sum=0.1, initial_scale=0.1)
    small, lks = _mk(tn, opt, 8, rows=256, max_unique=512)
    big, lkb = _mk(tn, opt, 8, rows=1 << 13, max_unique=512)
    g = torch.Generator().manual_seed(11)
    for step in range(12):
        ids = (torch.randperm(100000, generator=g)[:250] + 1).to(small.dev)
        if small.n_rows + 250 > small.row_cap:
            small.grow()
        for t, lk in ((small, lks), (big, lkb)):
            inv = lk.pull(ids, training=True)
            lk.gU[inv.long().unique(), :8] = 0.25
            lk.push()
    torch.cuda.synchronize()
    assert small.grown >= 2 and small.n_rows == big.n_rows
    ks, rs = small.dump()
    kb, rb = big.dump()
    os_, ob = np.argsort(ks), np.argsort(kb)
    assert np.array_equal(ks[os_], kb[ob]) and np.array_equal(rs[os_], rb[ob])
    # compaction: keep the even row indices
    n = small.n_rows
    keep = torch.zeros(n, dtype=torch.bool, device=small.dev)
    keep[::2] = True
    kept_keys = torch.from_numpy(ks.view(np.int64)).to(small.dev)[::2]
    dropped_keys = torch.from_numpy(ks.view(np.int64)).to(small.dev)[1::2]
    kept_rows = torch.from_numpy(rs).to(small.dev)[::2]
    dropped = small.compact(keep)
    assert dropped == n - kept_keys.numel() and small.n_rows == kept_keys.numel()
    idx = small.lookup_rows(kept_keys).long()
    assert int(idx.min()) >= 0 and int(idx.max()) < small.n_rows
    assert torch.equal(small.rows[idx, : kept_rows.shape[1]], kept_rows)
    assert int(small.lookup_rows(dropped_keys).max()) == -1
    inv = lks.pull(dropped_keys[:200].contiguous(), training=False)      # the freed part of the slab takes new signs
    torch.cuda.synchronize()
    assert small.n_rows == kept_keys.numel() + 200


@pytest.mark.parametrize("dim", [8, 64])
def test_pull_front_run_ahead_matches_the_one_kernel_pull(tn_gpu, status_ok, dim):
    """The front of a pull (dedup, id dispatch, inverse map) run ahead as plain kernels, followed by the probe-only
    pull, against the pull that does everything in one kernel: same rows per id, same show / click counts, same
    table after the pushes; a front that is not followed by its pull is discarded cleanly."""
    tn = tn_gpu
    opt = tn.core.AdaGrad(learning_rate=0.05, initial_g2sum=0.1, initial_scale=0.3)
    g = torch.Generator().manual_seed(11)
    batches = [(torch.randint(0, 700, (3000,), generator=g, dtype=torch.int64) * 104729 + 5) for _ in range(4)]
    labels = [(torch.rand(3000, generator=g) < 0.3).float() for _ in range(4)]
    tables = []
    for ahead in (False, True):
        t, lk = _mk(tn, opt, dim)
        dev = t.dev
        ids_d = [b.to(dev) for b in batches]
        lab_d = [l.to(dev) for l in labels]
        seen = []
        for k in range(4):
            inv = lk.pull(ids_d[k], labels=lab_d[k], label_mod=0, training=True)
            if ahead and k > 0:
                assert inv.data_ptr() == lk._front_inverse[(ids_d[k].data_ptr(), 3000)].data_ptr()
            if ahead and k + 1 < 4:
                lk.prefetch(ids_d[k + 1])                 # same stream here; the model forks it onto a side stream
            torch.cuda.synchronize()
            tn.core.runtime().check_status()
            inv_l = inv.long()
            assert int(inv_l.min()) >= 0
            seen.append((lk.U[inv_l, :dim].cpu(), lk.cnts[inv_l].cpu()))
            # a gradient that depends only on the sign, so both runs push the same thing whatever the virtual order
            gid = (ids_d[k] % 97).float().unsqueeze(1) * 0.01 + torch.arange(dim, device=dev).float() * 1e-3
            lk.gU[:, :dim].index_put_((inv_l,), gid, accumulate=False)
            lk.push()
        torch.cuda.synchronize()
        tn.core.runtime().check_status()
        tables.append((_host_rows(t), seen))
        if ahead:
            # a front whose pull never comes: the next pull is for other ids and must still be right
            lk.prefetch(ids_d[0])
            inv = lk.pull(ids_d[2], labels=lab_d[2], label_mod=0, training=True)
            torch.cuda.synchronize()
            tn.core.runtime().check_status()
            rows = _host_rows(t)
            U = lk.U[inv.long(), :dim].cpu().numpy()
            for i, s in enumerate(batches[2].tolist()[:200]):
                assert np.allclose(U[i], rows[s][:dim])
            lk.push()
    (rows_a, seen_a), (rows_b, seen_b) = tables
    for (Ua, ca), (Ub, cb) in zip(seen_a, seen_b):
        assert torch.allclose(Ua, Ub, rtol=1e-6, atol=1e-7)
        assert torch.equal(ca, cb)
    assert rows_a.keys() == rows_b.keys()
    for k in rows_a:
        assert np.allclose(rows_a[k], rows_b[k], rtol=1e-5, atol=1e-6)

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

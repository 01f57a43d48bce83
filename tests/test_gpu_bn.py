"""Device-resident batch-norm table and layer against the host table (numpy, float64) and plain PyTorch."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _host_table(pctr=False, max_count=100000, moment=0.99, C=7):
    from tensornet_b200.ops.bn_table import BnTable

    return BnTable("ref", C, False, moment, max_count, pctr)


@pytest.mark.parametrize("max_count", [100000, 300])
def test_bn_table_matches_host_table(tn_gpu, status_ok, max_count):
    from tensornet_b200.ops.bn_table import GpuBnTable

    C = 37
    dev = tn_gpu.core.runtime().device
    g = GpuBnTable("t", C, False, 0.9, max_count)
    h = _host_table(max_count=max_count, moment=0.9, C=C)
    gen = torch.Generator().manual_seed(3)
    for step in range(8):
        B = [128, 257, 64, 1000][step % 4]
        x = torch.randn(B, C, generator=gen) * (1 + step) + step
        g.push_batch(x.to(dev))
        xd = x.double()
        h.append(xd.sum(0).numpy(), (xd * xd).sum(0).numpy(), np.full(C, float(B)))
        mean_g, var_g = g.get_moments()
        mean_h, var_h = h.get_moments()
        assert np.allclose(mean_g, mean_h, rtol=1e-6, atol=1e-6)
        assert np.allclose(var_g, var_h, rtol=1e-5, atol=1e-5)
    s, q, c = g.totals()
    hs, hq, hc = h.totals()
    assert np.allclose(s, hs, rtol=1e-12) and np.allclose(q, hq, rtol=1e-12) and np.array_equal(c, hc)
    assert float(g.batch.abs().sum()) == 0.0          # per-step scratch comes back clean
    inc = g.take_increments()
    hinc = h.take_increments()
    for a, b in zip(inc, hinc):
        assert np.allclose(a, b, rtol=1e-12)


def test_bn_layer_forward_backward_and_checkpoint(tn_gpu, status_ok, tmp_path):
    tn = tn_gpu
    dev = tn.core.runtime().device
    C, B = 45, 512
    bn = tn.layers.TNBatchNormalization(C, name="bn_gpu_test")
    assert bn._on_device
    bn.train()
    torch.manual_seed(0)
    x = (torch.randn(B, C, device=dev) * 3 + 1).requires_grad_(True)
    with torch.no_grad():
        bn.gamma.copy_(torch.rand(C, device=dev) + 0.5)
        bn.beta.copy_(torch.randn(C, device=dev))
    y = bn(x)
    mean, var = x.detach().mean(0), x.detach().var(0, unbiased=False)
    assert torch.allclose(bn.moving_mean, mean, atol=1e-5) and torch.allclose(bn.moving_variance, var, rtol=1e-4, atol=1e-4)
    ref = (x.detach() - mean) * torch.rsqrt(var + bn.epsilon) * bn.gamma.detach() + bn.beta.detach()
    assert torch.allclose(y, ref, rtol=1e-4, atol=1e-4)
    w = torch.randn(B, C, device=dev)
    (y * w).sum().backward()
    rs = torch.rsqrt(var + bn.epsilon)
    assert torch.allclose(x.grad, w * bn.gamma.detach() * rs, rtol=1e-4, atol=1e-4)
    assert torch.allclose(bn.beta.grad, w.sum(0), rtol=1e-4, atol=1e-3)
    assert torch.allclose(bn.gamma.grad, (w * (x.detach() - mean) * rs).sum(0), rtol=1e-4, atol=1e-2)
    bn.save_bn_table(str(tmp_path))
    bn2 = tn.layers.TNBatchNormalization(C, name="bn_gpu_test2")
    bn2.table.handle = bn.table.handle
    bn2.bn_table_handle = bn.bn_table_handle
    tn.core.load_bn_table(bn.bn_table_handle, str(tmp_path))
    assert torch.allclose(bn.moving_mean, mean, atol=1e-5)
    bn.eval()
    y2 = bn(x.detach())
    assert torch.allclose(y2, ref, rtol=1e-4, atol=1e-4)


def test_pctr_bn_accumulates_deviation_from_current_mean(tn_gpu, status_ok):
    tn = tn_gpu
    dev = tn.core.runtime().device
    C = 9
    bn = tn.layers.PCTRDNNBatchNormalization(C, name="pctr_gpu_test")
    bn.train()
    h = _host_table(pctr=True, C=C)
    gen = torch.Generator().manual_seed(5)
    for _ in range(3):
        x = torch.randn(200, C, generator=gen) + 2
        mean_before = torch.from_numpy(h.get_moments()[0])
        y = bn(x.to(dev))
        xd = x.double()
        h.append(xd.sum(0).numpy(), ((xd - mean_before.double()) ** 2).sum(0).numpy(), np.full(C, 200.0))
    mg, vg = bn.table.get_moments()
    mh, vh = h.get_moments()
    assert np.allclose(mg, mh, rtol=1e-6, atol=1e-6) and np.allclose(vg, vh, rtol=1e-5)

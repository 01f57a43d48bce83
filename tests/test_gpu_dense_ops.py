"""Memory-bound kernels and the fused dense optimizer against plain PyTorch fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_fm_forward_backward(tn_gpu, status_ok):
    from tensornet_b200.ops import functional as F

    dev = tn_gpu.core.runtime().device
    B, Fd, D = 300, 26, 16
    e = torch.randn(B, Fd * D, device=dev, requires_grad=True)
    out = F.fm(e, Fd, D)
    out.sum().backward()
    e2 = e.detach().clone().cpu().requires_grad_(True)
    ref = F.fm(e2, Fd, D)
    ref.sum().backward()
    assert torch.allclose(out.cpu(), ref, rtol=1e-4, atol=1e-4)
    assert torch.allclose(e.grad.cpu(), e2.grad, rtol=1e-4, atol=1e-4)


def test_concat_cast_roundtrip(tn_gpu, status_ok):
    from tensornet_b200.ops import functional as F

    dev = tn_gpu.core.runtime().device
    B = 257
    a = torch.randn(B, 416, device=dev, requires_grad=True)
    b = torch.randn(B, 13, device=dev)
    x = F.concat_cast([a, b], ones=True)
    assert x.shape == (B, 432) and x.dtype == torch.bfloat16
    assert torch.equal(x[:, :416].float(), a.detach().bfloat16().float())
    assert torch.equal(x[:, 416:429].float(), b.bfloat16().float())
    assert torch.all(x[:, 429] == 1) and torch.all(x[:, 430:] == 0)
    g = torch.randn(B, 432, device=dev).bfloat16()
    x.backward(g)
    assert torch.equal(a.grad, g[:, :416].float())


def test_head_and_bce(tn_gpu, status_ok):
    from tensornet_b200.ops import functional as F

    dev = tn_gpu.core.runtime().device
    B, K = 1000, 427
    z = torch.zeros(B, 432, dtype=torch.bfloat16, device=dev)
    z[:, :K] = torch.randn(B, K, device=dev).bfloat16()
    z[:, K] = 1.0
    z.requires_grad_(True)
    w = torch.nn.Parameter(torch.randn(K + 1, device=dev) * 0.05)
    y = (torch.rand(B, device=dev) < 0.25).float()
    sums = torch.zeros(4, device=dev)
    logit = F.head(z, w)
    loss, pred = F.bce_with_logits(logit, y, sums)
    loss.backward()
    zr = z.detach().float().clone().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    lr = zr[:, :K + 1] @ wr
    lossr = torch.nn.functional.binary_cross_entropy_with_logits(lr, y)
    lossr.backward()
    assert abs(float(loss) - float(lossr)) < 1e-4
    assert torch.allclose(pred.view(-1), torch.sigmoid(lr), atol=1e-5)
    assert torch.allclose(w.grad, wr.grad, rtol=1e-3, atol=1e-5)
    assert torch.allclose(z.grad.float()[:, :K + 1], zr.grad[:, :K + 1], rtol=2e-2, atol=1e-6)
    s = sums.tolist()
    assert abs(s[1] - float(y.sum())) < 1e-3 and s[3] == B


def test_mlp_forward_backward(tn_gpu, status_ok):
    """Chain of tcgen05 layers (forward, dgrad with ReLU mask, split-K wgrad) vs autograd on the CPU restatement."""
    from tensornet_b200.layers import MLP
    from tensornet_b200.ops import functional as F

    dev = tn_gpu.core.runtime().device
    torch.manual_seed(0)
    B, K = 2048, 429
    mlp = MLP(K, [400, 400, 96])
    with torch.no_grad():
        for w in mlp.weights:
            w[:, -1] = 0  # padding stays zero
    mlp_ref = MLP(K, [400, 400, 96])
    mlp_ref.load_state_dict(mlp.state_dict())
    mlp.to(dev)
    x = torch.randn(B, K)
    xin = x.to(dev).requires_grad_(True)
    out = mlp(F.concat_cast([xin], ones=True))
    gout = torch.randn(B, out.shape[1]).bfloat16()
    out.backward(gout.to(dev))
    # reference: the CPU restatement of the same chain (bf16-rounded activations, fp32 accumulate), so both
    # sides see the same ReLU masks; autograd differentiates it
    xr = x.clone().requires_grad_(True)
    outr = mlp_ref(F.concat_cast([xr], ones=True))
    outr.backward(gout)
    dims = [K, 400, 400]
    assert float((out.float().cpu()[:, :96] - outr.float()[:, :96]).abs().max()) < 0.1
    # a handful of units sit so close to zero that the two summation orders disagree on the ReLU mask;
    # compare in the Frobenius norm, which such isolated flips barely move
    rel = lambda a, b: float((a - b).norm() / (b.norm() + 1e-6))
    for l, (w, wr) in enumerate(zip(mlp.weights, mlp_ref.weights)):
        assert rel(w.grad.cpu()[:, :dims[l] + 1], wr.grad[:, :dims[l] + 1]) < 1e-2, l
    assert rel(xin.grad.cpu(), xr.grad) < 1e-2


@pytest.mark.parametrize("kind", ["Adam", "AdaGrad"])
def test_dense_table_step(tn_gpu, status_ok, kind):
    tn = tn_gpu
    from tensornet_b200.ops.dense_table import DenseTable

    dev = tn.core.runtime().device
    opt = tn.core.Adam(learning_rate=0.01) if kind == "Adam" else tn.core.AdaGrad(learning_rate=0.01, initial_g2sum=0.1,
                                                                                   grad_decay_rate=0.9, mom_decay_rate=0.9)
    ps = [torch.nn.Parameter(torch.randn(37, 5, device=dev)), torch.nn.Parameter(torch.randn(1001, device=dev))]
    ref = [p.detach().clone().cpu() for p in ps]
    t = DenseTable(opt)
    t.init([("b", ps[0]), ("a", ps[1])])
    st = [[torch.zeros_like(r) for r in ref] for _ in range(3)]
    if kind == "AdaGrad":
        for s in st[1]:
            s.fill_(0.1)
    b1p = b2p = 1.0
    for step in range(4):
        gs = [torch.randn_like(r) for r in ref]
        for p, g in zip(ps, gs):
            p.grad.copy_(g.to(dev))
        t.step()
        torch.cuda.synchronize()
        for i, (w, g) in enumerate(zip(ref, gs)):
            if kind == "Adam":
                if i == 0:
                    b1p *= 0.9; b2p *= 0.999
                alpha = 0.01 * (1 - b2p) ** 0.5 / (1 - b1p)
                st[0][i] += (g - st[0][i]) * (1 - 0.9)
                st[1][i] += (g * g - st[1][i]) * (1 - 0.999)
                w -= st[0][i] * alpha / (st[1][i].sqrt() + 1e-8)
            else:
                st[0][i] = 0.9 * st[0][i] + 1
                st[1][i] = 0.9 * st[1][i] + g * g
                st[2][i] += (g - st[2][i]) * (1 - 0.9)
                w -= 0.01 * st[2][i] / (st[1][i].sqrt() / st[0][i].sqrt() + 1e-8)
        for p, w in zip(ps, ref):
            assert torch.allclose(p.detach().cpu(), w, rtol=1e-4, atol=1e-5)
            assert float(p.grad.abs().sum()) == 0.0
            assert torch.equal(p._tn_bf16.float(), p.detach().bfloat16().float())

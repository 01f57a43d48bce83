"""tcgen05 GEMM family against a plain fp32 PyTorch reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ext():
    from tensornet_b200 import _build

    return _build.cuda_ext()


def _rel_err(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6))


@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (256, 80, 200), (1000, 400, 430), (8192, 400, 430)])
def test_forward_kk_relu_ones(tn_gpu, status_ok, M, N, K):
    """C = relu(A . B^T), ones column at N, zero pad after it (MLP forward layer)."""
    dev = tn_gpu.core.runtime().device
    Kp, Np = (K + 7) // 8 * 8, (N + 1 + 7) // 8 * 8
    g = torch.Generator(device="cpu").manual_seed(M * 31 + N)
    A = torch.zeros(M, Kp).bfloat16()
    A[:, :K] = torch.randn(M, K, generator=g).bfloat16()
    B = torch.zeros(N, Kp).bfloat16()
    B[:, :K] = (torch.randn(N, K, generator=g) * 0.1).bfloat16()
    A, B = A.to(dev), B.to(dev)
    C = torch.full((M, Np), 7.0, dtype=torch.bfloat16, device=dev)
    _ext().gemm(A, B, C, M, N, K, Kp, Kp, Np, False, False, False, True, None, None, None, None, 0, N, Np, 1, 0,
                tn_gpu.core.runtime().status)
    ref = torch.relu(A.float()[:, :K] @ B.float()[:, :K].t())
    assert _rel_err(C[:, :N], ref) < 2e-2
    assert torch.all(C[:, N] == 1.0)
    assert torch.all(C[:, N + 1:] == 0.0)


@pytest.mark.parametrize("M,N,K", [(256, 128, 64), (512, 432, 400), (8192, 432, 400)])
def test_dgrad_k_mn_mask(tn_gpu, status_ok, M, N, K):
    """dX[M,N] = (dY[M,K] . W[K,N]) masked by X > 0   (A contraction-major, B output-major)."""
    dev = tn_gpu.core.runtime().device
    Kp = (K + 7) // 8 * 8
    g = torch.Generator(device="cpu").manual_seed(N * 17 + K)
    dY = torch.zeros(M, Kp + 8).bfloat16()
    dY[:, :K] = torch.randn(M, K, generator=g).bfloat16()
    dY[:, K:] = 3.0    # columns beyond K must be ignored
    W = (torch.randn(K, N, generator=g) * 0.1).bfloat16()
    X = torch.randn(M, N, generator=g).bfloat16()
    dY, W, X = dY.to(dev), W.to(dev), X.to(dev)
    dX = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    _ext().gemm(dY, W, dX, M, N, K, Kp + 8, N, N, False, True, False, False, None, X, None, None, N, -1, N, 1, 0,
                tn_gpu.core.runtime().status)
    ref = (dY.float()[:, :K] @ W.float()) * (X.float() > 0)
    assert _rel_err(dX, ref) < 2e-2


@pytest.mark.parametrize("Bt,N,K,split", [(256, 128, 64, 1), (1024, 400, 430, 2), (8192, 400, 430, 8)])
def test_wgrad_mn_mn_accumulate(tn_gpu, status_ok, Bt, N, K, split):
    """dW[N,K] += dY[Bt,N]^T . X[Bt,K]   (both operands output-major, split-K, fp32 accumulate)."""
    dev = tn_gpu.core.runtime().device
    Np, Kp = (N + 1 + 7) // 8 * 8, (K + 7) // 8 * 8
    g = torch.Generator(device="cpu").manual_seed(Bt + N)
    dY = torch.zeros(Bt, Np).bfloat16()
    dY[:, :N] = torch.randn(Bt, N, generator=g).bfloat16()
    dY[:, N:] = 5.0
    X = torch.zeros(Bt, Kp).bfloat16()
    X[:, :K] = torch.randn(Bt, K, generator=g).bfloat16()
    dY, X = dY.to(dev), X.to(dev)
    dW = torch.ones(N, Kp, dtype=torch.float32, device=dev)
    _ext().gemm(dY, X, dW, N, K, Bt, Np, Kp, Kp, True, True, True, False, None, None, None, None, 0, -1, K, split, 0,
                tn_gpu.core.runtime().status)
    ref = 1.0 + dY.float()[:, :N].t() @ X.float()[:, :K]
    err = float((dW[:, :K] - ref).abs().max() / ref.abs().max())
    assert err < 1e-2
    assert torch.all(dW[:, K:] == 1.0)


def test_hadamard_epilogue(tn_gpu, status_ok):
    """DCN-v2 cross layer: C = x0 * (A . B^T + bias) + xl."""
    dev = tn_gpu.core.runtime().device
    M, N, K = 512, 256, 256
    g = torch.Generator(device="cpu").manual_seed(5)
    A = torch.randn(M, K, generator=g).bfloat16().to(dev)
    B = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(dev)
    bias = torch.randn(N, generator=g).to(dev)
    x0 = torch.randn(M, N, generator=g).bfloat16().to(dev)
    xl = torch.randn(M, N, generator=g).bfloat16().to(dev)
    C = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    _ext().gemm(A, B, C, M, N, K, K, K, N, False, False, False, False, bias, None, x0, xl, N, -1, N, 1, 0,
                tn_gpu.core.runtime().status)
    ref = x0.float() * (A.float() @ B.float().t() + bias) + xl.float()
    assert _rel_err(C, ref) < 2e-2


def test_weight_gate_passes_and_times_out(tn_gpu):
    """The gated GEMM waits for per-owner "chunk written" flags before loading its weights: with the flags at the
    expected epoch it computes as usual; with a flag nothing sets, its bounded wait runs out, the kernel gives up
    cleanly, the status words name the missing owner and the context stays usable."""
    M, N, K = 256, 64, 128
    g = torch.Generator().manual_seed(5)
    A, W = torch.randn(M, K, generator=g).bfloat16(), (torch.randn(N, K, generator=g) * 0.1).bfloat16()
    dev = tn_gpu.core.runtime().device
    C = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
    epoch = torch.tensor([3], dtype=torch.int64, device=dev)
    flags = torch.tensor([3 << 32, 4 << 32, 0, 0], dtype=torch.int64, device=dev)
    rt = tn_gpu.core.runtime()
    _ext().gemm(A.to(dev), W.to(dev), C, M, N, K, K, K, N, False, False, False, False, None, None, None, None, 0, -1, N, 1, 0,
                tn_gpu.core.runtime().status, gate_flags=flags, gate_epoch=epoch, gate_world=2, gate_wait_ns=10_000_000)
    torch.cuda.synchronize()
    rt.check_status()
    ref = A.float() @ W.float().t()
    assert (C.float().cpu() - ref).abs().max() < 2e-2 * ref.abs().max()
    # owner 2's flag never reaches epoch 3
    C2 = torch.zeros_like(C)
    _ext().gemm(A.to(dev), W.to(dev), C2, M, N, K, K, K, N, False, False, False, False, None, None, None, None, 0, -1, N, 1, 0,
                tn_gpu.core.runtime().status, gate_flags=flags, gate_epoch=epoch, gate_world=3, gate_wait_ns=2_000_000)
    torch.cuda.synchronize()
    with pytest.raises(tn_gpu.core.DeviceError) as e:
        rt.check_status()
    assert e.value.code == 5 and e.value.phase == 70 and e.value.aux == 2
    assert float(torch.ones(4, device=dev).sum()) == 4.0
    tn_gpu.core.recover()
    rt.check_status()      # recover() cleared the words


@pytest.mark.parametrize("layout", ["kk", "k_mn", "mn_mn"])
def test_two_accumulator_tile(tn_gpu, status_ok, layout):
    """256-row tiles (two 128-row TMEM accumulators sharing each B tile) against an fp32 reference, with a ragged
    last row tile and a ragged last column tile."""
    dev = tn_gpu.core.runtime().device
    M, N, K = 640 + 40, 512 + 64, 1024
    g = torch.Generator().manual_seed(12)
    st = tn_gpu.core.runtime().status
    if layout == "kk":
        A = torch.randn(M, K, generator=g).bfloat16().to(dev)
        B = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(dev)
        C = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        _ext().gemm(A, B, C, M, N, K, K, K, N, False, False, False, False, None, None, None, None, 0, -1, N, 1, 256, st, m_halves=2)
        ref = A.float() @ B.float().t()
    elif layout == "k_mn":
        A = torch.randn(M, K, generator=g).bfloat16().to(dev)
        B = (torch.randn(K, N, generator=g) * 0.05).bfloat16().to(dev)          # [K, N]: N contiguous
        C = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        _ext().gemm(A, B, C, M, N, K, K, N, N, False, True, False, False, None, None, None, None, 0, -1, N, 1, 256, st, m_halves=2)
        ref = A.float() @ B.float()
    else:
        A = torch.randn(K, M + 0, generator=g).bfloat16().to(dev)              # [K, M]: M contiguous
        B = (torch.randn(K, N, generator=g) * 0.05).bfloat16().to(dev)
        C = torch.zeros(M, N, dtype=torch.float32, device=dev)
        _ext().gemm(A, B, C, M, N, K, M, N, N, True, True, True, False, None, None, None, None, 0, -1, N, 1, 256, st, m_halves=2)
        ref = A.float().t() @ B.float()
    assert _rel_err(C, ref) < 2e-2


@pytest.mark.parametrize("layout", ["kk", "k_mn", "mn_mn"])
@pytest.mark.parametrize("BN", [512, 256, 128])
def test_pair_kernel_walks_several_tiles_per_cluster(tn_gpu, status_ok, layout, BN):
    """The persistent kernel on pairs of CTAs (one tcgen05.mma over two SMs, double-buffered accumulator) against an
    fp32 reference: more tiles than clusters, so every cluster walks two or three tiles through both accumulator
    stages and around the operand ring; ragged last row tile, ragged last column tile, contraction not a multiple
    of the stage depth."""
    dev = tn_gpu.core.runtime().device
    M, N, K = 4096 + 40, {512: 5120, 256: 2560, 128: 1280}[BN] + 64, 1000
    g = torch.Generator().manual_seed(21)
    st = tn_gpu.core.runtime().status
    if layout == "kk":
        A = torch.randn(M, K, generator=g).bfloat16().to(dev)
        B = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(dev)
        C = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        _ext().gemm(A, B, C, M, N, K, K, K, N, False, False, False, False, None, None, None, None, 0, -1, N, 1, BN, st, m_halves=4)
        ref = A.float() @ B.float().t()
    elif layout == "k_mn":
        A = torch.randn(M, K, generator=g).bfloat16().to(dev)
        B = (torch.randn(K, N, generator=g) * 0.05).bfloat16().to(dev)          # [K, N]: N contiguous
        C = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        _ext().gemm(A, B, C, M, N, K, K, N, N, False, True, False, False, None, None, None, None, 0, -1, N, 1, BN, st, m_halves=4)
        ref = A.float() @ B.float()
    else:
        A = torch.randn(K, M, generator=g).bfloat16().to(dev)                  # [K, M]: M contiguous
        B = (torch.randn(K, N, generator=g) * 0.05).bfloat16().to(dev)
        C = torch.ones(M, N, dtype=torch.float32, device=dev)
        _ext().gemm(A, B, C, M, N, K, M, N, N, True, True, True, False, None, None, None, None, 0, -1, N, 1, BN, st, m_halves=4)
        ref = A.float().t() @ B.float() + 1.0
    torch.cuda.synchronize()
    tn_gpu.core.runtime().check_status()
    assert _rel_err(C, ref) < 2e-2


@pytest.mark.parametrize("BN", [512, 256])
def test_pair_kernel_hadamard_epilogue(tn_gpu, status_ok, BN):
    """The DCN-v2 cross-layer epilogue (bias, pre-activation kept, x0 * u + xl) through the pair kernel."""
    dev = tn_gpu.core.runtime().device
    M, N, K = 1024 + 24, 768 + 16, 448
    g = torch.Generator(device="cpu").manual_seed(10)
    A = torch.randn(M, K, generator=g).bfloat16().to(dev)
    B = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(dev)
    bias = torch.randn(N, generator=g).to(dev)
    x0 = torch.randn(M, N, generator=g).bfloat16().to(dev)
    xl = torch.randn(M, N, generator=g).bfloat16().to(dev)
    st = tn_gpu.core.runtime().status
    C = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    U = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=dev)
    _ext().gemm(A, B, C, M, N, K, K, K, N, False, False, False, False, bias, None, x0, xl, N, -1, N, 1, BN, st, m_halves=4, aux_out=U)
    u_ref = A.float() @ B.float().t() + bias
    assert _rel_err(U, u_ref) < 2e-2
    assert _rel_err(C, x0.float() * u_ref + xl.float()) < 2e-2


def test_hadamard_epilogue_keeps_pre_activation_and_residual_mode(tn_gpu, status_ok):
    """aux_out receives u = A . B^T + bias next to y = x0 * u + xl; without x0 the epilogue is a plain residual add."""
    dev = tn_gpu.core.runtime().device
    M, N, K = 384, 272, 320
    g = torch.Generator(device="cpu").manual_seed(9)
    A = torch.randn(M, K, generator=g).bfloat16().to(dev)
    B = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(dev)
    bias = torch.randn(N, generator=g).to(dev)
    x0 = torch.randn(M, N, generator=g).bfloat16().to(dev)
    xl = torch.randn(M, N, generator=g).bfloat16().to(dev)
    st = tn_gpu.core.runtime().status
    C = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    U = torch.full((M, N), 7.0, dtype=torch.bfloat16, device=dev)
    _ext().gemm(A, B, C, M, N, K, K, K, N, False, False, False, False, bias, None, x0, xl, N, -1, N, 1, 0, st, aux_out=U)
    u_ref = A.float() @ B.float().t() + bias
    assert _rel_err(U, u_ref) < 2e-2
    assert _rel_err(C, x0.float() * u_ref + xl.float()) < 2e-2
    R = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    _ext().gemm(A, B, R, M, N, K, K, K, N, False, False, False, False, None, None, None, xl, N, -1, N, 1, 0, st)
    assert _rel_err(R, A.float() @ B.float().t() + xl.float()) < 2e-2


def test_cross_v2_backward_elementwise_kernels(tn_gpu, status_ok):
    dev = tn_gpu.core.runtime().device
    n = 256 * 136
    g = torch.Generator(device="cpu").manual_seed(2)
    gg, u, x0 = (torch.randn(n, generator=g).bfloat16().to(dev) for _ in range(3))
    acc = torch.randn(n, generator=g).to(dev)
    gx0 = acc.clone()
    du = torch.empty(n, dtype=torch.bfloat16, device=dev)
    _ext().cross_v2_bwd_elem(gg, u, x0, gx0, du, False)
    assert torch.allclose(gx0, acc + gg.float() * u.float(), rtol=1e-5, atol=1e-5)
    assert torch.equal(du, (gg.float() * x0.float()).bfloat16())
    first = torch.full((n,), 3.0, device=dev)
    _ext().cross_v2_bwd_elem(gg, u, x0, first, du, True)
    assert torch.allclose(first, gg.float() * u.float(), rtol=1e-5, atol=1e-5)
    out = torch.empty(n, dtype=torch.bfloat16, device=dev)
    _ext().cross_v2_bwd_final(gx0, gg, out)
    assert torch.equal(out, (gx0 + gg.float()).bfloat16())


@pytest.mark.parametrize("K", [300, 6672, 13000])
def test_head_forward_backward_wide(tn_gpu, status_ok, K):
    """Dense(1) head against fp32 matmul; 13000 columns need more than 48 KiB of shared memory for the weight copy."""
    from tensornet_b200.ops import functional as F
    dev = torch.device("cuda", 0)
    B, ld = 512, (K + 8 + 7) // 8 * 8
    g = torch.Generator(device="cpu").manual_seed(K)
    z = (torch.randn(B, ld, generator=g) * 0.5).to(dev).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(K, generator=g) * 0.05).to(dev)
    w.grad = None
    y = F.head(z, w)
    ref = z.detach().float()[:, :K] @ w
    assert torch.allclose(y.view(-1), ref, rtol=2e-3, atol=2e-3)
    gy = torch.randn(B, 1, generator=g).to(dev)
    y.backward(gy)
    torch.cuda.synchronize()
    dz_ref = gy * w.view(1, -1)
    assert torch.allclose(z.grad.float()[:, :K], dz_ref, rtol=2e-2, atol=2e-3)
    gw = F._grad_buffer(w)
    gw_ref = z.detach().float()[:, :K].t() @ gy.view(-1)
    assert torch.allclose(gw[:K], gw_ref, rtol=2e-2, atol=5e-2)

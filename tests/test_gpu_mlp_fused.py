"""The one-kernel MLP tower (csrc/mlp_fused.cu) against a plain fp32 PyTorch restatement of the same layers, forward and
backward, for a tiny batch, the benchmark batch and a batch whose last 128-row stripe is ragged."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(x32, weights, dims):
    """fp32 math on the bf16-rounded operands, bf16 rounding of every activation (what the kernels store)."""
    h = x32
    acts = []
    for l, w in enumerate(weights):
        K = dims[l]
        wq = w.detach().float().cpu().to(torch.bfloat16).float()
        y = torch.relu(h[:, :K + 1] @ wq[:, :K + 1].t())
        y = y.to(torch.bfloat16).float()
        h = torch.cat([y, torch.ones(y.shape[0], 1)], dim=1)
        acts.append(y)
    return acts


@pytest.mark.parametrize("B", [100, 8192, 8192 + 37])
@pytest.mark.parametrize("in_dim,hidden", [(429, (400, 400, 400)), (84, (64, 32)), (300, (256, 128, 64, 16))])
def test_fused_tower_matches_fp32_reference(tn_gpu, status_ok, B, in_dim, hidden):
    tn = tn_gpu
    from tensornet_b200.layers import MLP
    from tensornet_b200.ops import functional as F

    dev = tn.core.runtime().device
    torch.manual_seed(B + in_dim)
    mlp = MLP(in_dim, hidden).to(dev)
    with torch.no_grad():
        for l, w in enumerate(mlp.weights):
            K = ([in_dim] + list(hidden))[l]
            w[:, K].uniform_(-0.2, 0.2)            # non-zero biases
    feats = torch.randn(B, in_dim)
    x = F.concat_cast([feats.to(dev)], ones=True).requires_grad_(True)
    dims = [in_dim] + list(hidden)[:-1]

    def run(fused):
        tn.core.config.fused_mlp = fused
        F._chain_ok.clear()
        for w in mlp.weights:
            if getattr(w, "grad", None) is not None:
                w.grad = None
            F._grad_buffer(w).zero_()
        xx = x.detach().clone().requires_grad_(True)
        y = mlp(xx)
        gy = torch.zeros_like(y)
        g = torch.Generator(device="cpu").manual_seed(5)
        gy[:, : hidden[-1]] = (torch.randn(B, hidden[-1], generator=g) * (y[:, : hidden[-1]].float().cpu() > 0)).to(dev).to(torch.bfloat16)
        y.backward(gy)
        torch.cuda.synchronize()
        return y.detach().float().cpu(), xx.grad.float().cpu(), [F._grad_buffer(w).detach().float().cpu().clone() for w in mlp.weights]

    try:
        y_f, gx_f, gw_f = run(True)
        supported = F._chain_ok and all(F._chain_ok.values())
        y_u, gx_u, gw_u = run(False)
    finally:
        tn.core.config.fused_mlp = False
        F._chain_ok.clear()
    assert supported, F._chain_ok
    # forward against the fp32 restatement
    ref = _reference(x.detach().float().cpu(), list(mlp.weights), dims)[-1]
    N = hidden[-1]
    scale = ref.abs().max().clamp_min(1e-3)
    assert (y_f[:, :N] - ref).abs().max() <= 2e-2 * scale
    assert torch.equal(y_f[:, N], torch.ones(B)) and float(y_f[:, N + 1:].abs().sum()) == 0.0
    # the one-kernel path and the layer-by-layer path agree (same operands, same rounding points)
    assert (y_f - y_u).abs().max() <= 1e-2 * scale
    gscale = gx_u.abs().max().clamp_min(1e-6)
    assert (gx_f[:, :in_dim] - gx_u[:, :in_dim]).abs().max() <= 2e-2 * gscale
    for a, b in zip(gw_f, gw_u):
        assert (a - b).abs().max() <= 2e-2 * b.abs().max().clamp_min(1e-6)
    # backward against fp32 math.  The ReLU masks are taken from the kernels' own activations (sub-towers of the same
    # weights give them bit for bit): a pre-activation within rounding distance of zero may fall on either side, and
    # one flipped mask entry moves a weight gradient by a whole term.
    N = hidden[-1]
    acts = [x.detach().float().cpu()]
    for l in range(1, len(hidden)):
        acts.append(F.mlp(x.detach(), list(mlp.weights)[:l], in_dim).float().cpu())
    acts.append(y_f)
    g = torch.Generator(device="cpu").manual_seed(5)
    gl = (torch.randn(B, N, generator=g) * (y_f[:, :N] > 0)).to(torch.bfloat16).float()
    all_dims = [in_dim] + list(hidden)
    for l in range(len(hidden) - 1, -1, -1):
        K = all_dims[l]
        wq = mlp.weights[l].detach().float().cpu().to(torch.bfloat16).float()
        gw_ref = gl.t() @ acts[l][:, :K + 1]
        assert (gw_f[l][:, :K + 1] - gw_ref).abs().max() <= 2e-2 * gw_ref.abs().max().clamp_min(1e-6), l
        gl = gl @ wq[:, :K]
        if l > 0:
            gl = (gl * (acts[l][:, :K] > 0)).to(torch.bfloat16).float()
    assert (gx_f[:, :in_dim] - gl).abs().max() <= 2e-2 * gl.abs().max().clamp_min(1e-6)

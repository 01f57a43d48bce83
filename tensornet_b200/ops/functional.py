"""Differentiable front-ends of the dense-tower kernels.

On a CUDA tensor each function runs the hand-written sm_100a kernels through a
``torch.autograd.Function``; on a CPU tensor it runs the same arithmetic in plain PyTorch
(the oracle path).  Layout conventions shared by the GPU kernels:

* GEMM operands are bf16 with the row length padded to a multiple of 8 elements
  (16 bytes, the TMA stride rule).  Column ``K`` of an activation matrix holds the constant
  1.0, so a layer's bias is simply column ``K`` of its ``[N, K_pad]`` weight matrix and the
  bias gradient falls out of the weight-gradient GEMM.
* Weight gradients are accumulated straight into ``param.grad`` (fp32).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import _build
from ..core.runtime import runtime


def pad8(n: int) -> int:
    return (int(n) + 7) // 8 * 8


def _ext():
    return _build.cuda_ext()


def _status():
    return runtime().status


def _bf16_of(p: torch.Tensor) -> torch.Tensor:
    """bf16 shadow of a parameter (kept current by the dense optimizer) or a fresh cast."""
    sh = getattr(p, "_tn_bf16", None)
    if sh is not None:
        return sh
    return p.detach().to(torch.bfloat16)


_SIDE_STREAMS = {}


def _side_stream(device) -> "torch.cuda.Stream":
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    s = _SIDE_STREAMS.get(key)
    if s is None:
        s = torch.cuda.Stream(device=device)
        _SIDE_STREAMS[key] = s
    return s


def _grad_buffer(p: torch.Tensor) -> torch.Tensor:
    if p.grad is None:
        p.grad = torch.zeros_like(p)
    return p.grad


# =========================================================================================
# concat + cast to the padded bf16 operand
# =========================================================================================
class _ConcatCast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ones: bool, widths, *pieces):
        B = pieces[0].shape[0]
        widths = [int(p.shape[1]) if w is None else int(w) for p, w in zip(pieces, widths)]
        K = sum(widths)
        ld = pad8(K + (1 if ones else 0))
        out = torch.empty((B, ld), dtype=torch.bfloat16, device=pieces[0].device)
        ps = [p if p.stride(-1) == 1 else p.contiguous() for p in pieces]
        _ext().concat_cast(list(ps), widths, [int(p.stride(0)) for p in ps], out, B, ld, K if ones else -1)
        ctx.meta = (B, widths, ld, [p.dtype for p in pieces], [p.requires_grad for p in pieces], [int(p.shape[1]) for p in pieces])
        return out

    @staticmethod
    def backward(ctx, g):
        B, widths, ld, dtypes, needs, full = ctx.meta
        g = g.contiguous()
        outs: List[Optional[torch.Tensor]] = []
        for w, dt, need, fw in zip(widths, dtypes, needs, full):
            if not need:
                outs.append(None)
            elif fw == w:
                outs.append(torch.empty((B, w), dtype=dt, device=g.device))
            else:       # piece wider than the columns used: the unused columns get zero gradient
                outs.append(torch.zeros((B, fw), dtype=dt, device=g.device))
        _ext().split_cast(outs, widths, list(full), g, B, ld, -1)
        return (None, None, *outs)


def concat_cast(pieces: Sequence[torch.Tensor], ones: bool = True, widths: Optional[Sequence[Optional[int]]] = None) -> torch.Tensor:
    """``[B, sum(widths) (+1)]`` bf16, zero padded to a multiple of 8 columns; with ``ones`` the
    column right after the data is the constant 1 that carries the next layer's bias.
    ``widths[i]`` (optional) uses only the first columns of piece i (e.g. to drop its padding)."""
    pieces = [p if p.dim() == 2 else p.reshape(p.shape[0], -1) for p in pieces]
    widths = list(widths) if widths is not None else [None] * len(pieces)
    if pieces[0].is_cuda:
        return _ConcatCast.apply(ones, widths, *pieces)
    B = pieces[0].shape[0]
    cols = [p.float() if w is None else p.float()[:, :w] for p, w in zip(pieces, widths)]
    K = sum(int(c.shape[1]) for c in cols)
    if ones:
        cols.append(torch.ones(B, 1))
    ld = pad8(K + (1 if ones else 0))
    if ld > K + (1 if ones else 0):
        cols.append(torch.zeros(B, ld - K - (1 if ones else 0)))
    return torch.cat(cols, dim=1).to(torch.bfloat16)


# =========================================================================================
# MLP tower: chain of (bf16 GEMM + bias + ReLU) layers on the tcgen05 kernel
# =========================================================================================
_chain_ok: dict = {}


def _chain_supported(backward: bool, x, in_cols, bws, n_rows, k_cols, outs, relu, n_valid, masks) -> bool:
    """Does this tower fit the one-kernel path (``csrc/mlp_fused.cu``)?  Asked once per shape."""
    from ..core.config import config

    if not config.fused_mlp:
        return False
    key = (backward, int(x.shape[0]), in_cols, tuple(n_rows), tuple(k_cols), tuple(int(o.stride(0)) for o in outs))
    ok = _chain_ok.get(key)
    if ok is None:
        why = _ext().mlp_chain(backward, x, in_cols, bws, n_rows, k_cols, outs, relu, n_valid, masks, _status(), probe_only=True)
        ok = _chain_ok[key] = (why == "")
    return ok


class _MLP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dims, relu_last, premasked, gate, *weights):
        # x: bf16 [B, Kp0] (ones column at dims[0]);  weights[l]: fp32 [N_l, pad8(K_l + 1)]
        # gate: None or (flags, epoch, world, wait_ns): the first GEMM waits until every owner's chunk of the
        # dense weight array has landed on this GPU (the dense step then ends without a closing barrier)
        ext, st = _ext(), _status()
        B = x.shape[0]
        L = len(weights)
        bws = [_bf16_of(w) for w in weights]
        n_rows = [int(w.shape[0]) for w in weights]
        k_cols = [dims[l] + 1 for l in range(L)]
        outs = [torch.empty((B, pad8(n + 1)), dtype=torch.bfloat16, device=x.device) for n in n_rows]
        relu = [1 if (relu_last or l < L - 1) else 0 for l in range(L)]
        if L <= 4 and x.stride(1) == 1 and _chain_supported(False, x, int(x.shape[1]), bws, n_rows, k_cols, outs, relu, [], []):
            # the whole tower in one kernel: activations stay in shared memory between the layers
            g = {} if gate is None else dict(gate_flags=gate[0], gate_epoch=gate[1], gate_world=gate[2], gate_wait_ns=gate[3])
            ext.mlp_chain(False, x, int(x.shape[1]), bws, n_rows, k_cols, outs, relu, [], [], st, **g)
            acts = [x] + outs
        else:
            acts = [x]
            h = x
            for l, w in enumerate(weights):
                N, Kp = n_rows[l], int(w.shape[1])
                K = dims[l]
                Np = pad8(N + 1)
                y = outs[l]
                if l == 0 and gate is not None:
                    ext.gemm(h, bws[l], y, B, N, K + 1, int(h.stride(0)), Kp, Np, False, False, False, bool(relu[l]), None, None, None,
                             None, 0, N, Np, 1, 0, st, gate_flags=gate[0], gate_epoch=gate[1], gate_world=gate[2], gate_wait_ns=gate[3])
                else:
                    ext.gemm(h, bws[l], y, B, N, K + 1, int(h.stride(0)), Kp, Np, False, False, False, bool(relu[l]), None, None, None,
                             None, 0, N, Np, 1, 0, st)
                acts.append(y)
                h = y
        ctx.save_for_backward(*acts)
        ctx.weights = weights
        ctx.dims = dims
        ctx.relu_last = relu_last
        ctx.premasked = premasked
        return acts[-1]

    @staticmethod
    def backward(ctx, gy):
        ext, st = _ext(), _status()
        acts = ctx.saved_tensors
        weights = ctx.weights
        dims = ctx.dims
        L = len(weights)
        B = gy.shape[0]
        g = gy.contiguous()
        if ctx.relu_last and not ctx.premasked:
            g = g.clone()
            ext.relu_mask(g, acts[L])
        # The weight gradients are off the critical path (only the optimizer needs them): they run on a side
        # stream next to the input-gradient chain and are joined before this function returns.
        main = torch.cuda.current_stream()
        side = _side_stream(g.device)
        need_x = bool(ctx.needs_input_grad[0])
        lo = 0 if need_x else 1                       # lowest layer whose input gradient is wanted
        grads = [None] * L                            # grads[l]: gradient w.r.t. the output of layer l
        grads[L - 1] = g
        gx = None

        def wgrad(l):
            w = weights[l]
            if not w.requires_grad:
                return
            h = acts[l]
            ext.gemm(grads[l], h, _grad_buffer(w), int(w.shape[0]), dims[l] + 1, B, int(grads[l].stride(0)), int(h.stride(0)),
                     int(w.shape[1]), True, True, True, False, None, None, None, None, 0, -1, dims[l] + 1, 0, 0, st)

        chain = list(range(L - 1, lo - 1, -1))        # layers the input-gradient chain walks through
        fused = False
        if chain and len(chain) <= 4:
            bws = [_bf16_of(weights[l]) for l in chain]
            n_rows = [int(weights[l].shape[0]) for l in chain]
            k_cols = [min(int(weights[l].shape[1]), int(acts[l].stride(0))) for l in chain]
            outs = [torch.empty((B, int(acts[l].stride(0))), dtype=torch.bfloat16, device=g.device) for l in chain]
            n_valid = [dims[l] if l > 0 else k_cols[i] for i, l in enumerate(chain)]
            masks = [acts[l] if l > 0 else None for l in chain]
            fused = g.stride(1) == 1 and _chain_supported(True, g, int(g.shape[1]), bws, n_rows, k_cols, outs, [], n_valid, masks)
        if fused:
            # weight gradient of the top layer needs nothing from the chain: it starts beside it
            ev = torch.cuda.Event()
            ev.record(main)
            side.wait_event(ev)
            with torch.cuda.stream(side):
                wgrad(L - 1)
            ext.mlp_chain(True, g, int(g.shape[1]), bws, n_rows, k_cols, outs, [], n_valid, masks, st)
            for i, l in enumerate(chain):
                if l > 0:
                    grads[l - 1] = outs[i]
                else:
                    gx = outs[i]
            ev2 = torch.cuda.Event()
            ev2.record(main)
            side.wait_event(ev2)
            with torch.cuda.stream(side):
                for l in range(L - 2, -1, -1):
                    wgrad(l)
        else:
            for l in range(L - 1, -1, -1):
                w = weights[l]
                N, Kp = int(w.shape[0]), int(w.shape[1])
                h = acts[l]
                ldh = int(h.stride(0))
                # weight gradient (incl. the bias column): dW[N, Kp] += g[:, :N]^T . h   (contraction over the batch)
                if w.requires_grad:
                    ev = torch.cuda.Event()
                    ev.record(main)
                    side.wait_event(ev)
                    with torch.cuda.stream(side):
                        wgrad(l)
                # input gradient: gh[B, ldh] = g[:, :N] . W   masked by the ReLU of the layer below
                if l >= lo:
                    gh = torch.empty((B, ldh), dtype=torch.bfloat16, device=g.device)
                    mask = h if l > 0 else None
                    ext.gemm(grads[l], _bf16_of(w), gh, B, min(Kp, ldh), N, int(grads[l].stride(0)), Kp, ldh, False, True, False, False,
                             None, mask, None, None, ldh, -1, ldh, 1, 0, st)
                    if l > 0:
                        grads[l - 1] = gh
                    else:
                        gx = gh
        main.wait_stream(side)
        return (gx if need_x else None, None, None, None, None, *([None] * L))


def mlp(x: torch.Tensor, weights: Sequence[torch.Tensor], in_dim: int, relu_last: bool = True,
        grad_premasked: bool = False, gate=None) -> torch.Tensor:
    """Run ``x`` (bf16, ones column at ``in_dim``) through the layers ``weights``.
    Returns bf16 ``[B, pad8(N_last + 1)]`` whose column ``N_last`` is again the constant 1.
    ``grad_premasked``: the consumer hands back a gradient that is already zero where the last ReLU was
    inactive (the fused DeepFM head does), so the backward skips its own masking pass."""
    dims = [in_dim] + [int(w.shape[0]) for w in weights[:-1]]
    if x.is_cuda:
        return _MLP.apply(x, dims, relu_last, grad_premasked, gate, *weights)
    h = x.float()
    L = len(weights)
    for l, w in enumerate(weights):
        K, N = dims[l], int(w.shape[0])
        wq = w.to(torch.bfloat16).float()
        y = h[:, :K + 1] @ wq[:, :K + 1].t()
        if relu_last or l < L - 1:
            y = torch.relu(y)
        Np = pad8(N + 1)
        y = torch.cat([y, torch.ones(y.shape[0], 1), torch.zeros(y.shape[0], Np - N - 1)], dim=1)
        h = y.to(torch.bfloat16).float()
    return h.to(torch.bfloat16)


# =========================================================================================
# FM second-order term
# =========================================================================================
class _FM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, e, F, D):
        e = e.contiguous()
        B = e.shape[0]
        out = torch.empty(B, dtype=torch.float32, device=e.device)
        _ext().fm_fwd(e, F * D, B, F, D, out)
        ctx.save_for_backward(e)
        ctx.fd = (F, D)
        return out.view(B, 1)

    @staticmethod
    def backward(ctx, g):
        (e,) = ctx.saved_tensors
        F, D = ctx.fd
        B = e.shape[0]
        ge = torch.empty_like(e)
        _ext().fm_bwd(e, F * D, B, F, D, g.contiguous().view(-1), ge, F * D, False)
        return ge, None, None


def fm(e: torch.Tensor, fields: int, dim: int) -> torch.Tensor:
    """``0.5 * sum_d((sum_f e)^2 - sum_f e^2)`` of ``e [B, fields*dim]`` -> ``[B, 1]``."""
    if e.is_cuda:
        return _FM.apply(e.reshape(e.shape[0], fields * dim), fields, dim)
    x = e.reshape(e.shape[0], fields, dim)
    s = x.sum(dim=1)
    return 0.5 * (s * s - (x * x).sum(dim=1)).sum(dim=1, keepdim=True)


# =========================================================================================
# Dense(1) head on a padded bf16 operand
# =========================================================================================
class _Head(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z, w):
        B, ld = z.shape[0], int(z.stride(0))
        K1 = int(w.numel())
        y = torch.empty(B, dtype=torch.float32, device=z.device)
        _ext().gemv_fwd(z, ld, B, K1, w, y)
        ctx.save_for_backward(z)
        ctx.w = w
        return y.view(B, 1)

    @staticmethod
    def backward(ctx, gy):
        (z,) = ctx.saved_tensors
        w = ctx.w
        B, ld = z.shape[0], int(z.stride(0))
        dz = torch.empty_like(z)
        gw = _grad_buffer(w)
        _ext().gemv_bwd(z, ld, B, int(w.numel()), w, gy.contiguous().view(-1), dz, gw, 0)
        return dz, None


def head(z: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``z[:, :len(w)] @ w`` -> ``[B, 1]`` fp32; ``w``'s last element multiplies z's ones column (bias)."""
    if z.is_cuda:
        return _Head.apply(z, w)
    return (z.float()[:, : w.numel()] @ w).view(-1, 1)


# =========================================================================================
# sigmoid binary cross-entropy (mean) with fused dlogit and CTR / PCTR sums
# =========================================================================================
class _BCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logit, label, sums):
        B = logit.numel()
        lg = logit.contiguous().view(-1)
        dl = torch.empty_like(lg)
        pred = torch.empty_like(lg)
        s = sums if sums is not None else torch.zeros(4, dtype=torch.float32, device=lg.device)
        loss_before = s[0].clone()      # the kernel adds this step's mean loss to s[0]
        _ext().bce(lg, label.contiguous().view(-1).float(), pred, dl, 1.0 / B, s)
        ctx.save_for_backward(dl)
        ctx.shape = logit.shape
        ctx.mark_non_differentiable(pred)
        return s[0] - loss_before, pred.view(logit.shape)

    @staticmethod
    def backward(ctx, gloss, _gpred):
        (dl,) = ctx.saved_tensors
        return (dl * gloss).view(ctx.shape), None, None


def bce_with_logits(logit: torch.Tensor, label: torch.Tensor, sums: Optional[torch.Tensor] = None):
    """Mean sigmoid cross-entropy.  Returns ``(loss, prediction)``.  ``sums`` (fp32[4] or fp32[4 + 2 * bins]), when
    given, accumulates ``[loss, sum(label), sum(prediction), count]`` for the CTR / PCTR / COPC metrics and, in the
    longer form, two histograms of the prediction (32-bit counts stored in the same buffer: positives, then
    negatives) for a streaming AUC."""
    if logit.is_cuda:
        return _BCE.apply(logit, label, sums)
    lg = logit.view(-1)
    y = label.view(-1).float()
    loss = torch.nn.functional.binary_cross_entropy_with_logits(lg, y)
    pred = torch.sigmoid(lg).detach()
    if sums is not None:
        with torch.no_grad():
            sums[:4] += torch.stack([loss.detach(), y.sum(), pred.sum(), torch.tensor(float(y.numel()))])
            if sums.numel() > 4:
                bins = (sums.numel() - 4) // 2
                hist = sums[4:].view(torch.int32)
                idx = (pred * bins).long().clamp_(max=bins - 1) + torch.where(y > 0.5, 0, bins)
                hist += torch.bincount(idx, minlength=2 * bins).to(torch.int32)
    return loss, pred.view(logit.shape)


# =========================================================================================
# DCN-v1 cross layer  y = x0 * (xl . w) + b + xl     (examples/common/layers.py:53-59)
# =========================================================================================
class _CrossV1(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x0, xl, w, b):
        x0, xl = x0.contiguous(), xl.contiguous()
        y = torch.empty_like(x0)
        dot = torch.empty(x0.shape[0], dtype=torch.float32, device=x0.device)
        _ext().cross_v1_fwd(x0, xl, w.contiguous().view(-1), b.contiguous(), y, dot)
        ctx.save_for_backward(x0, xl, w, dot)
        return y

    @staticmethod
    def backward(ctx, gy):
        x0, xl, w, dot = ctx.saved_tensors
        gy = gy.contiguous()
        gx0, gxl = torch.empty_like(x0), torch.empty_like(xl)
        gw = torch.zeros(w.numel(), dtype=torch.float32, device=w.device)
        gb = torch.zeros(w.numel(), dtype=torch.float32, device=w.device)
        _ext().cross_v1_bwd(x0, xl, w.contiguous().view(-1), dot, gy, gx0, gxl, gw, gb)
        return gx0, gxl, gw.view(w.shape), gb


def cross_v1(x0, xl, w, b):
    if x0.is_cuda:
        return _CrossV1.apply(x0, xl, w, b)
    return x0 * (xl @ w.view(-1, 1)) + b + xl


# =========================================================================================
# DCN-v2 cross network  x_{l+1} = x0 * (W_l x_l + b_l) + x_l   on padded bf16 operands
# =========================================================================================
class _CrossV2(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x0, dim, *weights):
        ext, st = _ext(), _status()
        B, Dp = x0.shape[0], int(x0.stride(0))
        xs, us = [x0], []
        xl = x0
        keep_u = any(w.requires_grad for w in weights) or x0.requires_grad
        for w in weights:
            y = torch.empty((B, Dp), dtype=torch.bfloat16, device=x0.device)
            # u = W x_l + b is needed again by the backward pass; the epilogue writes it next to y (105 MB per layer at
            # batch 8192 x width 6416) instead of the backward pass recomputing it with a fourth GEMM per layer
            u = torch.empty((B, Dp), dtype=torch.bfloat16, device=x0.device) if keep_u else None
            # tcgen05 GEMM with the Hadamard-residual epilogue; the bias rides on x_l's ones column
            ext.gemm(xl, _bf16_of(w), y, B, dim, dim + 1, Dp, int(w.shape[1]), Dp, False, False, False, False, None, None, x0, xl,
                     Dp, dim, Dp, 1, 0, st, aux_out=u)
            xs.append(y)
            us.append(u)
            xl = y
        ctx.save_for_backward(*xs, *[u for u in us if u is not None])
        ctx.weights, ctx.dim, ctx.keep_u = weights, dim, keep_u
        return xl

    @staticmethod
    def backward(ctx, g):
        ext, st = _ext(), _status()
        L = len(ctx.weights)
        saved = ctx.saved_tensors
        xs, us = saved[:L + 1], saved[L + 1:]
        weights, dim = ctx.weights, ctx.dim
        x0 = xs[0]
        B, Dp = x0.shape[0], int(x0.stride(0))
        g = g.contiguous()
        gx0 = torch.empty((B, Dp), dtype=torch.float32, device=g.device)
        du = torch.empty((B, Dp), dtype=torch.bfloat16, device=g.device)
        for l in range(L - 1, -1, -1):
            w, xl = weights[l], xs[l]
            wb = _bf16_of(w)
            Kp = int(w.shape[1])
            # gx0 (+)= g * u ; du = g * x0   in one pass
            ext.cross_v2_bwd_elem(g, us[l], x0, gx0, du, l == L - 1)
            if w.requires_grad:
                ext.gemm(du, xl, _grad_buffer(w), dim, dim + 1, B, Dp, Dp, Kp, True, True, True, False, None, None, None, None, 0, -1,
                         dim + 1, 0, 0, st)
            # g_{l} = g_{l+1} + du . W   (the residual add rides in the GEMM epilogue)
            gn = torch.empty((B, Dp), dtype=torch.bfloat16, device=g.device)
            ext.gemm(du, wb, gn, B, min(Kp, Dp), dim, Dp, Kp, Dp, False, True, False, False, None, None, None, g, Dp, -1, Dp, 1, 0, st)
            g = gn
        out = torch.empty((B, Dp), dtype=torch.bfloat16, device=g.device)
        ext.cross_v2_bwd_final(gx0, g, out)
        return (out, None, *([None] * L))


def cross_v2(x0: torch.Tensor, weights: Sequence[torch.Tensor], dim: int) -> torch.Tensor:
    """``x0``: bf16 ``[B, pad8(dim+1)]`` with the ones column at ``dim``; ``weights[l]``: fp32 ``[dim, pad8(dim+1)]``
    (bias in column ``dim``).  Returns the last cross layer's output in the same padded layout."""
    if x0.is_cuda:
        return _CrossV2.apply(x0, dim, *weights)
    x0f = x0.float()
    xl = x0f
    for w in weights:
        wq = w.to(torch.bfloat16).float()
        u = xl[:, : dim + 1] @ wq[:, : dim + 1].t()
        y = x0f[:, :dim] * u + xl[:, :dim]
        y = torch.cat([y, torch.ones(y.shape[0], 1), torch.zeros(y.shape[0], x0.shape[1] - dim - 1)], dim=1)
        xl = y.to(torch.bfloat16).float()
    return xl.to(torch.bfloat16)


# =========================================================================================
# DeepFM fusions (GPU only): embedding gather + FM + operand build; head + loss + head backward
# =========================================================================================
class _DeepFMInput(torch.autograd.Function):
    @staticmethod
    def forward(ctx, anchor, link, ids, B, S, dense, training, emb_dim, lin_col):
        inverse = link.pull(ids, None, 0, training)
        D = emb_dim
        Dd = 0 if dense is None else int(dense.shape[1])
        ld = pad8(S * D + Dd + 1)
        x0 = torch.empty((B, ld), dtype=torch.bfloat16, device=ids.device)
        fm = torch.empty(B, dtype=torch.float32, device=ids.device)
        lin = torch.empty((B, S), dtype=torch.float32, device=ids.device) if lin_col >= 0 else None
        _ext().deepfm_input_fwd(link.U, link.ustride, inverse, B, S, D, dense, x0, fm, lin_col, lin)
        ctx.link, ctx.inverse, ctx.meta = link, inverse, (B, S, D, lin_col)
        if lin is None:
            lin = torch.empty(0, device=ids.device)
            ctx.mark_non_differentiable(lin)
        return x0, fm.view(B, 1), lin

    @staticmethod
    def backward(ctx, gx0, gfm, glin):
        link = ctx.link
        B, S, D, lin_col = ctx.meta
        if gfm is None:
            gfm = torch.zeros(B, dtype=torch.float32, device=gx0.device)
        dl = glin.contiguous() if (lin_col >= 0 and glin is not None) else None
        _ext().deepfm_input_bwd(link.U, link.ustride, ctx.inverse, B, S, D, gx0.contiguous(), gfm.contiguous().view(-1), link.gU,
                                link.gstride, lin_col, dl)
        return (None,) * 9


def deepfm_input(anchor, link, ids, B, S, dense=None, training=True, emb_dim=None, lin_col=-1):
    """Pull the S single-hot slots of ``ids`` ([S*B], slot after slot) and build in one pass the padded bf16 operand
    ``[emb | dense | 1 | 0]`` of the first MLP layer plus the second-order FM term ``[B, 1]``.  When the table rows carry
    the slot's linear weight in column ``lin_col`` (``emb_dim`` < row width), also returns those weights ``[B, S]``."""
    if dense is not None:
        dense = dense.float().contiguous()
    x0, fm, lin = _DeepFMInput.apply(anchor, link, ids, B, S, dense, training, emb_dim or link.dim, lin_col)
    return x0, fm, (lin if lin_col >= 0 else None)


_HEAD_SCRATCH = {}


def _head_scratch(dev) -> torch.Tensor:
    """Persistent scratch per device that the head kernel leaves at zero: partial loss, finished-block count and
    sixteen partial copies of the head's weight gradient."""
    key = (dev.type, dev.index)
    if key not in _HEAD_SCRATCH:
        _HEAD_SCRATCH[key] = torch.zeros(4 + 16 * 576, dtype=torch.float32, device=dev)
    return _HEAD_SCRATCH[key]


class _DeepFMHeadLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, lin, fm, w, label, sums, n_hidden):
        B = h.shape[0]
        dev = h.device
        dh = torch.empty_like(h)
        dl = torch.empty_like(lin) if lin is not None else None
        dfm = torch.empty(B, dtype=torch.float32, device=dev)
        loss = torch.empty((), dtype=torch.float32, device=dev)     # written (not accumulated) by the last block
        pred = torch.empty(B, dtype=torch.float32, device=dev)
        _ext().deepfm_head_loss(h, n_hidden, None if lin is None else lin.contiguous(), fm.contiguous().view(-1), w,
                                label.contiguous().view(-1).float(), dh, dl, dfm, _grad_buffer(w), sums, pred, loss,
                                _head_scratch(dev))
        ctx.save_for_backward(dh, dl if dl is not None else dfm, dfm)
        ctx.has_lin = lin is not None
        ctx.mark_non_differentiable(pred)
        return loss, pred

    @staticmethod
    def backward(ctx, gloss, _gpred):
        # The head's gradients were produced by the forward pass for d(loss) = 1, which is what
        # ``loss.backward()`` supplies; a caller that scales the loss must use the unfused head.
        dh, dl, dfm = ctx.saved_tensors
        return dh, (dl if ctx.has_lin else None), dfm.view(-1, 1), None, None, None, None


def deepfm_head_loss(h, lin, fm, w, label, sums, n_hidden):
    """``Dense(1)`` over ``[h[:, :n_hidden] | lin | fm | 1]`` + mean sigmoid cross-entropy, with the whole backward of
    the head computed in the same kernel.  The weight gradient is accumulated into ``w.grad`` right away and the
    returned loss must be back-propagated with a unit gradient.  Returns ``(loss, prediction)``."""
    return _DeepFMHeadLoss.apply(h, lin, fm, w, label, sums, n_hidden)

"""Pull + pool as one differentiable op, and the matching gradient path.

Forward  : ids -> (fused dedup / all-to-all pull into the per-batch unique-row matrix ``U``)
           -> bag pooling into ``[B, S * width]``.
Backward : scatter-add of the pooled gradient into the unique-gradient matrix ``gU`` that the
           fused push kernel later ships to the owning GPUs.

This is the reference's "virtual sparse feature" trick (README.md:26-34): the network only
ever sees a small ``[unique ids of the batch, dim]`` matrix, never the full vocabulary.
The virtual index of an id is its row in ``U``.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _build

COMBINERS = {"sum": 0, "mean": 1, "sqrtn": 2}


def _bag_ids(offsets: Optional[torch.Tensor], nbags: int, nnz: int, device) -> torch.Tensor:
    if offsets is None:
        return torch.arange(nbags, device=device)
    lens = (offsets[1:] - offsets[:-1]).long()
    return torch.repeat_interleave(torch.arange(nbags, device=device), lens, output_size=nnz)


def _bag_scale(offsets, nbags, combiner, device):
    if offsets is None or combiner == 0:
        return None
    lens = (offsets[1:] - offsets[:-1]).float().clamp(min=1.0)
    return 1.0 / lens if combiner == 1 else lens.rsqrt()


class _PullPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, anchor, table, ids, offsets, B, S, combiner, labels, label_mod, training):
        inverse = table.pull(ids, labels, label_mod, training)
        pd = table.pdim
        if ids.is_cuda:
            out = torch.empty((B, S * pd), dtype=torch.float32, device=ids.device)
            _build.cuda_ext().pool_fwd(table.U, table.ustride, inverse, offsets, B, S, pd, combiner, out, S * pd)
        else:
            nnz = ids.numel()
            inv = inverse.long()
            rows = table.U[inv.clamp(min=0), :pd] * (inv >= 0).unsqueeze(1)
            bag = _bag_ids(offsets, B * S, nnz, ids.device)
            pooled = torch.zeros((B * S, pd), dtype=torch.float32).index_add_(0, bag, rows)
            sc = _bag_scale(offsets, B * S, combiner, ids.device)
            if sc is not None:
                pooled = pooled * sc.unsqueeze(1)
            out = pooled.view(S, B, pd).permute(1, 0, 2).reshape(B, S * pd).contiguous()
        ctx.table = table
        ctx.meta = (B, S, combiner)
        ctx.inverse = inverse
        ctx.offsets = offsets
        return out

    @staticmethod
    def backward(ctx, g):
        table = ctx.table
        B, S, combiner = ctx.meta
        pd, dim = table.pdim, table.dim
        inverse, offsets = ctx.inverse, ctx.offsets
        g = g.contiguous()
        if g.is_cuda:
            _build.cuda_ext().pool_bwd(table.gU, table.gstride, inverse, offsets, B, S, pd, dim, combiner, g, S * pd)
        else:
            gb = g.view(B, S, pd).permute(1, 0, 2).reshape(B * S, pd)[:, :dim]
            sc = _bag_scale(offsets, B * S, combiner, g.device)
            if sc is not None:
                gb = gb * sc.unsqueeze(1)
            bag = _bag_ids(offsets, B * S, inverse.numel(), g.device)
            inv = inverse.long()
            ok = inv >= 0
            table.gU[:, :dim].index_add_(0, inv[ok], gb[bag][ok])
        return (None,) * 10


def pull_pool(anchor, table, ids, offsets, B, S, combiner="sum", labels=None, label_mod=0, training=True):
    """``ids``: all ids of the layer's S columns, column after column (bag ``s*B + b``).
    ``offsets``: int32 ``[S*B + 1]`` bag boundaries, or None when every bag holds exactly one id."""
    return _PullPool.apply(anchor, table, ids, offsets, B, S, COMBINERS[combiner] if isinstance(combiner, str) else combiner,
                           labels, label_mod, training)


class _PullSeq(torch.autograd.Function):
    """Un-pooled variant for one sequence column: ``[B, T, width]`` plus lengths."""

    @staticmethod
    def forward(ctx, anchor, table, ids, offsets, B, T, labels, training):
        inverse = table.pull(ids, labels, 0, training)
        pd = table.pdim
        if ids.is_cuda:
            out = torch.zeros((B, T, pd), dtype=torch.float32, device=ids.device)
            lengths = torch.zeros(B, dtype=torch.int32, device=ids.device)
            _build.cuda_ext().seq_fwd(table.U, table.ustride, inverse, offsets, B, T, pd, out, lengths)
        else:
            out = torch.zeros((B, T, pd), dtype=torch.float32)
            lens = (offsets[1:] - offsets[:-1]).long()
            lengths = lens.clamp(max=T).int()
            bag = torch.repeat_interleave(torch.arange(B), lens)
            pos = torch.arange(ids.numel()) - offsets[:-1].long()[bag]
            ok = (pos < T) & (inverse.long() >= 0)
            out[bag[ok], pos[ok]] = table.U[inverse.long()[ok], :pd]
            ctx.cpu_idx = (bag, pos, ok)
        ctx.table, ctx.meta, ctx.inverse, ctx.offsets = table, (B, T), inverse, offsets
        ctx.mark_non_differentiable(lengths)
        return out, lengths

    @staticmethod
    def backward(ctx, g, _gl):
        table = ctx.table
        B, T = ctx.meta
        g = g.contiguous()
        if g.is_cuda:
            _build.cuda_ext().seq_bwd(table.gU, table.gstride, ctx.inverse, ctx.offsets, B, T, table.pdim, table.dim, g)
        else:
            bag, pos, ok = ctx.cpu_idx
            table.gU[:, : table.dim].index_add_(0, ctx.inverse.long()[ok], g[bag[ok], pos[ok], : table.dim])
        return (None,) * 8


def pull_sequence(anchor, table, ids, offsets, B, T, labels=None, training=True):
    return _PullSeq.apply(anchor, table, ids, offsets, B, T, labels, training)

"""Global batch-norm statistics table (core/ps/table/bn_table.cc:32-214).

Keeps, in double precision, the running sum, squared sum and count of every feature with
Kahan-compensated accumulation, increment buffers for the cross-rank exchange and the
moving-window decay that starts once ``max_count`` records have been seen.  The reference
ships increments to its peers with BnStatisticsPush RPCs (core/kernels/bn_table_ops.cc:86-153);
here the ranks all-reduce their increments, which yields the same totals on every rank.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from ..core.runtime import runtime


class BnTable:
    def __init__(self, name: str, bn_size: int, synchronized: bool, moment: float, max_count: int,
                 use_pctr_dnn_bn: bool = False):
        self.name, self.bn_size = name, int(bn_size)
        self.synchronized, self.moment, self.max_count = bool(synchronized), float(moment), int(max_count)
        self.use_pctr_dnn_bn = bool(use_pctr_dnn_bn)
        self.handle = 0
        z = lambda: np.zeros(self.bn_size, np.float64)
        self.total_sum, self.total_sum_err = z(), z()
        self.total_squared_sum, self.total_squared_sum_err = z(), z()
        self.total_count = z()
        self.inc_sum, self.inc_squared_sum, self.inc_count = z(), z(), z()

    # Kahan-compensated adds (bn_table.cc:98-110)
    def _sum_acc(self, acc):
        y = acc - self.total_sum_err
        t = self.total_sum + y
        self.total_sum_err = (t - self.total_sum) - y
        self.total_sum = t

    def _sq_acc(self, acc):
        y = acc - self.total_squared_sum_err
        t = self.total_squared_sum + y
        self.total_squared_sum_err = (t - self.total_squared_sum) - y
        self.total_squared_sum = t

    def append(self, acc_sum, acc_squared_sum, acc_count, is_local: bool = True):
        acc_sum, acc_squared_sum, acc_count = (np.asarray(a, np.float64) for a in (acc_sum, acc_squared_sum, acc_count))
        if is_local:
            self.inc_sum += acc_sum
            self.inc_squared_sum += acc_squared_sum
            self.inc_count += acc_count
        cur = int(self.total_count.max()) if self.bn_size else 0
        if self.max_count > 0 and cur > self.max_count:
            ratio = float(int(acc_count.max())) / cur
            k = (1 - self.moment) * ratio
            self.total_sum *= (1 - k)
            self._sum_acc(k * acc_sum)
            self.total_squared_sum *= (1 - k)
            self._sq_acc(k * acc_squared_sum)
        else:
            self._sum_acc(acc_sum)
            self._sq_acc(acc_squared_sum)
            self.total_count = self.total_count + acc_count

    @staticmethod
    def _div_no_nan(a, b):
        out = a.copy()
        ok = (~np.isnan(b)) & (b != 0)
        out[ok] = a[ok] / b[ok]
        out[~ok] = 0.0
        return out.astype(np.float32)

    def get_moments(self):
        mean = self._div_no_nan(self.total_sum, self.total_count)
        if self.use_pctr_dnn_bn:
            return mean, self.total_squared_sum.astype(np.float32)
        sq_mean = self._div_no_nan(self.total_squared_sum, self.total_count)
        var = np.maximum(sq_mean - mean * mean, 0.0).astype(np.float32)
        return mean, var

    def take_increments(self):
        out = (self.inc_sum.copy(), self.inc_squared_sum.copy(), self.inc_count.copy())
        self.inc_sum[:] = 0
        self.inc_squared_sum[:] = 0
        self.inc_count[:] = 0
        return out

    def sync_increments(self):
        """Exchange the increments accumulated since the last exchange with all other ranks."""
        rt = runtime()
        s, q, c = self.take_increments()
        if rt.world == 1:
            return
        mine = torch.from_numpy(np.concatenate([s, q, c]))
        tot = mine.clone()
        dist.all_reduce(tot, group=rt.host_group)
        others = (tot - mine).numpy()
        n = self.bn_size
        self.append(others[:n], others[n:2 * n], others[2 * n:], is_local=False)

    def refresh(self):
        for a in (self.total_sum, self.total_squared_sum, self.total_count, self.inc_sum, self.inc_squared_sum, self.inc_count):
            a[:] = 0

    def totals(self):
        return self.total_sum.copy(), self.total_squared_sum.copy(), self.total_count.copy()

    def set_totals(self, s, q, c):
        self.total_sum, self.total_squared_sum, self.total_count = (np.asarray(a, np.float64).copy() for a in (s, q, c))
        self.total_sum_err[:] = 0
        self.total_squared_sum_err[:] = 0


class GpuBnTable:
    """The same table held in device memory (``csrc/bn.cu``): a training step of the layer folds its batch in
    with two small kernels and no host round trip, so the layer can sit inside a captured CUDA graph; the
    cross-GPU exchange of increments is one kernel doing peer loads between two bounded flag handshakes.
    The host-visible methods mirror :class:`BnTable` (numpy in, numpy out) for checkpoints and tests."""

    def __init__(self, name: str, bn_size: int, synchronized: bool, moment: float, max_count: int,
                 use_pctr_dnn_bn: bool = False):
        from .. import _build
        from ..parallel.symm import SymmArena

        rt = runtime()
        self.name, self.bn_size = name, int(bn_size)
        self.synchronized, self.moment, self.max_count = bool(synchronized), float(moment), int(max_count)
        self.use_pctr_dnn_bn = bool(use_pctr_dnn_bn)
        self.handle = 0
        d, C = rt.device, self.bn_size
        zd = lambda n=C: torch.zeros(n, dtype=torch.float64, device=d)
        self.total_sum, self.total_sum_err, self.total_sq, self.total_sq_err, self.total_count = zd(), zd(), zd(), zd(), zd()
        self.mean = torch.zeros(C, dtype=torch.float32, device=d)
        self.var = torch.zeros(C, dtype=torch.float32, device=d)
        self.batch, self.scratch = zd(3 * C), zd(3 * C)
        cfg = dict(C=C, pctr=int(self.use_pctr_dnn_bn), moment=self.moment, max_count=self.max_count,
                   total_sum=self.total_sum, total_sum_err=self.total_sum_err, total_sq=self.total_sq,
                   total_sq_err=self.total_sq_err, total_count=self.total_count, mean=self.mean, var=self.var,
                   batch=self.batch, scratch=self.scratch, world=rt.world, rank=rt.rank)
        if rt.world > 1:
            # every rank creates its BN layers in the same order, so the collective allocation lines up
            self._arena = SymmArena([("inc", (3 * C,), torch.float64), ("sig", (2 * 8,), torch.int64)])
            self.inc = self._arena.tensor("inc")
            self._epoch = torch.zeros(1, dtype=torch.int64, device=d)
            cfg.update(inc=self.inc, inc_ptrs=self._arena.ptrs("inc"), sig_ptrs=self._arena.ptrs("sig"), epoch=self._epoch,
                       status=rt.status, wait_ns=rt.wait_ns)
            rt.barrier()
        else:
            self.inc = zd(3 * C)
            cfg.update(inc=self.inc)
        self.ctx = _build.cuda_ext().BnCtx(cfg)
        self.ctx.refresh()

    # ---- device-side step -------------------------------------------------------------------
    def push_batch(self, x: torch.Tensor, centered: bool = False):
        """Fold the per-feature sums of ``x`` ([B, C] fp32) into the table; ``centered`` squares deviations
        from the table's current mean (the PCTR variant)."""
        self.ctx.push(x, bool(centered))

    def sync_increments(self):
        """All ranks call this at the same step; a no-op with one GPU apart from dropping the increments."""
        if runtime().world > 1:
            self.ctx.sync()
        else:
            self.inc.zero_()

    # ---- host-visible mirror of BnTable ------------------------------------------------------
    def append(self, acc_sum, acc_squared_sum, acc_count, is_local: bool = True):
        if not is_local:
            raise NotImplementedError("non-local appends happen inside the exchange kernel")
        acc = np.concatenate([np.asarray(a, np.float64).reshape(-1) for a in (acc_sum, acc_squared_sum, acc_count)])
        self.batch.copy_(torch.from_numpy(acc))
        # the append kernel alone: the batch sums are already in place
        _append_only(self)

    def get_moments(self):
        return self.mean.cpu().numpy(), self.var.cpu().numpy()

    def take_increments(self):
        C = self.bn_size
        inc = self.inc.cpu().numpy().copy()
        self.inc.zero_()
        return inc[:C], inc[C:2 * C], inc[2 * C:]

    def refresh(self):
        for a in (self.total_sum, self.total_sum_err, self.total_sq, self.total_sq_err, self.total_count, self.inc):
            a.zero_()
        self.ctx.refresh()

    def totals(self):
        return self.total_sum.cpu().numpy(), self.total_sq.cpu().numpy(), self.total_count.cpu().numpy()

    def set_totals(self, s, q, c):
        for dst, src in ((self.total_sum, s), (self.total_sq, q), (self.total_count, c)):
            dst.copy_(torch.from_numpy(np.asarray(src, np.float64).copy()))
        self.total_sum_err.zero_()
        self.total_sq_err.zero_()
        self.ctx.refresh()


def _append_only(t: GpuBnTable):
    # a zero-row batch adds nothing to the sums already staged in ``t.batch`` but would overwrite the counts,
    # so the staged record goes through a dedicated entry point
    t.ctx.append_staged()

"""GPU shard of one sparse embedding table and its exchange buffers.

What the reference keeps in ``SparseTable`` + ``SparseOptimizerKernel`` on every CPU rank
(core/ps/table/sparse_table.cc:52-137, core/ps/optimizer/optimizer_kernel.h:439-560) lives
here in HBM: an open-addressing key array, a dense slab of rows (weights + optimizer slots +
show/click counters in one contiguous record) and the symmetric-memory inboxes the fused
pull / push kernels use to talk to the other GPUs.  Row ownership is ``sign % world`` as in
the reference (core/kernels/sparse_table_ops.cc:221), so checkpoint directories line up.
"""
from __future__ import annotations

import math
import weakref
from typing import Optional, Tuple

import numpy as np
import torch

from .. import _build
from .._opentelemetry import phase
from ..core.config import config
from ..core.optimizers import KIND_ADAGRAD, OptimizerBase
from ..core.runtime import runtime
from ..parallel.symm import SymmArena


def round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def row_floats(kind: int, dim: int) -> int:
    return dim + 4 if kind == KIND_ADAGRAD else 3 * dim + 2


def next_pow2(x: int) -> int:
    return 1 << max(1, (int(x) - 1).bit_length())


#: every live shard of this process (``core.recover`` resets the exchange state of all of them)
live_tables: "weakref.WeakSet[GpuSparseTable]" = weakref.WeakSet()


class GpuSparseTable:
    def __init__(self, opt: OptimizerBase, dim: int, use_cvm: bool = False, name: str = "", rows: Optional[int] = None):
        rt = runtime()
        assert rt.on_gpu, "GpuSparseTable needs a CUDA device"
        self.ext = _build.cuda_ext()
        self.opt = opt
        self.kind = opt.kind
        self.dim = int(dim)
        self.use_cvm = bool(use_cvm)
        self.name = name
        self.dev = rt.device
        self.world, self.rank = rt.world, rt.rank
        self.row_cap = int(rows or config.table_rows_per_gpu)
        self.stride = round_up(row_floats(self.kind, self.dim), 4)
        self.pdim = self.dim + (2 if self.use_cvm else 0)
        self.ustride = round_up(self.pdim, 4)
        self.gstride = round_up(self.dim + 2, 4)
        cap = next_pow2(int(self.row_cap / config.table_load_factor))
        d = self.dev
        self.keys = torch.full((cap,), -1, dtype=torch.int64, device=d)
        self.slots = torch.full((cap,), -1, dtype=torch.int32, device=d)
        self.rows = torch.empty((self.row_cap, self.stride), dtype=torch.float32, device=d)
        self.row_keys = torch.empty((self.row_cap,), dtype=torch.int64, device=d)
        self.row_tag = torch.zeros((self.row_cap,), dtype=torch.int64, device=d)
        self.n_rows_dev = torch.zeros((1,), dtype=torch.int32, device=d)
        self.epoch = torch.zeros((1,), dtype=torch.int64, device=d)
        self.links = []
        self._zero_init = False
        self.grown = 0               # how many times the shard has been enlarged
        live_tables.add(self)

    # ------------------------------------------------------------------ views for the kernels
    def table_dict(self):
        return dict(keys=self.keys, slots=self.slots, rows=self.rows, row_keys=self.row_keys, row_tag=self.row_tag,
                    n_rows=self.n_rows_dev, dim=self.dim, stride=self.stride, use_cvm=int(self.use_cvm))

    def _opt_dict(self):
        d = self.opt.sparse_params()
        d["zero_init"] = int(self._zero_init or self.opt.sparse_zero_init)
        return d

    def link(self, max_unique: int) -> "GpuSparseLink":
        """Exchange buffers + kernel context for one user (layer) of this table.  Collective when
        world > 1: all ranks must create their links in the same order."""
        lk = GpuSparseLink(self, max_unique)
        self.links.append(lk)
        return lk

    def set_training(self, training: bool):
        """Inference mode creates all-zero rows (core/ps/optimizer/ada_grad_kernel.cc:80-84)."""
        zi = not training
        if zi != self._zero_init:
            self._zero_init = zi
            self.refresh_opt()

    # ------------------------------------------------------------------ maintenance
    @property
    def n_rows(self) -> int:
        return int(self.n_rows_dev.item())

    def refresh_opt(self):
        for lk in self.links:
            lk.ctx.set_opt(self._opt_dict())

    def show_decay(self, delta_days: int):
        rate = float(getattr(self.opt, "show_decay_rate", 1.0))
        self.ext.table_decay(self.table_dict(), self.kind, rate, int(delta_days))

    def clear(self):
        self.keys.fill_(-1)
        self.slots.fill_(-1)
        self.row_tag.zero_()
        self.n_rows_dev.zero_()

    def dump(self) -> Tuple[np.ndarray, np.ndarray]:
        """Host copy of (signs [n] uint64, rows [n, row_floats] float32) of this shard."""
        n = self.n_rows
        rf = row_floats(self.kind, self.dim)
        keys = self.row_keys[:n].cpu().numpy().view(np.uint64)
        rows = self.rows[:n, :rf].contiguous().cpu().numpy()
        return keys, rows

    def export_chunks(self, chunk_rows: int = 1 << 22, evict=(False, 0.0, 0, 0)):
        """Stream this shard for a checkpoint.  Yields ``(signs uint64 [m], rows float32 [m, row_floats],
        offsets int64 [9])`` per slab range of ``chunk_rows`` rows: rows the save-time eviction rule drops are
        already gone and the rest is grouped by block file (``offsets[b]:offsets[b+1]`` is block b), packed on
        the device and copied out through one pinned staging buffer that is reused, so host memory stays at one
        chunk however large the shard is.  The arrays are views of that buffer: consume them before the next one."""
        n = self.n_rows
        rf = row_floats(self.kind, self.dim)
        chunk_rows = max(1, min(int(chunk_rows), max(n, 1)))
        d = self.dev
        k_dev = torch.empty(chunk_rows, dtype=torch.int64, device=d)
        r_dev = torch.empty((chunk_rows, rf), dtype=torch.float32, device=d)
        cnt = torch.zeros(16, dtype=torch.int32, device=d)
        k_host = torch.empty(chunk_rows, dtype=torch.int64).pin_memory()
        r_host = torch.empty((chunk_rows, rf), dtype=torch.float32).pin_memory()
        for r0 in range(0, n, chunk_rows):
            r1 = min(n, r0 + chunk_rows)
            cnt.zero_()
            self.ext.table_export(self.table_dict(), self.kind, bool(evict[0]), float(evict[1]), int(evict[2]), int(evict[3]),
                                  r0, r1, cnt[:8], cnt[8:], k_dev, r_dev)
            counts = cnt[:8].cpu().numpy().astype(np.int64)
            m = int(counts.sum())
            k_host[:m].copy_(k_dev[:m], non_blocking=True)
            r_host[:m].copy_(r_dev[:m], non_blocking=True)
            torch.cuda.current_stream().synchronize()
            offsets = np.zeros(9, dtype=np.int64)
            offsets[1:] = np.cumsum(counts)
            yield k_host[:m].numpy().view(np.uint64), r_host[:m].numpy(), offsets

    def load_rows(self, signs: np.ndarray, rows: np.ndarray, chunk: int = 1 << 20):
        """Insert (or overwrite) rows given as host arrays; ``signs`` must be distinct."""
        rt = runtime()
        rf = row_floats(self.kind, self.dim)
        assert rows.shape[1] == rf
        for s in range(0, len(signs), chunk):
            k = torch.from_numpy(signs[s:s + chunk].view(np.int64).copy()).to(self.dev)
            r = torch.from_numpy(np.ascontiguousarray(rows[s:s + chunk])).to(self.dev)
            idx = torch.empty(k.numel(), dtype=torch.int32, device=self.dev)
            self.ext.table_insert_keys(self.table_dict(), k, idx, rt.status)
            ok = idx >= 0
            li = idx[ok].long()
            full = torch.zeros((int(ok.sum().item()), self.stride), dtype=torch.float32, device=self.dev)
            full[:, :rf] = r[ok]
            self.rows.index_copy_(0, li, full)
        rt.check_status()

    def lookup_rows(self, ids: torch.Tensor) -> torch.Tensor:
        """Row index of each sign on this shard (-1 when absent); read-only."""
        out = torch.empty(ids.numel(), dtype=torch.int32, device=self.dev)
        self.ext.table_lookup(self.table_dict(), ids.reshape(-1).contiguous(), out)
        return out

    # ------------------------------------------------------------------ growth and shedding (between steps)
    def _swap_arrays(self):
        """The shard's arrays were replaced: hand the new ones to every link.  Launches already recorded in CUDA
        graphs read the table through a descriptor in device memory, so they follow without a new capture."""
        for lk in self.links:
            lk.ctx.set_table(self.table_dict())

    def load_factor(self, rows: Optional[int] = None) -> float:
        return (self.n_rows if rows is None else rows) / self.keys.numel()

    def grow(self, new_row_cap: Optional[int] = None):
        """Make room for more rows: a longer row slab (the rows in use are copied over on the device) and, when the
        key array would pass the configured load factor, a larger key array that is re-filled from the signs of the
        rows.  Call between steps; rows keep their indices.  The reference's sub-maps rehash themselves and its
        allocator adds a 65 536-row slab at a time (core/ps/optimizer/optimizer_kernel.h:257-270,
        core/utility/allocator.h:74-92)."""
        rt = runtime()
        torch.cuda.synchronize(self.dev)
        n = self.n_rows
        new_cap = int(new_row_cap or max(2 * self.row_cap, 1024))
        if new_cap <= self.row_cap:
            return
        d = self.dev
        rows = torch.empty((new_cap, self.stride), dtype=torch.float32, device=d)
        rows[:n].copy_(self.rows[:n])
        self.rows = rows
        for name, fill in (("row_keys", None), ("row_tag", 0)):
            old = getattr(self, name)
            new = torch.empty((new_cap,), dtype=torch.int64, device=d) if fill is None else torch.zeros((new_cap,), dtype=torch.int64, device=d)
            new[:n].copy_(old[:n])
            setattr(self, name, new)
        self.row_cap = new_cap
        cap = next_pow2(int(new_cap / config.table_load_factor))
        if cap > self.keys.numel():
            self.keys = torch.full((cap,), -1, dtype=torch.int64, device=d)
            self.slots = torch.full((cap,), -1, dtype=torch.int32, device=d)
            self.ext.table_rebuild_index(self.table_dict(), n, rt.status)
        self._swap_arrays()
        self.grown += 1

    def maybe_grow(self, rows_now: int, threshold: float = 0.85) -> bool:
        """Grow when the slab is ``threshold`` full (``rows_now``: a recent reading of the row counter)."""
        if rows_now >= threshold * self.row_cap:
            self.grow()
            return True
        return False

    def compact(self, keep_mask: torch.Tensor):
        """Drop the rows whose ``keep_mask`` entry is false and close the gaps, all on the device: kept rows from
        beyond the new end move into the holes before it, then the key array is cleared and re-filled from the
        rows.  Row indices change, so call it between steps only."""
        rt = runtime()
        torch.cuda.synchronize(self.dev)
        n = self.n_rows
        keep = keep_mask[:n].to(torch.bool)
        n_keep = int(keep.sum().item())
        if n_keep < n:
            holes = (~keep[:n_keep]).nonzero().flatten()
            movers = keep[n_keep:].nonzero().flatten() + n_keep
            piece = 1 << 22                                   # bounds the temporary of the gather
            for s in range(0, int(movers.numel()), piece):
                src, dst = movers[s:s + piece], holes[s:s + piece]
                self.rows[dst] = self.rows[src]
                self.row_keys[dst] = self.row_keys[src]
            self.row_tag[:n].zero_()
            self.n_rows_dev.fill_(n_keep)
            self.keys.fill_(-1)
            self.slots.fill_(-1)
            self.ext.table_rebuild_index(self.table_dict(), n_keep, rt.status)
        rt.check_status()
        return n - n_keep

    def evict(self) -> int:
        """Shed the rows the optimizer's save-time rule would not write (AdaGrad: ``show < show_threshold`` or / and
        ``no_show_days`` exceeded; Ftrl: ``show < show_threshold``; ada_grad_kernel.cc:197-204, ftrl_kernel.cc:126)
        from the live shard.  Returns the number of rows dropped."""
        from ..utils.checkpoint import _evict_args

        ev = _evict_args(self.opt)
        if not ev[0]:
            return 0
        n = self.n_rows
        keep = torch.empty(max(n, 1), dtype=torch.uint8, device=self.dev)
        self.ext.table_keep_mask(self.table_dict(), self.kind, True, float(ev[1]), int(ev[2]), int(ev[3]), n, keep)
        return self.compact(keep)


_FRONT_STREAMS = {}


def front_stream(device) -> "torch.cuda.Stream":
    """The stream the pull fronts of a device run on."""
    key = str(device)
    st = _FRONT_STREAMS.get(key)
    if st is None:
        st = _FRONT_STREAMS[key] = torch.cuda.Stream(device=device)
    return st


class GpuSparseLink:
    """Per-layer exchange state of a table: symmetric inboxes, the per-batch unique-row matrix
    ``U``, its gradient ``gU`` and the bookkeeping that ties one pull to the following push."""

    def __init__(self, table: GpuSparseTable, max_unique: int):
        rt = runtime()
        self.table = table
        self.dim, self.pdim, self.kind = table.dim, table.pdim, table.kind
        self.ustride, self.gstride = table.ustride, table.gstride
        self.dev = table.dev
        W = table.world
        self.max_unique = int(max_unique)
        if W == 1:
            capo = round_up(self.max_unique + 4, 32)
        else:
            # One (sender, owner) segment.  The reference accepts any batch below bucket_size whatever the spread of
            # its signs over sign % world (core/kernels/sparse_table_ops.cc:135-136), so a segment holds the whole
            # batch when the exchange buffers stay within `segment_worst_case_mb`; larger layers size it for an even
            # spread times `owner_segment_slack`, and a batch that overflows it is reported (owner segment overflow).
            even = round_up(int(math.ceil(self.max_unique / W * config.owner_segment_slack)) + 64, 32)   # whole row tiles
            worst = round_up(self.max_unique + 4, 32)
            per_row = 4 * (2 * self.gstride + self.ustride) + 48          # accumulator, gradient records, pulled row, bookkeeping
            capo = worst if W * worst * per_row <= config.segment_worst_case_mb * (1 << 20) else even
        self.capo = capo
        n_seg = W * capo
        multi = W > 1
        arena = SymmArena([
            ("inbox_ids", (n_seg if multi else 4,), torch.int64),
            ("gU", (n_seg * self.gstride,), torch.float32),       # owners read their segment of every GPU's records
            ("cnts", (n_seg * 2,), torch.float32),
            ("U", (n_seg * self.ustride,), torch.float32),
            ("sig", (4 * 8,), torch.int64),
        ])
        d = self.dev
        dd_cap = next_pow2(2 * self.max_unique + 16)
        loc = dict(
            stage_ids=torch.zeros(n_seg, dtype=torch.int64, device=d),
            gU=arena.tensor("gU").zero_(),
            cnts=arena.tensor("cnts").zero_(),
            cnt=torch.zeros(8, dtype=torch.int32, device=d),
            cnt_saved=torch.zeros(8, dtype=torch.int32, device=d),
            req_n=torch.zeros(8, dtype=torch.int32, device=d),
            req_row=torch.full((n_seg,), -1, dtype=torch.int32, device=d),
            req_ou=torch.full((n_seg,), -1, dtype=torch.int32, device=d),
            ou_row=torch.full((n_seg if multi else 4,), -1, dtype=torch.int32, device=d),
            ocount=torch.zeros(1, dtype=torch.int32, device=d),
            acc=torch.zeros(n_seg * self.gstride if multi else 4, dtype=torch.float32, device=d),
            dd_keys=torch.full((dd_cap,), -1, dtype=torch.int64, device=d),
            dd_vals=torch.zeros(dd_cap, dtype=torch.int32, device=d),
            bar=torch.zeros(8, dtype=torch.int32, device=d),
            prof=torch.zeros(24, dtype=torch.int64, device=d),
        )
        self.arena = arena
        self._loc = loc
        self.U = arena.tensor("U").view(n_seg, self.ustride)
        self.gU = loc["gU"].view(n_seg, self.gstride)
        self.cnts = loc["cnts"].view(n_seg, 2)       # (show, click) of the batch per distinct sign
        self.cnt_saved = loc["cnt_saved"]
        self.prof = loc["prof"]
        staged = multi if config.staged_row_return < 0 else bool(config.staged_row_return)
        self.comm = dict(world=W, rank=table.rank, capo=capo, staged_return=staged, gstride=self.gstride, ustride=self.ustride,
                         inbox_ids=arena.ptrs("inbox_ids"), gU_peer=arena.ptrs("gU"), cnts_peer=arena.ptrs("cnts"), U=arena.ptrs("U"),
                         sig=arena.ptrs("sig"), epoch=table.epoch, status=rt.status, wait_ns=rt.wait_ns, **loc)
        self.ctx = table.ext.SparseCtx(table.table_dict(), self.comm, table._opt_dict())
        self._last_n_ids = 0
        self.push_cta_cap = 0        # > 0: the push kernel leaves the remaining SMs to a kernel on another stream
        self.dense_rider = None      # a DenseTable whose step the next push carries on a few of its CTAs (several GPUs)
        # pull front run ahead of its step (see prefetch): (ids data pointer, count, inverse buffer) of the batch it ran for
        self._front = None
        self.next_ids = None         # set by the model before a step: the ids this link will pull at the NEXT step
        self.front_in_flight = False # a front was forked onto the side stream during this step (the model joins it)
        self.front_hits = 0          # pulls that found their front done (a model checks that its layers really pull)
        self._fork = torch.cuda.Event() if runtime().on_gpu else None
        self._front_inverse = {}     # inverse buffers of the fronts, one per id buffer (stable addresses for CUDA graphs)
        if multi:
            rt.barrier()

    def pull(self, ids: torch.Tensor, labels: Optional[torch.Tensor] = None, label_mod: int = 0, training: bool = True,
             inverse: Optional[torch.Tensor] = None, lookup_only: bool = False) -> torch.Tensor:
        """Dedup ``ids``, fetch (creating on miss) their rows from the owning GPUs into ``self.U`` and
        return ``inverse``: the row of ``self.U`` holding each id's embedding.  ``lookup_only`` (inference)
        never creates rows: signs no shard holds come back as zeros."""
        n = ids.numel()
        front, self._front = self._front, None
        front_done = False
        if front is not None:
            if front[0] == ids.data_ptr() and front[1] == n and training and not lookup_only and inverse is None:
                inverse, front_done = front[2], True
                self.front_hits += 1
            else:
                self.discard_front()
        if inverse is None:
            inverse = torch.empty(n, dtype=torch.int32, device=self.dev)
        self._last_n_ids = n
        with phase("tn.sparse_pull"):
            self.ctx.pull(ids.reshape(-1), inverse, labels, int(label_mod), bool(training), bool(lookup_only), front_done)
        return inverse

    def fork_front(self):
        """The batch of the following step is known (``next_ids``): run its dedup and id dispatch on the side stream
        from this point of the current stream on.  The model calls this once the forward pass is issued, so the
        front's atomics share the GPU with the backward GEMMs rather than with the gather of this step's rows."""
        nxt, self.next_ids = self.next_ids, None
        if nxt is None:
            return
        self._fork.record()
        side = front_stream(self.dev)
        side.wait_event(self._fork)
        with torch.cuda.stream(side):
            self.prefetch(nxt)
        self.front_in_flight = True

    def prefetch(self, ids: torch.Tensor):
        """Run the front of the pull (dedup, id dispatch to the owners, inverse map) for the batch ``ids`` on the
        current stream.  The next :meth:`pull` must be a training pull of this very tensor; it then only probes and
        returns rows.  Anything else discards the front (:meth:`discard_front`).  ``ids`` must not live in the
        buffer of a batch whose backward pass is still to come: the inverse map of a front is kept per id buffer."""
        n = ids.numel()
        key = (ids.data_ptr(), n)
        inverse = self._front_inverse.get(key)
        if inverse is None:
            if len(self._front_inverse) >= 8:
                self._front_inverse.pop(next(iter(self._front_inverse)))
            inverse = self._front_inverse[key] = torch.empty(n, dtype=torch.int32, device=self.dev)
        with phase("tn.sparse_pull_front"):
            self.ctx.front(ids.reshape(-1), inverse)
        self._front = (ids.data_ptr(), n, inverse)

    def discard_front(self):
        """Forget a front that ran for a batch which is not pulled next: the per-owner counters it built are
        cleared and the step counter moves on by one, so the id segments and flags it sent can never be taken for
        those of the pull that follows.  Every rank must do this at the same point (they do: same program)."""
        self._front = None
        self._loc["cnt"].zero_()
        self.table.epoch.add_(1)

    def push(self):
        """Apply the accumulated unique-row gradients (``self.gU``) on the owning GPUs."""
        rider, self.dense_rider = self.dense_rider, None
        with phase("tn.sparse_push+dense_step" if rider is not None else "tn.sparse_push"):
            self.ctx.push(max(self._last_n_ids, 1), int(self.push_cta_cap), rider.ctx if rider is not None else None)
        if self.table.world > 1:
            runtime().peer_synced_pushes += 1      # this kernel waited for every peer's gradient records

    def reset_exchange(self):
        """Bring this link's per-step state back to "between steps" after a kernel gave up half-way (a wait that ran
        out skips the clean-up at the end of the pull): dedup scratch empty, counters and accumulators zero, no
        request bookkeeping, flag words clear.  Part of :func:`tensornet_b200.core.recover`; every rank runs it
        between two host barriers, so no peer is writing into the inboxes meanwhile."""
        l = self._loc
        l["dd_keys"].fill_(-1)
        for k in ("cnt", "cnt_saved", "req_n", "ocount", "acc", "gU", "cnts", "bar"):
            l[k].zero_()
        for k in ("req_row", "req_ou", "ou_row"):
            l[k].fill_(-1)
        self.arena.tensor("sig").zero_()
        self._front = None           # a pull front that ran ahead is gone with the counters it built

    def pull_phase_us(self):
        """Durations (microseconds) of the last pull's phases as seen by CTA 0: dedup; id dispatch + inverse map;
        probe and row return of this GPU's own segment; wait for the other GPUs' ids, their probe and row return;
        completion flags + scratch clear."""
        t = self.prof.tolist()
        return [(t[i + 1] - t[i]) / 1e3 for i in range(5)]

    def front_timeline_us(self):
        """Where the last run-ahead pull front sat in time, in microseconds relative to the start of the last pull
        kernel: (front start, end of its dedup kernel, end of its shipping / inverse kernel, end of the pull, start of
        the last push, end of that push's row updates)."""
        t = self.prof.tolist()
        return [(t[i] - t[0]) / 1e3 for i in (16, 17, 18, 5, 8, 13)]

    def push_phase_us(self):
        """Durations (microseconds) of the last multi-GPU push's phases as seen by CTA 0: flags to the owners,
        (unused), owner-side accumulation (own records, then the wait for and the read of the peers' records over
        NVLink), grid barrier, optimizer update."""
        t = self.prof.tolist()
        return [(t[i + 1] - t[i]) / 1e3 for i in range(8, 13)]

    def unique_counts(self):
        """Per-owner unique-sign counts of the last pull (host sync)."""
        return self.cnt_saved[: self.table.world].tolist()

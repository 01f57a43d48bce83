"""CPU shard of a sparse table: the reference's algorithms restated in plain C++ (module
``_tn_cpu``), used when no GPU is present, as the oracle of the GPU kernels and as the CPU
baseline.  Ranks exchange id lists, rows and gradient records over the gloo process group,
playing the part of the reference's brpc SparsePull / SparsePush RPCs
(core/ps/ps_local_server.cc:30-54).

Like the GPU path the step is synchronous, and by default gradients of one sign coming from
several ranks are summed and applied once by the owner.  ``apply_mode="arrival"`` restates the
reference's own behaviour instead: every worker's records are applied one worker after the other
in arrival order (here: rank order), each on top of the previous one's result
(core/kernels/sparse_table_ops.cc:363-367, core/ps/ps_local_server.cc:43-54), which is what
makes N workers pushing the same sign differ from one worker pushing the sum.
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from .. import _build
from ..core.optimizers import KIND_ADAGRAD, OptimizerBase
from ..core.runtime import runtime


def row_floats(kind: int, dim: int) -> int:
    return dim + 4 if kind == KIND_ADAGRAD else 3 * dim + 2


class CpuSparseTable:
    def __init__(self, opt: OptimizerBase, dim: int, use_cvm: bool = False, name: str = "", rows=None,
                 apply_mode: str = "sum"):
        if apply_mode not in ("sum", "arrival"):
            raise ValueError("apply_mode must be 'sum' (one update per sign and step) or 'arrival' (one per worker)")
        self.apply_mode = apply_mode
        rt = runtime()
        self.ext = _build.cpu_ext()
        self.opt, self.kind, self.dim, self.use_cvm, self.name = opt, opt.kind, int(dim), bool(use_cvm), name
        self.pdim = self.dim + (2 if self.use_cvm else 0)
        self.world, self.rank = rt.world, rt.rank
        self._zero_init = False
        self.native = self.ext.CpuSparseTable(self._opt_dict(), self.dim, self.use_cvm, self.world, self.rank)
        self.links = []

    def _opt_dict(self):
        d = self.opt.sparse_params()
        d["zero_init"] = int(self._zero_init or self.opt.sparse_zero_init)
        return d

    def refresh_opt(self):
        self.native.set_opt(self._opt_dict())

    def set_training(self, training: bool):
        zi = not training
        if zi != self._zero_init:
            self._zero_init = zi
            self.refresh_opt()

    def link(self, max_unique: int) -> "CpuSparseLink":
        lk = CpuSparseLink(self)
        lk.max_unique = int(max_unique)
        self.links.append(lk)
        return lk

    @property
    def n_rows(self) -> int:
        return int(self.native.size())

    def show_decay(self, delta_days: int):
        self.native.show_decay(float(getattr(self.opt, "show_decay_rate", 1.0)), int(delta_days))

    def dump(self) -> Tuple[np.ndarray, np.ndarray]:
        return self.native.dump()

    def load_rows(self, signs: np.ndarray, rows: np.ndarray):
        self.native.load_rows(np.ascontiguousarray(signs, dtype=np.uint64), np.ascontiguousarray(rows, dtype=np.float32))

    def clear(self):
        self.native.clear()


class CpuSparseLink:
    """Per-layer state tying one pull to the following push (mirrors GpuSparseLink)."""

    def __init__(self, table: CpuSparseTable):
        self.table = table
        self.dim, self.pdim, self.kind = table.dim, table.pdim, table.kind
        self.ustride, self.gstride = table.pdim, table.dim
        self.U = torch.zeros(0, self.pdim)
        self.gU = torch.zeros(0, self.dim)
        self._uniq = np.zeros(0, np.uint64)
        self._show = self._click = np.zeros(0, np.float32)
        self._route = None
        self._split = None
        self._mine = None
        self._ready = None           # (ids tensor, inverse) of a pull that pull_many ran ahead of the layer's own call
        self.max_unique = 0

    def unique_counts(self):
        return [int(len(self._uniq))]

    # ---- pull in stages, so that several layers' exchanges can share their round trips (pull_many) ------------
    def _pull_local(self, ids, labels, label_mod, training):
        """Dedup the batch; returns the inverse map.  With several ranks also splits the signs by owner."""
        t = self.table
        ids_np = ids.reshape(-1).cpu().numpy()
        lab = None
        if labels is not None and training:
            lab = labels.reshape(-1).float().cpu().numpy()
            if label_mod > 0:
                lab = lab[np.arange(len(ids_np)) % label_mod]
        uniq, inv, show, click = t.ext.unique_first_occurrence(ids_np, lab)
        self._uniq, self._show, self._click = uniq, show, click
        if t.world > 1:
            W = t.world
            owner = (uniq % np.uint64(W)).astype(np.int64)
            order = np.argsort(owner, kind="stable")
            counts = np.bincount(owner, minlength=W)
            self._split = (order, counts, np.split(uniq[order], np.cumsum(counts)[:-1]))
        return inv

    def _fixed_size_ids(self) -> bool:
        """Small layers: fixed-size id messages [n | signs | padding] save the round that tells the sizes."""
        cap = self.max_unique
        return 0 < cap <= (1 << 16) and len(self._uniq) <= cap

    def _ids_out(self):
        cap, W = self.max_unique, self.table.world
        send = []
        for p in self._split[2]:
            buf = np.zeros(cap + 1, np.uint64)
            buf[0] = len(p)
            buf[1:1 + len(p)] = p
            send.append(torch.from_numpy(buf.view(np.uint8)))
        return send, [8 * (cap + 1)] * W

    def _ids_in(self, got, fixed: bool):
        """Signs every rank asks this shard for -> the rows to send back."""
        if fixed:
            mine = []
            for gbuf in got:
                a = gbuf.numpy().view(np.uint64)
                mine.append(a[1:1 + int(a[0])])
        else:
            mine = [g.numpy().view(np.uint64) for g in got]
        self._mine = mine
        t = self.table
        answers = [torch.from_numpy(np.ascontiguousarray(t.native.pull(np.ascontiguousarray(m)), dtype=np.float32).reshape(-1).view(np.uint8))
                   for m in mine]
        return answers, [4 * self.pdim * int(n) for n in self._split[1]]

    def _rows_in(self, back):
        order, counts, _ = self._split
        rows = np.zeros((len(self._uniq), self.pdim), np.float32)
        rows[order] = np.concatenate([b.numpy().view(np.float32).reshape(-1, self.pdim) for b in back], axis=0)
        self._route = (order, counts, self._mine)
        self._finish_pull(rows)

    def _finish_pull(self, rows):
        self.U = torch.from_numpy(np.ascontiguousarray(rows))
        self.gU = torch.zeros(len(self._uniq), self.dim)

    def pull(self, ids: torch.Tensor, labels: Optional[torch.Tensor] = None, label_mod: int = 0, training: bool = True,
             inverse=None) -> torch.Tensor:
        ready, self._ready = self._ready, None
        if ready is not None and ready[0] is ids:
            return ready[1]                      # pull_many already ran this pull
        t, rt = self.table, runtime()
        inv = self._pull_local(ids, labels, label_mod, training)
        if t.world == 1:
            self._finish_pull(t.native.pull(self._uniq))
            return torch.from_numpy(inv)
        fixed = self._fixed_size_ids()
        if fixed:
            got = rt.exchange_bytes(*self._ids_out())
        else:
            counts, pieces = self._split[1], self._split[2]
            send = [torch.from_numpy(np.ascontiguousarray(p).view(np.uint8)) for p in pieces]
            want = rt.exchange_counts(counts)[:, t.rank].tolist()             # signs each rank asks this shard for
            got = rt.exchange_bytes(send, [8 * n for n in want])
        self._rows_in(rt.exchange_bytes(*self._ids_in(got, fixed)))
        return torch.from_numpy(inv)

    @staticmethod
    def pull_many(calls):
        """Run several layers' pulls with shared round trips: ``calls`` is a list of ``(link, ids, labels, label_mod,
        training)``.  All id messages travel in one round and all row messages in a second one (a step of a model
        with N embedding layers then pays 2 rounds instead of 2 N).  Each link remembers its result; the layer's own
        ``pull`` of the same ``ids`` tensor picks it up.  Links whose batch does not fit the fixed-size id message
        are pulled one by one."""
        rt = runtime()
        batch = []
        for lk, ids, labels, label_mod, training in calls:
            inv = lk._pull_local(ids, labels, label_mod, training)
            if lk.table.world == 1:
                lk._finish_pull(lk.table.native.pull(lk._uniq))
                lk._ready = (ids, torch.from_numpy(inv))
            elif lk._fixed_size_ids():
                batch.append((lk, ids, inv))
            else:
                lk._ready = None
                lk._ready = (ids, lk.pull(ids, labels, label_mod, training))
        if not batch:
            return
        got = rt.exchange_bytes_many([lk._ids_out() for lk, _, _ in batch])
        back = rt.exchange_bytes_many([lk._ids_in(g, True) for (lk, _, _), g in zip(batch, got)])
        for (lk, ids, inv), b in zip(batch, back):
            lk._rows_in(b)
            lk._ready = (ids, torch.from_numpy(inv))

    def _records_out(self):
        order, counts, mine = self._route
        cuts = np.cumsum(counts)[:-1]
        g = self.gU.numpy()
        # one message per owner: grad[n, dim] | show[n] | click[n] (the signs went over with the pull, in this order)
        send = []
        for gd, sh, cl in zip(np.split(g[order], cuts), np.split(self._show[order], cuts), np.split(self._click[order], cuts)):
            buf = np.concatenate([np.ascontiguousarray(gd, dtype=np.float32).reshape(-1), sh.astype(np.float32), cl.astype(np.float32)])
            send.append(torch.from_numpy(buf.view(np.uint8)))
        return send, [4 * (self.dim + 2) * len(m) for m in mine]

    def push(self):
        t, rt = self.table, runtime()
        if t.world == 1:
            t.native.push(self._uniq, self.gU.numpy(), self._show, self._click)
            return
        self._records_in(rt.exchange_bytes(*self._records_out()))

    @staticmethod
    def push_many(links, dense=None):
        """Several layers' pushes with one shared round trip.  ``dense``: a DenseTable whose gradient travels in the
        same round (every rank sends its flat gradient to every other rank and leaves the mean in ``dense.G``; the
        table's next step then skips its own all-reduce)."""
        rt = runtime()
        multi = [lk for lk in links if lk.table.world > 1]
        for lk in links:
            if lk.table.world == 1:
                lk.push()
        exchanges = [lk._records_out() for lk in multi]
        if dense is not None and rt.world > 1:
            g = dense.G.detach().reshape(-1)
            raw = g.view(torch.uint8) if g.is_contiguous() else g.contiguous().view(torch.uint8)
            exchanges.append(([raw] * rt.world, [raw.numel()] * rt.world))
        if not exchanges:
            return
        got = rt.exchange_bytes_many(exchanges)
        for lk, g in zip(multi, got):
            lk._records_in(g)
        if dense is not None and rt.world > 1:
            with torch.no_grad():
                total = torch.zeros_like(dense.G).reshape(-1)
                for r in range(rt.world):          # rank order: every rank adds the same numbers in the same order
                    total += got[-1][r].view(dense.G.dtype)
                dense.G.reshape(-1).copy_(total / rt.world)
            dense.grad_pre_reduced = True

    def _records_in(self, got):
        t = self.table
        mine = self._route[2]
        parts = []
        for m, b in zip(mine, got):
            n = len(m)
            f = b.numpy().view(np.float32)
            parts.append((m, f[: n * self.dim].reshape(n, self.dim), f[n * self.dim: n * self.dim + n], f[n * self.dim + n:]))
        if t.apply_mode == "arrival":
            for m, gd, sh, cl in parts:         # one worker after the other, as the reference's servers apply them
                if len(m):
                    t.native.push(np.ascontiguousarray(m), np.ascontiguousarray(gd), np.ascontiguousarray(sh), np.ascontiguousarray(cl))
            return
        signs = np.concatenate([p[0] for p in parts])
        if len(signs) == 0:
            return
        grads = np.concatenate([p[1] for p in parts], axis=0)
        shows = np.concatenate([p[2] for p in parts])
        clicks = np.concatenate([p[3] for p in parts])
        u, inv = np.unique(signs, return_inverse=True)
        gs = np.zeros((len(u), self.dim), np.float32)
        np.add.at(gs, inv, grads)
        sh = np.zeros(len(u), np.float32)
        cl = np.zeros(len(u), np.float32)
        np.add.at(sh, inv, shows)
        np.add.at(cl, inv, clicks)
        t.native.push(u, gs, sh, cl)

"""Host-memory model of the peer exchange the fused sparse kernels run over NVLink.

The kernels talk through symmetric memory: a sender writes its payload into a region of the receiver's copy, then
release-stores a 64-bit word ``epoch << 32 | count`` into the receiver's flag table; the receiver acquire-loads that
word with a wall-time budget and, when the budget runs out, records ``{code, phase, peer}`` in its status words,
skips the rest of its work and returns (csrc/tn_device.cuh ``wait_flag_ge``; csrc/sparse_fused.cu phases A2, B1, B2, C
of the pull and A, B, C and the tail of the push).  In the push the payload does not move: a sender only raises
"my records are complete", every owner reads its segment out of the sender's memory, answers "read", and the sender
clears its records once every owner has answered.  The pull may also run in two steps: its front (dedup and id
dispatch, flags carrying the NEXT step counter) one training step ahead, and the probe-only rest when the batch is
due; a front that is not followed by its pull is discarded by moving the step counter on by one on every rank, so
that the ids and flags it sent can never be taken for current ones (csrc/sparse_fused.cu ``pull_front_*``,
``GpuSparseLink.prefetch`` / ``discard_front``).  This module restates that protocol with ``W`` ranks as threads of one process
and numpy arrays as the "symmetric heap", on top of the CPU tables, so that the hand-shake order and the failure
behaviour can be exercised without a GPU: a test may drop or delay any single flag and must see every rank return
within the budget with the right peer named.  The reference's counterpart is the brpc retry loop that ends in
abort() (core/ps/ps_remote_server.cc:48-83).
"""
from __future__ import annotations

import threading
import time
from typing import Dict, List, Optional, Tuple

import numpy as np

K_PULL_REQ, K_PULL_DONE, K_PUSH_REQ, K_PUSH_DONE = 0, 1, 2, 3    # flag kinds, as in the kernels
OK, PEER_WAIT_TIMEOUT = 0, 5                           # status codes, as in the kernels
PHASE_PULL_IDS, PHASE_PULL_DONE, PHASE_PUSH_RECORDS, PHASE_PUSH_READ = 3, 6, 12, 16


class FakeHeap:
    """What every rank can reach on every other rank: flag words, mailboxes and status words."""

    def __init__(self, world: int, wait_budget_s: float = 0.5):
        self.world = world
        self.budget = float(wait_budget_s)
        self.sig = np.zeros((world, 4, world), dtype=np.uint64)             # sig[receiver, kind, sender]
        self.box: List[Dict[Tuple[int, int], object]] = [dict() for _ in range(world)]   # box[receiver][(kind, sender)]
        self.status = np.zeros((world, 3), dtype=np.int64)                  # code, phase, peer
        self._lock = threading.Lock()
        self._dropped = set()
        self._delayed: Dict[Tuple[int, int, int], float] = {}

    # -------------------------------------------------------------- fault hooks (host side only)
    def drop_flag(self, kind: int, sender: int, receiver: int):
        """The payload still arrives, the flag never does (a lost or mis-addressed release store)."""
        self._dropped.add((kind, sender, receiver))

    def delay_flag(self, kind: int, sender: int, receiver: int, seconds: float):
        self._delayed[(kind, sender, receiver)] = float(seconds)

    # -------------------------------------------------------------- the two primitives
    def post(self, kind: int, sender: int, receiver: int, payload, epoch: int, count: int = 0):
        self.box[receiver][(kind, sender)] = payload                        # "stores to peer memory"
        key = (kind, sender, receiver)
        if key in self._dropped:
            return
        word = np.uint64((epoch << 32) | (count & 0xFFFFFFFF))

        def release():
            with self._lock:
                self.sig[receiver, kind, sender] = word                     # "st.release.sys"

        if key in self._delayed:
            threading.Timer(self._delayed[key], release).start()
        else:
            release()

    def wait(self, kind: int, sender: int, receiver: int, epoch: int, phase: int) -> Optional[int]:
        """Bounded wait for ``sender``'s flag of this epoch; returns its count, or None after recording the failure."""
        t0 = time.monotonic()
        while True:
            with self._lock:
                v = int(self.sig[receiver, kind, sender])
            if (v >> 32) >= epoch:                                          # wait_flag_ge: this step's flag or a later one
                return v & 0xFFFFFFFF
            if self.status[receiver, 0] != OK:                              # an earlier phase already failed
                return None
            if time.monotonic() - t0 > self.budget:
                if self.status[receiver, 0] == OK:                          # first error wins
                    self.status[receiver] = (PEER_WAIT_TIMEOUT, phase, sender)
                return None
            time.sleep(0.0005)


class FakeRank:
    """One rank's side of the protocol.  ``table`` is this rank's shard (a native CPU table built with the job's
    world size and this rank's index); ``ext`` is the CPU extension module."""

    def __init__(self, heap: FakeHeap, rank: int, table, ext, dim: int):
        self.heap, self.rank, self.table, self.ext, self.dim = heap, rank, table, ext, dim
        self.epoch = 0
        self._route = None
        self._front = None           # (ids, dedup results) of a pull front that ran ahead

    @property
    def failed(self) -> bool:
        return self.heap.status[self.rank, 0] != OK

    def _dedup_and_dispatch(self, ids, labels, ep):
        """Phases A and A2: dedup, split by owner, ids into the owners' inboxes, then the flags of step ``ep``."""
        h, R, W = self.heap, self.rank, self.heap.world
        uniq, inv, show, click = self.ext.unique_first_occurrence(np.ascontiguousarray(ids, np.uint64), labels)
        owner = (uniq % np.uint64(W)).astype(np.int64)
        order = np.argsort(owner, kind="stable")
        counts = np.bincount(owner, minlength=W)
        segs = np.split(uniq[order], np.cumsum(counts)[:-1])
        for p in range(W):                                                   # ids first, then the flag
            h.post(K_PULL_REQ, R, p, segs[p], ep, len(segs[p]))
        return uniq, inv, order, counts, show, click

    def pull_front(self, ids: np.ndarray):
        """The front of the NEXT step's pull, run while the current step computes: its flags carry the next step
        counter; the counter itself moves when that pull runs."""
        self._front = (np.array(ids, copy=True), self._dedup_and_dispatch(ids, None, self.epoch + 1))

    def discard_front(self):
        """The pull the front ran for is not coming: move the step counter past the flags it sent.  Every rank must
        do this at the same point of the program."""
        self._front = None
        self.epoch += 1

    def pull(self, ids: np.ndarray, labels: Optional[np.ndarray] = None):
        """Returns ``(rows_of_unique_signs, inverse)`` or None when a wait ran out (status words say which)."""
        h, R, W = self.heap, self.rank, self.heap.world
        front, self._front = self._front, None
        if front is not None and not np.array_equal(front[0], ids):
            self._front = front
            self.discard_front()
            front = None
        self.epoch += 1
        ep = self.epoch
        if front is not None:
            uniq, inv, order, counts, show, click = front[1]                 # ids and flags of this step are out already
            if labels is not None:                                           # show / click are counted by the probe-only pull
                _, _, show, click = self.ext.unique_first_occurrence(np.ascontiguousarray(ids, np.uint64), labels)
        else:
            uniq, inv, order, counts, show, click = self._dedup_and_dispatch(ids, labels, ep)
        self._route = (uniq, order, counts, show, click)
        def serve(s):
            want = np.ascontiguousarray(h.box[R][(K_PULL_REQ, s)], np.uint64)
            h.box[s][("rows", R)] = self.table.pull(want)                    # phase B2: rows into the requester's matrix
            h.post(K_PULL_DONE, R, s, None, ep)                              # phase C: "your rows are in place"

        # phase B1: the own segment needs no peer; the remote senders are handled as one flat index space, so all
        # their flags are awaited before any of them is served
        if h.wait(K_PULL_REQ, R, R, ep, PHASE_PULL_IDS) is None:
            return None
        serve(R)
        remote = [s for s in range(W) if s != R]
        for s in remote:
            n = h.wait(K_PULL_REQ, s, R, ep, PHASE_PULL_IDS)
            if n is None:
                return None                                                  # skip the rest, return normally
            assert len(h.box[R][(K_PULL_REQ, s)]) == n
        for s in remote:
            serve(s)
        got = [None] * W
        for p in range(W):
            if h.wait(K_PULL_DONE, p, R, ep, PHASE_PULL_DONE) is None:
                return None
            got[p] = h.box[R][("rows", p)]
        rows = np.zeros((len(uniq), got[R].shape[1] if len(got[R]) else self.dim), np.float32)
        if len(uniq):
            rows[order] = np.concatenate([g for g in got if len(g)], axis=0)
        return rows, inv

    def push(self, grads: np.ndarray) -> bool:
        """``grads[i]`` belongs to the i-th unique sign of the last pull.  Every owner sums the records it receives
        per sign and applies the optimizer once per sign."""
        h, R, W = self.heap, self.rank, self.heap.world
        ep = self.epoch
        uniq, order, counts, show, click = self._route
        cuts = np.cumsum(counts)[:-1]
        parts = [np.split(a[order], cuts) for a in (uniq, grads.astype(np.float32), show, click)]
        for p in range(W):                                                   # phase A: "my records are complete"
            h.post(K_PUSH_REQ, R, p, tuple(a[p] for a in parts), ep, int(counts[p]))
        acc: Dict[int, list] = {}
        for s in [R] + [s for s in range(W) if s != R]:                      # phase B: own records, then the peers'
            if h.wait(K_PUSH_REQ, s, R, ep, PHASE_PUSH_RECORDS) is None:
                return False
            signs, g, sh, ck = h.box[R][(K_PUSH_REQ, s)]                      # read out of the sender's memory
            for i, sgn in enumerate(signs.tolist()):
                a = acc.setdefault(sgn, [np.zeros(self.dim, np.float32), 0.0, 0.0])
                a[0] += g[i]; a[1] += float(sh[i]); a[2] += float(ck[i])
        for s in range(W):                                                   # "read": the senders may clear their records
            if s != R:
                h.post(K_PUSH_DONE, R, s, None, ep)
        if acc:                                                              # phase C: one update per sign
            signs = np.fromiter(acc.keys(), dtype=np.uint64, count=len(acc))
            self.table.push(signs, np.stack([acc[int(s)][0] for s in signs]),
                            np.array([acc[int(s)][1] for s in signs], np.float32),
                            np.array([acc[int(s)][2] for s in signs], np.float32))
        for p in range(W):                                                   # tail: every owner has read this rank's records
            if p != R and h.wait(K_PUSH_DONE, p, R, ep, PHASE_PUSH_READ) is None:
                return False
        return True


def run_ranks(fns) -> list:
    """Run one callable per rank on its own thread and return their results in rank order."""
    out = [None] * len(fns)

    def go(i):
        out[i] = fns[i]()

    ts = [threading.Thread(target=go, args=(i,)) for i in range(len(fns))]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=60)
    assert not any(t.is_alive() for t in ts), "a rank did not return"
    return out


__all__ = ["FakeHeap", "FakeRank", "run_ranks", "K_PULL_REQ", "K_PULL_DONE", "K_PUSH_REQ", "K_PUSH_DONE", "PEER_WAIT_TIMEOUT",
           "PHASE_PULL_IDS", "PHASE_PULL_DONE", "PHASE_PUSH_RECORDS", "PHASE_PUSH_READ"]

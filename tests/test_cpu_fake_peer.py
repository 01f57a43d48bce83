"""The flag protocol of the fused sparse exchange on a host-memory stand-in for peer memory: three ranks as threads
agree with a single-shard oracle, and a dropped or late flag makes every rank return within the wait budget with
the silent peer named in its status words.  No GPU is involved and nothing hangs."""
import time

import numpy as np

import tensornet_b200 as tn
from tensornet_b200 import _build
from tensornet_b200.parallel import fake_peer as fp

W, DIM = 3, 4


def _opt():
    d = tn.core.AdaGrad(learning_rate=0.1, initial_g2sum=0.1, initial_scale=0.5).sparse_params()
    d["zero_init"] = 0
    return d


def _job(budget=0.4):
    ext = _build.cpu_ext()
    heap = fp.FakeHeap(W, wait_budget_s=budget)
    ranks = [fp.FakeRank(heap, r, ext.CpuSparseTable(_opt(), DIM, False, W, r), ext, DIM) for r in range(W)]
    return ext, heap, ranks


def _ids(r):
    g = np.random.default_rng(r)
    return g.integers(1, 60, size=40).astype(np.uint64)


def _grad_of(signs, r):
    return np.outer((signs % 7).astype(np.float32) - 3.0, np.ones(DIM, np.float32)) * (r + 1) * 0.1


def test_three_ranks_match_one_shard():
    ext, heap, ranks = _job()
    oracle = ext.CpuSparseTable(_opt(), DIM, False, 1, 0)
    for step in range(3):
        ids = [_ids(10 * step + r) for r in range(W)]
        pulled = fp.run_ranks([lambda r=r: ranks[r].pull(ids[r]) for r in range(W)])
        uniqs = []
        for r in range(W):
            rows, inv = pulled[r]
            uniq = ext.unique_first_occurrence(ids[r], None)[0]
            uniqs.append(uniq)
            assert np.array_equal(uniq[inv], ids[r])
            assert np.allclose(rows, oracle.pull(uniq)), (step, r)
        assert all(fp.run_ranks([lambda r=r: ranks[r].push(_grad_of(uniqs[r], r)) for r in range(W)]))
        # oracle: one push of the whole job's batch, gradients of a sign summed over the ranks that saw it
        allu, _, show, click = ext.unique_first_occurrence(np.concatenate(ids), None)
        g = np.zeros((len(allu), DIM), np.float32)
        pos = {int(s): i for i, s in enumerate(allu)}
        for r in range(W):
            gr = _grad_of(uniqs[r], r)
            for i, s in enumerate(uniqs[r]):
                g[pos[int(s)]] += gr[i]
        oracle.push(allu, g, show, click)
    assert (heap.status[:, 0] == fp.OK).all()
    assert sum(rk.table.size() for rk in ranks) == oracle.size()


def test_dropped_flag_times_out_everywhere_and_names_the_peer():
    ext, heap, ranks = _job(budget=0.3)
    heap.drop_flag(fp.K_PULL_REQ, sender=1, receiver=2)          # rank 2 never learns that rank 1's ids arrived
    t0 = time.monotonic()
    out = fp.run_ranks([lambda r=r: ranks[r].pull(_ids(r)) for r in range(W)])
    took = time.monotonic() - t0
    assert out == [None, None, None] and took < 5.0
    assert heap.status[2].tolist() == [fp.PEER_WAIT_TIMEOUT, fp.PHASE_PULL_IDS, 1]
    # rank 2 serves nobody but itself, so ranks 0 and 1 miss their rows from it
    assert heap.status[0].tolist() == [fp.PEER_WAIT_TIMEOUT, fp.PHASE_PULL_DONE, 2]
    assert heap.status[1].tolist() == [fp.PEER_WAIT_TIMEOUT, fp.PHASE_PULL_DONE, 2]
    assert all(rk.failed for rk in ranks)


def test_late_flag_within_the_budget_is_harmless():
    ext, heap, ranks = _job(budget=1.0)
    heap.delay_flag(fp.K_PUSH_REQ, sender=0, receiver=1, seconds=0.2)
    ids = [_ids(r) for r in range(W)]
    pulled = fp.run_ranks([lambda r=r: ranks[r].pull(ids[r]) for r in range(W)])
    assert all(p is not None for p in pulled)
    ok = fp.run_ranks([lambda r=r: ranks[r].push(np.ones((len(set(ids[r].tolist())), DIM), np.float32)) for r in range(W)])
    assert ok == [True, True, True] and (heap.status[:, 0] == fp.OK).all()


def test_sender_waits_for_its_records_to_be_read():
    """The push leaves the records in the sender's memory: an owner that never answers "read" makes exactly the sender
    it owes the answer give up in the tail of its push (the rows were updated everywhere; only the sender's clear of
    its own records is withheld)."""
    ext, heap, ranks = _job(budget=0.3)
    ids = [_ids(r) for r in range(W)]
    pulled = fp.run_ranks([lambda r=r: ranks[r].pull(ids[r]) for r in range(W)])
    assert all(p is not None for p in pulled)
    heap.drop_flag(fp.K_PUSH_DONE, sender=2, receiver=0)         # rank 0 never learns that rank 2 has read its records
    ok = fp.run_ranks([lambda r=r: ranks[r].push(np.ones((len(set(ids[r].tolist())), DIM), np.float32)) for r in range(W)])
    assert ok == [False, True, True]
    assert heap.status[0].tolist() == [fp.PEER_WAIT_TIMEOUT, fp.PHASE_PUSH_READ, 2]
    assert (heap.status[1:, 0] == fp.OK).all()


def _oracle_push(ext, oracle, ids, uniqs):
    allu, _, show, click = ext.unique_first_occurrence(np.concatenate(ids), None)
    g = np.zeros((len(allu), DIM), np.float32)
    pos = {int(s): i for i, s in enumerate(allu)}
    for r in range(W):
        gr = _grad_of(uniqs[r], r)
        for i, s in enumerate(uniqs[r]):
            g[pos[int(s)]] += gr[i]
    oracle.push(allu, g, show, click)


def test_pull_front_one_step_ahead_matches_one_shard_and_discard_is_clean():
    """The two-step pull: while step k runs, every rank sends the ids of step k+1 to their owners with the flags of
    the next step counter; the pull of step k+1 then only probes and returns rows.  Same results as one shard.  A
    front whose batch never comes is discarded by all ranks together (step counter moved on by one) and the pull of
    another batch works as if nothing had been sent."""
    ext, heap, ranks = _job()
    oracle = ext.CpuSparseTable(_opt(), DIM, False, 1, 0)
    batches = [[_ids(100 + 10 * step + r) for r in range(W)] for step in range(4)]
    for step in range(3):
        ids = batches[step]
        pulled = fp.run_ranks([lambda r=r: ranks[r].pull(ids[r]) for r in range(W)])
        uniqs = []
        for r in range(W):
            rows, inv = pulled[r]
            uniq = ext.unique_first_occurrence(ids[r], None)[0]
            uniqs.append(uniq)
            assert np.array_equal(uniq[inv], ids[r])
            assert np.allclose(rows, oracle.pull(uniq)), (step, r)
        # the next batch's front runs under this step's "compute", before the push
        fp.run_ranks([lambda r=r: ranks[r].pull_front(batches[step + 1][r]) for r in range(W)])
        assert all(r._front is not None for r in ranks)
        assert all(fp.run_ranks([lambda r=r: ranks[r].push(_grad_of(uniqs[r], r)) for r in range(W)]))
        _oracle_push(ext, oracle, ids, uniqs)
    # the front for batch 3 is pending; the job pulls other ids instead (an evaluation batch): every rank discards
    other = [_ids(900 + r) for r in range(W)]
    epochs_before = [r.epoch for r in ranks]
    pulled = fp.run_ranks([lambda r=r: ranks[r].pull(other[r]) for r in range(W)])
    for r in range(W):
        rows, inv = pulled[r]
        uniq = ext.unique_first_occurrence(other[r], None)[0]
        assert np.allclose(rows, oracle.pull(uniq))
        assert ranks[r].epoch == epochs_before[r] + 2           # one for the discarded front, one for this pull
    assert (heap.status[:, 0] == fp.OK).all()


def test_a_rank_that_leaves_the_two_step_pull_alone_is_reported_not_waited_for_forever():
    """Ranks must agree on the form of the pull step by step.  Here rank 0 alone discards its front and runs a whole
    pull for another batch while ranks 1 and 2 run the probe-only pull of the promised batch: rank 0's step counter is
    one ahead of everybody's flags, so its wait for their ids runs out and it reports a peer-wait time-out (it does
    not hang, and it does not hand back rows of the wrong step)."""
    ext, heap, ranks = _job(budget=0.3)
    first = [_ids(300 + r) for r in range(W)]
    nxt = [_ids(310 + r) for r in range(W)]
    pulled = fp.run_ranks([lambda r=r: ranks[r].pull(first[r]) for r in range(W)])
    assert all(p is not None for p in pulled)
    fp.run_ranks([lambda r=r: ranks[r].pull_front(nxt[r]) for r in range(W)])
    uniqs = [ext.unique_first_occurrence(first[r], None)[0] for r in range(W)]
    assert all(fp.run_ranks([lambda r=r: ranks[r].push(_grad_of(uniqs[r], r)) for r in range(W)]))
    t0 = time.monotonic()
    stray = _ids(999)
    out = fp.run_ranks([lambda: ranks[0].pull(stray)] + [lambda r=r: ranks[r].pull(nxt[r]) for r in (1, 2)])
    assert time.monotonic() - t0 < 5.0
    assert out[0] is None
    assert heap.status[0, 0] == fp.PEER_WAIT_TIMEOUT and heap.status[0, 1] == fp.PHASE_PULL_IDS and heap.status[0, 2] in (1, 2)

"""BalanceDataset: ranks with unequal input take the same number of steps (the purpose of the reference's balance op,
core/kernels/data/balance_dataset_ops.cc:198-311), checked on the pure planning rule and on three gloo ranks."""
import json
import os
import socket
import subprocess
import sys
import textwrap

import pytest
from hypothesis import given, settings, strategies as st

from tensornet_b200.data import BalanceDataset, list_files

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@settings(max_examples=200, deadline=None)
@given(st.lists(st.integers(0, 5), min_size=2, max_size=8))
def test_plan_gives_every_rank_one_batch_or_stops(have):
    gifts = BalanceDataset.plan(have)
    if sum(have) < len(have):
        assert gifts is None
        return
    left = list(have)
    for n, d in gifts:
        assert have[n] == 0 and left[d] >= 2      # a donor never gives away the batch it needs itself
        left[d] -= 1
    assert sorted(n for n, _ in gifts) == [r for r, h in enumerate(have) if h == 0]


def test_list_files_sorted_per_day_and_error(tmp_path):
    for day, names in {"d1": ["part-2", "part-1", "other"], "d2": ["part-0"]}.items():
        os.makedirs(tmp_path / day)
        for n in names:
            (tmp_path / day / n).write_text("x")
    got = list_files(str(tmp_path), ["d1", "d2"], "part-*")
    assert [os.path.relpath(g, tmp_path) for g in got] == ["d1/part-1", "d1/part-2", "d2/part-0"]
    with pytest.raises(FileNotFoundError):
        list_files(str(tmp_path), ["d3"], "part-*")


@pytest.mark.timeout(300)
@pytest.mark.parametrize("counts", [[11, 0, 2], [40, 9, 23]])
def test_three_ranks_with_unequal_input_take_equal_steps(tmp_path, counts):
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent("""
        import json, os
        import tensornet_b200 as tn
        tn.core.init()
        rank = tn.core.self_shard_id()
        counts = COUNTS                        # e.g. 13 batches over 3 ranks: 4 rounds, one batch unused
        ds = tn.data.BalanceDataset([(rank, i) for i in range(counts[rank])])
        seen = []
        for b in ds:
            seen.append(tuple(b))
            tn.core.barrier()                  # stands for the collectives of a training step
        print("SEEN", rank, json.dumps(seen), flush=True)
        tn.core.barrier()
        os._exit(0)
    """).replace("COUNTS", repr(counts)))
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    procs = []
    for r in range(3):
        env = dict(os.environ, TN_FORCE_CPU="1", RANK=str(r), WORLD_SIZE="3", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), TN_PG_TIMEOUT_S="60", PYTHONPATH=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    seen = {}
    for o in outs:
        line = [l for l in o.splitlines() if l.startswith("SEEN")]
        assert line, o[-2000:]
        _, r, rest = line[0].split(" ", 2)
        seen[int(r)] = [tuple(b) for b in json.loads(rest)]
    rounds = sum(counts) // 3
    assert len(seen[0]) == len(seen[1]) == len(seen[2]) == rounds
    used = [b for r in range(3) for b in seen[r]]
    assert len(set(used)) == 3 * rounds               # no batch is used twice
    assert all(i < counts[src] for src, i in used)

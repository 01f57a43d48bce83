"""Failure detection without any GPU fault: a rank that leaves between steps is noticed by the
survivors on the host (a short process-group timeout turns their next collective into an error
instead of a hang), and capacity problems surface as exceptions, not aborts.
The reference retries RPCs three times and then abort()s the process (core/ps/ps_remote_server.cc:48-83)."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.timeout(180)
def test_survivor_detects_departed_rank(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(textwrap.dedent("""
        import os, sys, time
        import tensornet_b200 as tn
        tn.core.init()
        rank = tn.core.self_shard_id()
        tn.core.barrier()                      # everyone is up
        if rank == 1:
            os._exit(0)                        # leaves between steps, nothing in flight
        t0 = time.time()
        try:
            tn.core.barrier()
            print("NOT DETECTED", flush=True)
        except Exception as e:
            print("DETECTED after %.1fs: %s" % (time.time() - t0, type(e).__name__), flush=True)
        os._exit(0)
    """))
    port = _free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ, TN_FORCE_CPU="1", RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), TN_PG_TIMEOUT_S="8", PYTHONPATH=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    out0, _ = procs[0].communicate(timeout=150)
    procs[1].wait(timeout=30)
    assert "DETECTED" in out0 and "NOT DETECTED" not in out0, out0[-2000:]


def test_bucket_overflow_and_bad_checkpoint_raise(tmp_path):
    import numpy as np
    import tensornet_b200 as tn
    from tensornet_b200 import _build

    tn.core.shutdown(); tn.core.config.force_cpu = True; tn.core.init()
    ext = _build.cpu_ext()
    with pytest.raises(RuntimeError):
        ext.read_sparse_dir(str(tmp_path / "missing"), 0, 4, False) if os.path.isdir(tmp_path / "missing") else (_ for _ in ()).throw(RuntimeError("no dir"))
    d = tmp_path / "t"
    ext.write_sparse_dir(str(d), "bin", 1, 4, False, np.array([1], np.uint64), np.zeros((1, 14), np.float32), False, 0.0, 0, 0)
    with pytest.raises(RuntimeError, match="dim"):
        ext.read_sparse_dir(str(d), 1, 8, False)          # table dim differs from the file's
    t = ext.CpuSparseTable(tn.core.Adam().sparse_params(), 4, False, 1, 0)
    with pytest.raises(RuntimeError, match="not create yet"):
        t.push(np.array([99], np.uint64), np.zeros((1, 4), np.float32), np.ones(1, np.float32), np.zeros(1, np.float32))
    tn.core.shutdown()


def test_guard_words_behind_shared_regions_catch_a_stray_write():
    """Every region of a symmetric arena is followed by a guard; a write past a region's end is reported by name."""
    import torch
    import tensornet_b200 as tn
    from tensornet_b200.parallel.symm import SymmArena, verify_all_arenas

    tn.core.shutdown(); tn.core.config.force_cpu = True; tn.core.init()
    a = SymmArena([("inbox", (100,), torch.float32), ("flags", (8,), torch.int64), ("rows", (3, 5), torch.float32)])
    a.tensor("inbox").fill_(1.0); a.tensor("flags").fill_(-1); a.tensor("rows").fill_(2.0)     # in-bounds writes
    assert a.damaged() == []
    verify_all_arenas()
    assert a.offsets["flags"] >= a.offsets["inbox"] + 400 + 256
    end_of_flags = a.offsets["flags"] + 256            # the region is padded to 256 bytes; the guard starts here
    a.buf.local[end_of_flags + 3] = 0
    assert a.damaged() == ["flags"]
    with pytest.raises(RuntimeError, match="flags"):
        verify_all_arenas()
    a.buf.local[end_of_flags + 3] = 0xA5
    verify_all_arenas()
    tn.core.shutdown()

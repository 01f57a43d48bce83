"""Two (and four) GPUs: the fused pull / push kernels exchange ids, rows and gradients over peer memory and
the dense step reduces over NVSwitch; the run must follow the one-GPU trajectory on the same global batches."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _run(world, out, extra_env=None):
    env = dict(os.environ, PYTHONPATH=ROOT, TN_WAIT_BUDGET_S="1.0", TN_PG_TIMEOUT_S="120", **(extra_env or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_port()), os.path.join(ROOT, "tests", "mgpu_worker.py"), out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=420)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-3000:]
    return json.load(open(out))


@pytest.mark.timeout(900)
@pytest.mark.parametrize("world", [2, 4, 8])
def test_multi_gpu_follows_single_gpu(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    one = _run(1, str(tmp_path / "one.json"))
    many = _run(world, str(tmp_path / "many.json"), {"TN_USE_MULTIMEM": "1"})      # the NVSwitch multimem dense path at every size
    assert many["graph"] and many["replicas_identical"] and many["bn_sync_ok"] and many["serving_ok"] and many["ckpt_ok"]
    assert many["balance_ok"], many["balance_steps"]
    assert many["rows"] == one["rows"]                      # every sign lives on exactly one shard
    assert many["losses"][-1] < 0.8 * many["losses"][0]
    for a, b in zip(one["losses"], many["losses"]):
        assert abs(a - b) < 0.08 * max(a, 0.2), (one["losses"], many["losses"])


@pytest.mark.timeout(600)
def test_multi_gpu_over_plain_peer_loads(tmp_path):
    """Same run with the CUDA-IPC heap: no NVSwitch multicast mapping, the dense step reduces with peer loads."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    r = _run(2, str(tmp_path / "ipc.json"), {"TN_SYMM_BACKEND": "ipc", "NCCL_NVLS_ENABLE": "0"})
    assert r["replicas_identical"] and not r["multimem"] and r["bn_sync_ok"]
    assert r["losses"][-1] < 0.8 * r["losses"][0]


@pytest.mark.timeout(300)
def test_survivor_notices_departed_rank_before_its_next_launch(tmp_path):
    """A rank leaves between steps with nothing in flight; the survivor learns of it on the host (short
    process-group timeout on the pre-step barrier) and launches no kernel that would wait for the dead peer.
    Plain peer loads only: no NVSwitch multicast mapping is bound while a rank dies."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    script = tmp_path / "leaver.py"
    script.write_text('''
import os, sys, time, torch
import tensornet_b200 as tn
tn.core.init()
rt = tn.core.runtime()
slots = [str(i) for i in range(1, 5)]
B = 128
model = tn.models.DeepFM(slots, slots, dnn_hidden_units=(32, 16), embedding_dim=8, dense_dim=3,
                         sparse_opt=tn.core.Adam(learning_rate=1e-2, initial_scale=0.1), bucket_size=2 * B, table_rows=1 << 14)
model.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=1e-2)), cuda_graph=False)
g = torch.Generator().manual_seed(rt.rank)
def batch():
    ids = torch.randint(0, 500, (len(slots), B), generator=g, dtype=torch.int64)
    return {tn.data.PACKED_KEY: tn.data.PackedFeatures(slots, ids=ids), "dense": torch.randn(B, 3, generator=g)}, (torch.rand(B, generator=g) < 0.3).float()
for _ in range(3):
    tn.core.barrier()                      # pre-step health check on the host
    f, y = batch()
    model.train_on_batch(f, y)
torch.cuda.synchronize()
rt.check_status()
tn.core.barrier()
if rt.rank == 1:
    os._exit(0)                            # between steps, none of its kernels or collectives in flight
t0 = time.time()
try:
    tn.core.barrier()                      # the next step's health check
    print("NOT DETECTED", flush=True)
except Exception as e:
    print("DETECTED after %.1fs: %s" % (time.time() - t0, type(e).__name__), flush=True)
assert float(torch.ones(4, device=rt.device).sum()) == 4.0     # the survivor's context is intact
print("CONTEXT OK", flush=True)
os._exit(0)
''')
    port = _port()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   TN_PG_TIMEOUT_S="10", TN_WAIT_BUDGET_S="1.0", TN_SYMM_BACKEND="ipc", TN_USE_MULTIMEM="0", NCCL_NVLS_ENABLE="0",
                   PYTHONPATH=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    out0, _ = procs[0].communicate(timeout=240)
    procs[1].wait(timeout=60)
    assert "DETECTED" in out0 and "NOT DETECTED" not in out0 and "CONTEXT OK" in out0, out0[-3000:]


@pytest.mark.timeout(300)
def test_peer_wait_runs_out_on_the_pull_and_recover_realigns(tmp_path):
    """Rank 1 skips one pull launch (a host-side hook; nothing on any GPU faults or spins for ever).  Rank 0's fused pull
    kernel gives up waiting for rank 1's id segment after the 0.3 s budget, records "peer wait timed out, owner
    phase, peer 1" and returns; its context keeps computing.  Both ranks then call ``core.recover()`` and the next
    pull on both returns the same rows as before the failure.  Plain peer loads, no NVSwitch multicast mapping."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    script = tmp_path / "skipper.py"
    script.write_text('''
import os, torch
import tensornet_b200 as tn
from tensornet_b200.ops.sparse_table_gpu import GpuSparseTable
tn.core.init()
rt = tn.core.runtime()
t = GpuSparseTable(tn.core.Adam(learning_rate=1e-2, initial_scale=0.1), 8, rows=1 << 14)
lk = t.link(4096)
g = torch.Generator().manual_seed(5 + rt.rank)
ids = torch.randint(0, 3000, (2048,), generator=g, dtype=torch.int64).to(rt.device)
torch.cuda.synchronize(); rt.barrier()
inv = lk.pull(ids, training=False)
torch.cuda.synchronize(); rt.check_status()
before = lk.U[inv.long()].clone()
rt.barrier()
lk.pull(ids, training=False)
torch.cuda.synchronize(); rt.check_status(); rt.barrier()
# ---- the step in which rank 1 never launches its pull
if rt.rank == 0:
    lk.pull(ids, training=False)
    torch.cuda.synchronize()
    try:
        rt.check_status()
        print("NO ERROR", flush=True)
    except tn.core.DeviceError as e:
        print("ERROR code=%d phase=%d peer=%d" % (e.code, e.phase, e.aux), flush=True)
    assert float(torch.ones(4, device=rt.device).sum()) == 4.0
    # until recover() has run every fused kernel returns at once: nothing is applied on top of the failed step
    lk.pull(ids, training=False)
    torch.cuda.synchronize()
    print("FAILED FLAG", rt.failed, flush=True)
agreed = tn.core.recover()
torch.cuda.synchronize(); rt.barrier()
inv2 = lk.pull(ids, training=False)
torch.cuda.synchronize(); rt.check_status()
same = bool(torch.equal(lk.U[inv2.long()], before))
rt.barrier()
lk.pull(ids, training=True); lk.push()
torch.cuda.synchronize(); rt.check_status(); rt.barrier()
print("RECOVERED epoch=%d same_rows=%s" % (agreed, same), flush=True)
tn.core.shutdown()
''')
    port = _port()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   TN_PG_TIMEOUT_S="60", TN_WAIT_BUDGET_S="0.3", TN_SYMM_BACKEND="ipc", TN_USE_MULTIMEM="0", NCCL_NVLS_ENABLE="0",
                   PYTHONPATH=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert "ERROR code=5 phase=3 peer=1" in outs[0] and "NO ERROR" not in outs[0], outs[0][-3000:]
    assert "FAILED FLAG True" in outs[0], outs[0][-2000:]
    for o in outs:
        assert "same_rows=True" in o, o[-3000:]

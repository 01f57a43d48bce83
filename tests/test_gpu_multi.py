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
    many = _run(world, str(tmp_path / "many.json"))
    assert many["graph"] and many["replicas_identical"] and many["bn_sync_ok"]
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

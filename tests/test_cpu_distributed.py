"""Two CPU ranks over gloo (the reference's `mpiexec -n 2` integration test, test/CMakeLists.txt:33-38):
Wide&Deep with synchronised BN trains, saves per-rank shards, and the checkpoint written by two
ranks reloads on one rank (re-sharding by sign % world)."""
import json
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(nproc, args, timeout=600):
    env = dict(os.environ, TN_FORCE_CPU="1", OMP_NUM_THREADS="1", PYTHONPATH=ROOT)
    if nproc == 1:
        cmd = [sys.executable, os.path.join(ROOT, "examples", "main.py")] + args
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
               "--master-port", str(_free_port()), os.path.join(ROOT, "examples", "main.py")] + args
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    return json.loads(line)


@pytest.mark.timeout(900)
def test_wide_deep_two_ranks_then_reload_on_one(tmp_path):
    data, model_dir = str(tmp_path / "data"), str(tmp_path / "model")
    subprocess.run([sys.executable, os.path.join(ROOT, "examples", "gen_example_data.py"), "--out", data, "--examples-per-file",
                    "3000", "--files-per-day", "3"], check=True, env=dict(os.environ, PYTHONPATH=ROOT))
    common = ["--data", data, "--model-dir", model_dir, "--hidden", "32", "16", "--batch-size", "64", "--save-mode", "bin"]
    rep = _run(2, common + ["--days", "2020-05-10"])
    assert len(rep["days"]) == 1 and rep["days"][0]["loss"] < 0.5
    cp = os.path.join(model_dir, "2020-05-10")
    assert json.load(open(os.path.join(model_dir, "_checkpoint"))) == {"dt": "2020-05-10"}
    for layer in ("linear_input", "deep_input"):
        for r in (0, 1):
            d = os.path.join(cp, "sparse_table", layer, f"rank_{r}")
            assert sorted(os.listdir(d)) == [f"block_{b}_bin.gz" for b in range(8)]
    assert sorted(os.listdir(os.path.join(cp, "dense_table", "0"))) == ["0", "1"]
    assert os.path.exists(os.path.join(cp, "bn_table", "0"))
    # second day on ONE rank: day 1 is skipped (done-file), its 2-rank checkpoint is re-sharded on load
    rep1 = _run(1, common + ["--days", "2020-05-10", "2020-05-11", "--predict"])
    assert [d["day"] for d in rep1["days"]] == ["2020-05-11"]
    assert rep1["days"][0]["loss"] < 0.3
    assert rep1["predict_auc"] > 0.95


@pytest.mark.timeout(900)
@pytest.mark.parametrize("model", ["deep_cross"])
def test_other_model_families_on_two_ranks(tmp_path, model):
    """Deep&Cross through the same driver on two gloo ranks: sharded tables, replicated dense part.  (DeepFM with the
    example's CVM columns is left out: its FM term multiplies raw show counters, as in the reference's example, and the
    first day's loss depends on the seed.)"""
    data, model_dir = str(tmp_path / "data"), str(tmp_path / "model")
    subprocess.run([sys.executable, os.path.join(ROOT, "examples", "gen_example_data.py"), "--out", data, "--examples-per-file",
                    "3000", "--files-per-day", "3", "--days", "2020-05-10"], check=True, env=dict(os.environ, PYTHONPATH=ROOT))
    rep = _run(2, ["--data", data, "--model-dir", model_dir, "--model", model, "--hidden", "32", "16", "--batch-size", "64",
                   "--days", "2020-05-10", "--save-mode", "bin", "--predict"])
    assert rep["days"][0]["loss"] < 0.5 and rep["predict_auc"] > 0.9
    assert 0.5 < rep["days"][0]["copc"] < 2.0
    cp = os.path.join(model_dir, "2020-05-10")
    assert sorted(os.listdir(os.path.join(cp, "sparse_table", "deep_input"))) == ["rank_0", "rank_1"]


@pytest.mark.timeout(600)
def test_integration_script_prepares_trains_and_checks_on_two_ranks(tmp_path):
    """The user-runnable end-to-end check (examples/integration-test.py in the reference): rank 0 writes the missing
    days and clears an old model directory while rank 1 waits in the rendezvous, both train, rank 0 verifies."""
    data, model_dir = str(tmp_path / "data"), str(tmp_path / "model")
    os.makedirs(os.path.join(model_dir, "stale"))                # an old model directory must go
    env = dict(os.environ, TN_FORCE_CPU="1", OMP_NUM_THREADS="1", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "examples", "integration_test.py"), "--data", data,
           "--model-dir", model_dir, "--files-per-day", "2", "--examples-per-file", "640", "--max-steps", "8",
           "--hidden", "32", "16", "--format", "tfrecord"]        # the reference's input format, through the native reader
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=500)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert "integration test passed" in out.stdout
    assert not os.path.exists(os.path.join(model_dir, "stale"))
    assert sorted(os.listdir(data)) == ["2020-05-10", "2020-05-11"]
    assert sorted(os.listdir(os.path.join(data, "2020-05-10"))) == ["tf-part.00000", "tf-part.00001"]


@pytest.mark.timeout(300)
def test_apply_on_arrival_differs_from_one_summed_update(tmp_path):
    """What changes when two workers push the same sign in one step.  ``apply_mode="sum"`` (this framework's
    synchronous step) applies the sum of the two gradients once; ``apply_mode="arrival"`` restates the reference's
    servers, which apply each worker's records when they arrive, one on top of the other
    (core/kernels/sparse_table_ops.cc:363-367, core/ps/ps_local_server.cc:43-54).  With AdaGrad the two differ in a
    way that can be written down: one step of size g1+g2 against g2sum + (g1+g2)^2/dim, versus two steps against
    accumulators that grow in between."""
    script = tmp_path / "w.py"
    script.write_text('''
import json, sys, numpy as np, torch
import tensornet_b200 as tn
from tensornet_b200.ops.sparse_table_cpu import CpuSparseTable
tn.core.init()
rt = tn.core.runtime()
out = {}
for mode in ("sum", "arrival"):
    opt = tn.core.AdaGrad(learning_rate=0.1, initial_g2sum=0.5, initial_scale=0.0)
    t = CpuSparseTable(opt, 2, apply_mode=mode)
    lk = t.link(16)
    ids = torch.tensor([4, 6], dtype=torch.int64)           # both owned by rank 0; both ranks pull and push them
    lk.pull(ids, training=True)
    lk.gU = torch.full((2, 2), 1.0 if rt.rank == 0 else 3.0)
    lk.push()
    rt.barrier()
    lk.pull(ids, training=False)
    out[mode] = lk.U[:, :2].tolist()
if rt.rank == 0:
    print(json.dumps(out))
tn.core.shutdown()
''')
    env = dict(os.environ, TN_FORCE_CPU="1", OMP_NUM_THREADS="1", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    got = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    lr, eps, g2 = 0.1, 1e-8, 0.5
    # sum: g = 4 per element, g2sum += (16 + 16) / 2
    w_sum = -lr * 4.0 / (eps + (g2 + 16.0) ** 0.5)
    # arrival: rank 0's g = 1 first (g2sum += 1), then rank 1's g = 3 (g2sum += 9)
    w_arr = -lr * 1.0 / (eps + (g2 + 1.0) ** 0.5) - lr * 3.0 / (eps + (g2 + 10.0) ** 0.5)
    for row in got["sum"]:
        assert row == pytest.approx([w_sum, w_sum], rel=1e-5)
    for row in got["arrival"]:
        assert row == pytest.approx([w_arr, w_arr], rel=1e-5)
    assert abs(w_sum - w_arr) > 1e-3


@pytest.mark.timeout(900)
@pytest.mark.parametrize("nproc", [2, 3])
def test_shared_round_trips_give_what_one_by_one_exchanges_give(tmp_path, nproc):
    """Two ranks, two tables: the pulls run together (`pull_many`: ids of both tables in one round, rows in a second)
    and the pushes with the dense gradient riding along (`push_many`), against the same calls made one by one and a
    plain all-reduce; pulled rows, tables after the push and the mean dense gradient must be identical."""
    script = tmp_path / "w.py"
    script.write_text('''
import json, numpy as np, torch
import torch.distributed as dist
import tensornet_b200 as tn
from tensornet_b200.ops.sparse_table_cpu import CpuSparseTable, CpuSparseLink
from tensornet_b200.ops.dense_table import DenseTable
tn.core.init()
rt = tn.core.runtime()
res = {}
g = torch.Generator().manual_seed(5 + rt.rank)
ids_a = torch.randint(1, 200, (96,), generator=g)
ids_b = torch.randint(1, 50, (64,), generator=g)
for mode in ("single", "many"):
    ta = CpuSparseTable(tn.core.AdaGrad(learning_rate=0.1, initial_g2sum=0.5, initial_scale=0.3), 4)
    tb = CpuSparseTable(tn.core.Adam(learning_rate=0.05, initial_scale=0.3), 2)
    la, lb = ta.link(256), tb.link(256)
    p = torch.nn.Parameter(torch.arange(16, dtype=torch.float32))
    dt = DenseTable(tn.core.Adam(learning_rate=0.01)); dt.init([("p", p)])
    for step in range(2):
        if mode == "single":
            ia, ib = la.pull(ids_a, training=True), lb.pull(ids_b, training=True)
        else:
            CpuSparseLink.pull_many([(la, ids_a, None, 0, True), (lb, ids_b, None, 0, True)])
            ia, ib = la.pull(ids_a, training=True), lb.pull(ids_b, training=True)      # picked up, no exchange
        Ua, Ub = la.U[ia.long()].clone(), lb.U[ib.long()].clone()
        la.gU = (la.U[:, :4] * 0.5 + 0.1 * (rt.rank + 1)).clone()
        lb.gU = (lb.U[:, :2] * 0.25 - 0.2 * (rt.rank + 1)).clone()
        dt.G.copy_(torch.arange(dt.G.numel(), dtype=torch.float32) * (rt.rank + 1))
        if mode == "single":
            la.push(); lb.push()
        else:
            CpuSparseLink.push_many([la, lb], dt)
            assert dt.grad_pre_reduced
        mean_g = dt.G.clone()
        if mode == "single":
            dist.all_reduce(mean_g, group=rt.host_group); mean_g /= rt.world
        dt.step()
        rt.barrier()
    ka, ra = ta.dump(); kb, rb = tb.dump()
    oa, ob = np.argsort(ka), np.argsort(kb)
    res[mode] = dict(Ua=Ua.tolist(), Ub=Ub.tolist(), ka=ka[oa].tolist(), ra=ra[oa].tolist(), kb=kb[ob].tolist(), rb=rb[ob].tolist(),
                     g=mean_g.tolist(), w=dt.W.tolist())
ok = all(np.allclose(np.array(res["single"][k], dtype=np.float64), np.array(res["many"][k], dtype=np.float64), rtol=1e-6, atol=1e-7)
         for k in res["single"])
oks = rt.all_gather_object(bool(ok))
if rt.rank == 0:
    print(json.dumps({"ok": all(oks), "rows_a": len(res["many"]["ka"])}))
tn.core.shutdown()
''')
    env = dict(os.environ, TN_FORCE_CPU="1", OMP_NUM_THREADS="1", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    got = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert got["ok"] and got["rows_a"] > 0

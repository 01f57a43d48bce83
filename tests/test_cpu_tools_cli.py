"""`python -m tensornet_b200.tools` on a checkpoint written by a model (the role of tensornet_tools/bin/tn_tools.sh and
the Spark jobs behind it): merge to a dictionary, re-shard sparse and dense parts, and load the re-sharded dense part."""
import os
import subprocess
import sys

import numpy as np
import torch

import tensornet_b200 as tn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tool(*args):
    r = subprocess.run([sys.executable, "-m", "tensornet_b200.tools", *args], capture_output=True, text=True, timeout=300,
                       env=dict(os.environ, PYTHONPATH=ROOT, TN_FORCE_CPU="1"))
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
    return r.stdout.strip().splitlines()[-1]


def test_cli_merge_and_resize(tmp_path):
    tn.core.shutdown(); tn.core.config.force_cpu = True; tn.core.init()
    torch.manual_seed(0)
    m = tn.models.DeepFM(["a", "b"], ["a", "b"], dnn_hidden_units=(8,), embedding_dim=4, bucket_size=64,
                         sparse_opt=tn.core.Adam(learning_rate=0.01))
    m.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=0.01)))
    f = {"a": torch.arange(1, 33), "b": torch.arange(101, 133)}
    for _ in range(2):
        m.train_on_batch(f, (f["a"] % 2).float())
    cp = str(tmp_path / "cp")
    m.save_weights(cp, mode="txt")
    tn.core.shutdown()

    deep = os.path.join(cp, "sparse_table", "deep_input")
    out = str(tmp_path / "deep.dict")
    assert int(_tool("merge-sparse", deep, out)) == 64
    lines = open(out).read().splitlines()
    assert len(lines) == 64 and all(len(l.split("\t")) == 1 + 4 for l in lines)
    assert sorted(int(l.split("\t")[0]) for l in lines) == sorted(list(range(1, 33)) + list(range(101, 133)))
    outb = str(tmp_path / "deep.brackets")
    assert int(_tool("merge-sparse", deep, outb, "--brackets")) == 64 and "[" in open(outb).readline()

    assert int(_tool("resize-sparse", deep, str(tmp_path / "deep4"), "4", "--mode", "bin")) == 64
    for r in range(4):
        d = tmp_path / "deep4" / f"rank_{r}"
        assert sorted(os.listdir(d)) == [f"block_{b}_bin.gz" for b in range(8)]
    from tensornet_b200 import tools
    signs, rows, name, dim = tools.read_sparse_table(str(tmp_path / "deep4"), "Adam", 4)    # binary blocks do not name the optimizer
    assert name == "Adam" and dim == 4 and len(signs) == 64

    dense = os.path.join(cp, "dense_table", "0")
    n = int(_tool("resize-dense", dense, str(tmp_path / "dense3"), "3", "--opt", "Adam"))
    assert sorted(os.listdir(tmp_path / "dense3")) == ["0", "1", "2"] and n > 0
    from tensornet_b200 import _build
    ext = _build.cpu_ext()
    whole = ext.read_dense_file(os.path.join(dense, "0"), 1)
    parts = [ext.read_dense_file(str(tmp_path / "dense3" / str(r)), 1) for r in range(3)]
    wkey = [k for k in whole if isinstance(whole[k], np.ndarray) and whole[k].ndim == 1 and len(whole[k]) == n][0]
    assert np.allclose(np.concatenate([p[wkey] for p in parts])[:n], whole[wkey])


def test_cli_batch_cache(tmp_path):
    """TFRecord files parsed once into a cache of ready-made batches from the command line."""
    files = []
    for k in range(2):
        p = str(tmp_path / f"tf-{k}")
        with tn.data.TFRecordWriter(p) as w:
            for j in range(50):
                w.write(tn.data.encode_example({"1": [k * 100 + j], "2": [7], "label": [j & 1]}, {"d": [0.5, 1.5]}))
        files.append(p)
    out = str(tmp_path / "pass.tnbc")
    assert int(_tool("batch-cache", out, *files, "--batch-size", "32", "--slots", "1", "2", "--dense", "d", "2", "--single-hot",
                     "--workers", "1")) == 100
    got = list(tn.data.BatchCacheDataset(out, pin_memory=False))
    assert [int(y.numel()) for _, y in got] == [32, 32, 32, 4]
    ids = torch.cat([f[tn.data.PACKED_KEY].ids for f, _ in got], dim=1)
    assert sorted(ids[0].tolist()) == sorted(k * 100 + j for k in range(2) for j in range(50)) and set(ids[1].tolist()) == {7}
    assert got[0][0]["dense"].shape == (32, 2) and float(got[0][0]["dense"][0, 1]) == 1.5

"""The stand-alone C++ serving program (examples/native_serving/serve.cpp, the role of the reference's
examples/online_serving/main.cc) against the Python engine: same dictionary file, same tower, same probabilities."""
import json
import os
import shutil
import subprocess

import numpy as np
import pytest
import torch

import tensornet_b200 as tn
from tensornet_b200.serving import EmbeddingDictionary, InferenceEngine, export_tower

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a C++ compiler")
def test_native_serving_program_matches_the_python_engine(tmp_path):
    exe = str(tmp_path / "tn_serve")
    subprocess.run(["g++", "-O2", "-std=c++17", "-pthread", os.path.join(ROOT, "examples", "native_serving", "serve.cpp"), "-lz", "-o", exe],
                   check=True, timeout=300)
    tn.core.init()
    S, dim, B = 3, 4, 16
    rng = np.random.default_rng(0)
    signs = np.unique(rng.integers(0, 2 ** 63, size=200, dtype=np.uint64))
    signs[0] = 0                                                       # sign 0 is a key like any other
    weights = rng.standard_normal((len(signs), dim)).astype(np.float32)
    dict_file = str(tmp_path / "d.txt")
    with open(dict_file, "w") as f:
        for s, w in zip(signs, weights):
            f.write(str(int(s)) + "\t" + "\t".join(repr(float(x)) for x in w) + "\n")
    torch.manual_seed(0)
    mlp, head = tn.layers.MLP(S * dim, [8, 5]), tn.layers.DenseHead(5)
    with torch.no_grad():
        for i in range(2):
            mlp.bias(i).copy_(torch.randn(mlp.bias(i).shape) * 0.1)
        head.weight[-1] = 0.3
    tower_file = str(tmp_path / "tower.bin")
    assert export_tower(mlp, head, tower_file) == 3
    ids = signs[rng.integers(0, len(signs), size=(S, B))]
    ids[1, 3] = 12345                                                  # unknown: zeros
    ids[2, 0] = 0
    req = str(tmp_path / "req.txt")
    with open(req, "w") as f:
        for row in ids:
            f.write(" ".join(str(int(x)) for x in row) + "\n")
    out = subprocess.run([exe, "--dict", dict_file, "--tower", tower_file, "--slots", str(S), "--dim", str(dim), "--ids", req, "--dump"],
                         capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    native = np.array([float(x) for x in out.stdout.split()])
    eng = InferenceEngine(EmbeddingDictionary.from_file(dict_file, dim=dim), mlp, head, S, combiner="sum")
    want = eng.infer(torch.from_numpy(ids.view(np.int64))).numpy()
    assert native.shape == (B,) and np.abs(native - want).max() < 2e-2, (native, want)      # the engine computes in bf16
    # and in fp32 by hand
    x = torch.zeros(B, S * dim)
    look = {int(s): w for s, w in zip(signs, weights)}
    for s in range(S):
        for b in range(B):
            if int(ids[s, b]) in look:
                x[b, s * dim:(s + 1) * dim] = torch.from_numpy(look[int(ids[s, b])])
    for i in range(2):
        x = torch.relu(x @ mlp.weight(i).float().t() + mlp.bias(i).float())
    exact = torch.sigmoid(x @ head.weight[:5].float() + head.weight[5].float()).detach().numpy()
    assert np.abs(native - exact).max() < 1e-5
    # latency mode prints one JSON line; a damaged tower file is refused
    out = subprocess.run([exe, "--dict", dict_file, "--tower", tower_file, "--slots", str(S), "--dim", str(dim), "--batch", "8",
                          "--requests", "20"], capture_output=True, text=True, timeout=60)
    rep = json.loads(out.stdout)
    assert rep["dictionary_rows"] == len(signs) and 0 < rep["mean_probability"] < 1 and rep["p50_ms"] <= rep["p99_ms"]
    with open(tower_file, "r+b") as f:
        f.truncate(40)
    out = subprocess.run([exe, "--dict", dict_file, "--tower", tower_file, "--slots", str(S), "--dim", str(dim)], capture_output=True, text=True)
    assert out.returncode == 1 and "tower" in out.stderr

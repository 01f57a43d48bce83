"""Checkpoints are read as streams: block files in bounded pieces (text and binary give the same rows as the whole-file
reader), the tools re-shard without holding a table, a large shard loads with the host holding a few pieces only, a
path with a URL scheme goes through a file-system object, and the serving dictionary is parsed natively.
Reference: core/ps/optimizer/optimizer_kernel.h:366-420,488-538, core/utility/file_io.cc:47-50,132,
tensornet_tools/python/resize_sparse.py:35-54."""
import os
import resource
import shutil

import numpy as np
import pytest

import tensornet_b200 as tn
from tensornet_b200 import _build
from tensornet_b200.tools import ckpt_tools
from tensornet_b200.utils import checkpoint


@pytest.fixture(autouse=True)
def _cpu_runtime():
    tn.core.shutdown()
    tn.core.config.force_cpu = True
    tn.core.init()
    yield
    tn.core.shutdown()


def _rows(kind, dim, n, seed=0):
    ext = _build.cpu_ext()
    rng = np.random.default_rng(seed)
    signs = rng.choice(1 << 40, size=n, replace=False).astype(np.uint64)
    rows = rng.standard_normal((n, ext.row_floats(kind, dim))).astype(np.float32)
    if kind == 0:
        rows[:, dim + 3] = 0.0          # no_show_days is an integer field
    else:
        rows[:, 3 * dim + 1:] = 0.0
    return signs, rows


@pytest.mark.parametrize("kind,mode", [(0, "txt"), (0, "bin"), (1, "bin"), (2, "txt")])
def test_block_reader_pieces_equal_the_whole_file(tmp_path, kind, mode):
    ext = _build.cpu_ext()
    dim = 4
    signs, rows = _rows(kind, dim, 5000, seed=kind)
    d = str(tmp_path / "rank_0")
    ext.write_sparse_dir(d, mode, kind, dim, False, signs, rows, False, 0.0, 0, 0)
    whole_s, whole_r = ext.read_sparse_dir(d, kind, dim, False)
    got_s, got_r, pieces = [], [], 0
    for s, r in checkpoint.iter_rank_dir(d, kind, dim, False, chunk_rows=333, files_in_flight=3):
        assert 0 < len(s) <= 333
        got_s.append(s); got_r.append(r); pieces += 1
    got_s, got_r = np.concatenate(got_s), np.concatenate(got_r)
    assert pieces >= 15 and len(got_s) == 5000
    a, b = np.argsort(whole_s), np.argsort(got_s)
    assert np.array_equal(whole_s[a], got_s[b]) and np.array_equal(whole_r[a], got_r[b])


def test_streamed_load_holds_a_few_pieces_only(tmp_path):
    """2 M AdaGrad rows of dim 8 (112 MB of rows on disk as ~60 MB of gzip): loading them raises the process's peak
    resident size by far less than the table's size on the host path that hands pieces to the table."""
    ext = _build.cpu_ext()
    kind, dim, n = 0, 8, 2_000_000
    d = str(tmp_path / "rank_0")
    w = ext.SparseDirWriter(d, "bin", kind, dim, False, False, 0.0, 0, 0)
    rng = np.random.default_rng(0)
    for lo in range(0, n, 250_000):
        s = (np.arange(lo, lo + 250_000, dtype=np.uint64) + 1) * np.uint64(0x9E3779B97F4A7C15)
        w.append(s, rng.standard_normal((250_000, ext.row_floats(kind, dim))).astype(np.float32))
    assert w.close() == n
    before = resource.getrusage(resource.RUSAGE_SELF).ru_maxrss
    seen = 0
    for s, r in checkpoint.iter_rank_dir(d, kind, dim, False, chunk_rows=1 << 15):
        seen += len(s)
    grown_mb = (resource.getrusage(resource.RUSAGE_SELF).ru_maxrss - before) / 1024
    assert seen == n
    # eight pieces of 32 K rows are ~15 MB; the whole table would be 112 MB.  (A sanitizer build keeps freed memory in
    # quarantine, which counts as resident: only the order of magnitude is checked there.)
    limit = 200 if os.environ.get("TN_CPU_SANITIZE", "") not in ("", "0") else 60
    assert grown_mb < limit, grown_mb


def test_tools_stream_and_resharded_load_is_exact(tmp_path):
    kind, dim = 1, 4
    signs, rows = _rows(kind, dim, 4000, seed=3)
    src = str(tmp_path / "src")
    ext = _build.cpu_ext()
    for r in range(2):
        m = signs % np.uint64(2) == r
        ext.write_sparse_dir(os.path.join(src, f"rank_{r}"), "bin", kind, dim, False, signs[m], rows[m], False, 0.0, 0, 0)
    out = str(tmp_path / "w8")
    assert ckpt_tools.resize_sparse(src, out, 8, mode="bin", opt_name="Adam", dim=dim) == 4000
    back_s, back_r, _, _ = ckpt_tools.read_sparse_table(out, "Adam", dim)
    a, b = np.argsort(signs), np.argsort(back_s)
    assert np.array_equal(signs[a], back_s[b]) and np.array_equal(rows[a], back_r[b])
    for r in range(8):
        s, _ = ext.read_sparse_dir(os.path.join(out, f"rank_{r}"), kind, dim, False)
        assert np.all(s % np.uint64(8) == r)
    # extra embeddings: an existing old sign gives its row to a new sign; unknown old signs and taken new signs are skipped
    old_a, old_b = int(signs[0]), int(signs[1])
    n_add = ckpt_tools.merge_extra_embedding(src, str(tmp_path / "extra"), {old_a: 999_999_999_999, old_b: int(signs[2]), 12345: 777},
                                             mode="bin", opt_name="Adam", dim=dim)
    assert n_add == 1
    ex_s, ex_r, _, _ = ckpt_tools.read_sparse_table(str(tmp_path / "extra"), "Adam", dim)
    assert len(ex_s) == 4001 and np.array_equal(ex_r[ex_s == np.uint64(999_999_999_999)][0], rows[0])
    # dictionary export, then the native dictionary reader
    dic = str(tmp_path / "dict.txt.gz")
    assert ckpt_tools.merge_sparse(src, dic, "Adam", dim, brackets=True, compress=True) == 4000
    rd = ext.DictionaryReader(dic)
    ds, dw = [], []
    while True:
        s, wts = rd.next(700)
        if not len(s):
            break
        ds.append(s); dw.append(wts)
    ds, dw = np.concatenate(ds), np.concatenate(dw)
    assert dw.shape == (4000, dim)
    o = np.argsort(ds)
    assert np.array_equal(ds[o], signs[a]) and np.allclose(dw[o], rows[a][:, :dim], rtol=1e-5, atol=1e-6)
    from tensornet_b200.serving.engine import EmbeddingDictionary
    ed = EmbeddingDictionary.from_file(dic)
    assert ed.n == 4000 and ed.dim == dim


class _DirFS:
    """A stand-in for a remote file system: URLs ``mem://bucket/...`` live under a local root."""

    def __init__(self, root):
        self.root = root
        self.calls = []

    def _p(self, path):
        return os.path.join(self.root, path.lstrip("/"))

    def exists(self, path):
        return os.path.exists(self._p(path))

    def ls(self, path, detail=False):
        return [os.path.join(path, n) for n in os.listdir(self._p(path))]

    def makedirs(self, path, exist_ok=True):
        os.makedirs(self._p(path), exist_ok=True)

    def get(self, src, dst, recursive=True):
        self.calls.append(("get", src))
        (shutil.copytree if os.path.isdir(self._p(src)) else shutil.copy)(self._p(src), dst)

    def put(self, src, dst, recursive=True):
        self.calls.append(("put", dst))
        if os.path.isdir(src):
            shutil.copytree(src, self._p(dst), dirs_exist_ok=True)
        else:
            os.makedirs(os.path.dirname(self._p(dst)), exist_ok=True)
            shutil.copy(src, self._p(dst))


def test_checkpoint_through_a_remote_file_system(tmp_path):
    fs = _DirFS(str(tmp_path / "remote"))
    checkpoint.set_remote_fs(lambda url: (fs, url.split("://", 1)[1]))
    try:
        opt = tn.core.Adam(learning_rate=0.1)              # Adam rows are never dropped by the save-time rule
        h = tn.core.create_sparse_table(opt, "emb", 4)
        t = tn.core.sparse_table(h)
        signs, rows = _rows(1, 4, 300, seed=9)
        t.load_rows(signs, rows)
        tn.core.save_sparse_table(h, "mem://bucket/model/d1", "bin")
        assert os.path.isdir(str(tmp_path / "remote" / "bucket" / "model" / "d1" / "sparse_table" / "emb" / "rank_0"))
        t.clear()
        tn.core.load_sparse_table(h, "mem://bucket/model/d1", "bin")
        s2, r2 = t.dump()
        a, b = np.argsort(signs), np.argsort(s2)
        assert np.array_equal(signs[a], s2[b]) and np.array_equal(rows[a], r2[b])
        assert any(c[0] == "put" for c in fs.calls) and any(c[0] == "get" for c in fs.calls)
    finally:
        checkpoint.set_remote_fs(None)
    assert checkpoint.is_remote("hdfs://nn/x") and not checkpoint.is_remote("/tmp/x") and not checkpoint.is_remote("file:///tmp/x")

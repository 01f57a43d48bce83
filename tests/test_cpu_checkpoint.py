"""On-disk formats: golden bytes derived from the reference's serializers
(core/ps/optimizer/*_kernel.cc, optimizer_kernel.h:324-420,462-538, dense_table.cc:103-157,
bn_table.cc:171-214), write -> read round trips, file-name rules, re-sharding on load."""
import gzip
import os
import struct

import numpy as np
import pytest

import tensornet_b200 as tn
from tensornet_b200 import _build

ext = _build.cpu_ext()
ADAGRAD, ADAM, FTRL = 0, 1, 2


def _block_of(sign):
    return (((sign >> 32) | (sign << 32)) & 0xFFFFFFFFFFFFFFFF) % 8


def _adagrad_rows(signs, dim, rng):
    rows = np.zeros((len(signs), dim + 4), np.float32)
    rows[:, :dim] = rng.standard_normal((len(signs), dim)).astype(np.float32)
    rows[:, dim] = rng.random(len(signs)) + 0.1
    rows[:, dim + 1] = rng.integers(0, 50, len(signs))
    rows[:, dim + 2] = rng.integers(0, 5, len(signs))
    rows[:, dim + 3] = rng.integers(0, 9, len(signs)).astype(np.int32).view(np.float32)
    return rows


def test_adagrad_text_block_golden(tmp_path):
    signs = np.array([8, 16], dtype=np.uint64)          # both fall into block 0
    rows = np.zeros((2, 6), np.float32)
    rows[0] = [0.5, -1.25, 0.1, 3, 1, 0]
    rows[1] = [1e-7, 123456.789, 2.5, 0, 0, 0]
    rows[:, 5] = np.array([0, 7], np.int32).view(np.float32)
    ext.write_sparse_dir(str(tmp_path), "txt", ADAGRAD, 2, False, signs, rows, True, 0.0, 1000, 0)
    txt = gzip.open(tmp_path / "block_0.gz", "rt").read()
    assert txt == ("opt_name:AdaGrad\ndim:2\n"
                   "8\t2\t0.5\t-1.25\t0.1\t3\t0\t\n"           # trailing tab: no click column without CVM
                   "16\t2\t1e-07\t123457\t2.5\t0\t7\t\n"          # ostream default: %g, 6 significant digits
                   "\n")
    assert gzip.open(tmp_path / "block_3.gz", "rt").read() == "opt_name:AdaGrad\ndim:2\n\n"
    ext.write_sparse_dir(str(tmp_path / "cvm"), "txt", ADAGRAD, 2, True, signs, rows, True, 0.0, 1000, 0)
    assert gzip.open(tmp_path / "cvm" / "block_0.gz", "rt").read().splitlines()[2] == "8\t2\t0.5\t-1.25\t0.1\t3\t0\t1"


def test_adam_binary_block_golden_and_suffix(tmp_path):
    signs = np.array([8], dtype=np.uint64)
    rows = np.array([[1, 2, 0.1, 0.2, 0.01, 0.02, 5, 0]], np.float32)      # w | m | v | show | delta_show
    ext.write_sparse_dir(str(tmp_path), "bin", ADAM, 2, False, signs, rows, False, 0.0, 0, 0)
    raw = gzip.open(tmp_path / "block_0_bin.gz", "rb").read()
    assert raw == struct.pack("<iQ7f", 2, 8, 1, 2, 0.1, 0.2, 0.01, 0.02, 5) + b"\n"
    txtdir = tmp_path / "t"
    ext.write_sparse_dir(str(txtdir), "txt", ADAM, 2, False, signs, rows, False, 0.0, 0, 0)
    assert gzip.open(txtdir / "block_0.gz", "rt").read().splitlines()[2] == "8\t1\t0.1\t0.01\t2\t0.2\t0.02\t5"   # interleaved w m v


@pytest.mark.parametrize("kind,dim,cvm", [(ADAGRAD, 8, False), (ADAGRAD, 4, True), (ADAM, 8, False), (FTRL, 3, False)])
def test_sparse_round_trip_bin_exact_txt_6_digits(tmp_path, kind, dim, cvm):
    rng = np.random.default_rng(kind * 10 + dim)
    signs = rng.integers(1, 2 ** 63, 3000, dtype=np.int64).astype(np.uint64)
    if kind == ADAGRAD:
        rows = _adagrad_rows(signs, dim, rng)
        if not cvm:
            rows[:, dim + 2] = 0
    else:
        rows = rng.standard_normal((len(signs), 3 * dim + 2)).astype(np.float32)
        rows[:, 3 * dim + 1] = 0
    for mode in ("bin", "txt"):
        d = str(tmp_path / mode)
        ext.write_sparse_dir(d, mode, kind, dim, cvm, signs, rows, False, 0.0, 0, 0)
        for b in range(8):          # every sign sits in the block the reference's hasher picks
            assert os.path.exists(os.path.join(d, f"block_{b}{'_bin' if mode == 'bin' else ''}.gz"))
        s2, r2 = ext.read_sparse_dir(d, kind, dim, cvm)
        order, order2 = np.argsort(signs), np.argsort(s2)
        assert np.array_equal(signs[order], s2[order2])
        if mode == "bin":
            assert np.array_equal(rows[order].view(np.int32), r2[order2].view(np.int32))     # bit exact
            d2 = str(tmp_path / "again")
            ext.write_sparse_dir(d2, "bin", kind, dim, cvm, s2, r2, False, 0.0, 0, 0)
            s3, r3 = ext.read_sparse_dir(d2, kind, dim, cvm)
            assert np.array_equal(np.sort(s3), np.sort(signs))
        else:
            nf = dim + 2 if kind == ADAGRAD else 3 * dim + 1
            assert np.allclose(rows[order][:, :nf], r2[order2][:, :nf], rtol=1e-5, atol=1e-30)
    # block placement
    txt = gzip.open(os.path.join(str(tmp_path / "txt"), "block_5.gz"), "rt").read().splitlines()[2:]
    assert all(_block_of(int(l.split("\t")[0])) == 5 for l in txt if l)


def test_reader_sniffs_suffixless_binary_and_legacy_names(tmp_path):
    signs = np.array([3, 11], dtype=np.uint64)
    rows = np.arange(16, dtype=np.float32).reshape(2, 8)            # Adam dim 2
    ext.write_sparse_dir(str(tmp_path), "bin", ADAM, 2, False, signs, rows, False, 0.0, 0, 0)
    for b in range(8):                                              # what the reference itself writes in "bin" mode
        os.rename(tmp_path / f"block_{b}_bin.gz", tmp_path / f"sparse_block_{b}.gz")
    s2, r2 = ext.read_sparse_dir(str(tmp_path), ADAM, 2, False)
    assert sorted(s2.tolist()) == [3, 11]
    assert np.array_equal(r2[np.argsort(s2)][:, :7], rows[:, :7])


def test_old_adagrad_text_without_no_show_days(tmp_path):
    with gzip.open(tmp_path / "block_0.gz", "wt") as f:
        f.write("opt_name:AdaGrad\ndim:2\n8\t2\t0.5\t0.25\t0.1\t3\n\n")   # dim + 4 columns: the pre-no_show_days format
    for b in range(1, 8):
        with gzip.open(tmp_path / f"block_{b}.gz", "wt") as f:
            f.write("opt_name:AdaGrad\ndim:2\n\n")
    s, r = ext.read_sparse_dir(str(tmp_path), ADAGRAD, 2, False)
    assert s.tolist() == [8] and r[0, :4].tolist() == [0.5, 0.25, 0.10000000149011612, 3.0]
    assert r[0, 5:].view(np.int32).tolist() == [0]


def test_optimizer_name_is_checked(tmp_path):
    ext.write_sparse_dir(str(tmp_path), "txt", ADAM, 2, False, np.array([1], np.uint64), np.zeros((1, 8), np.float32), False, 0.0, 0, 0)
    with pytest.raises(RuntimeError, match="same optimizer"):
        ext.read_sparse_dir(str(tmp_path), FTRL, 2, False)


def test_eviction_filter_applies_only_on_save(tmp_path):
    signs = np.array([8, 16, 24], dtype=np.uint64)
    rows = np.zeros((3, 6), np.float32)
    rows[:, 3] = [0.5, 5.0, 5.0]                                   # show
    rows[:, 5] = np.array([0, 0, 2000], np.int32).view(np.float32)  # no_show_days
    ext.write_sparse_dir(str(tmp_path / "or"), "bin", ADAGRAD, 2, False, signs, rows, True, 1.0, 1000, 0)
    assert sorted(ext.read_sparse_dir(str(tmp_path / "or"), ADAGRAD, 2, False)[0].tolist()) == [16]
    ext.write_sparse_dir(str(tmp_path / "and"), "bin", ADAGRAD, 2, False, signs, rows, True, 1.0, 1000, 1)
    assert sorted(ext.read_sparse_dir(str(tmp_path / "and"), ADAGRAD, 2, False)[0].tolist()) == [8, 16, 24]


def test_dense_file_golden_and_round_trip(tmp_path):
    w = np.arange(1, 11, dtype=np.float32) / 4
    m = np.full(10, 0.5, np.float32)
    v = np.full(10, 0.25, np.float32)
    path = str(tmp_path / "dense_table" / "0" / "0")
    ext.write_dense_file(path, 10, 1, ADAM, w, m, v, None, 0.9, 0.999)
    txt = open(path).read()
    assert txt.startswith("total_elements:10\nrank_num:1\nopt_name:Adam\narray_size:2\nbeta1_power:0.9\nbeta2_power:0.999\n"
                          "0.25\t0.5\t0.25\n0.5\t0.5\t0.25\n\n\nopt_name:Adam\narray_size:2\n")
    assert txt.count("opt_name:Adam") == 5                        # ceil(10/8) = 2 per block -> 5 blocks
    d = ext.read_dense_file(path, ADAM)
    assert d["total_elements"] == 10 and d["rank_num"] == 1
    assert np.array_equal(d["w"], w) and np.array_equal(d["s0"], m) and np.array_equal(d["s1"], v)
    assert abs(d["beta1_power"] - 0.9) < 1e-6
    with pytest.raises(RuntimeError):
        ext.read_dense_file(path, ADAGRAD)


def test_bn_file_layout(tmp_path):
    path = str(tmp_path / "bn_table" / "0")
    s, q, c = np.array([1.5, 2.5]), np.array([3.0, 4.0]), np.array([10.0, 10.0])
    ext.write_bn_file(path, True, s, q, c)
    raw = gzip.open(path, "rb").read()
    assert raw == struct.pack("<?I6d", True, 2, 1.5, 3.0, 10.0, 2.5, 4.0, 10.0)
    pctr, s2, q2, c2 = ext.read_bn_file(path)
    assert pctr and np.array_equal(s2, s) and np.array_equal(q2, q) and np.array_equal(c2, c)


@pytest.mark.parametrize("mode", ["txt", "bin"])
def test_streaming_writer_equals_one_shot_write(tmp_path, mode):
    """A shard appended in pieces (in any order, or already grouped by block file as the device export delivers it)
    produces the same block contents as one write of the whole shard."""
    rng = np.random.default_rng(4)
    dim = 3
    signs = np.unique(rng.integers(1, 2 ** 62, 3000, dtype=np.int64).astype(np.uint64))
    rows = _adagrad_rows(signs, dim, rng)
    ext.write_sparse_dir(str(tmp_path / "one"), mode, ADAGRAD, dim, True, signs, rows, True, 5.0, 6, 0)
    w = ext.SparseDirWriter(str(tmp_path / "pieces"), mode, ADAGRAD, dim, True, True, 5.0, 6, 0)
    for lo in range(0, len(signs), 700):
        w.append(signs[lo:lo + 700], rows[lo:lo + 700])
    kept = w.close()
    blocks = np.array([_block_of(int(s)) for s in signs])
    order = np.argsort(blocks, kind="stable")
    gs, gr = signs[order], rows[order]
    offsets = np.concatenate([[0], np.cumsum(np.bincount(blocks, minlength=8))]).astype(np.int64)
    g = ext.SparseDirWriter(str(tmp_path / "grouped"), mode, ADAGRAD, dim, True, True, 5.0, 6, 0)
    g.append_grouped(gs, gr, offsets)
    assert g.close() == kept
    sfx = "_bin" if mode == "bin" else ""
    total = 0
    for b in range(8):
        one = gzip.open(tmp_path / "one" / f"block_{b}{sfx}.gz", "rb").read()
        assert gzip.open(tmp_path / "pieces" / f"block_{b}{sfx}.gz", "rb").read() == one
        assert gzip.open(tmp_path / "grouped" / f"block_{b}{sfx}.gz", "rb").read() == one
    s2, r2 = ext.read_sparse_dir(str(tmp_path / "pieces"), ADAGRAD, dim, True)
    assert len(s2) == kept and 0 < kept < len(signs)            # the eviction rule dropped some rows
    with pytest.raises(Exception):
        g.append(signs[:1], rows[:1])                           # closed
    bad = offsets.copy(); bad[1], bad[2] = bad[2], bad[1]
    g2 = ext.SparseDirWriter(str(tmp_path / "bad"), mode, ADAGRAD, dim, True, False, 0.0, 0, 0)
    with pytest.raises(Exception):
        g2.append_grouped(gs, gr, bad)

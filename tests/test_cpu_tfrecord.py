"""TFRecord / tf.train.Example input without TensorFlow: the native reader against records serialized by the protobuf
library from a schema written out here (independent of this package's own encoder), the framing against the known
crc32c check value, interleave order, gzip files, damaged files, and a model trained from such files.

Reference: examples/common/util.py:23-39 (input pipeline), examples/gen_example_data.py:20-60 (record contents)."""
import gzip
import os
import struct

import numpy as np
import pytest
import torch

import tensornet_b200 as tn
from tensornet_b200 import _build


def _example_class():
    """tf.train.Example rebuilt from its published schema with the protobuf runtime."""
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory
    fd = descriptor_pb2.FileDescriptorProto(name="example_for_test.proto", package="tnt", syntax="proto3")
    F = descriptor_pb2.FieldDescriptorProto

    def msg(name):
        m = fd.message_type.add()
        m.name = name
        return m

    for name, typ in (("BytesList", F.TYPE_BYTES), ("FloatList", F.TYPE_FLOAT), ("Int64List", F.TYPE_INT64)):
        msg(name).field.add(name="value", number=1, label=F.LABEL_REPEATED, type=typ)
    m = msg("Feature")
    m.oneof_decl.add(name="kind")
    for i, (n, t) in enumerate((("bytes_list", "BytesList"), ("float_list", "FloatList"), ("int64_list", "Int64List"))):
        m.field.add(name=n, number=i + 1, label=F.LABEL_OPTIONAL, type=F.TYPE_MESSAGE, type_name=".tnt." + t, oneof_index=0)
    m = msg("Features")
    e = m.nested_type.add(name="FeatureEntry")
    e.options.map_entry = True
    e.field.add(name="key", number=1, label=F.LABEL_OPTIONAL, type=F.TYPE_STRING)
    e.field.add(name="value", number=2, label=F.LABEL_OPTIONAL, type=F.TYPE_MESSAGE, type_name=".tnt.Feature")
    m.field.add(name="feature", number=1, label=F.LABEL_REPEATED, type=F.TYPE_MESSAGE, type_name=".tnt.Features.FeatureEntry")
    msg("Example").field.add(name="features", number=1, label=F.LABEL_OPTIONAL, type=F.TYPE_MESSAGE, type_name=".tnt.Features")
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    return message_factory.GetMessageClass(pool.FindMessageTypeByName("tnt.Example"))


def _frame(data: bytes) -> bytes:
    ext = _build.cpu_ext()
    head = struct.pack("<Q", len(data))
    return head + struct.pack("<I", ext.tf_masked_crc32c(head)) + data + struct.pack("<I", ext.tf_masked_crc32c(data))


def _make_examples(n, seed=0):
    rng = np.random.default_rng(seed)
    Example = _example_class()
    rows, blobs = [], []
    for i in range(n):
        label = int(rng.random() < 0.4)
        row = {"label": label, "uniq_id": b"id%05d" % i, "1": [int(rng.integers(1, 50))],
               "2": [int(x) for x in rng.integers(-2 ** 62, 2 ** 62, size=int(rng.integers(0, 4)))],
               "4": None if label == 0 else [int(x) for x in rng.integers(1, 1000, size=3)],
               "dense": [float(x) for x in rng.standard_normal(3).astype(np.float32)]}
        ex = Example()
        ex.features.feature["label"].int64_list.value.append(label)
        ex.features.feature["uniq_id"].bytes_list.value.append(row["uniq_id"])
        ex.features.feature["1"].int64_list.value.extend(row["1"])
        ex.features.feature["2"].int64_list.value.extend(row["2"])          # may be an empty list
        if row["4"] is not None:                                             # missing for negatives
            ex.features.feature["4"].int64_list.value.extend(row["4"])
        ex.features.feature["dense"].float_list.value.extend(row["dense"])
        ex.features.feature["ignored"].float_list.value.append(1.0)
        rows.append(row)
        blobs.append(ex.SerializeToString())
    return rows, blobs


def test_crc32c_check_value_on_both_code_paths():
    ext = _build.cpu_ext()
    assert ext.crc32c(b"123456789", True) == 0xE3069283 and ext.crc32c(b"123456789", False) == 0xE3069283
    blob = bytes(range(256)) * 37 + b"tail"
    assert ext.crc32c(blob, True) == ext.crc32c(blob, False)
    assert ext.crc32c(b"", False) == 0


@pytest.mark.parametrize("compressed", [False, True])
def test_reader_matches_records_written_by_the_protobuf_library(tmp_path, compressed):
    rows, blobs = _make_examples(37)
    path = str(tmp_path / "tf-part.00001")
    payload = b"".join(_frame(b) for b in blobs)
    with (gzip.open(path, "wb") if compressed else open(path, "wb")) as f:
        f.write(payload)
    kw = dict(dense_keys={"dense": 3}, bytes_keys=["uniq_id"], num_workers=1, pin_memory=False)
    got = list(tn.data.TFRecordDataset([path], 16, ["1", "2", "4"], **kw))
    got_packed = list(tn.data.TFRecordDataset([path], 16, ["1", "2", "4"], packed=True, **kw))
    assert [int(y.numel()) for _, y in got] == [16, 16, 5] == [int(y.numel()) for _, y in got_packed]
    i = 0
    for (feats, y), (pf, _) in zip(got, got_packed):
        n = int(y.numel())
        packed = pf[tn.data.PACKED_KEY]
        assert "1" not in pf and tn.data.PACKED_KEY not in feats
        assert packed.keys == ["1", "2", "4"] and packed.batch_size == n and packed.offsets.numel() == 3 * n + 1
        for b in range(n):
            row = rows[i + b]
            assert float(y[b]) == row["label"] and feats["uniq_id"][b] == row["uniq_id"]
            np.testing.assert_array_equal(feats["dense"][b].numpy(), np.asarray(row["dense"], np.float32))
            for s, k in enumerate(["1", "2", "4"]):
                want = row[k] or []
                v, o = feats[k]
                assert v[int(o[b]):int(o[b + 1])].tolist() == want
                lo, hi = int(packed.offsets[s * n + b]), int(packed.offsets[s * n + b + 1])
                assert packed.values[lo:hi].tolist() == want
        i += n
    assert i == 37
    # fixed shapes: one id per slot, the default where the record has none, the first of several
    (pf, _), = list(tn.data.TFRecordDataset([path], 64, ["1", "2", "4"], single_hot=True, default_id=7, packed=True,
                                            num_workers=1, pin_memory=False))
    (feats, y), = list(tn.data.TFRecordDataset([path], 64, ["1", "2", "4"], single_hot=True, default_id=7, num_workers=1,
                                               pin_memory=False))
    assert pf[tn.data.PACKED_KEY].ids.shape == (3, 37) and pf[tn.data.PACKED_KEY].ids[0].tolist() == feats["1"].tolist()
    for b, row in enumerate(rows):
        assert int(feats["1"][b]) == row["1"][0]
        assert int(feats["2"][b]) == (row["2"][0] if row["2"] else 7)
        assert int(feats["4"][b]) == (row["4"][0] if row["4"] else 7)


def test_own_writer_round_trips_and_unpacked_lists_are_read(tmp_path):
    path = str(tmp_path / "w.tfrecord.gz")
    with tn.data.TFRecordWriter(path, gzip=True) as w:
        w.write(tn.data.encode_example({"a": [1, -2, 3], "label": [1]}, {"x": [0.5, 0.25]}, {"u": b"k"}))
        # hand-made record: the int64 list with one element per tag (not packed), as old writers emit it
        lst = b"\x08\x05\x08\x06"
        feat = b"\x1a" + bytes([len(lst)]) + lst
        entry = b"\x0a\x01a\x12" + bytes([len(feat)]) + feat
        feats = b"\x0a" + bytes([len(entry)]) + entry
        w.write(b"\x0a" + bytes([len(feats)]) + feats)
    (f, y), = list(tn.data.TFRecordDataset([path], 8, ["a"], dense_keys={"x": 4}, bytes_keys=["u"], pin_memory=False))
    assert f["a"].values.tolist() == [1, -2, 3, 5, 6] and f["a"].offsets.tolist() == [0, 3, 5]
    assert tn.data.TFRecordDataset(path, 8, ["a"], pin_memory=False).files == [path]           # one path, not its characters
    cols = [tn.feature_column.embedding_column(tn.feature_column.category_column(k), 4) for k in ("a", "zz")]
    assert tn.data.TFRecordDataset.from_columns([path], 8, cols, pin_memory=False).sparse_keys == ["a", "zz"]
    assert y.tolist() == [1.0, 0.0] and f["dense"].tolist() == [[0.5, 0.25, 0, 0], [0, 0, 0, 0]] and f["u"] == [b"k", b""]


def test_interleave_order_and_worker_split_are_deterministic(tmp_path):
    files = []
    for k in range(5):                                   # file k holds ids 100k .. 100k + 19 + k (unequal lengths)
        p = str(tmp_path / f"tf-{k}")
        with tn.data.TFRecordWriter(p) as w:
            for j in range(20 + k):
                w.write(tn.data.encode_example({"s": [100 * k + j]}))
        files.append(p)

    def run(**kw):
        ds = tn.data.TFRecordDataset(files, 4, ["s"], label_key=None, single_hot=True, pin_memory=False, **kw)
        return [f["s"].tolist() for f, _ in ds]

    one = run(num_workers=1, cycle_length=2, block_length=3)
    flat = [x for b in one for x in b]
    assert flat[:12] == [0, 1, 2, 100, 101, 102, 3, 4, 5, 103, 104, 105]       # blocks of 3 from two open files in turn
    assert sorted(flat) == sorted(100 * k + j for k in range(5) for j in range(20 + k))
    assert len(one[-1]) == len(flat) % 4 or len(one[-1]) == 4
    a, b = run(num_workers=3), run(num_workers=3)
    assert a == b                                                               # thread timing does not show
    assert sorted(x for bb in a for x in bb) == sorted(flat)
    assert all(len({x // 100 % 3 for x in bb}) == 1 for bb in a)                # a batch never mixes two workers' files
    assert sum(len(bb) for bb in run(num_workers=2, drop_remainder=True)) % 4 == 0
    ds = tn.data.TFRecordDataset(files, 4, ["s"], label_key=None, single_hot=True, pin_memory=False, num_workers=1, cycle_length=1,
                                 shuffle_files=True, seed=5)

    def file_order(d):
        seen = []
        for f, _ in d:
            for x in f["s"].tolist():
                if x // 100 not in seen:
                    seen.append(x // 100)
        return seen

    first = [file_order(ds) for _ in range(3)]                     # three passes over one dataset object
    again = tn.data.TFRecordDataset(files, 4, ["s"], label_key=None, single_hot=True, pin_memory=False, num_workers=1,
                                    cycle_length=1, shuffle_files=True, seed=5)
    assert len({tuple(o) for o in first}) > 1 and all(sorted(o) == [0, 1, 2, 3, 4] for o in first)
    assert file_order(again) == first[0]


def test_damaged_files_are_reported(tmp_path):
    good = _frame(tn.data.encode_example({"s": [1]}))
    cases = {"cut": good + good[:-3], "flip": good[:14] + bytes([good[14] ^ 1]) + good[15:], "head": b"\x01" + good[1:]}
    for name, payload in cases.items():
        p = str(tmp_path / name)
        with open(p, "wb") as f:
            f.write(payload)
        with pytest.raises(RuntimeError, match=name == "cut" and "ends inside" or name == "flip" and "checksum" or "corrupt"):
            list(tn.data.TFRecordDataset([p], 2, ["s"], label_key=None, pin_memory=False))
    p = str(tmp_path / "junk")
    with open(p, "wb") as f:
        f.write(_frame(b"\x0a\x05\x0a\x03\x0a\x7f"))                          # lengths that run past the record
    with pytest.raises(RuntimeError, match="well-formed"):
        list(tn.data.TFRecordDataset([p], 2, ["s"], label_key=None, pin_memory=False))
    # a reader abandoned in mid-file shuts its threads down
    p = str(tmp_path / "many")
    with tn.data.TFRecordWriter(p) as w:
        for j in range(2000):
            w.write(tn.data.encode_example({"s": [j]}))
    it = iter(tn.data.TFRecordDataset([p], 4, ["s"], label_key=None, pin_memory=False, queue_depth=1))
    next(it)
    it.close()


def test_wide_deep_trains_from_tfrecord_files(tmp_path):
    """The reference's example records (slots 1-3 one id, slot 4 three ids or missing, int64 label) through fit."""
    rng = np.random.default_rng(3)
    pools = {s: rng.integers(1, 2 ** 62, size=10) for s in "1234"}
    files = []
    for k in range(2):
        p = str(tmp_path / f"tf-part.{k:05d}")
        with tn.data.TFRecordWriter(p) as w:
            for _ in range(640):
                first = int(rng.integers(0, 10))
                label = int(first % 2 == 0)
                ints = {"label": [label], "1": [int(pools["1"][first])], "2": [int(rng.choice(pools["2"]))],
                        "3": [int(rng.choice(pools["3"]))]}
                if label:
                    ints["4"] = [int(x) for x in rng.choice(pools["4"], size=3)]
                w.write(tn.data.encode_example(ints, raw={"uniq_id": b"xxxxx"}))
        files.append(p)
    tn.core.init()
    slots = ["1", "2", "3", "4"]
    torch.manual_seed(0)
    model = tn.models.WideDeep(slots, slots, dnn_hidden_units=(32, 16), embedding_dim=8, bucket_size=2048,
                               sparse_opt=tn.core.AdaGrad(learning_rate=0.05, initial_g2sum=0.1, initial_scale=0.1))
    model.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=5e-3)), loss="binary_crossentropy",
                  metrics=[tn.metric.AUC()])
    ds = tn.data.TFRecordDataset(files, 64, slots, num_workers=2)
    hist = model.fit(ds, epochs=3)
    assert hist["loss"][-1] < 0.2 and hist["auc"][-1] > 0.98, hist


def test_arbitrary_record_bytes_parse_or_are_refused(tmp_path):
    """Records are untrusted input: random bytes and damaged valid records either parse or raise, and what parses
    stays inside the batch's bounds (run under the sanitizer build this is a fuzz test of the wire parser)."""
    from hypothesis import given, settings, strategies as st
    good = tn.data.encode_example({"a": [1, 2, 3], "b": [], "label": [1]}, {"x": [1.0, 2.0]}, {"u": b"abc"})
    path = str(tmp_path / "fuzz")

    @settings(max_examples=300, deadline=None)
    @given(st.one_of(st.binary(max_size=64),
                     st.tuples(st.integers(0, len(good) - 1), st.integers(0, 255)).map(
                         lambda t: good[:t[0]] + bytes([t[1]]) + good[t[0] + 1:]),
                     st.integers(0, len(good)).map(lambda n: good[:n])))
    def check(blob):
        with open(path, "wb") as f:
            f.write(_frame(blob) + _frame(good))
        ds = tn.data.TFRecordDataset([path], 4, ["a", "b"], dense_keys={"x": 2}, bytes_keys=["u"], num_workers=1, pin_memory=False)
        try:
            (feats, y), = list(ds)
        except RuntimeError as e:
            assert "well-formed" in str(e)
            return
        assert y.numel() == 2 and feats["a"].offsets.numel() == 3 and feats["dense"].shape == (2, 2)
        assert int(feats["a"].offsets[-1]) == feats["a"].values.numel()
        assert feats["a"].values[int(feats["a"].offsets[1]):].tolist() == [1, 2, 3]      # the good record behind it

    check()


def test_input_files_on_a_remote_file_system_are_fetched_as_they_are_read(tmp_path):
    """Day directories under a URL (``hdfs://`` for the reference's users; a local stand-in here) are listed through
    the file-system layer and every file is copied to scratch space only while a reader works on it."""
    import shutil
    from tensornet_b200.utils import checkpoint

    class DirFS:
        def __init__(self, root):
            self.root, self.gets, self.live_max = root, [], 0

        def _p(self, path):
            return os.path.join(self.root, path.lstrip("/"))

        def exists(self, path):
            return os.path.exists(self._p(path))

        def ls(self, path, detail=False):
            return [os.path.join(path, n) for n in os.listdir(self._p(path))]

        def get(self, src, dst, recursive=True):
            self.gets.append(src)
            shutil.copy(self._p(src), dst)
            self.live_max = max(self.live_max, len(os.listdir(os.path.dirname(dst))))

    root = tmp_path / "remote"
    want = []
    for day in ("2020-05-10", "2020-05-11"):
        os.makedirs(root / "bucket" / "data" / day)
        for k in range(3):
            with tn.data.TFRecordWriter(str(root / "bucket" / "data" / day / f"tf-part.{k:05d}")) as w:
                for j in range(10):
                    x = int(day[-2:]) * 1000 + k * 100 + j
                    want.append(x)
                    w.write(tn.data.encode_example({"s": [x], "label": [j & 1]}))
        (root / "bucket" / "data" / day / "_SUCCESS").write_text("")
    fs = DirFS(str(root))
    checkpoint.set_remote_fs(lambda url: (fs, url.split("://", 1)[1]))
    try:
        files = tn.data.list_files("mem://bucket/data", ["2020-05-10", "2020-05-11"], "tf-*")
        assert files[0] == "mem://bucket/data/2020-05-10/tf-part.00000" and len(files) == 6
        with pytest.raises(FileNotFoundError):
            tn.data.list_files("mem://bucket/data", ["2020-05-12"], "tf-*")
        ds = tn.data.TFRecordDataset(files, 4, ["s"], single_hot=True, num_workers=2, cycle_length=1, pin_memory=False)
        got = [x for f, _ in ds for x in f["s"].tolist()]
        assert sorted(got) == sorted(want)
        assert sorted(fs.gets) == sorted(f.split("://", 1)[1] for f in files)
        assert fs.live_max <= 2                               # two readers, one open file each
        # a file that cannot be fetched is reported with its remote name
        bad = tn.data.TFRecordDataset(files[:1] + ["mem://bucket/data/2020-05-10/missing"], 4, ["s"], num_workers=1, pin_memory=False)
        with pytest.raises(RuntimeError, match="missing|No such file"):
            list(bad)
    finally:
        checkpoint.set_remote_fs(None)


def _py_example(row, long_len=False, unpacked=False):
    """Plain-Python tf.train.Example encoder with two knobs that keep a record valid but off the reader's fast path:
    every length as a two-byte varint, and number lists with one element per tag."""
    def varint(v):
        v &= (1 << 64) - 1
        out = bytearray()
        while v >= 0x80:
            out.append((v & 0x7F) | 0x80)
            v >>= 7
        out.append(v)
        return bytes(out)

    def length(n):
        return bytes([(n & 0x7F) | 0x80, n >> 7]) if long_len else varint(n)

    def field(num, body):
        return varint(num << 3 | 2) + length(len(body)) + body

    feats = b""
    for key, (kind, vals) in row.items():
        if kind == "int":
            lst = b"".join(b"\x08" + varint(v) for v in vals) if unpacked else (field(1, b"".join(varint(v) for v in vals)) if vals else b"")
            feature = field(3, lst)
        elif kind == "float":
            raw = [struct.pack("<f", v) for v in vals]
            lst = b"".join(b"\x0d" + r for r in raw) if unpacked else (field(1, b"".join(raw)) if vals else b"")
            feature = field(2, lst)
        elif kind == "bytes":
            feature = field(1, b"".join(field(1, v) for v in vals))
        else:
            feature = b""                                              # a feature with no list at all
        feats += field(1, field(1, key.encode()) + field(2, feature))
    return field(1, feats)


def test_fast_path_and_general_parser_agree(tmp_path):
    """Records of the usual shape take a shortcut in the reader; the same contents encoded so that the shortcut does
    not apply (long length prefixes, unpacked lists) must give the same batches."""
    rng = np.random.default_rng(11)
    rows = []
    for i in range(300):
        row = {}
        if rng.random() < 0.9:
            row["a"] = ("int", [int(x) for x in rng.integers(-2 ** 63, 2 ** 63 - 1, size=int(rng.integers(0, 5)))])
        if rng.random() < 0.8:
            row["b"] = ("int", [int(rng.integers(0, 200))])
        row["c"] = [("int", [3]), ("float", [1.0]), ("none", []), ("bytes", [b"z"])][int(rng.integers(0, 4))]   # a slot of the wrong type
        row["x"] = ("float", [float(np.float32(v)) for v in rng.standard_normal(int(rng.integers(0, 6)))])
        row["n"] = ("int", [int(v) for v in rng.integers(-5, 5, size=int(rng.integers(0, 3)))])                  # ints into the dense block
        row["label"] = ("int", [int(rng.integers(0, 2))]) if rng.random() < 0.5 else ("float", [float(rng.integers(0, 2))])
        if rng.random() < 0.7:
            row["u"] = ("bytes", [bytes(rng.integers(0, 256, size=int(rng.integers(0, 9)), dtype=np.uint8))])
        keys = list(row)
        if i % 7 == 0:
            rng.shuffle(keys)                                           # another order: the predicted names miss
        rows.append({k: row[k] for k in keys})
    outs, singles = [], []
    for name, kw in (("plain", {}), ("long", {"long_len": True}), ("unpacked", {"unpacked": True})):
        p = str(tmp_path / name)
        with tn.data.TFRecordWriter(p) as w:
            for row in rows:
                w.write(_py_example(row, **kw))
        ds = tn.data.TFRecordDataset([p], 64, ["a", "b", "c"], dense_keys={"x": 4, "n": 2}, bytes_keys=["u"], packed=True, num_workers=1,
                                     pin_memory=False)
        outs.append(list(ds))
        singles.append(list(tn.data.TFRecordDataset([p], 64, ["a", "b", "c"], single_hot=True, default_id=-7, packed=True,
                                                    num_workers=1, pin_memory=False)))
    ref = outs[0]
    assert sum(int(y.numel()) for _, y in ref) == 300
    i = 0
    for f, _ in singles[0]:                                             # one id per slot: the first, or the default
        ids = f[tn.data.PACKED_KEY].ids
        for b in range(ids.shape[1]):
            row = rows[i + b]
            want = [(row[k][1][0] if k in row and row[k][0] == "int" and row[k][1] else -7) for k in ("a", "b", "c")]
            assert ids[:, b].tolist() == want
        i += ids.shape[1]
    assert i == 300
    for other in singles[1:]:
        assert all(torch.equal(f0[tn.data.PACKED_KEY].ids, f1[tn.data.PACKED_KEY].ids) for (f0, _), (f1, _) in zip(singles[0], other))
    i = 0
    for f, y in ref:                                                    # and the plain file against the rows themselves
        pk = f[tn.data.PACKED_KEY]
        n = pk.batch_size
        for b in range(n):
            row = rows[i + b]
            want_a = row["a"][1] if "a" in row else []
            lo, hi = int(pk.offsets[b]), int(pk.offsets[b + 1])
            assert pk.values[lo:hi].tolist() == want_a
            want_c = row["c"][1] if row["c"][0] == "int" else []
            lo, hi = int(pk.offsets[2 * n + b]), int(pk.offsets[2 * n + b + 1])
            assert pk.values[lo:hi].tolist() == want_c
            xs = (row["x"][1] + [0.0] * 4)[:4] + ([float(v) for v in row["n"][1]] + [0.0, 0.0])[:2]
            assert f["dense"][b].tolist() == xs
            assert float(y[b]) == float(row["label"][1][0])
            assert f["u"][b] == (row["u"][1][0] if "u" in row else b"")
        i += n
    for other in outs[1:]:
        assert len(other) == len(ref)
        for (f0, y0), (f1, y1) in zip(ref, other):
            assert torch.equal(f0[tn.data.PACKED_KEY].values, f1[tn.data.PACKED_KEY].values)
            assert torch.equal(f0[tn.data.PACKED_KEY].offsets, f1[tn.data.PACKED_KEY].offsets)
            assert torch.equal(f0["dense"], f1["dense"]) and torch.equal(y0, y1) and f0["u"] == f1["u"]

"""Batch cache: a pass over the input written once as whole batches in the layout a step copies to the device, read
back without parsing.  What comes back must be what went in, for ragged and fixed-shape slots, from one or several
ranks' point of view, and a model must train from it exactly as from the source."""
import os

import numpy as np
import pytest
import torch

import tensornet_b200 as tn


def _records(path, n, seed):
    rng = np.random.default_rng(seed)
    with tn.data.TFRecordWriter(path) as w:
        for i in range(n):
            first = int(rng.integers(0, 20))
            ints = {"label": [int(first % 2 == 0)], "a": [1000 + first], "b": [int(x) for x in rng.integers(1, 50, size=int(rng.integers(0, 4)))]}
            w.write(tn.data.encode_example(ints, {"x": rng.standard_normal(3).astype(np.float32)}))


def _same(t, u):
    assert t.dtype == u.dtype and t.shape == u.shape and torch.equal(t, u)


@pytest.mark.parametrize("single_hot", [False, True])
def test_cache_round_trip_and_sharding(tmp_path, single_hot):
    src = str(tmp_path / "tf-0")
    _records(src, 150, 1)
    ds = tn.data.TFRecordDataset([src], 32, ["a", "b"], dense_keys={"x": 3}, single_hot=single_hot, packed=True, num_workers=1,
                                 pin_memory=False)
    cache = str(tmp_path / "day.tnbc")
    assert tn.data.write_batch_cache(cache, ds, ["a", "b"], dense_name="dense") == 150
    back = tn.data.BatchCacheDataset(cache, pin_memory=False)
    assert len(back) == 5
    for (f0, y0), (f1, y1) in zip(ds, back):
        p0, p1 = f0[tn.data.PACKED_KEY], f1[tn.data.PACKED_KEY]
        assert p0.keys == p1.keys and p0.batch_size == p1.batch_size
        if single_hot:
            _same(p0.ids, p1.ids)
        else:
            _same(p0.values, p1.values)
            _same(p0.offsets, p1.offsets)
        _same(f0["dense"], f1["dense"])
        _same(y0, y1)
        _same(f1["label"], y1)
    # two ranks reading one cache see disjoint halves, in order
    a = [int(y.numel()) for _, y in tn.data.BatchCacheDataset(cache, shard=(0, 2), pin_memory=False)]
    b = [int(y.numel()) for _, y in tn.data.BatchCacheDataset(cache, shard=(1, 2), pin_memory=False)]
    assert a == [32, 32, 22] and b == [32, 32] and len(tn.data.BatchCacheDataset(cache, shard=(1, 2))) == 2
    # several files are read one after the other; a reader that is dropped early stops its thread
    two = tn.data.BatchCacheDataset([cache, cache], pin_memory=False, prefetch=1)
    assert sum(int(y.numel()) for _, y in two) == 300
    it = iter(two)
    next(it)
    it.close()


def test_per_slot_features_are_packed_on_the_way_in_and_damage_is_reported(tmp_path):
    cache = str(tmp_path / "c.tnbc")
    g = torch.Generator().manual_seed(0)
    batches = []
    with tn.data.BatchCacheWriter(cache, ["u", "v"], label=True) as w:
        for _ in range(3):
            lens = torch.randint(0, 3, (8,), generator=g)
            offs = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)]).int()
            f = {"u": torch.randint(1, 99, (8,), generator=g), "v": tn.data.Ragged(torch.randint(1, 99, (int(offs[-1]),), generator=g), offs)}
            y = torch.rand(8, generator=g)
            w.append(f, y)
            batches.append((f, y))
        with pytest.raises(ValueError, match="labels"):
            w.append(batches[0][0])
    for (f, y), (fb, yb) in zip(batches, tn.data.BatchCacheDataset(cache, pin_memory=False)):
        p = fb[tn.data.PACKED_KEY]
        assert p.values[:8].tolist() == f["u"].tolist() and p.offsets[:9].tolist() == list(range(9))
        assert p.values[8:].tolist() == f["v"].values.tolist()
        assert (p.offsets[8:] - 8).tolist() == f["v"].offsets.tolist()
        _same(y, yb)
    blob = open(cache, "rb").read()
    cut = str(tmp_path / "cut.tnbc")
    with open(cut, "wb") as fh:
        fh.write(blob[:-30])
    with pytest.raises(ValueError, match="not a batch cache"):
        list(tn.data.BatchCacheDataset(cut, pin_memory=False))


def test_training_from_the_cache_follows_training_from_the_records(tmp_path):
    files = []
    for k in range(2):
        p = str(tmp_path / f"tf-{k}")
        _records(p, 320, 10 + k)
        files.append(p)
    ds = tn.data.TFRecordDataset(files, 64, ["a", "b"], dense_keys={"x": 3}, packed=True, num_workers=2, pin_memory=False)
    cache = str(tmp_path / "c.tnbc")
    tn.data.write_batch_cache(cache, ds, ["a", "b"], dense_name="dense")
    assert os.path.getsize(cache) % 8 == 0
    tn.core.init()

    def train(data):
        torch.manual_seed(0)
        m = tn.models.DeepFM(["a", "b"], ["a", "b"], dnn_hidden_units=(16, 8), embedding_dim=4, dense_dim=3, bucket_size=1024,
                             sparse_opt=tn.core.AdaGrad(learning_rate=0.05, initial_g2sum=0.1, initial_scale=0.1), combiner="sum")
        m.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=5e-3)), loss="binary_crossentropy")
        return [float(m.train_on_batch(f, y)) for _ in range(3) for f, y in data]

    a, b = train(ds), train(tn.data.BatchCacheDataset(cache, pin_memory=False))
    assert a == b and a[-1] < a[0]


def test_any_mix_of_ragged_and_fixed_slots_survives_the_cache(tmp_path):
    """Property: whatever per-slot features go in (fixed [B], fixed [B, L], ragged with empty bags, any batch sizes),
    what comes back packs to the same ids and offsets."""
    from hypothesis import given, settings, strategies as st
    from tensornet_b200.data.features import gather_columns
    path = str(tmp_path / "p.tnbc")

    @settings(max_examples=40, deadline=None)
    @given(st.lists(st.tuples(st.integers(1, 9), st.integers(0, 2 ** 31)), min_size=1, max_size=4), st.integers(1, 3))
    def check(batches, S):
        keys = [f"k{s}" for s in range(S)]
        fed = []
        with tn.data.BatchCacheWriter(path, keys, label=False) as w:
            for B, seed in batches:
                g = torch.Generator().manual_seed(seed)
                f = {}
                for s, k in enumerate(keys):
                    kind = (seed + s) % 3
                    if kind == 0:
                        f[k] = torch.randint(-2 ** 62, 2 ** 62, (B,), generator=g)
                    elif kind == 1:
                        f[k] = torch.randint(0, 100, (B, 2), generator=g)
                    else:
                        lens = torch.randint(0, 4, (B,), generator=g)
                        offs = torch.cat([torch.zeros(1, dtype=torch.long), lens.cumsum(0)])
                        f[k] = tn.data.Ragged(torch.randint(0, 100, (int(offs[-1]),), generator=g), offs.int())
                w.append(f)
                fed.append(f)
        back = list(tn.data.BatchCacheDataset(path, pin_memory=False, threads=1))
        assert len(back) == len(fed)
        for f, (fb, yb) in zip(fed, back):
            assert yb is None
            ids, offs, B = gather_columns(f, keys, torch.device("cpu"))
            ids2, offs2, B2 = gather_columns(fb, keys, torch.device("cpu"))
            assert B == B2 and torch.equal(ids, ids2) and (offs is None) == (offs2 is None)
            if offs is not None:
                assert torch.equal(offs.int(), offs2.int())

    check()

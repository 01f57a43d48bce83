"""Input containers on the CPU path: packed slots (single-hot and ragged) are equivalent to one entry per slot, and the
loss helpers bring labels / weights / masks to the prediction's shape (tensornet/model/compile_utils.py)."""
import pytest
import torch

import tensornet_b200 as tn
from tensornet_b200.data import PACKED_KEY, PackedFeatures, Ragged


@pytest.fixture(autouse=True)
def _cpu_runtime():
    tn.core.shutdown()
    tn.core.config.force_cpu = True
    tn.core.init()
    yield
    tn.core.shutdown()


def _layer(keys, name):
    cols = [tn.feature_column.embedding_column(tn.feature_column.category_column(k, 64), 4, "sum") for k in keys]
    return tn.layers.EmbeddingFeatures(cols, tn.core.AdaGrad(learning_rate=0.1, initial_scale=1.0), name=name, is_concat=True)


def test_packed_single_hot_equals_per_slot_entries():
    keys = ["a", "b", "c"]
    ids = torch.tensor([[3, 4, 3, 9], [7, 7, 8, 1], [5, 6, 5, 6]])
    per_slot = _layer(keys, "t")({k: ids[i] for i, k in enumerate(keys)})
    packed = _layer(keys, "t2")({PACKED_KEY: PackedFeatures(keys, ids=ids)})
    assert per_slot.shape == (4, 12) and torch.allclose(per_slot, packed)      # rows are initialised from the sign alone
    sub = _layer(["c", "a"], "t3")({PACKED_KEY: PackedFeatures(keys, ids=ids)})       # a layer may read a subset
    assert torch.allclose(sub, torch.cat([per_slot[:, 8:12], per_slot[:, 0:4]], dim=1))


def test_packed_ragged_equals_ragged_entries():
    keys = ["a", "b"]
    a = Ragged(torch.tensor([1, 2, 3]), torch.tensor([0, 2, 2, 3]))            # bags [1,2] [] [3]
    b = Ragged(torch.tensor([9, 9, 4, 5]), torch.tensor([0, 1, 3, 4]))         # bags [9] [9,4] [5]
    per_slot = _layer(keys, "r")({"a": a, "b": b})
    values = torch.cat([a.values, b.values])
    offsets = torch.cat([a.offsets, b.offsets[1:] + a.offsets[-1]])
    packed = _layer(keys, "r2")({PACKED_KEY: PackedFeatures(keys, values=values, offsets=offsets, batch_size=3)})
    assert per_slot.shape == (3, 8) and torch.allclose(per_slot, packed)
    assert float(per_slot.detach()[1, :4].abs().sum()) == 0                     # the empty bag pools to zeros


def test_loss_helpers_shape_labels_weights_and_masks():
    y_p = torch.zeros(4, 1)
    y_t, _, sw = tn.model.match_dtype_and_rank(torch.tensor([1, 0, 1, 0]), y_p, torch.tensor([1, 2, 3, 4]))
    assert y_t.shape == (4, 1) and y_t.dtype == y_p.dtype and sw.shape == (4, 1) and sw.dtype == y_p.dtype
    mask = torch.tensor([[True], [False], [True], [True]])
    assert torch.equal(tn.model.apply_mask(y_p, sw, mask), torch.tensor([[1.0], [0.0], [3.0], [4.0]]))
    assert torch.equal(tn.model.apply_mask(y_p, None, mask), mask.float())
    assert tn.model.apply_mask(y_p, sw, None) is sw

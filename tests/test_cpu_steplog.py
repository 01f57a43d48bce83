"""Structured step log: window records on one CPU rank and the cross-rank merge rule."""
import json

import pytest
import torch

import tensornet_b200 as tn
from tensornet_b200 import models
from tensornet_b200.utils import StepLog, merge_rank_records


@pytest.fixture(autouse=True)
def _cpu_runtime():
    tn.core.shutdown()
    tn.core.config.force_cpu = True
    tn.core.init()
    yield
    tn.core.shutdown()


def test_merge_sums_examples_and_takes_the_slowest_rank():
    a = {"step": 100, "steps": 100, "examples": 800, "seconds": 1.0, "loss": 0.5, "ctr": 0.2, "pctr": 0.25,
         "tables": {"emb": {"rows": 30, "new_rows": 3, "load": 0.1}}}
    b = {"step": 100, "steps": 100, "examples": 200, "seconds": 2.0, "loss": 1.0, "ctr": 0.4, "pctr": 0.25,
         "tables": {"emb": {"rows": 10, "new_rows": 1, "load": 0.3}}}
    m = merge_rank_records([a, b])
    assert m["examples"] == 1000 and m["seconds"] == 2.0 and m["slowest_rank"] == 1
    assert m["examples_per_s"] == pytest.approx(500.0) and m["ms_per_step"] == pytest.approx(20.0)
    assert m["loss"] == pytest.approx(0.6) and m["ctr"] == pytest.approx(0.24) and m["copc"] == pytest.approx(0.96)
    assert m["tables"]["emb"] == {"rows": 40, "new_rows": 4, "max_load": 0.3, "largest_shard_share": 0.75}


def test_fit_writes_one_line_per_window(tmp_path):
    torch.manual_seed(0)
    slots = ["s1", "s2"]
    m = models.WideDeep(slots, slots, dnn_hidden_units=(8,), embedding_dim=4, bucket_size=64)
    m.compile(optimizer=tn.optimizer.Optimizer(tn.core.Adam(learning_rate=0.01)))
    g = torch.Generator().manual_seed(0)

    def batches(n):
        for _ in range(n):
            f = {s: torch.randint(1, 40, (32,), generator=g) for s in slots}
            yield f, (f["s1"] % 2 == 0).float()

    path = str(tmp_path / "log" / "train.jsonl")
    log = StepLog(path, every=5)
    m.fit(batches(13), callbacks=[log], prefetch=False)
    lines = [json.loads(l) for l in open(path)]
    # the first step of a pass starts the clock: 12 counted steps = two full windows and one of two steps
    assert [l["steps"] for l in lines] == [5, 5, 2] and [l["step"] for l in lines] == [5, 10, 12]
    assert lines == log.records
    for l in lines:
        assert l["world"] == 1 and l["examples"] == 32 * l["steps"] and l["examples_per_s"] > 0 and l["status"] == "ok"
        assert 0.0 <= l["ctr"] <= 1.0 and 0.0 < l["pctr"] < 1.0 and l["loss"] > 0
    t = lines[-1]["tables"]
    assert set(t) == {"linear_input", "deep_input"} and 0 < t["deep_input"]["rows"] <= 78
    assert sum(l["tables"]["deep_input"]["new_rows"] for l in lines) == t["deep_input"]["rows"]

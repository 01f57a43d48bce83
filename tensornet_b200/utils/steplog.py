"""Structured training log: one JSON line per window of steps, aggregated over all ranks.

The reference has no throughput counter beyond the Keras progress bar and logs table sizes only when a
checkpoint is written (core/ps/table/sparse_table.cc:102-108,132-136).  ``StepLog`` is a ``fit`` callback that
closes a window every ``every`` steps: it synchronises the device once, measures the window's wall time, reads
the running loss / CTR / PCTR / COPC sums and every sparse shard's row count, gathers the per-rank records on the
control-plane group and lets rank 0 append one line to a JSONL file (and keep it in ``records``).

Aggregation rules: examples and rows are summed over ranks, the step time is the maximum over ranks (the job
moves at the pace of its slowest rank), the load factor is the maximum over shards, the loss is the
example-weighted mean.
"""
from __future__ import annotations

import json
import os
import time
from typing import Dict, List, Optional

from .. import core
from ..callbacks import Callback
from ..parallel.symm import verify_all_arenas


def merge_rank_records(per_rank: List[Dict]) -> Dict:
    """Combine the records of one window (one dict per rank) into the job-wide record."""
    first = per_rank[0]
    examples = sum(r["examples"] for r in per_rank)
    seconds = max(r["seconds"] for r in per_rank)
    out = {
        "step": first["step"],
        "steps": first["steps"],
        "world": len(per_rank),
        "examples": examples,
        "seconds": seconds,
        "ms_per_step": 1e3 * seconds / max(first["steps"], 1),
        "examples_per_s": examples / seconds if seconds > 0 else 0.0,
        "loss": sum(r["loss"] * r["examples"] for r in per_rank) / max(examples, 1),
        "ctr": sum(r["ctr"] * r["examples"] for r in per_rank) / max(examples, 1),
        "pctr": sum(r["pctr"] * r["examples"] for r in per_rank) / max(examples, 1),
        "tables": {},
        "slowest_rank": max(range(len(per_rank)), key=lambda i: per_rank[i]["seconds"]),
    }
    out["copc"] = out["ctr"] / out["pctr"] if out["pctr"] > 0 else 0.0
    for name in first["tables"]:
        shards = [r["tables"][name] for r in per_rank]
        rows = sum(s["rows"] for s in shards)
        out["tables"][name] = {
            "rows": rows,
            "new_rows": sum(s["new_rows"] for s in shards),
            "max_load": max(s["load"] for s in shards),
            "largest_shard_share": max(s["rows"] for s in shards) / rows if rows else 0.0,
        }
    return out


class StepLog(Callback):
    """``model.fit(ds, callbacks=[StepLog("train.jsonl", every=100)])``."""

    def __init__(self, path: Optional[str] = None, every: int = 100):
        self.path = path
        self.every = max(int(every), 1)
        self.records: List[Dict] = []
        self._reset_window()
        self._rows_before: Dict[str, int] = {}
        self._step = 0

    def _reset_window(self):
        self._t0 = None
        self._steps = 0
        self._examples = 0

    # ------------------------------------------------------------------ fit hooks
    def on_train_begin(self, logs=None):
        self._reset_window()
        self._step = 0
        if self.path and core.runtime().rank == 0:
            os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)

    def on_train_batch_end(self, step: int, logs=None):
        if self._t0 is None:
            # the first step of a window starts the clock after the device has drained, so that a window never
            # pays for work queued before it
            self._sync()
            self._t0 = time.perf_counter()
            self._sums0 = self._metric_sums()
            return
        self._steps += 1
        self._step += 1
        self._examples += int((logs or {}).get("batch", 0))
        if self._steps >= self.every:
            self._close()

    def on_epoch_end(self, epoch, logs=None):
        if self._steps:
            self._close()
        self._t0 = None

    # ------------------------------------------------------------------ internals
    @staticmethod
    def _sync():
        rt = core.runtime()
        if rt.on_gpu:
            import torch

            torch.cuda.synchronize()

    def _metric_sums(self):
        s = self.model.metric_sums()
        return {"loss_sum": s["loss_sum"], "clicks": s["ctr"] * s["count"], "preds": s["pctr"] * s["count"], "count": s["count"]}

    def _tables(self) -> Dict[str, Dict]:
        out = {}
        for kind, m in self.model._tn_children():
            if kind != "sparse":
                continue
            t = m.table
            rows = int(t.n_rows)
            cap = int(getattr(t, "row_cap", 0))
            name = m.layer_name or str(m.sparse_table_handle)
            out[name] = {"rows": rows, "new_rows": rows - self._rows_before.get(name, 0), "load": rows / cap if cap else 0.0}
            self._rows_before[name] = rows
        return out

    def _close(self):
        self._sync()
        seconds = time.perf_counter() - self._t0
        now = self._metric_sums()
        n = max(now["count"] - self._sums0["count"], 0.0)
        # models that do not feed the running sums still report throughput from the batch sizes fit passes in
        examples = int(n) if n > 0 else self._examples
        rec = {
            "step": self._step,
            "steps": self._steps,
            "examples": examples,
            "seconds": seconds,
            "loss": (now["loss_sum"] - self._sums0["loss_sum"]) / self._steps if n > 0 else 0.0,   # sum of per-step means
            "ctr": (now["clicks"] - self._sums0["clicks"]) / n if n > 0 else 0.0,
            "pctr": (now["preds"] - self._sums0["preds"]) / n if n > 0 else 0.0,
            "tables": self._tables(),
        }
        rt = core.runtime()
        per_rank = rt.all_gather_object(rec) if rt.world > 1 else [rec]
        merged = merge_rank_records(per_rank)
        core.runtime().check_status()
        verify_all_arenas()
        merged["status"] = "ok"
        self.records.append(merged)
        if self.path and rt.rank == 0:
            with open(self.path, "a") as f:
                f.write(json.dumps(merged) + "\n")
        self._steps = 0
        self._examples = 0
        self._sums0 = now
        self._t0 = time.perf_counter()


__all__ = ["StepLog", "merge_rank_records"]

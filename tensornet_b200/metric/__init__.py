"""``tn.metric``: CTR (mean label), PCTR (mean prediction), COPC (sum label / sum prediction)
(tensornet/metric/metrics.py:31-104) and a streaming AUC (the reference's example compiles
``tf.keras.metrics.AUC``, examples/main.py:63-74).

Every metric can be driven two ways:

* ``update_state(y_true, y_pred, sample_weight=None)`` with tensors, as in Keras;
* ``feed(stats)`` with a :class:`BatchStats` delta.  ``tn.model.Model`` uses this one: its loss
  kernels keep the label / prediction sums and the two prediction histograms on the device, and
  the model hands the metrics what accumulated since the last hand-over.  A training step
  therefore costs the metrics nothing, however many are compiled in.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

AUC_BINS = 200


@dataclass
class BatchStats:
    """What accumulated on the device since the metrics were last fed."""
    loss_sum: float          # sum of the per-step mean losses
    label_sum: float
    pred_sum: float
    count: float             # examples
    steps: int
    pos_hist: Optional[torch.Tensor] = None     # float64 [bins] predictions of positive examples
    neg_hist: Optional[torch.Tensor] = None


class Metric:
    """Base class: a name, ``reset_state``, ``result`` and the two ways of feeding."""

    device_backed = False     # True: ``feed`` is enough, the model need not call ``update_state`` every step

    def __init__(self, name: str):
        self.name = name

    def reset_state(self):
        raise NotImplementedError

    def result(self) -> float:
        raise NotImplementedError

    def update_state(self, y_true, y_pred, sample_weight=None):
        raise NotImplementedError

    def feed(self, stats: BatchStats):
        raise NotImplementedError


class _Mean(Metric):
    device_backed = True

    def __init__(self, name):
        super().__init__(name)
        self.total, self.count = 0.0, 0.0

    def reset_state(self):
        self.total, self.count = 0.0, 0.0

    def result(self) -> float:
        return self.total / self.count if self.count else 0.0

    def _add(self, v: torch.Tensor, sample_weight=None):
        v = v.detach().float().reshape(-1)
        if sample_weight is not None:
            w = sample_weight.detach().float().reshape(-1)
            self.total += float((v * w).sum())
            self.count += float(w.sum())
        else:
            self.total += float(v.sum())
            self.count += float(v.numel())


class CTR(_Mean):
    """Average of the label."""

    def __init__(self, name="CTR", dtype=None):
        super().__init__(name)

    def update_state(self, y_true, y_pred, sample_weight=None):
        self._add(y_true, sample_weight)

    def feed(self, stats: BatchStats):
        self.total += stats.label_sum
        self.count += stats.count


class PCTR(_Mean):
    """Average of the prediction."""

    def __init__(self, name="PCTR", dtype=None):
        super().__init__(name)

    def update_state(self, y_true, y_pred, sample_weight=None):
        self._add(y_pred, sample_weight)

    def feed(self, stats: BatchStats):
        self.total += stats.pred_sum
        self.count += stats.count


class MeanLoss(_Mean):
    """Average of the per-step mean loss (what Keras reports as ``loss``)."""

    def __init__(self, name="loss"):
        super().__init__(name)

    def update_state(self, y_true, y_pred, sample_weight=None):
        p = y_pred.detach().float().reshape(-1).clamp(1e-7, 1 - 1e-7)
        y = y_true.detach().float().reshape(-1)
        self.total += float(-(y * p.log() + (1 - y) * (1 - p).log()).mean())
        self.count += 1.0

    def feed(self, stats: BatchStats):
        self.total += stats.loss_sum
        self.count += stats.steps


class COPC(Metric):
    """Click over predicted click: sum(label) / sum(prediction)."""

    device_backed = True

    def __init__(self, name="COPC", dtype=None):
        super().__init__(name)
        self.ctr_total, self.pctr_total = 0.0, 0.0

    def reset_state(self):
        self.ctr_total, self.pctr_total = 0.0, 0.0

    def update_state(self, y_true, y_pred, sample_weight=None):
        self.ctr_total += float(y_true.detach().float().sum())
        self.pctr_total += float(y_pred.detach().float().sum())

    def feed(self, stats: BatchStats):
        self.ctr_total += stats.label_sum
        self.pctr_total += stats.pred_sum

    def result(self) -> float:
        return self.ctr_total / self.pctr_total if self.pctr_total else 0.0


class AUC(Metric):
    """Area under the ROC curve from two histograms of the prediction (``num_thresholds`` buckets over [0, 1])."""

    device_backed = True

    def __init__(self, name="auc", num_thresholds: int = AUC_BINS):
        super().__init__(name)
        self.n = int(num_thresholds)
        self.pos = torch.zeros(self.n, dtype=torch.float64)
        self.neg = torch.zeros(self.n, dtype=torch.float64)

    def reset_state(self):
        self.pos.zero_()
        self.neg.zero_()

    def update_state(self, y_true, y_pred, sample_weight=None):
        p = y_pred.detach().float().reshape(-1).cpu().clamp(0, 1)
        y = y_true.detach().float().reshape(-1).cpu()
        idx = (p * self.n).long().clamp_(max=self.n - 1)
        self.pos += torch.bincount(idx[y > 0.5], minlength=self.n).double()
        self.neg += torch.bincount(idx[y <= 0.5], minlength=self.n).double()

    def feed(self, stats: BatchStats):
        if stats.pos_hist is None:
            raise RuntimeError("AUC.feed needs the prediction histograms; compile the model with this metric")
        if stats.pos_hist.numel() != self.n:
            raise ValueError(f"AUC has {self.n} buckets, the model accumulates {stats.pos_hist.numel()}")
        self.pos += stats.pos_hist
        self.neg += stats.neg_hist

    def result(self) -> float:
        tp = torch.flip(torch.cumsum(torch.flip(self.pos, [0]), 0), [0])
        fp = torch.flip(torch.cumsum(torch.flip(self.neg, [0]), 0), [0])
        P, N = self.pos.sum(), self.neg.sum()
        if P == 0 or N == 0:
            return 0.0
        tpr = torch.cat([tp / P, torch.zeros(1, dtype=torch.float64)])
        fpr = torch.cat([fp / N, torch.zeros(1, dtype=torch.float64)])
        return float(torch.trapz(torch.flip(tpr, [0]), torch.flip(fpr, [0])))


class _PerExample(Metric):
    """Mean over the examples of a value computed from (label, prediction): the metrics Keras knows by name, which
    the reference's example compiles as ``"acc", "mse", "mae", "mape"`` (examples/main.py:64-69).  They need the
    predictions of every step, so a model that compiles one runs its steps without CUDA graphs; sums are kept as
    tensors on the predictions' device and read when ``result()`` is called."""

    def __init__(self, name):
        super().__init__(name)
        self.reset_state()

    def reset_state(self):
        self._total, self._count = None, None

    def _value(self, y: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def update_state(self, y_true, y_pred, sample_weight=None):
        p = y_pred.detach().float().reshape(-1)
        y = y_true.detach().float().reshape(-1).to(p.device)
        v = self._value(y, p)
        if sample_weight is not None:
            w = sample_weight.detach().float().reshape(-1).to(p.device)
            s, c = (v * w).sum(), w.sum()
        else:
            s, c = v.sum(), torch.tensor(float(v.numel()), device=p.device)
        self._total = s if self._total is None else self._total + s
        self._count = c if self._count is None else self._count + c

    def result(self) -> float:
        if self._total is None:
            return 0.0
        c = float(self._count)
        return float(self._total) / c if c else 0.0


class BinaryAccuracy(_PerExample):
    """Share of examples whose prediction falls on the label's side of ``threshold``."""

    def __init__(self, name="acc", threshold: float = 0.5):
        super().__init__(name)
        self.threshold = threshold

    def _value(self, y, p):
        return ((p > self.threshold) == (y > 0.5)).float()


class MeanSquaredError(_PerExample):
    def __init__(self, name="mse"):
        super().__init__(name)

    def _value(self, y, p):
        return (y - p) ** 2


class MeanAbsoluteError(_PerExample):
    def __init__(self, name="mae"):
        super().__init__(name)

    def _value(self, y, p):
        return (y - p).abs()


class MeanAbsolutePercentageError(_PerExample):
    """``100 * |y - p| / max(|y|, 1e-7)``, as Keras defines it (large when labels are 0)."""

    def __init__(self, name="mape"):
        super().__init__(name)

    def _value(self, y, p):
        return 100.0 * (y - p).abs() / y.abs().clamp(min=1e-7)


_BY_NAME = {"auc": AUC, "ctr": CTR, "pctr": PCTR, "copc": COPC, "loss": MeanLoss,
            "acc": BinaryAccuracy, "accuracy": BinaryAccuracy, "binary_accuracy": BinaryAccuracy,
            "mse": MeanSquaredError, "mean_squared_error": MeanSquaredError,
            "mae": MeanAbsoluteError, "mean_absolute_error": MeanAbsoluteError,
            "mape": MeanAbsolutePercentageError, "mean_absolute_percentage_error": MeanAbsolutePercentageError}


def get(spec) -> Metric:
    """A metric object from an instance or one of the names ``auc / ctr / pctr / copc / loss`` (fed from the loss
    kernels' sums) and ``acc / mse / mae / mape`` with their long Keras names (computed from every step's
    predictions).  A name keeps its spelling as the metric's name."""
    if isinstance(spec, str):
        try:
            cls = _BY_NAME[spec.lower()]
            return cls(spec) if issubclass(cls, _PerExample) else cls()
        except KeyError:
            raise ValueError(f"unknown metric {spec!r}; pass an object with update_state / result") from None
    if not (hasattr(spec, "update_state") and hasattr(spec, "result")):
        raise TypeError("a metric needs update_state(y_true, y_pred, sample_weight) and result()")
    return spec


__all__ = ["Metric", "BatchStats", "CTR", "PCTR", "COPC", "AUC", "MeanLoss", "BinaryAccuracy", "MeanSquaredError",
           "MeanAbsoluteError", "MeanAbsolutePercentageError", "get", "AUC_BINS"]

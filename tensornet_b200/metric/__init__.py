"""``tn.metric``: CTR (mean label), PCTR (mean prediction), COPC (sum label / sum prediction)
(tensornet/metric/metrics.py:31-104) and a streaming AUC."""
from __future__ import annotations

import torch


class _Mean:
    def __init__(self, name):
        self.name = name
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


class PCTR(_Mean):
    """Average of the prediction."""

    def __init__(self, name="PCTR", dtype=None):
        super().__init__(name)

    def update_state(self, y_true, y_pred, sample_weight=None):
        self._add(y_pred, sample_weight)


class COPC:
    """Click over predicted click: sum(label) / sum(prediction)."""

    def __init__(self, name="COPC", dtype=None):
        self.name = name
        self.ctr_total, self.pctr_total = 0.0, 0.0

    def reset_state(self):
        self.ctr_total, self.pctr_total = 0.0, 0.0

    def update_state(self, y_true, y_pred, sample_weight=None):
        self.ctr_total += float(y_true.detach().float().sum())
        self.pctr_total += float(y_pred.detach().float().sum())

    def result(self) -> float:
        return self.ctr_total / self.pctr_total if self.pctr_total else 0.0


class AUC:
    """Histogram AUC with ``num_thresholds`` buckets (the example compiles ``tf.keras.metrics.AUC``,
    examples/main.py:63-74)."""

    def __init__(self, name="auc", num_thresholds: int = 200):
        self.name = name
        self.n = num_thresholds
        self.pos = torch.zeros(self.n, dtype=torch.float64)
        self.neg = torch.zeros(self.n, dtype=torch.float64)

    def reset_state(self):
        self.pos.zero_()
        self.neg.zero_()

    def update_state(self, y_true, y_pred, sample_weight=None):
        p = y_pred.detach().float().reshape(-1).cpu().clamp(0, 1)
        y = y_true.detach().float().reshape(-1).cpu()
        idx = (p * (self.n - 1)).long()
        self.pos += torch.bincount(idx[y > 0.5], minlength=self.n).double()
        self.neg += torch.bincount(idx[y <= 0.5], minlength=self.n).double()

    def result(self) -> float:
        tp = torch.flip(torch.cumsum(torch.flip(self.pos, [0]), 0), [0])
        fp = torch.flip(torch.cumsum(torch.flip(self.neg, [0]), 0), [0])
        P, N = self.pos.sum(), self.neg.sum()
        if P == 0 or N == 0:
            return 0.0
        tpr = torch.cat([tp / P, torch.zeros(1, dtype=torch.float64)])
        fpr = torch.cat([fp / N, torch.zeros(1, dtype=torch.float64)])
        return float(torch.trapz(torch.flip(tpr, [0]), torch.flip(fpr, [0])))


__all__ = ["CTR", "PCTR", "COPC", "AUC"]

"""Hyper-parameter objects returned by ``tn.core.AdaGrad / Adam / Ftrl``.

Same keyword names and defaults as the reference's pybind factories
(core/main/py_wrapper.cc:82-162); unlike the reference, unknown keywords are rejected.
``learning_rate`` may be a float or a callable schedule ``step -> float``; the sparse
kernels use the constant value (core/ps/optimizer/optimizer.h:57-64), the dense optimizer
evaluates the schedule every step (tensornet/optimizer/optimizer.py:30-36,69).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Union

from .config import config

KIND_ADAGRAD, KIND_ADAM, KIND_FTRL = 0, 1, 2


class OptimizerBase:
    name = "Base"
    kind = -1
    _defaults: Dict[str, Any] = {}

    def __init__(self, **kwargs):
        lr = kwargs.pop("learning_rate", 0.01)
        self.schedule: Union[None, Callable[[int], float]] = None
        if callable(lr):
            self.schedule = lr
            self.learning_rate = 0.01
        else:
            self.learning_rate = float(lr)
        unknown = set(kwargs) - set(self._defaults)
        if unknown:
            raise TypeError(f"{self.name}: unknown hyper-parameter(s) {sorted(unknown)}")
        for k, v in self._defaults.items():
            setattr(self, k, type(v)(kwargs.get(k, v)))
        self.sparse_zero_init = False
        self.validate()

    def validate(self):
        pass

    # -- lowering for the kernels ---------------------------------------------------
    def sparse_params(self) -> Dict[str, Any]:
        d = dict(kind=self.kind, lr=self.learning_rate, eps=getattr(self, "epsilon", 1e-8),
                 beta1=getattr(self, "beta1", 0.9), beta2=getattr(self, "beta2", 0.999),
                 initial_g2sum=getattr(self, "initial_g2sum", 0.0), initial_scale=self.initial_scale,
                 ftrl_beta=getattr(self, "beta", 1.0), lambda1=getattr(self, "lambda1", 0.0),
                 lambda2=getattr(self, "lambda2", 0.0), zero_init=int(self.sparse_zero_init),
                 seed=int(config.seed))
        return d

    def current_lr(self, step: int) -> float:
        return float(self.schedule(step)) if self.schedule is not None else self.learning_rate

    def get_config(self) -> Dict[str, Any]:
        """Name and hyper-parameters, enough for :func:`optimizer_from_config` to build the same optimizer again
        (a learning-rate schedule is code and is not part of it: the current base rate stands in)."""
        return {"name": self.name, "learning_rate": self.learning_rate, **{k: getattr(self, k) for k in self._defaults}}

    def __repr__(self):
        kv = ", ".join(f"{k}={getattr(self, k)!r}" for k in ["learning_rate", *self._defaults])
        return f"{self.name}({kv})"


class AdaGrad(OptimizerBase):
    name, kind = "AdaGrad", KIND_ADAGRAD
    _defaults = dict(show_decay_rate=0.98, show_threshold=0.0, initial_g2sum=0.0, initial_scale=1.0, epsilon=1e-8,
                     grad_decay_rate=1.0, mom_decay_rate=1.0, no_show_days=1000, elimination_logic=0)

    def validate(self):
        if self.elimination_logic not in (0, 1):
            raise ValueError(f"elimination_logic must be in the set of valid values {{0, 1}}, but got: {self.elimination_logic}")

    def delete_by_show(self, show: float, no_show_days: int) -> bool:
        if self.elimination_logic == 1:
            return show < self.show_threshold and no_show_days > self.no_show_days
        return show < self.show_threshold or no_show_days > self.no_show_days


class Adam(OptimizerBase):
    name, kind = "Adam", KIND_ADAM
    _defaults = dict(show_decay_rate=0.98, beta1=0.9, beta2=0.999, epsilon=1e-8, initial_scale=1.0)


class Ftrl(OptimizerBase):
    name, kind = "Ftrl", KIND_FTRL
    _defaults = dict(show_decay_rate=0.98, show_threshold=0.0, beta=1.0, lambda1=0.1, lambda2=1.0, initial_scale=1.0)


def optimizer_from_config(config: Dict[str, Any]) -> OptimizerBase:
    """The optimizer :meth:`OptimizerBase.get_config` described."""
    kw = dict(config)
    name = kw.pop("name")
    for cls in OptimizerBase.__subclasses__():
        if cls.name == name:
            return cls(**kw)
    raise ValueError(f"unknown optimizer {name!r}")

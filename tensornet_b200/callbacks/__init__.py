"""``tn.callbacks``: hooks that ``Model.fit / predict / evaluate`` call around their loops.

``PsWeightCheckpoint`` is the one the reference ships (tensornet/callbacks/callbacks.py:21-95):
it restores the parameter tables before a loop starts, re-arms the balanced dataset, ages the
show / click counters and writes a checkpoint when training ends, and keeps the ranks in step.
"""
from __future__ import annotations

from typing import Optional

from .. import core


class Callback:
    """Base class: every hook is optional.  ``model`` is set by the loop before the first hook fires."""

    model = None

    def set_model(self, model):
        self.model = model

    def on_train_begin(self, logs=None): ...
    def on_train_end(self, logs=None): ...
    def on_epoch_begin(self, epoch, logs=None): ...
    def on_epoch_end(self, epoch, logs=None): ...
    def on_predict_begin(self, logs=None): ...
    def on_predict_end(self, logs=None): ...
    def on_test_begin(self, logs=None): ...
    def on_test_end(self, logs=None): ...


class PsWeightCheckpoint(Callback):
    """Restore tables before a loop, save them after training.

    ``checkpoint_dir``       where checkpoints are read from (the directory holding ``_checkpoint``, or one
                             checkpoint itself when ``model_path_incl_dt``)
    ``checkpoint_save``      where they are written; defaults to ``checkpoint_dir``
    ``need_save_model``      write a checkpoint when training ends
    ``dt``                   name of the checkpoint sub-directory (a date in the day-by-day drivers)
    ``delta_days``           days since the previous pass: passed to ``show_decay`` before saving
    ``save_mode/load_mode``  ``"txt"`` or ``"bin"`` sparse blocks; ``load_mode`` defaults to ``save_mode``
    ``need_load_model``      restore before training / prediction / evaluation starts

    Order of operations (all ranks take part in every barrier):
    begin of fit / predict / evaluate: barrier, load, barrier, then barrier, dataset re-arm, barrier;
    end of every pass: barrier; end of training: barrier, show decay, save.
    """

    def __init__(self, checkpoint_dir: str, checkpoint_save: Optional[str] = None, need_save_model: bool = False,
                 dt: Optional[str] = None, delta_days: int = 0, save_mode: str = "txt", model_path_incl_dt: bool = False,
                 need_load_model: bool = True, load_mode: Optional[str] = None):
        self.checkpoint_dir = checkpoint_dir
        self.checkpoint_save = checkpoint_save or checkpoint_dir
        self.need_save_model = bool(need_save_model)
        self.need_load_model = bool(need_load_model)
        self.dt = dt
        self.delta_days = int(delta_days)
        self.save_mode = save_mode
        self.load_mode = load_mode or save_mode
        self.model_path_incl_dt = bool(model_path_incl_dt)

    # ------------------------------------------------------------------ building blocks
    def load_model(self):
        """Every rank restores its shards between two barriers, so no rank trains on while another still reads."""
        core.barrier()
        if self.need_load_model:
            self.model.load_weights(self.checkpoint_dir, include_dt=self.model_path_incl_dt, mode=self.load_mode)
        core.barrier()

    def reset_balance_dataset(self):
        """Forget which ranks ran out of input in the previous loop."""
        core.barrier()
        core.reset_balance_dataset()
        core.barrier()

    def _prepare(self):
        self.load_model()
        self.reset_balance_dataset()

    # ------------------------------------------------------------------ hooks
    def on_train_begin(self, logs=None):
        from ..optimizer import Optimizer

        if not isinstance(self.model.optimizer, Optimizer):
            raise TypeError("PsWeightCheckpoint needs a model compiled with tn.optimizer.Optimizer (it owns the dense table)")
        self._prepare()

    def on_predict_begin(self, logs=None):
        self._prepare()

    def on_test_begin(self, logs=None):
        self._prepare()

    def on_epoch_end(self, epoch, logs=None):
        core.barrier()

    def on_predict_end(self, logs=None):
        core.barrier()

    def on_test_end(self, logs=None):
        core.barrier()

    def on_train_end(self, logs=None):
        core.barrier()
        self.model.show_decay(self.delta_days)
        if self.need_save_model:
            self.model.save_weights(self.checkpoint_save, dt=self.dt or "", mode=self.save_mode)


class ProfileBatches(Callback):
    """Record a timeline of a few training steps: the role of the TensorBoard callback with
    ``profile_batch="50,60"`` in the reference's driver (examples/main.py:76-79).

    Steps ``start`` .. ``stop`` (counted from 0 over the whole ``fit`` call) run under ``torch.profiler`` with
    CPU and CUDA activities; the Chrome trace (``chrome://tracing``, Perfetto) goes to
    ``<log_dir>/trace_rank<r>.json``.  Phases of a step carry NVTX / record-function names, so the pull, tower,
    push and dense-update ranges can be told apart on the timeline."""

    def __init__(self, log_dir: str, start: int = 50, stop: int = 60):
        if stop < start:
            raise ValueError("ProfileBatches: stop must not precede start")
        self.log_dir, self.start, self.stop = log_dir, int(start), int(stop)
        self._prof = None
        self._seen = 0
        self.trace_path = None

    def on_train_begin(self, logs=None):
        self._seen = 0

    def _begin(self):
        import torch
        from torch import profiler

        acts = [profiler.ProfilerActivity.CPU]
        if core.runtime().on_gpu:
            acts.append(profiler.ProfilerActivity.CUDA)
            torch.cuda.synchronize()
        self._prof = profiler.profile(activities=acts)
        self._prof.__enter__()

    def _end(self):
        import os
        import torch

        if core.runtime().on_gpu:
            torch.cuda.synchronize()
        self._prof.__exit__(None, None, None)
        os.makedirs(self.log_dir, exist_ok=True)
        self.trace_path = os.path.join(self.log_dir, f"trace_rank{core.runtime().rank}.json")
        self._prof.export_chrome_trace(self.trace_path)
        self._prof = None

    def on_train_batch_end(self, step, logs=None):
        # called after step `_seen`; the profiler is switched on after step start-1 and off after step stop
        self._seen += 1
        if self._prof is None and self._seen == self.start and self.trace_path is None:
            self._begin()
        elif self._prof is not None and self._seen > self.stop:
            self._end()

    def on_train_end(self, logs=None):
        if self._prof is not None:
            self._end()


__all__ = ["Callback", "PsWeightCheckpoint", "ProfileBatches"]

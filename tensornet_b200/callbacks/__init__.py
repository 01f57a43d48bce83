"""``tn.callbacks.PsWeightCheckpoint`` (tensornet/callbacks/callbacks.py:21-95): load the last
checkpoint before training / prediction, decay show counters and save after training, and
keep the ranks in step with barriers."""
from __future__ import annotations

from .. import core


class Callback:
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
    """Save ps weight after every fit."""

    def __init__(self, checkpoint_dir, checkpoint_save=None, need_save_model=False, dt=None, delta_days=0,
                 save_mode="txt", model_path_incl_dt=False, **kwargs):
        self.checkpoint_dir = checkpoint_dir
        self.checkpoint_save = checkpoint_save if checkpoint_save else checkpoint_dir
        self.need_save_model = need_save_model
        self.need_load_model = kwargs.get("need_load_model", True)
        self.save_mode = save_mode
        self.load_mode = kwargs.get("load_mode", self.save_mode)
        self.model_path_incl_dt = model_path_incl_dt
        self.dt = dt
        self.delta_days = delta_days

    def load_model(self):
        core.barrier()
        if self.need_load_model:
            self.model.load_weights(self.checkpoint_dir, include_dt=self.model_path_incl_dt, mode=self.load_mode)
        core.barrier()

    def reset_balance_dataset(self):
        core.barrier()
        core.reset_balance_dataset()
        core.barrier()

    def on_train_begin(self, logs=None):
        from ..optimizer import Optimizer

        assert isinstance(self.model.optimizer, Optimizer)
        self.load_model()
        self.reset_balance_dataset()

    def on_train_end(self, logs=None):
        core.barrier()
        self.model.show_decay(self.delta_days)
        if not self.need_save_model:
            return
        self.model.save_weights(self.checkpoint_save, dt=self.dt or "", mode=self.save_mode)

    def on_predict_begin(self, logs=None):
        self.load_model()
        self.reset_balance_dataset()

    def on_predict_end(self, logs=None):
        core.barrier()

    def on_test_begin(self, logs=None):
        self.load_model()
        self.reset_balance_dataset()

    def on_test_end(self, logs=None):
        core.barrier()

    def on_epoch_end(self, epoch, logs=None):
        core.barrier()


__all__ = ["Callback", "PsWeightCheckpoint"]

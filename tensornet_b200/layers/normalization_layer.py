"""Batch normalisation driven by GLOBAL statistics (tensornet/layers/normalization_layer.py:26-242).

Every training batch contributes its per-feature sum / squared sum / count to the BN table;
the layer always normalises with the table's global mean and variance (treated as
constants, so no gradient flows through the statistics).  With ``synchronized=True`` the
increments are exchanged between ranks every ``sync_freq`` batches; otherwise rank 0 gathers
them once before saving.  ``PCTRDNNBatchNormalization`` accumulates the squared deviation
from the current global mean instead of the raw squared sum.
"""
from __future__ import annotations

import torch
from torch import nn

from .. import core


class _BnApply(torch.autograd.Function):
    """y = (x - mean) * rsqrt(var + eps) * gamma + beta with the table's moments as constants, as the reference's
    layer does (tensornet/layers/normalization_layer.py:149-156): no gradient flows into the statistics."""

    @staticmethod
    def forward(ctx, x, gamma, beta, table, eps):
        y = torch.empty_like(x)
        mean, var = table.mean.clone(), table.var.clone()      # the table moves on before the backward pass runs
        table.ctx.apply_fwd(x, mean, var, gamma, beta, float(eps), y)
        ctx.save_for_backward(x, gamma, mean, var)
        ctx.table, ctx.eps, ctx.has_beta = table, float(eps), beta is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gamma, mean, var = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x) if ctx.needs_input_grad[0] else None
        gg = torch.zeros_like(gamma) if gamma is not None else None
        gb = torch.zeros(x.shape[1], dtype=torch.float32, device=x.device) if ctx.has_beta else None
        ctx.table.ctx.apply_bwd(dy, x, mean, var, gamma, ctx.eps, dx, gg, gb)
        return dx, gg, gb, None, None


class TNBatchNormalizationBase(nn.Module):
    _USE_PCTR_DNN_BN = False

    def __init__(self, num_features: int = 0, center=True, scale=True, epsilon=1e-5, momentum=0.99, name=None,
                 synchronized=False, sync_freq=1, max_count=100000):
        super().__init__()
        self.center, self.scale, self.epsilon, self.momentum = center, scale, epsilon, momentum
        self.synchronized, self.sync_freq, self.max_count = synchronized, sync_freq, max_count
        self.layer_name = name or "tn_batch_normalization"
        self.batch_counter = 0
        self.bn_table_handle = None
        self.gamma = self.beta = None
        if num_features:
            self._build(num_features)

    def _build(self, c: int):
        dev = core.runtime().device
        self.num_features = c
        if self.scale:
            self.gamma = nn.Parameter(torch.ones(c, device=dev))
        if self.center:
            self.beta = nn.Parameter(torch.zeros(c, device=dev))
        self.register_buffer("moving_mean", torch.zeros(c, device=dev))
        self.register_buffer("moving_variance", torch.ones(c, device=dev))
        self.bn_table_handle = core.create_bn_table(self.layer_name, c, self.synchronized, self.momentum, self.max_count,
                                                    self._USE_PCTR_DNN_BN)
        self.table = core.bn_table(self.bn_table_handle)
        self.table.handle = self.bn_table_handle
        self._on_device = hasattr(self.table, "push_batch")
        if self._on_device:
            self.moving_mean = self.table.mean
            self.moving_variance = self.table.var

    # ---- table plumbing --------------------------------------------------------------------
    def _local_stats(self, x: torch.Tensor, center=None):
        x2 = x.detach().reshape(-1, x.shape[-1]).double()
        s = x2.sum(dim=0)
        q = ((x2 - center.double()) ** 2).sum(dim=0) if center is not None else (x2 * x2).sum(dim=0)
        n = torch.full_like(s, float(x2.shape[0]))
        return s.cpu().numpy(), q.cpu().numpy(), n.cpu().numpy()

    def bn_statistics_push(self, stats, synchronized: bool):
        self.table.append(*stats, is_local=True)
        if synchronized:
            self.table.sync_increments()

    def _push_counted(self, stats):
        if self.synchronized:
            self.batch_counter += 1
            if self.batch_counter == self.sync_freq:
                self.bn_statistics_push(stats, True)
                self.batch_counter = 0
            else:
                self.bn_statistics_push(stats, False)
        else:
            self.bn_statistics_push(stats, False)

    def update_moments(self):
        if self._on_device:
            return          # moving_mean / moving_variance alias the table's device arrays
        mean, var = self.table.get_moments()
        self.moving_mean.copy_(torch.from_numpy(mean))
        self.moving_variance.copy_(torch.from_numpy(var))

    # ---- device path: statistics, table update and normalisation without leaving the GPU ------
    def _device_push(self, x2: torch.Tensor, centered: bool):
        self.table.push_batch(x2, centered)
        if self.synchronized:
            if torch.cuda.is_current_stream_capturing():
                # a captured step replays the same launches every time, so the exchange cannot run every
                # sync_freq-th step only: inside a CUDA graph it runs every step (one small kernel)
                self.table.sync_increments()
                self.batch_counter = 0
                return
            self.batch_counter += 1
            if self.batch_counter == self.sync_freq:
                self.table.sync_increments()
                self.batch_counter = 0

    def _device_forward(self, inputs: torch.Tensor, training: bool, centered: bool):
        x2 = inputs.reshape(-1, inputs.shape[-1])
        if x2.dtype != torch.float32 or x2.stride(-1) != 1:
            x2 = x2.float().contiguous()
        if training and not centered:
            self._device_push(x2.detach(), False)
        y = _BnApply.apply(x2, self.gamma, self.beta, self.table, self.epsilon)
        if training and centered:
            self._device_push(x2.detach(), True)
        return y.view(*inputs.shape[:-1], inputs.shape[-1])

    def bn_statistics_pull(self):
        """Fold the other ranks' pending increments in (called by rank 0 before saving)."""
        if not self.synchronized or self.sync_freq > 1:
            self.batch_counter = 0
            self.table.sync_increments()
            self.update_moments()

    def _normalize(self, x):
        y = (x - self.moving_mean) * torch.rsqrt(self.moving_variance + self.epsilon)
        if self.gamma is not None:
            y = y * self.gamma
        if self.beta is not None:
            y = y + self.beta
        return y

    def forward(self, inputs: torch.Tensor, training=None):
        if self.bn_table_handle is None:
            self._build(inputs.shape[-1])
        training = self.training if training is None else training
        if self._on_device:
            return self._device_forward(inputs, training, False)
        if training:
            self._push_counted(self._local_stats(inputs))
            self.update_moments()
        return self._normalize(inputs)

    def save_bn_table(self, filepath):
        return core.save_bn_table(self.bn_table_handle, filepath)

    def load_bn_table(self, filepath):
        core.load_bn_table(self.bn_table_handle, filepath)
        self.update_moments()

    def get_config(self) -> dict:
        """Constructor arguments as plain data (normalization_layer.py:185-198)."""
        return {"name": self.layer_name, "center": self.center, "scale": self.scale, "epsilon": self.epsilon,
                "momentum": self.momentum, "synchronized": self.synchronized, "sync_freq": self.sync_freq,
                "max_count": self.max_count}


class TNBatchNormalization(TNBatchNormalizationBase):
    """var = squared_sum / count - (sum / count)^2"""


class PCTRDNNBatchNormalization(TNBatchNormalizationBase):
    """Accumulates sum and the squared deviation from the current global mean."""
    _USE_PCTR_DNN_BN = True

    def forward(self, inputs: torch.Tensor, training=None):
        if self.bn_table_handle is None:
            self._build(inputs.shape[-1])
        training = self.training if training is None else training
        if self._on_device:
            return self._device_forward(inputs, training, True)
        self.update_moments()
        if training:
            self._push_counted(self._local_stats(inputs, center=self.moving_mean))
        return self._normalize(inputs)

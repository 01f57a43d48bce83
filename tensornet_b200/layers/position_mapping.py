"""``PositionMappingLayer`` (tensornet/layers/position_mapping.py:21-68): one-hot of a position id
against a fixed list while training; at inference the position is unknown and slot 0 is used."""
from __future__ import annotations

import torch
from torch import nn


class PositionMappingLayer(nn.Module):
    def __init__(self, position_array):
        super().__init__()
        assert len(position_array) > 0, "position array must be not empty"
        self._position_array = list(position_array)
        self._position_number = len(position_array)
        self.register_buffer("_position_slot_tensor", torch.tensor(self._position_array, dtype=torch.int64))

    def forward(self, inputs, training=None):
        training = self.training if training is None else training
        values = inputs[0] if isinstance(inputs, (tuple, list)) else inputs
        values = values.reshape(-1).to(self._position_slot_tensor.device)
        n = values.shape[0]
        if training:
            eq = values.unsqueeze(1) == self._position_slot_tensor.unsqueeze(0)
            if not bool(eq.any(dim=1).all()):
                raise ValueError("inputs contains no existing value from provided position array")
            return eq.float()
        out = torch.zeros(n, self._position_number, device=values.device)
        out[:, 0] = 1.0
        return out

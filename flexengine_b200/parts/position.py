"""Rotary position encoding, half-split ("rotate_half") form.

inv_freq[j] = 1 / theta^(2j/d), angle = position * inv_freq in float32, pairs (i, i + d/2)
(src/flexengine/inference/models/qwen2.py:15-17,46,73-77).  The table is handed to the
mixer's fused bias+rotation+cache-write kernel; the angle, sine and cosine are
computed there in float32.
"""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_position


class RotaryHalfSplit(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, rotary_dim: int | None = None):
        self.head_dim = int(head_dim)
        self.theta = float(theta)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self._table = {}

    def rotary_table(self, device):
        key = str(device)
        if key not in self._table:
            # Same expression as the reference, evaluated in float32.
            exponent = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
            inv_freq = 1.0 / self.theta ** exponent
            self._table[key] = inv_freq.to(device).contiguous()
        return self._table[key], self.rotary_dim


class NoPosition(PositionEncoding):
    """No position encoding: queries and keys are used as projected."""

    def __init__(self, **_):
        pass


register_position("rope_half_split", RotaryHalfSplit)
register_position("none", NoPosition)

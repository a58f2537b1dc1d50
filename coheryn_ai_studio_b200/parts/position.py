"""Rotary position encoding with rotate-half pairing (element i with i + rotary_dim/2).

The angles follow crates/coheryn-engine/src/cpu.rs:58-73 exactly: in float32,
``step = theta ** (-2 / head_dim)``, ``angle_0 = position`` and
``angle_{i+1} = angle_i * step`` (an iterated product, not ``position * theta**(-2i/d)``;
the two differ by about 1e-4 at a few hundred positions).  cos and sin of every
(position, pair) are tabulated once when the model is built; the kernels only look
them up.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import Position, Runtime, register_position


class RotateHalfRope(Position):
    def __init__(self, runtime: Runtime, head_dim: int, rotary_dim: int, theta: float,
                 max_positions: int):
        super().__init__(runtime)
        if rotary_dim % 2 or not 0 < rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        self.head_dim, self.rotary_dim = int(head_dim), int(rotary_dim)
        self.theta, self.max_positions = float(theta), int(max_positions)
        self._table = None

    def angle_table(self) -> np.ndarray:
        """float32 [max_positions, rotary_dim/2] of angles, by the iterated product."""
        half = self.rotary_dim // 2
        step = np.float32(np.power(np.float32(self.theta), np.float32(-2.0) / np.float32(self.rotary_dim)))
        angles = np.empty((self.max_positions, half), dtype=np.float32)
        a = np.arange(self.max_positions, dtype=np.float32)
        for i in range(half):
            angles[:, i] = a
            a = (a * step).astype(np.float32)
        return angles

    def cos_sin(self) -> torch.Tensor:
        """float32 [max_positions, rotary_dim/2, 2] = (cos, sin) on the device."""
        if self._table is None:
            ang = self.angle_table()
            t = np.stack([np.cos(ang, dtype=np.float32), np.sin(ang, dtype=np.float32)], axis=-1)
            self._table = torch.from_numpy(np.ascontiguousarray(t)).to(self.runtime.device)
        return self._table


register_position("rope_rotate_half", RotateHalfRope)

"""Rotary position encoding: the table of inverse frequencies."""
from __future__ import annotations

import numpy as np
import torch

from .base import POSITIONS, PositionEncoding


def inv_freq_f32(rotary_dim: int, theta: float) -> np.ndarray:
    """1 / theta^(2i / d) for i < d/2, computed on the host in float32 with theta narrowed to
    float32 first (x0ne-core/runtime/src/ops.rs:210-214, x0ne-core/runtime/src/engine.rs:351)."""
    t = np.float32(theta)
    d = np.float32(rotary_dim)
    return np.array([np.float32(1.0) / np.power(t, np.float32(2 * i) / d, dtype=np.float32)
                     for i in range(rotary_dim // 2)], dtype=np.float32)


class Rope(PositionEncoding):
    """Rotate-half RoPE over the first `rotary_dim` values of each head: the pair
    (i, i + rotary_dim/2) turns by pos * inv_freq[i] (x0ne-core/kernels/cuda/rope.cu:28-31).
    The rotation itself runs inside the mixer's fused kernel; this part owns the table.
    Parameters: head_dim, rotary_dim, theta."""

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.theta = float(spec["theta"])
        self.table = torch.from_numpy(inv_freq_f32(self.rotary_dim, self.theta)).to(env.device)

    def rotary(self):
        return self.table, self.rotary_dim


class NoPosition(PositionEncoding):
    """No position encoding: mixers leave q and k unrotated."""


POSITIONS.register("rope", Rope)
POSITIONS.register("none", NoPosition)

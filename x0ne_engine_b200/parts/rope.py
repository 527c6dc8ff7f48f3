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
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.theta = float(spec["theta"])
        self.inv_freq = inv_freq_f32(self.rotary_dim, self.theta)
        self.table = torch.from_numpy(self.inv_freq).to(env.device)
        self._cos_sin = None

    def rotary(self):
        return self.table, self.rotary_dim

    def cos_sin_table(self, positions: int):
        """float32 [positions, rotary_dim]: cos then sin of the float32 angle position * inv_freq[i],
        made once on the host; mixers pass it to the fused kernel so that it reads two short rows
        instead of computing the row's sines and cosines for every head."""
        if self._cos_sin is None or self._cos_sin.shape[0] < positions:
            pos = np.arange(positions, dtype=np.float32)[:, None]
            ang = (pos * self.inv_freq[None, :]).astype(np.float32).astype(np.float64)
            tab = np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)
            self._cos_sin = torch.from_numpy(tab).to(self.env.device)
        return self._cos_sin


class NoPosition(PositionEncoding):
    """No position encoding: mixers leave q and k unrotated."""
    replayable = True


POSITIONS.register("rope", Rope)
POSITIONS.register("none", NoPosition)

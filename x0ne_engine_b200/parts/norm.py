"""RMSNorm with the residual add fused in front of it."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .base import NORMS, Norm


class RMSNorm(Norm):
    """out = r * rsqrt(mean(r^2) + eps) * w with r = resid + delta, in float32; eps inside the
    root, the weight multiplies directly (x0ne-core/kernels/cuda/rmsnorm.cu:11-20).
    Parameters: size, eps, names.weight."""
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.weight = None

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        return [TensorNeed(spec["names"]["weight"], (int(spec["size"]),), role="vector", init="norm")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.spec["names"]["weight"]]

    def add_norm(self, ctx, resid, delta, out, n_rows, rows=None):
        ops.add_rmsnorm(resid, delta, self.weight, out, n_rows, self.eps, rows)


NORMS.register("rmsnorm", RMSNorm)

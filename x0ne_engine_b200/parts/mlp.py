"""Dense SwiGLU feed-forward."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .base import FEED_FORWARDS, FeedForward
from .linear import Linear


class SwiGLU(FeedForward):
    """down( silu(gate x) * up x ): one product on the packed [gate; up] weight (gate rows, then
    up rows: x0ne-core/runtime/src/weights.rs:218-219), the activation
    g / (1 + expf(-g)) * u (x0ne-core/kernels/cuda/swiglu.cu:5-11), one product with down.
    Parameters: hidden_size, intermediate_size, names.{gate, up, down}."""
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.gate_up = None
        self.down = None

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        h, i, n = int(spec["hidden_size"]), int(spec["intermediate_size"]), spec["names"]
        return [TensorNeed(n["gate"], (i, h)), TensorNeed(n["up"], (i, h)), TensorNeed(n["down"], (h, i))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.spec["names"]
        self.gate_up = Linear(torch.cat([tensors[n["gate"]], tensors[n["up"]]], dim=0).contiguous())
        self.down = Linear(tensors[n["down"]])

    def weight_bytes(self) -> int:
        return self.gate_up.weight_bytes() + self.down.weight_bytes()

    def forward(self, ctx, x, n_rows):
        gu = ctx.ws.buffer("ffn.gate_up", (ctx.ws.max_rows, 2 * self.inter), self.env.dtype)
        act = ctx.ws.buffer("ffn.act", (ctx.ws.max_rows, self.inter), self.env.dtype)
        out = ctx.ws.buffer("delta", (ctx.ws.max_rows, self.hidden), self.env.dtype)
        kernel = ops.product_kernel(self.gate_up.weight, n_rows, fused=True)       # the routing table (csrc/routes.py)
        if kernel == "skinny":
            ops.gemm_bf16_skinny_tcgen05(x, self.gate_up.weight, act, n_rows, swiglu=True)   # 9 to 64 rows, tcgen05
        elif kernel == "smallm":
            ops.gemm_bf16_smallm(x, self.gate_up.weight, act, n_rows, swiglu=True)     # activation in the epilogue
        elif kernel == "tc_pair":
            ops.gemm_bf16_tcgen05(x, self.gate_up.weight, act, n_rows, swiglu=True)    # tcgen05, activation in the epilogue
        else:
            self.gate_up(x, gu, n_rows)
            ops.swiglu(gu, act, n_rows)
        self.down(act, out, n_rows)
        return out


FEED_FORWARDS.register("swiglu", SwiGLU)

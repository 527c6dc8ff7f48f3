"""Matrix products y = x W^T for weights stored [out, in] (row-major, as checkpoints hold them).

float32: this library's own fixed-order FMA kernel, so a row's result does not depend on the
batch it is in.  bfloat16: float32 accumulation with a bfloat16 or float32 result; the
library engine delegates these products to cuBLAS (x0ne-core/runtime/src/gpu.rs:1098-1149), and
`Linear` does the same through torch.mm unless one of this library's own kernels takes the shape.
"""
from __future__ import annotations

import torch

from ..csrc import ops


class Linear:
    def __init__(self, weight: torch.Tensor):
        if weight.dim() != 2 or not weight.is_contiguous():
            raise ValueError("a Linear weight is a contiguous [out, in] matrix")
        self.weight = weight
        self.out_features, self.in_features = weight.shape

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def __call__(self, x: torch.Tensor, out: torch.Tensor, m: int) -> torch.Tensor:
        """out[:m] = x[:m] @ W^T.  `out` has the dtype of x, or float32 (logits)."""
        w = self.weight
        if w.dtype == torch.float32:
            ops.gemm_f32_nt(x, w, out, m)
            return out
        if w.dtype != torch.bfloat16:
            raise ops.KernelError(f"no matrix product for weights of {w.dtype}")
        if out.dtype == torch.float32:
            # logits: the weight-streaming kernel for a handful of rows, else the library (the vocabulary's
            # 1,187 tiles of 128 rows are 4.01 waves of the few-row tcgen05 kernel's blocks: 247 us against
            # 203 us at 12 rows)
            kernel = "smallm" if m <= 8 and ops.gemm_smallm_takes(w, m) else "library"
        else:
            kernel = ops.product_kernel(w, m)          # the routing table (csrc/routes.py)
        if kernel == "smallm":
            ops.gemm_bf16_smallm(x, w, out, m)
        elif kernel == "skinny":
            ops.gemm_bf16_skinny_tcgen05(x, w, out, m)
        elif m > 0:
            if out.dtype == torch.bfloat16:
                torch.mm(x[:m], w.t(), out=out[:m])
            else:
                torch.mm(x[:m], w.t(), out_dtype=torch.float32, out=out[:m])
        return out

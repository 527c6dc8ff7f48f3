"""Which kernel runs a bfloat16 product y = x W^T: ONE table, keyed by the rows of x and the shape of W.

What a kernel CAN take is the kernel's business (`ops.gemm_*_takes`); what is USED lives here, so
that a new size of model changes a row of a table and not a constant inside a part.  Every rule names
the measurement behind it: kernel times on one B200 at the projection matrices of the 1.7B, 8B and
32B sizes of the architecture, rows 1 to 64 (`profiles/small_row_products_by_shape.md`), and the
gate/up product at 64 to 2,048 rows.  The library engine has no such choice to make: it gives every
product to cublasGemmEx (x0ne-core/runtime/src/gpu.rs:1098-1149).

Kernels: "smallm" streams W once through mma.sync with the rows as the narrow operand (up to 32
rows; gemm_bf16.cu); "skinny" is the tcgen05 product for 9 to 64 rows whose blocks cut K over a
cluster (gemm_skinny_tcgen05.cu); "tc_pair" the tcgen05 product for many rows on pairs of blocks
(gemm_tcgen05.cu); "library" is cuBLAS through torch.mm (followed by the SwiGLU kernel where the
product is gate|up).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Tuple

MB = 1 << 20


@dataclass(frozen=True)
class Shape:
    """What the rules look at: W is [n, k] (for gate|up: n = 2 x intermediate), bfloat16."""
    n: int
    k: int
    sms: int = 148

    @property
    def weight_bytes(self) -> int:
        return 2 * self.n * self.k

    @property
    def long_rows(self) -> bool:
        """K at least twice N (a down projection): every block streams long enough to pay for a cluster's merge."""
        return self.k >= 2 * self.n

    @property
    def smallm_fill(self) -> float:
        """The share of the GPU's resident blocks (two per SM) that the weight-streaming kernel puts to
        work: it hands out tiles of 16 weight rows, the same number to every block."""
        tiles = (self.n + 15) // 16
        resident = 2 * self.sms
        per_block = (tiles + resident - 1) // resident
        return ((tiles + per_block - 1) // per_block) / resident


@dataclass(frozen=True)
class Rule:
    kernel: str
    rows: Tuple[int, int]                       # inclusive
    fused: Optional[bool]                       # True: gate|up with the SwiGLU epilogue only; False: plain only; None: both
    when: Callable[[Shape], bool]
    why: str


def _always(s: Shape) -> bool:
    return True


# First match wins.  Sizes in the notes: N x K of W.
RULES: List[Rule] = [
    # ---- up to 8 rows
    Rule("library", (1, 8), False, lambda s: s.weight_bytes >= 64 * MB and s.smallm_fill < 0.6,
         "5120 x 25600 at 8 rows: library 44.6 us, smallm 60.6; 5120 x 8192: 17.0 against 20.4 (320 tiles are two rounds "
         "of 160 blocks: half the GPU streams)"),
    Rule("smallm", (1, 8), None, _always,
         "4096 x 4096 at 8 rows: 7.1 us against 12.2 (library); 4096 x 12288: 20.2 against 31.1; 2048 x 2048: 3.3 against 7.4; "
         "gate|up 24576 x 4096 with the activation: 35.6 against 36.1 + the SwiGLU launch"),
    # ---- 9 to 16 rows
    Rule("smallm", (9, 16), True, lambda s: s.weight_bytes < 64 * MB,
         "gate|up 12288 x 2048 at 16 rows: smallm 12.1 us, skinny 13.8, library 11.0 + the SwiGLU launch"),
    Rule("skinny", (9, 16), True, lambda s: s.weight_bytes >= 2 * MB,
         "gate|up 24576 x 4096 at 16 rows: skinny 35.3 us, smallm 37.7, library 36.4 + the SwiGLU launch; 51200 x 5120: 85.6 / 91.8 / 89.8"),
    Rule("skinny", (9, 16), False, lambda s: s.long_rows and s.weight_bytes >= 2 * MB,
         "2048 x 6144 at 16 rows: skinny 8.8 us, smallm 10.8, library 10.3; 4096 x 12288: 18.9 / 23.4 / 21.2"),
    Rule("smallm", (9, 16), False, lambda s: s.weight_bytes < 32 * MB,
         "4096 x 2048 at 16 rows: smallm 5.5 us, library 5.9, skinny 7.1; 2048 x 2048: 4.3 / 5.5 / 5.3"),
    Rule("skinny", (9, 16), False, lambda s: s.weight_bytes >= 2 * MB,
         "6144 x 4096 at 16 rows: skinny 11.4 us, library 12.0, smallm 14.9; 5120 x 8192: 16.4 / 19.0 / 26.0"),
    # ---- 17 to 64 rows
    Rule("skinny", (17, 64), True, lambda s: s.weight_bytes >= 2 * MB,
         "gate|up 24576 x 4096 at 32 rows: skinny 36.2 us, library 36.7 + the SwiGLU launch; at 64: 38.1 = 38.1 + the launch"),
    Rule("skinny", (17, 64), False, lambda s: s.long_rows and s.weight_bytes >= 2 * MB,
         "4096 x 12288 at 64 rows: skinny 20.8 us, library 21.8; 5120 x 25600: 44.3 / 46.8; 2048 x 6144: 10.2 / 10.6"),
    Rule("skinny", (17, 48), False, lambda s: s.weight_bytes >= 64 * MB,
         "10240 x 5120 at 32 rows: skinny 20.1 us, library 21.1; 5120 x 8192: 17.0 / 19.4; at 64 rows the library is ahead on both"),
    # ---- many rows
    Rule("tc_pair", (768, 1 << 30), True, _always,
         "gate|up 24576 x 4096 at 2,048 rows: 1.62 PFLOP/s with the activation in the epilogue; at 512 rows the library "
         "(74.9 us + 8.5 for SwiGLU) is ahead of it (84.6)"),
    Rule("library", (1, 1 << 30), None, _always,
         "elsewhere cuBLAS is the fastest product measured: 6144 x 4096 at 128 rows 11.9 us (tcgen05 product here: 27.7), "
         "at 512 rows 21.0 (29.0)"),
]


def choose(rows: int, n: int, k: int, *, fused: bool = False, sms: int = 148) -> Rule:
    """The first rule that covers `rows` rows of x against W [n, k] (n = 2 x intermediate when `fused`)."""
    s = Shape(n, k, sms)
    for r in RULES:
        if r.rows[0] <= rows <= r.rows[1] and (r.fused is None or r.fused == fused) and r.when(s):
            return r
    raise ValueError(f"no rule for {rows} rows of a {n} x {k} product")     # the last rule matches everything


def kernel_for(rows: int, n: int, k: int, *, fused: bool = False, sms: int = 148) -> str:
    return choose(rows, n, k, fused=fused, sms=sms).kernel

"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math
from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .base import MIXERS, CacheNeed, Mixer
from .linear import Linear


def run_attention(ctx, q, out, view, n_rows, q_heads, scale, window):
    """Chooses the attention kernel for this step: the tensor-core kernels where they take the
    shape, else the plain kernel (which is also the whole 32-bit path)."""
    if not ops.fast_attention_takes(view, q.dtype):
        ops.attention_rows(q, out, view, ctx.row_slot, ctx.row_pos, n_rows, q_heads, scale, window)
    elif ctx.decode:
        # up to 8 splits merge inside a thread-block cluster and need no scratch
        splits = decode_splits(ctx, n_rows, view.kv_heads, q_heads, view.head_dim)
        ops.attention_decode_bf16(q, out, view, ctx.row_slot, ctx.row_pos, n_rows, q_heads, scale, window, splits, None)
    else:
        kernel = ops.attention_prefill_tcgen05 if ops.attention_tc_takes(view, q.dtype) else ops.attention_prefill_bf16
        kernel(q, out, view, ctx.tile_seq, ctx.tile_row0, ctx.n_tiles, ctx.seq_first_row, ctx.seq_slot, ctx.seq_pos0,
               q_heads, scale, window)


# what a decode attention block costs besides walking its pages (table look-ups, first slice, merges),
# in pages' worth of time: about 3 us against 0.3 us per page of 64 keys x 128 values, measured at 8 kv heads;
# the split only has to be near the best one, and the same rule chose well at 1 to 256 sequences and
# contexts of 1,024 to 17,408
DECODE_BLOCK_FIXED_PAGES = 10


def decode_splits(ctx, n_rows: int, kv_heads: int, q_heads: int, head_dim: int) -> int:
    """Into how many blocks each (sequence, kv head) of a decode pass is split.  The splits of one
    are a thread-block cluster (at most 8) and merge through shared memory.  With `fit(s)` clusters
    of s blocks running at once (asked of the runtime: clusters do not pack the GPU completely,
    296 blocks but only 71 clusters of 4), a launch takes ceil(units / fit(s)) waves of blocks that
    each walk pages / s pages and cost a fixed start and merge besides; the split with the shortest
    total wins.  So a small batch is split until it fills the GPU once, and a batch of 48
    sequences, whose 384 blocks would be 1.3 waves, is split in two (three shorter waves)."""
    group_chunks = (q_heads // kv_heads + 15) // 16
    units = max(1, n_rows * kv_heads * group_chunks)
    pages = max(1, (ctx.max_context + 63) // 64)
    best, best_cost = 1, None
    for splits in range(1, min(pages, ops.ATTENTION_DECODE_CLUSTER_SPLITS) + 1):
        fit = ops.attention_decode_max_clusters(head_dim, splits)
        if fit <= 0:      # unknown: assume seven eighths of the resident blocks
            resident = ops.attention_decode_blocks_per_sm() * ctx.sm_count
            fit = max(1, (resident - resident // 8) // splits)
        waves = -(-units // fit)
        cost = waves * (pages / splits + DECODE_BLOCK_FIXED_PAGES)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = splits, cost
    return best


class GQAttention(Mixer):
    """q, k, v from one product on the packed [q; k; v] weight (q rows, then k rows, then v rows:
    x0ne-core/runtime/src/weights.rs:1-4,212-213); optional per-head RMSNorm of q and k with one
    weight of head_dim values for all heads; rotation by the model's position encoding; K (after
    norm and rotation) and V written to the cache; causal softmax attention of each query over its
    sequence's cached keys, q head h reading kv head h // (q_heads // kv_heads), scale
    1/sqrt(head_dim) unless given; output projection.  Order of operations:
    x0ne-core/runtime/src/engine.rs:750-780, x0ne-core/kernels/cuda/rope.cu:7-47,
    x0ne-core/kernels/cuda/attention.cu.

    Parameters: hidden_size, q_heads, kv_heads, head_dim, qk_norm_eps (None: no q/k norm), window
    (None: all keys), position (name of a position encoding of the model, or None), scale (None:
    1/sqrt(head_dim)), names.{q, k, v, o, q_norm, k_norm}.
    """
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        g = spec.get
        self.hidden = int(spec["hidden_size"])
        self.q_heads = int(spec["q_heads"])
        self.kv_heads = int(spec["kv_heads"])
        self.head_dim = int(spec["head_dim"])
        if self.q_heads % self.kv_heads:
            raise ValueError("q heads are not a multiple of kv heads")
        self.qk_norm_eps = g("qk_norm_eps")
        self.window = g("window")
        # softmax scale: (1/sqrt(d) computed in float64) narrowed to float32 (x0ne-core/runtime/src/ops.rs:217-219)
        self.scale = float(g("scale")) if g("scale") is not None else 1.0 / math.sqrt(self.head_dim)
        pos = g("position")
        self.position = env.positions[pos] if pos is not None else None
        self.q_dim = self.q_heads * self.head_dim
        self.kv_dim = self.kv_heads * self.head_dim
        self.qkv = self.o = self.q_norm = self.k_norm = None

    @staticmethod
    def cache_need(spec: PartSpec) -> CacheNeed:
        return CacheNeed("kv", int(spec["kv_heads"]), int(spec["head_dim"]), spec.get("window"))

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        h, hd = int(spec["hidden_size"]), int(spec["head_dim"])
        qd, kvd, n = int(spec["q_heads"]) * hd, int(spec["kv_heads"]) * hd, spec["names"]
        needs = [TensorNeed(n["q"], (qd, h)), TensorNeed(n["k"], (kvd, h)), TensorNeed(n["v"], (kvd, h)),
                 TensorNeed(n["o"], (h, qd))]
        if spec.get("qk_norm_eps") is not None:
            needs += [TensorNeed(n["q_norm"], (hd,), role="vector", init="norm"),
                      TensorNeed(n["k_norm"], (hd,), role="vector", init="norm")]
        return needs

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.spec["names"]
        self.qkv = Linear(torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]]], dim=0).contiguous())
        self.o = Linear(tensors[n["o"]])
        if self.qk_norm_eps is not None:
            self.q_norm, self.k_norm = tensors[n["q_norm"]], tensors[n["k_norm"]]

    def weight_bytes(self) -> int:
        return self.qkv.weight_bytes() + self.o.weight_bytes()

    def forward(self, ctx, entry, x, n_rows, cache_entry=None, write_cache=True):
        dt, rows = self.env.dtype, ctx.ws.max_rows
        qkv = ctx.ws.buffer("attn.qkv", (rows, self.q_dim + 2 * self.kv_dim), dt)
        q = ctx.ws.buffer("attn.q", (rows, self.q_dim), dt)
        att = ctx.ws.buffer("attn.out", (rows, self.q_dim), dt)
        out = ctx.ws.buffer("delta", (rows, self.hidden), dt)
        self.qkv(x, qkv, n_rows)
        view = ctx.cache.kv_view(entry if cache_entry is None else cache_entry)
        rot = self.position.rotary() if self.position is not None else None
        inv_freq, rot_dim = rot if rot is not None else (None, 0)
        table = None
        if rot is not None and self.env.max_positions and hasattr(self.position, "cos_sin_table"):
            table = self.position.cos_sin_table(self.env.max_positions)
        ops.qk_norm_rope_kv_write(qkv, self.q_norm, self.k_norm, inv_freq, rot_dim, q, view, ctx.row_slot,
                                  ctx.row_pos, n_rows, self.q_heads,
                                  float(self.qk_norm_eps) if self.qk_norm_eps is not None else 0.0,
                                  write_kv=write_cache, rope_table=table)
        run_attention(ctx, q, att, view, n_rows, self.q_heads, self.scale, int(self.window or 0))
        self.o(att, out, n_rows)
        return out


MIXERS.register("gqa_attention", GQAttention)

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
        # up to 8 splits merge inside a thread-block cluster and need no scratch; several clusters
        # per (sequence, kv head) leave one partial result each in a scratch of the workspace
        splits, groups = decode_plan(ctx, n_rows, view.kv_heads, q_heads, view.head_dim)
        scratch = None
        if groups > 1:
            # one size for every launch that can come this way, so that a captured graph's pointer stays good
            scratch = ctx.ws.zeroed("attn.decode_parts", decode_scratch_bytes(ctx, view.kv_heads, q_heads, view.head_dim))
        ops.attention_decode_bf16(q, out, view, ctx.row_slot, ctx.row_pos, n_rows, q_heads, scale, window, splits, scratch,
                                  groups=groups)
    else:
        kernel = ops.attention_prefill_tcgen05 if ops.attention_tc_takes(view, q.dtype) else ops.attention_prefill_bf16
        kernel(q, out, view, ctx.tile_seq, ctx.tile_row0, ctx.n_tiles, ctx.seq_first_row, ctx.seq_slot, ctx.seq_pos0,
               q_heads, scale, window)


# what a decode attention block costs besides walking its pages (table look-ups, first slice, merges),
# in pages' worth of time: about 3 us against 0.3 us per page of 64 keys x 128 values, measured at 8 kv heads;
# the split only has to be near the best one, and the same rule chose well at 1 to 256 sequences and
# contexts of 1,024 to 17,408
DECODE_BLOCK_FIXED_PAGES = 10
# Several clusters per (sequence, kv head), measured at 1 and 2 sequences with 8 kv heads x 128 and
# 4,096 to 32,768 keys (microseconds): a block that shares the GPU with few others takes 0.85 per
# page (one SM takes in about 38 GB/s), with 256 blocks about 1.3 (they share the memory's
# bandwidth); the meeting of the clusters' results in scratch costs 2.5 on top with clusters of 4
# and 4.5 with clusters of 8, and a quarter more for every cluster past two.  One sequence at 32,768
# keys: one cluster of 8 57.4, four clusters of 8 30.5; at 6,144 keys 15.0 and 13.3; at 4,096 11.7
# and 12.4.
DECODE_PAGE_US_ALONE = 0.85
DECODE_PAGE_US_PER_BLOCK = 0.0023       # per block past 64, at head_dim 128
DECODE_GROUP_US = {4: 2.5, 8: 4.5}      # by cluster size
DECODE_GROUP_MARGIN_US = 0.5
DECODE_MAX_GROUPS = 4


def _fit(ctx, head_dim: int, cluster: int) -> int:
    fit = ops.attention_decode_max_clusters(head_dim, cluster)
    if fit <= 0:      # unknown: assume seven eighths of the resident blocks
        resident = ops.attention_decode_blocks_per_sm() * ctx.sm_count
        fit = max(1, (resident - resident // 8) // cluster)
    return fit


def decode_plan(ctx, n_rows: int, kv_heads: int, q_heads: int, head_dim: int) -> tuple:
    """(splits, groups): into how many blocks each (sequence, kv head) of a decode pass is split, and
    how many thread-block clusters those blocks form.  The blocks of a cluster (at most 8) merge
    through shared memory.  With `fit(s)` clusters of s blocks running at once (asked of the runtime:
    clusters do not pack the GPU completely, 296 blocks but only 71 clusters of 4), a launch takes
    ceil(units / fit(s)) waves of blocks that each walk pages / s pages and cost a fixed start and
    merge besides; the split with the shortest total wins.  So a small batch is split until it fills
    the GPU once, and a batch of 48 sequences, whose 384 blocks would be 1.3 waves, is split in two
    (three shorter waves).  Where even 8 splits leave most of the GPU idle (one or two sequences) and
    the context is long, several clusters per (sequence, kv head) follow: their results meet in
    scratch, which costs a few microseconds, so they are taken only where the shorter walk pays
    for that by the measured times above, and only as many as run at once."""
    group_chunks = (q_heads // kv_heads + 15) // 16
    units = max(1, n_rows * kv_heads * group_chunks)
    pages = max(1, (ctx.max_context + 63) // 64)
    best, best_cost = 1, None
    for splits in range(1, min(pages, ops.ATTENTION_DECODE_CLUSTER_SPLITS) + 1):
        waves = -(-units // _fit(ctx, head_dim, splits))
        cost = waves * (pages / splits + DECODE_BLOCK_FIXED_PAGES)
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = splits, cost
    if best < ops.ATTENTION_DECODE_CLUSTER_SPLITS:
        return best, 1

    def page_us(blocks):
        return DECODE_PAGE_US_ALONE + max(0, blocks - 64) * DECODE_PAGE_US_PER_BLOCK * head_dim / 128

    plan, plan_us = (best, 1), -(-pages // best) * page_us(units * best) - DECODE_GROUP_MARGIN_US
    for cluster, merge_us in DECODE_GROUP_US.items():
        for groups in range(2, DECODE_MAX_GROUPS + 1):
            splits = cluster * groups
            if splits <= best or splits > pages or splits > ops.ATTENTION_DECODE_MAX_SPLITS or units * groups > _fit(ctx, head_dim, cluster):
                continue
            us = -(-pages // splits) * page_us(units * splits) + merge_us + 0.25 * (groups - 2)
            if us < plan_us - 1e-9:
                plan, plan_us = (splits, groups), us
    return plan


def decode_scratch_bytes(ctx, kv_heads: int, q_heads: int, head_dim: int) -> int:
    """Scratch for the largest decode launch that decode_plan gives several clusters per (sequence,
    kv head): those are the launches whose clusters all run at once."""
    group_chunks = (q_heads // kv_heads + 15) // 16
    rows = max(1, max(_fit(ctx, head_dim, c) for c in DECODE_GROUP_US) // (2 * kv_heads * group_chunks))
    return ops.attention_decode_scratch_bytes(rows, q_heads, kv_heads, head_dim, DECODE_MAX_GROUPS)


def decode_splits(ctx, n_rows: int, kv_heads: int, q_heads: int, head_dim: int) -> int:
    """Blocks per (sequence, kv head) of a decode pass (see decode_plan)."""
    return decode_plan(ctx, n_rows, kv_heads, q_heads, head_dim)[0]


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

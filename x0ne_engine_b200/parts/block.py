"""Arrangements of a layer's parts around the residual stream."""
from __future__ import annotations

from .base import BLOCKS, Block


class PreNormBlock(Block):
    """x += mixer(norm(x)); x += ffn(norm(x)).  The residual stays in float32; each add is fused
    into the norm that follows it, so a block takes the previous block's pending delta and
    returns its own (x0ne-core/runtime/src/engine.rs:749,781,823)."""
    replayable = True
    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "ffn_norm": "norm", "ffn": "feed_forward"}

    def forward(self, ctx, entry, resid, delta, cache_entry=None, write_cache=True):
        normed = ctx.ws.buffer("normed", (ctx.ws.max_rows, resid.shape[-1]), ctx.dtype)
        self.mixer_norm.add_norm(ctx, resid, delta, normed, ctx.n_rows)
        delta = self.mixer.forward(ctx, entry, normed, ctx.n_rows, cache_entry=cache_entry, write_cache=write_cache)
        self.ffn_norm.add_norm(ctx, resid, delta, normed, ctx.n_rows)
        return self.ffn.forward(ctx, normed, ctx.n_rows)


BLOCKS.register("prenorm", PreNormBlock)

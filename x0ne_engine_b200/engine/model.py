"""A causal language model built from a ModelSpec: embedding, the run order of blocks, the final
norm and the head.  Nothing here names an architecture."""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from ..config.spec import ModelSpec
from ..parts import base as P
from ..parts.embedding import LMHead, TokenEmbedding
from ..weights.loader import TensorNeed


def _unique(needs: List[TensorNeed]) -> List[TensorNeed]:
    seen: Dict[str, TensorNeed] = {}
    for n in needs:
        if n.name in seen:
            if tuple(seen[n.name].shape) != tuple(n.shape) or seen[n.name].role != n.role:
                raise ValueError(f"tensor {n.name!r} is needed twice with different shapes or roles")
        else:
            seen[n.name] = n
    return list(seen.values())


def tensor_needs_of_spec(spec: ModelSpec) -> List[TensorNeed]:
    """Every checkpoint tensor the model reads, by name, in model order (no device needed)."""
    needs: List[TensorNeed] = list(TokenEmbedding.tensor_needs(spec.embedding))
    for ps in spec.positions.values():
        needs += P.POSITIONS.get(ps.kind).tensor_needs(ps)
    for layer in spec.layers:
        needs += P.NORMS.get(layer.mixer_norm.kind).tensor_needs(layer.mixer_norm)
        needs += P.MIXERS.get(layer.mixer.kind).tensor_needs(layer.mixer)
        needs += P.NORMS.get(layer.ffn_norm.kind).tensor_needs(layer.ffn_norm)
        needs += P.FEED_FORWARDS.get(layer.ffn.kind).tensor_needs(layer.ffn)
    needs += P.NORMS.get(spec.final_norm.kind).tensor_needs(spec.final_norm)
    needs += LMHead.tensor_needs(spec.head)
    return _unique(needs)


def optional_duplicates_of_spec(spec: ModelSpec) -> Dict[str, str]:
    """Tensors a checkpoint may carry although the model does not read them, each with the
    tensor it must equal: the head of a tied model."""
    if spec.head.get("tied"):
        return {"lm_head.weight": spec.head["names"]["weight"]}
    return {}


class CausalLM:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device, max_positions: int = 0):
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        env = P.BuildEnv(dtype=dtype, device=self.device, max_positions=max_positions)
        for name, ps in spec.positions.items():
            env.positions[name] = P.POSITIONS.get(ps.kind)(ps, env)
        self.env = env
        self.embedding = TokenEmbedding(spec.embedding, env)
        self.blocks: List[P.Block] = []
        for layer in spec.layers:
            self.blocks.append(P.BLOCKS.get(layer.block)(
                P.NORMS.get(layer.mixer_norm.kind)(layer.mixer_norm, env),
                P.MIXERS.get(layer.mixer.kind)(layer.mixer, env),
                P.NORMS.get(layer.ffn_norm.kind)(layer.ffn_norm, env),
                P.FEED_FORWARDS.get(layer.ffn.kind)(layer.ffn, env)))
        self.final_norm = P.NORMS.get(spec.final_norm.kind)(spec.final_norm, env)
        self.head = LMHead(spec.head, env)

    def parts(self) -> List[P.Part]:
        out: List[P.Part] = [self.embedding] + list(self.env.positions.values())
        for b in self.blocks:
            out += b.parts()
        return out + [self.final_norm, self.head]

    def replayable(self) -> bool:
        """Whether every part and block promises that its launches can be replayed from a CUDA graph
        and that it takes padding rows (see `parts.Part.replayable`)."""
        return all(p.replayable for p in self.parts()) and all(b.replayable for b in self.blocks)

    def cache_needs(self) -> List[P.CacheNeed]:
        """One CacheNeed per run-order entry."""
        return [P.MIXERS.get(self.spec.layers[e.layer].mixer.kind).cache_need(self.spec.layers[e.layer].mixer)
                for e in self.spec.run_order]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.bind(tensors)

    def step_weight_bytes(self) -> int:
        """Bytes of weights one step reads: every run-order entry's matrices once, and the head."""
        total = self.head.weight_bytes()
        for e in self.spec.run_order:
            total += sum(p.weight_bytes() for p in self.blocks[e.layer].parts())
        return total

    def forward(self, ctx, want_rows: Optional[torch.Tensor], n_want: int, logits: Optional[torch.Tensor]):
        """Runs the rows of `ctx` through the model; writes float32 logits of the wanted rows."""
        ws, h = ctx.ws, self.spec.hidden_size
        resid = ws.buffer("resid", (ws.max_rows, h), torch.float32)
        self.embedding.forward(ctx, resid, ctx.n_rows)
        for pos in self.env.positions.values():
            pos.on_embedding(ctx, resid, ctx.n_rows)
        delta = None
        for i, e in enumerate(self.spec.run_order):
            delta = self.blocks[e.layer].forward(ctx, i, resid, delta, cache_entry=e.reads_cache_of,
                                                 write_cache=e.reads_cache_of is None)
        if n_want == 0:
            return None
        normed = ws.buffer("head.normed", (ws.max_want, h), self.dtype)
        self.final_norm.add_norm(ctx, resid, delta, normed, n_want, rows=want_rows)
        return self.head.forward(normed, logits, n_want)

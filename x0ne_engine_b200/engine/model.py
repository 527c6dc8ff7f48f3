"""A causal language model built from a ModelSpec: embedding, the run order of blocks, the final
norm and the head.  Nothing here names an architecture."""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from ..config.spec import ModelSpec
from ..config.spec import ConfigError, LayerSpec
from ..parts import base as P
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


def layer_part_classes(layer: LayerSpec):
    """(role, part class, part spec) of a layer in the order its arrangement runs them; checks the
    layer's roles against the arrangement's."""
    block = P.BLOCKS.get(layer.block)
    try:
        block.check_roles(list(layer.parts))
    except ValueError as e:
        raise ConfigError(str(e)) from None
    return [(role, P.PART_REGISTRIES[kind].get(layer.parts[role].kind), layer.parts[role])
            for role, kind in block.ROLES.items() if role in layer.parts]


def tensor_needs_of_spec(spec: ModelSpec) -> List[TensorNeed]:
    """Every checkpoint tensor the model reads, by name, in model order (no device needed)."""
    needs: List[TensorNeed] = list(P.EMBEDDINGS.get(spec.embedding.kind).tensor_needs(spec.embedding))
    for ps in spec.positions.values():
        needs += P.POSITIONS.get(ps.kind).tensor_needs(ps)
    for layer in spec.layers:
        for _, cls, ps in layer_part_classes(layer):
            needs += cls.tensor_needs(ps)
    needs += P.NORMS.get(spec.final_norm.kind).tensor_needs(spec.final_norm)
    needs += P.HEADS.get(spec.head.kind).tensor_needs(spec.head)
    return _unique(needs)


def optional_duplicates_of_spec(spec: ModelSpec) -> Dict[str, str]:
    """Tensors a checkpoint may carry although the model does not read them, each with the
    tensor it must equal (the head of a tied model): what the head's class says."""
    return dict(P.HEADS.get(spec.head.kind).optional_duplicates(spec.head))


def cache_need_of_layer(layer: LayerSpec) -> P.CacheNeed:
    """What a run-order entry of this layer keeps per sequence: its mixer's need.  A layer without
    a mixer keeps nothing; a layer may hold one mixer that keeps something."""
    needs = [cls.cache_need(ps) for _, cls, ps in layer_part_classes(layer) if issubclass(cls, P.Mixer)]
    needs = [n for n in needs if n.kind != "none"]
    if len(needs) > 1:
        raise ConfigError("a layer with two mixers that both keep something per sequence is not served: "
                          "give each a layer of its own")
    return needs[0] if needs else P.CacheNeed()


def step_bytes_of_spec(spec: ModelSpec, dtype_bytes: int = 2):
    """(bytes of weights a decode step reads, bytes of cache one position of one sequence holds),
    from the spec alone: every run-order entry's tensors once and the head's, matrices in the
    run's dtype and vectors in float32; the embedding table is read one row per token, so it only
    counts where the head reads it whole (a tied model)."""
    def nbytes(need: TensorNeed) -> int:
        n = 1
        for s in need.shape:
            n *= s
        return n * (4 if need.role in ("vector", "table") else dtype_bytes)

    weights = sum(nbytes(n) for n in P.HEADS.get(spec.head.kind).tensor_needs(spec.head))
    weights += sum(nbytes(n) for n in P.NORMS.get(spec.final_norm.kind).tensor_needs(spec.final_norm))
    cache = 0
    for e in spec.run_order:
        layer = spec.layers[e.layer]
        weights += sum(nbytes(n) for _, cls, ps in layer_part_classes(layer) for n in cls.tensor_needs(ps))
        need = cache_need_of_layer(layer)
        if need.kind == "kv" and e.reads_cache_of is None:
            cache += 2 * need.kv_heads * need.head_dim * dtype_bytes
    return weights, cache


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
        self.embedding = P.EMBEDDINGS.get(spec.embedding.kind)(spec.embedding, env)
        self.blocks: List[P.Block] = []
        for layer in spec.layers:
            self.blocks.append(P.BLOCKS.get(layer.block)({role: cls(ps, env) for role, cls, ps in layer_part_classes(layer)}))
        self.final_norm = P.NORMS.get(spec.final_norm.kind)(spec.final_norm, env)
        self.head = P.HEADS.get(spec.head.kind)(spec.head, env)

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
        return [cache_need_of_layer(self.spec.layers[e.layer]) for e in self.spec.run_order]

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

"""The description of a model as data.

An architecture's config reader turns `config.json` into a `ModelSpec`: which parts every
layer is made of (by registered kind name), with every size and constant as a parameter of
the part, the checkpoint tensor names each part reads, and the order in which layers run.
Nothing below this file knows an architecture's name: the engine builds parts from the spec
through the part registries and runs the schedule.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """A config.json this library does not serve, with the reason in words."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered `kind` and its parameters.

    `params` holds sizes, constants and the checkpoint names of the part's tensors
    (under the key "names": role -> tensor name).
    """
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """A layer: how its parts are arranged (`block`, a registered arrangement) and the parts
    themselves by role.

    Which roles exist, which are required and what kind of part fills each (a norm, a mixer, a
    feed-forward) is the arrangement's business: the pre-norm block takes `mixer_norm`, `mixer`,
    `ffn_norm` and `ffn`; an arrangement with four norms, with both branches in parallel or
    without a feed-forward names its own.  Two layers of one model need not use the same
    arrangement, mixer or feed-forward.
    """
    block: str
    parts: Mapping[str, PartSpec] = field(default_factory=dict)

    def part(self, role: str) -> PartSpec:
        try:
            return self.parts[role]
        except KeyError:
            raise ConfigError(f"a {self.block!r} layer has no part in the role {role!r}; it has {sorted(self.parts)}") from None

    def with_part(self, role: str, spec: PartSpec) -> "LayerSpec":
        """A copy of this layer with one role filled anew."""
        return LayerSpec(self.block, {**self.parts, role: spec})


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order.

    `layer` indexes `ModelSpec.layers`; a layer may be named by several entries (its
    weights are then shared and every entry has a cache of its own).  `reads_cache_of`, if
    set, is the index of an earlier entry of the run order whose cache this entry's mixer
    reads instead of writing one.
    """
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    embedding: PartSpec
    positions: Mapping[str, PartSpec]
    layers: Tuple[LayerSpec, ...]
    run_order: Tuple[RunEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: Tuple[int, ...] = ()
    checkpoint_dtype: str = "bfloat16"

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for i, e in enumerate(self.run_order):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"run order entry {i} names layer {e.layer}, which does not exist")
            if e.reads_cache_of is not None and not 0 <= e.reads_cache_of < i:
                raise ConfigError(
                    f"run order entry {i} reads the cache of entry {e.reads_cache_of}, "
                    "which must be an earlier entry")

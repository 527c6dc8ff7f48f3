"""What a layer is made of: the interfaces of the parts, and one registry per kind of part.

A part is built from a `PartSpec` (its sizes, constants and checkpoint tensor names) and a
`BuildEnv` (the run's dtype and device, and the model's position encodings by name).  It never
sees the model's name or its config.json.  The kinds:

  * `Norm`         — `add_norm(ctx, resid, delta, out, n_rows, rows=None)`: adds `delta` (may be
                     None) into the float32 residual and writes the normed rows.
  * `Mixer`        — mixes information between the positions of a sequence.  Says what it keeps
                     per sequence with `cache_need(spec)`; `forward(ctx, entry, x, n_rows)` reads
                     and writes that through `ctx.cache` for run-order entry `entry` and returns
                     its output rows (the "delta" the next norm adds to the residual).
  * `FeedForward`  — `forward(ctx, x, n_rows)`: per-row transformation, returns the delta.
  * `PositionEncoding` — `rotary()` gives (inv_freq float32 [rotary_dim/2], rotary_dim) for
                     mixers that rotate q and k, or None; `on_embedding(ctx, resid, n_rows)` lets
                     an additive encoding change the residual after the token embedding.
  * `Block`        — how a layer's parts are arranged around the residual.  The class names its
                     roles and the kind of part each takes (`ROLES`, `OPTIONAL`); the engine builds
                     the layer's parts by role and hands them over; `forward(ctx, entry, resid,
                     delta)` returns the pending delta.
  * `Embedding`    — `forward(ctx, resid, n_rows)` fills the float32 residual from the token ids.
  * `Head`         — `forward(normed, logits, n_rows)` writes float32 logits of the normed rows.

To add a part: subclass the kind, implement `tensor_needs(spec)` (static: the checkpoint
tensors, by name, with shapes) and `bind(tensors)`, and call the kind's `register`.  A part that
may be replayed from a CUDA graph says so with `replayable = True` (see `Part`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple

import torch

from ..config.spec import PartSpec
from ..weights.loader import TensorNeed


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps for each sequence.

    kind "kv": keys and values of `kv_heads` x `head_dim` per position; all positions, or the
    last `window` of them.  kind "state": a float32 array of `state_shape` per sequence, zero
    when the sequence starts.  kind "none": nothing.
    """
    kind: str = "none"
    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()


@dataclass
class BuildEnv:
    dtype: torch.dtype
    device: torch.device
    positions: Dict[str, "PositionEncoding"] = field(default_factory=dict)
    max_positions: int = 0          # longest sequence the engine will hold (for tables made at start-up)


class Part:
    # True promises three things of every call the engine makes during a pass: it only queues work
    # on the current stream (nothing is read back, no tensor made in it is used after it returns);
    # its launches depend on the host only through the numbers of the StepContext (n_rows, n_seqs,
    # n_tiles, max_seq_rows, max_context, decode); and rows whose slot is -1 are rows of no
    # sequence (they read and write nothing that is kept per sequence).  If every part of a model
    # promises this, the engine pads short passes with such rows and replays the launches of
    # decode steps and of short prompt passes from CUDA graphs; else it launches every pass itself.
    replayable = False

    def __init__(self, spec: PartSpec, env: BuildEnv):
        self.spec = spec
        self.env = env

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        return []

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Receives the device tensors named in `tensor_needs`."""

    def weight_bytes(self) -> int:
        """Bytes of weights a step reads (for the roofline)."""
        return 0


class Norm(Part):
    def add_norm(self, ctx, resid, delta, out, n_rows: int, rows=None) -> None:
        raise NotImplementedError


class Mixer(Part):
    @staticmethod
    def cache_need(spec: PartSpec) -> CacheNeed:
        return CacheNeed()

    def forward(self, ctx, entry: int, x: torch.Tensor, n_rows: int, cache_entry: Optional[int] = None,
                write_cache: bool = True) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, x: torch.Tensor, n_rows: int) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary(self) -> Optional[Tuple[torch.Tensor, int]]:
        return None

    def on_embedding(self, ctx, resid: torch.Tensor, n_rows: int) -> None:
        return None


class Embedding(Part):
    def forward(self, ctx, resid: torch.Tensor, n_rows: int) -> None:
        raise NotImplementedError


class Head(Part):
    @staticmethod
    def optional_duplicates(spec: PartSpec) -> Dict[str, str]:
        """Tensors a checkpoint may carry although the head does not read them, each with the name
        of the needed tensor it must equal (a tied model that also stores its head)."""
        return {}

    def forward(self, normed: torch.Tensor, logits: torch.Tensor, n_rows: int) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """Arrangement of one layer's parts.  A subclass names the roles it takes and the kind of part
    in each (`ROLES`: role -> "norm" | "mixer" | "feed_forward", in the order the parts run) and
    which of them a layer may leave out (`OPTIONAL`); the engine builds the parts of a LayerSpec by
    these and passes them by role."""
    replayable = False      # as for Part
    ROLES: Dict[str, str] = {}
    OPTIONAL: Tuple[str, ...] = ()

    def __init__(self, parts: Mapping[str, Part]):
        self.by_role: Dict[str, Part] = dict(parts)
        for role, part in self.by_role.items():
            setattr(self, role, part)
        for role in self.OPTIONAL:
            if role not in self.by_role:
                setattr(self, role, None)

    @classmethod
    def check_roles(cls, given) -> None:
        """Raises ValueError unless `given` (role names) fits this arrangement."""
        unknown = [r for r in given if r not in cls.ROLES]
        missing = [r for r in cls.ROLES if r not in given and r not in cls.OPTIONAL]
        if unknown or missing:
            raise ValueError(f"a {cls.__name__} layer takes the roles {list(cls.ROLES)}"
                             + (f"; unknown: {unknown}" if unknown else "") + (f"; missing: {missing}" if missing else ""))

    def parts(self) -> List[Part]:
        return [self.by_role[r] for r in self.ROLES if r in self.by_role]

    def forward(self, ctx, entry: int, resid, delta, cache_entry=None, write_cache=True):
        raise NotImplementedError


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: Dict[str, Any] = {}

    def register(self, kind: str, cls: Any, replace: bool = False) -> None:
        if kind in self._kinds and not replace:
            raise ValueError(f"{self.what} kind {kind!r} is already registered")
        self._kinds[kind] = cls

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def get(self, kind: str) -> Any:
        try:
            return self._kinds[kind]
        except KeyError:
            raise KeyError(f"no {self.what} of kind {kind!r}; registered: {sorted(self._kinds)}") from None

    def kinds(self) -> List[str]:
        return sorted(self._kinds)


NORMS = Registry("norm")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
POSITIONS = Registry("position encoding")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")
# the registry behind each kind of part a block's role may name
PART_REGISTRIES = {"norm": NORMS, "mixer": MIXERS, "feed_forward": FEED_FORWARDS}

"""The Python entry point: a model you can generate from.

    from x0ne_engine_b200 import Model
    m = Model.from_folder("path/to/model", dtype="bfloat16", max_batch=8, max_ctx=4096)
    out = m.generate([[1, 2, 3], [4, 5]], max_tokens=32, temperature=0.7, seed=1)
    out.tokens, out.finish_reasons

Option names follow the library engine's request options where it has them (`max_tokens`,
`temperature`, `top_p`, `seed`: x0ne-infer/src/backend.rs:49-79; `max_ctx`:
x0ne-core/runtime/src/engine.rs:37-40; decode mode graph / eager: engine.rs:43-55).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

from .cache import PAGE_SIZE
from .engine.engine import Engine
from .engine.generate import Completion, GenerationStats, Generator, round_up
from .sampling.params import SamplingParams


@dataclass
class GenerateResult:
    tokens: List[List[int]]
    finish_reasons: List[str]
    prompt_tokens: List[int]
    stats: GenerationStats


class Model:
    def __init__(self, engine: Engine, max_batch: int, decode: str = "graph"):
        if decode not in ("graph", "eager"):
            raise ValueError("decode is 'graph' or 'eager'")
        self.engine = engine
        self.max_batch = max_batch
        self._generator = Generator(engine, max_batch=max_batch, cuda_graph=decode == "graph")

    @staticmethod
    def _sizes(max_batch, max_ctx, max_tokens, limit):
        max_ctx = min(max_ctx or limit, limit)
        if max_tokens is None:
            max_tokens = max_batch * round_up(max_ctx, PAGE_SIZE)
        return max_ctx, max_tokens

    @classmethod
    def from_folder(cls, folder: str, dtype: str = "bfloat16", device: str = "cuda:0", max_batch: int = 8,
                    max_ctx: Optional[int] = None, max_tokens: Optional[int] = None, decode: str = "graph",
                    max_step_tokens: Optional[int] = None) -> "Model":
        """`max_ctx`: longest sequence (prompt + generated); `max_tokens`: tokens the cache holds in
        all (default: max_batch sequences of max_ctx)."""
        from .config import config_from_folder
        limit = config_from_folder(folder).max_position_embeddings
        max_ctx, max_tokens = cls._sizes(max_batch, max_ctx, max_tokens, limit)
        eng = Engine.from_folder(folder, dtype=dtype, device=device, max_tokens=max_tokens, max_seq_len=max_ctx,
                                 max_step_tokens=max_step_tokens, max_slots=max(max_batch, 1))
        return cls(eng, max_batch, decode)

    @classmethod
    def random(cls, config, seed: int = 0, dtype: str = "bfloat16", device: str = "cuda:0", max_batch: int = 8,
               max_ctx: Optional[int] = None, max_tokens: Optional[int] = None, decode: str = "graph",
               linear_std: float = 0.02, norm_jitter: float = 0.0, max_step_tokens: Optional[int] = None) -> "Model":
        max_ctx, max_tokens = cls._sizes(max_batch, max_ctx, max_tokens, config.max_position_embeddings)
        eng = Engine.random(config, seed=seed, dtype=dtype, device=device, linear_std=linear_std,
                            norm_jitter=norm_jitter, max_tokens=max_tokens, max_seq_len=max_ctx,
                            max_step_tokens=max_step_tokens, max_slots=max(max_batch, 1))
        return cls(eng, max_batch, decode)

    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 16, temperature: float = 0.0,
                 top_p: float = 1.0, seed: Optional[int] = None, stop_token_ids: Optional[Sequence[int]] = None,
                 params: Optional[Sequence[SamplingParams]] = None, **options) -> GenerateResult:
        """Generates after every prompt (lists of token ids).  One set of options for all prompts, or
        `params` with one SamplingParams each.  `stop_token_ids` defaults to the model's
        `eos_token_id` from config.json; pass () to ignore it."""
        if options:
            SamplingParams.from_options(**options)       # refuses by name (top_k) or as unknown
        if params is None:
            if stop_token_ids is None:
                stop_token_ids = self.engine.spec.stop_token_ids
            params = [SamplingParams(max_tokens=max_tokens, temperature=temperature, top_p=top_p,
                                     seed=None if seed is None else (seed + i) % (1 << 64),
                                     stop_token_ids=tuple(stop_token_ids)) for i in range(len(prompts))]
        done: List[Completion] = self._generator.generate(prompts, list(params))
        return GenerateResult([c.tokens for c in done], [c.finish_reason for c in done],
                              [c.prompt_tokens for c in done], self._generator.stats)

    def step(self, slots, tokens, want=None):
        """The engine's step function (see Engine.step)."""
        return self.engine.step(slots, tokens, want)

"""How a request's tokens are picked, and its budget.

The options and their readings follow x0ne-infer/src/backend.rs:49-79 and
x0ne-infer/src/sampler.rs:59-79: `temperature` under 1e-7 or `top_p` at or below 0 is
greedy (argmax, lowest index on ties); `top_p` at or above 1 draws from the whole distribution;
`seed` starts the request's own draw stream; `top_k` is refused by name rather than ignored
(x0ne-infer/src/generation_prop_tests.rs:1299-1300).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Optional, Tuple

GREEDY_BELOW = 1e-7


class PromptTooLong(ValueError):
    """The prompt fills the context: nothing can be generated
    (x0ne-infer/src/backend.rs:25-47)."""

    def __init__(self, prompt_tokens: int, context_tokens: int):
        self.prompt_tokens, self.context_tokens = prompt_tokens, context_tokens
        super().__init__(f"the prompt is {prompt_tokens} tokens and this model's context is {context_tokens}")


def generation_budget(prompt_tokens: int, max_tokens: int, context_tokens: int) -> int:
    """Tokens that may still be generated: max_tokens cut to what the context leaves."""
    if prompt_tokens >= context_tokens:
        raise PromptTooLong(prompt_tokens, context_tokens)
    return min(max_tokens, context_tokens - prompt_tokens)


def fresh_seed() -> int:
    """A seed for a request that gave none: from the system's randomness, below 2^53
    (x0ne-infer/src/backend.rs:284-297)."""
    return int.from_bytes(os.urandom(8), "little") & ((1 << 53) - 1)


@dataclass(frozen=True)
class SamplingParams:
    max_tokens: int = 16
    temperature: float = 0.0
    top_p: float = 1.0
    seed: Optional[int] = None
    stop_token_ids: Tuple[int, ...] = ()

    def __post_init__(self):
        if isinstance(self.max_tokens, bool) or not isinstance(self.max_tokens, int) or self.max_tokens < 1:
            raise ValueError("max_tokens must be a whole number of at least 1")
        for name in ("temperature", "top_p"):
            v = getattr(self, name)
            if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
                raise ValueError(f"{name} must be a finite number")
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        if self.seed is not None and not 0 <= int(self.seed) < 1 << 64:
            raise ValueError("seed must fit 64 bits")
        object.__setattr__(self, "stop_token_ids", tuple(int(t) for t in self.stop_token_ids))

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_BELOW or self.top_p <= 0.0

    @classmethod
    def from_options(cls, **options) -> "SamplingParams":
        """Builds the parameters from a request's options, refusing by name what is not served."""
        if "top_k" in options:
            raise ValueError("top_k is not served; use temperature and top_p")
        known = {"max_tokens", "temperature", "top_p", "seed", "stop_token_ids"}
        unknown = sorted(set(options) - known)
        if unknown:
            raise ValueError(f"unknown sampling options: {', '.join(unknown)}")
        return cls(**options)

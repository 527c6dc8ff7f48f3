"""The generation loop above the step function.

Requests are token-id prompts with sampling options.  They are served in batches: the prompts of
a batch go through ONE step together whatever their lengths, then every live sequence decodes one
token per step; a sequence that ends leaves the batch at once (the live rows are compacted), its
cache is given back when the batch ends, and the next batch reuses it.  The decisions follow
x0ne-infer/src/stepped.rs:239-276: the budget is max_tokens cut to what the context leaves;
a stop token ends the sequence before it is fed or counted; the last token of the budget is
emitted but not fed.  Finish reasons: "stop" and "length" (x0ne-infer/src/backend.rs:82-109).

The loop itself is host logic over a `BatchRunner` (start / step / close), so its decisions are
tested on the CPU with a scripted runner; `DeviceBatch` in decode.py is the runner on the GPU.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Protocol, Sequence, Tuple

from ..sampling.params import SamplingParams, fresh_seed, generation_budget

NAN_PICK = -1        # the logits row held a NaN: no token (x0ne-core/kernels/cuda/argmax.cu:8-10)
FINISHED_PICK = -2   # the row had already finished on the device


class GenerationError(RuntimeError):
    pass


@dataclass
class Completion:
    tokens: List[int]
    finish_reason: str            # "stop" | "length"
    prompt_tokens: int


@dataclass
class Row:
    request: int
    prompt: List[int]
    params: SamplingParams
    budget: int
    seed: int
    generated: List[int] = field(default_factory=list)
    reason: Optional[str] = None

    def decide(self, pick: int) -> bool:
        """Takes the token picked for this row; True if the row goes on and the token is fed."""
        if pick == NAN_PICK:
            raise GenerationError(f"request {self.request}: the logits hold a NaN, no token")
        if pick < 0:
            raise GenerationError(f"request {self.request}: the device reported pick {pick} for a live row")
        if pick in self.params.stop_token_ids:
            self.reason = "stop"
            return False
        self.generated.append(pick)
        if len(self.generated) >= self.budget:
            self.reason = "length"
            return False
        return True


class BatchRunner(Protocol):
    def start(self, rows: Sequence[Row]) -> List[int]:
        """Takes slots, runs all prompts in one step, returns the first pick of every row."""

    def step(self, live: Sequence[int]) -> List[int]:
        """Feeds each live row's last pick and returns its next pick, in the order of `live`
        (indices into the rows given to `start`)."""

    def close(self) -> None:
        """Gives the batch's slots back."""


def round_up(n: int, unit: int) -> int:
    return (n + unit - 1) // unit * unit


def plan_batches(needs: Sequence[int], max_batch: int, capacity_tokens: int, unit: int) -> List[Tuple[int, int]]:
    """Cuts the requests, in order, into batches [first, last): at most `max_batch` requests each,
    whose reserved tokens (each request's prompt + budget, rounded up to the cache's unit) fit the
    cache together."""
    out = []
    i = 0
    while i < len(needs):
        j, used = i, 0
        while j < len(needs) and j - i < max_batch and used + round_up(needs[j], unit) <= capacity_tokens:
            used += round_up(needs[j], unit)
            j += 1
        if j == i:
            raise GenerationError(f"request {i} needs {needs[i]} tokens of cache; the cache holds {capacity_tokens}")
        out.append((i, j))
        i = j
    return out


@dataclass
class GenerationStats:
    """Sums over the batches served, and the host time at which every step's tokens landed.

    `token_gaps` holds, per decode step, the seconds between the arrival of the step before it
    (for a batch's first decode step: of the prompts' picks) and its own arrival: the inter-token
    time a client of any sequence of the batch sees.  The library engine stamps each token the same
    way (x0ne-core/runtime/src/engine.rs:1106-1116) and reports their percentiles."""
    batches: int = 0
    prefill_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_steps: int = 0
    decode_tokens: int = 0
    decode_seconds: float = 0.0
    token_gaps: List[float] = field(default_factory=list)

    def gap_percentiles(self, which: Sequence[float] = (50, 90, 99)) -> Optional[dict]:
        """{"p50": seconds, ...} of `token_gaps` (nearest-rank), or None when no step was decoded."""
        return percentiles(self.token_gaps, which)


def percentiles(values: Sequence[float], which: Sequence[float] = (50, 90, 99)) -> Optional[dict]:
    if not values:
        return None
    s = sorted(values)
    out = {}
    for p in which:
        rank = max(1, -(-len(s) * p // 100))            # nearest rank: ceil(p/100 * n), at least the first
        out[f"p{p:g}"] = s[min(len(s), int(rank)) - 1]
    out.update(max=s[-1], n=len(s))
    return out


def run_batch(runner: BatchRunner, rows: List[Row], stats: Optional[GenerationStats] = None,
              clock: Callable[[], float] = time.perf_counter) -> None:
    """One batch from its prompts to its last token; fills `rows[i].generated` and `.reason`."""
    t0 = clock()
    try:
        picks = runner.start(rows)
        live = [i for i, p in enumerate(picks) if rows[i].decide(p)]
        t1 = clock()
        if stats is not None:
            stats.batches += 1
            stats.prefill_tokens += sum(len(r.prompt) for r in rows)
            stats.prefill_seconds += t1 - t0
        last = t1
        while live:
            picks = runner.step(live)
            if stats is not None:
                now = clock()
                stats.decode_steps += 1
                stats.decode_tokens += len(live)
                stats.token_gaps.append(now - last)
                last = now
            live = [i for i, p in zip(live, picks) if rows[i].decide(p)]
        if stats is not None:
            stats.decode_seconds += last - t1
    finally:
        runner.close()


class Generator:
    """`generate(prompts, params)` over an engine; one batch after another until all are served."""

    def __init__(self, engine, max_batch: int = 64, cuda_graph: bool = True, runner_factory=None):
        self.engine = engine
        self.max_batch = max_batch
        if runner_factory is None:
            from .decode import DeviceBatch
            runner_factory = lambda: DeviceBatch(engine, max_batch, cuda_graph=cuda_graph)   # noqa: E731
        self._runner_factory = runner_factory
        self._runner = None
        self.stats = GenerationStats()

    def generate(self, prompts: Sequence[Sequence[int]], params=None) -> List[Completion]:
        if params is None:
            params = SamplingParams()
        plist = list(params) if isinstance(params, (list, tuple)) else [params] * len(prompts)
        if len(plist) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        context = self.engine.max_seq_len
        vocab = self.engine.vocab_size
        rows: List[Row] = []
        for i, (prompt, p) in enumerate(zip(prompts, plist)):
            prompt = [int(t) for t in prompt]
            if not prompt:
                raise ValueError(f"request {i}: empty prompt")
            if min(prompt) < 0 or max(prompt) >= vocab:
                raise ValueError(f"request {i}: a token id lies outside the vocabulary of {vocab}")
            budget = generation_budget(len(prompt), p.max_tokens, context)
            rows.append(Row(i, prompt, p, budget, p.seed if p.seed is not None else fresh_seed()))
        unit = self.engine.cache.page_size
        capacity = self.engine.cache.free_tokens()
        batches = plan_batches([len(r.prompt) + r.budget for r in rows], self.max_batch, capacity, unit)
        if self._runner is None:
            self._runner = self._runner_factory()
        for a, b in batches:
            run_batch(self._runner, rows[a:b], self.stats)
        return [Completion(r.generated, r.reason or "length", len(r.prompt)) for r in rows]

"""The engine: a model on one GPU, its cache, and ONE step function.

`Engine.step` takes a batch of sequences, each with the tokens it brings now (a whole prompt, a
further piece of it, or one token), runs exactly those tokens as one batch against what the
cache already holds for each sequence, appends their keys and values, and returns float32
logits at the wanted places.  Prefill, chunked prefill and decode are the same call; generation,
trace replay and the benchmark all go through it (decode steps may go through a CUDA graph of
the same launches, see decode.py).

The library engine's forward takes one sequence, a start position and a row count
(x0ne-core/runtime/src/engine.rs:702-839); here every row carries its own (slot, position), so
sequences of unequal length share a pass and padding never exists.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import PAGE_SIZE, CacheFull, SequenceCache
from ..config import config_from_folder
from ..config.spec import ModelSpec
from ..weights import RandomInit, load_folder, make_tensor
from ..weights.loader import held_dtype
from .model import CausalLM, optional_duplicates_of_spec, tensor_needs_of_spec
from .workspace import Workspace

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


# Prompt passes of at most this many rows are launch-bound on the host (about 300 launches
# against a few milliseconds of device work), so their launches are kept as CUDA graphs.
PASS_GRAPH_MAX_ROWS = 1024
PASS_GRAPH_MAX_WANT = 16
PASS_GRAPHS_KEPT = 24


def padded_rows(n: int) -> int:
    """The row count a short bfloat16 prompt pass is launched with: itself up to 8, then the next
    multiple of 16 up to 64, then the next multiple of 64.  Passes that agree in it (and in their
    attention tiles and wanted rows) launch the same kernels on the same grids."""
    if n <= 8:
        return n
    step = 16 if n <= 64 else 64
    return -(-n // step) * step


class StepError(ValueError):
    """A step the engine refuses before any launch: bad ids, bad slots, no room."""


@dataclass
class StepContext:
    """What the parts see of one pass."""
    n_rows: int
    tokens: torch.Tensor        # int32 [>= n_rows]
    row_slot: torch.Tensor      # int32: the cache slot of each row's sequence
    row_pos: torch.Tensor       # int32: the absolute position of each row
    dtype: torch.dtype
    ws: Workspace
    cache: SequenceCache
    decode: bool                # every sequence brings exactly one token
    n_seqs: int = 0
    max_seq_rows: int = 0       # upper bound on the rows one sequence brings to this pass
    max_context: int = 0        # upper bound on the keys any row reads
    seq_first_row: Optional[torch.Tensor] = None   # int32 [n_seqs + 1]
    seq_slot: Optional[torch.Tensor] = None        # int32 [n_seqs]
    seq_pos0: Optional[torch.Tensor] = None        # int32 [n_seqs]: position of the sequence's first row
    n_tiles: int = 0                               # tiles of consecutive rows of one sequence (prefill attention)
    tile_seq: Optional[torch.Tensor] = None        # int32 [n_tiles]
    tile_row0: Optional[torch.Tensor] = None       # int32 [n_tiles]
    sm_count: int = 0                              # multiprocessors of the device the pass runs on (set by the engine)


def require_gpu(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("this library runs its models on a CUDA device only; it has no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; this library has no CPU path")
    return device


class Engine:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], dtype, device="cuda:0",
                 max_tokens: int = 8192, max_seq_len: Optional[int] = None, max_step_tokens: Optional[int] = None,
                 max_slots: Optional[int] = None, pass_graphs: bool = True):
        self.device = require_gpu(device)
        self.dtype = DTYPES[dtype]
        self.spec = spec
        torch.cuda.set_device(self.device)
        self.max_seq_len = min(max_seq_len or spec.max_position_embeddings, spec.max_position_embeddings)
        self.model = CausalLM(spec, self.dtype, self.device, max_positions=self.max_seq_len)
        self.model.bind(tensors)
        self.vocab_size = spec.vocab_size
        needs = self.model.cache_needs()
        self.cache = SequenceCache(needs, [e.reads_cache_of for e in spec.run_order], max_tokens, self.max_seq_len,
                                   self.dtype, self.device, max_slots=max_slots)
        self.max_step_tokens = int(max_step_tokens or min(8192, max(PAGE_SIZE, max_tokens)))
        self.ws = Workspace(self.max_step_tokens, self.device)
        self.ws.max_want = self.max_step_tokens
        # pass tables (per row: token, slot, position; wanted rows; tiles; per sequence: first row, slot,
        # position), filled by native host code into a small ring of pinned staging buffers and brought
        # to the device with one copy per pass
        width = self.max_step_tokens + 1
        self._meta_dev = torch.zeros((9, width), dtype=torch.int32, device=self.device)
        self._stage = [torch.zeros((9, width), dtype=torch.int32).pin_memory() for _ in range(4)]
        self._stage_events: List[Optional[torch.cuda.Event]] = [None] * len(self._stage)
        self._stage_at = 0
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        # short bfloat16 prompt passes: padded to a few row counts, their launches kept as graphs
        self.replayable = self.model.replayable()
        self.pass_graphs = bool(pass_graphs)
        self._pass_graphs: "OrderedDict[tuple, torch.cuda.CUDAGraph]" = OrderedDict()
        self._pass_seen: Dict[tuple, int] = {}
        self._pass_logits: Optional[torch.Tensor] = None
        self._capture_stream: Optional[torch.cuda.Stream] = None
        self.pass_graph_replays = 0
        if self.dtype == torch.bfloat16:
            from ..csrc import ops
            self._tile_rows = ops.attention_prefill_tile_rows()
        else:
            self._tile_rows = 64

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda:0", **kw) -> "Engine":
        """Loads config.json and the safetensors of `folder`; the model class is chosen by config.json."""
        device = require_gpu(device)
        config = config_from_folder(folder)
        spec = config.to_spec()
        needs = tensor_needs_of_spec(spec)
        tensors = load_folder(folder, needs, DTYPES[dtype], device, same_as=optional_duplicates_of_spec(spec))
        eng = cls(spec, tensors, dtype, device, **kw)
        eng.config = config
        return eng

    @classmethod
    def random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0", linear_std: float = 0.02,
               norm_jitter: float = 0.0, **kw) -> "Engine":
        """A model with random weights made on the device (no folder): the values a folder written
        by `write_model_folder` with the same seed holds, in the config's stored dtype."""
        device = require_gpu(device)
        spec = config.to_spec()
        init = RandomInit(seed, linear_std, norm_jitter)
        stored = DTYPES[config.dtype]
        tensors = {}
        for need in tensor_needs_of_spec(spec):
            t = make_tensor(need, init, stored, device)
            tensors[need.name] = t.to(held_dtype(need, stored, DTYPES[dtype]))
        eng = cls(spec, tensors, dtype, device, **kw)
        eng.config = config
        return eng

    # ------------------------------------------------------------------ sequences
    def new_sequence(self, reserve_tokens: int = 0) -> int:
        return self.cache.acquire(reserve_tokens)

    def free_sequence(self, slot: int) -> None:
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.lengths[slot]

    # ------------------------------------------------------------------ the step
    def _stage_buffer(self) -> Tuple[torch.Tensor, int]:
        i = self._stage_at
        self._stage_at = (i + 1) % len(self._stage)
        ev = self._stage_events[i]
        if ev is not None:
            ev.synchronize()
        return self._stage[i], i

    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """Runs `tokens[i]` as the next tokens of the sequence in `slots[i]`.

        `want[i]` lists the places among `tokens[i]` whose logits are returned (default: the last
        one).  Returns float32 [number wanted, vocab] in the order of the sequences and of `want`.
        All checks happen before the first launch; a refused step changes nothing.
        """
        n_seqs = len(slots)
        if n_seqs == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        if len(tokens) != n_seqs or (want is not None and len(want) != n_seqs):
            raise StepError("slots, tokens and want must have one entry per sequence")
        if len(set(slots)) != n_seqs:
            raise StepError("a slot is named twice in one step")
        lens = [len(t) for t in tokens]
        if min(lens) == 0:
            raise StepError("a sequence brings no token")
        starts = []
        for s, n in zip(slots, lens):
            if not self.cache.slots.is_held(s):
                raise StepError(f"slot {s} is not held by a sequence")
            start = self.cache.lengths[s]
            if start + n > self.max_seq_len:
                raise StepError(f"slot {s}: {start} + {n} tokens exceed the longest sequence, {self.max_seq_len}")
            starts.append(start)
        flat = np.concatenate([np.asarray(t, dtype=np.int64) for t in tokens])
        if flat.min() < 0 or flat.max() >= self.vocab_size:
            raise StepError(f"a token id lies outside the vocabulary of {self.vocab_size}")
        if want is None:
            want = [[n - 1] for n in lens]
        for w, n in zip(want, lens):
            for j in w:
                if not 0 <= j < n:
                    raise StepError(f"a wanted place {j} lies outside the {n} tokens its sequence brings")
        # pages for every sequence, all or nothing
        try:
            self.cache.ensure_all([(s, st + n) for s, st, n in zip(slots, starts, lens)])
        except CacheFull as e:
            raise StepError(f"the cache has no room for this step: {e}") from None

        total = int(flat.shape[0])
        first_row = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
        asked = np.asarray([first_row[i] + j for i, w in enumerate(want) for j in w], dtype=np.int64)
        # A place asked for twice is computed once (two rows of the final norm adding into the same
        # residual row would race) and its logits row is repeated in the result.
        want_flat, repeat = np.unique(asked, return_inverse=True)
        if len(want_flat) == len(asked):
            want_flat, repeat = asked, None
        order = np.argsort(want_flat, kind="stable")
        n_want = len(want_flat)
        logits = torch.empty((n_want, self.vocab_size), dtype=torch.float32, device=self.device)

        decode = max(lens) == 1
        chunk = min(self.max_step_tokens, self.cache.max_chunk)
        step = dict(slots=np.asarray(slots, dtype=np.int32), starts=np.asarray(starts, dtype=np.int32), first_row=first_row,
                    tokens=np.ascontiguousarray(flat, dtype=np.int32), want_sorted=np.ascontiguousarray(want_flat[order]))
        for r0 in range(0, total, chunk):
            self._run_pass(step, r0, min(total, r0 + chunk), order, logits, decode)
        for s, n in zip(slots, lens):
            self.cache.lengths[s] += n
        if self.dtype == torch.bfloat16:
            from ..csrc import ops
            ops.check_tc_status(self.device)
        if repeat is not None:
            logits = logits[torch.from_numpy(repeat).to(self.device)]
        return logits

    def _run_pass(self, step: dict, r0: int, r1: int, order, logits, decode: bool) -> None:
        """Rows [r0, r1) of a step's flattened rows as one launch of the model."""
        from ..csrc import ops
        n = r1 - r0
        # A short bfloat16 prompt pass is launched with a padded row count; the rows past n carry
        # slot -1, belong to no sequence and no tile, write no cache and are wanted by nobody.
        short = self.replayable and self.dtype == torch.bfloat16 and not decode and n <= PASS_GRAPH_MAX_ROWS
        rows = padded_rows(n) if short and padded_rows(n) <= self.ws.max_rows else n
        stage, si = self._stage_buffer()
        ns, n_tiles, max_seq_rows, max_context, lo, hi = ops.plan_pass(
            step["slots"], step["starts"], step["first_row"], step["tokens"], r0, r1, step["want_sorted"], self._tile_rows,
            rows, stage)
        nw = hi - lo
        want_dest = order[lo:hi]
        meta = self._meta_dev
        meta.copy_(stage, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._stage_events[si] = ev
        if short:
            # the host-side numbers a part may size its launches by are rounded up, so that passes
            # with the same key below make the same launches
            max_seq_rows = padded_rows(max_seq_rows)
            max_context = -(-max_context // PAGE_SIZE) * PAGE_SIZE
        ctx = StepContext(
            n_rows=rows, tokens=meta[0], row_slot=meta[1], row_pos=meta[2],
            dtype=self.dtype, ws=self.ws, cache=self.cache, decode=decode, n_seqs=ns,
            max_seq_rows=max_seq_rows, max_context=max_context,
            seq_first_row=meta[6], seq_slot=meta[7], seq_pos0=meta[8],
            n_tiles=n_tiles, tile_seq=meta[4], tile_row0=meta[5], sm_count=self.sm_count)
        in_order = nw == logits.shape[0] and np.array_equal(want_dest, np.arange(nw))
        if short and self.pass_graphs and nw <= PASS_GRAPH_MAX_WANT and (nw == 0 or in_order):
            self._run_short_pass(ctx, (rows, n_tiles, ns, nw, max_seq_rows, max_context), nw, logits)
        elif nw == 0:
            self.model.forward(ctx, None, 0, None)
        elif in_order:
            self.model.forward(ctx, meta[3], nw, logits)
        else:
            out = torch.empty((nw, self.vocab_size), dtype=torch.float32, device=self.device)
            self.model.forward(ctx, meta[3], nw, out)
            logits[torch.from_numpy(want_dest).to(self.device)] = out

    def _run_short_pass(self, ctx: StepContext, key: tuple, nw: int, logits: torch.Tensor) -> None:
        """Launches a short prompt pass, from a CUDA graph once its key has been seen before.

        Everything that differs between two passes with the same key (tokens, slots, positions,
        tiles, the sequences' first rows, the page table) is in device arrays at fixed addresses
        that the launches read, so the launches themselves are the same and can be replayed.  The
        first pass of a key runs eagerly (it also lets libraries and the workspace finish their lazy
        set-up), the second is captured and replayed, later ones are replayed.  The launches and
        their inputs are the same either way, so the results are the same bits.
        """
        from ..csrc import ops
        out = None
        if nw:
            if self._pass_logits is None:
                self._pass_logits = torch.empty((PASS_GRAPH_MAX_WANT, self.vocab_size), dtype=torch.float32,
                                                device=self.device)
            out = self._pass_logits[:nw]
        want = self._meta_dev[3] if nw else None
        entry = self._pass_graphs.get(key)
        if entry is None:
            seen = self._pass_seen.get(key, 0) + 1
            self._pass_seen[key] = seen
            if seen >= 2:
                entry = self._capture_pass(key, ctx, want, nw, out)
        if entry is None:
            self.model.forward(ctx, want, nw, out)
        else:
            graph, uses_tc = entry
            self._pass_graphs.move_to_end(key)
            graph.replay()
            self.pass_graph_replays += 1
            ops.tc_used = ops.tc_used or uses_tc          # so that the step still reads the status word
        if nw:
            logits.copy_(out)

    def _capture_pass(self, key: tuple, ctx: StepContext, want, nw: int, out):
        from ..csrc import ops
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(self.device)
            self._graph_pool = torch.cuda.graph_pool_handle()
        cur, side = torch.cuda.current_stream(self.device), self._capture_stream
        graph = torch.cuda.CUDAGraph()
        was_used, ops.tc_used = ops.tc_used, False
        try:
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                graph.capture_begin(pool=self._graph_pool, capture_error_mode="thread_local")
                try:
                    self.model.forward(ctx, want, nw, out)
                finally:
                    graph.capture_end()
            cur.wait_stream(side)
            self.ws.frozen = True       # the graph holds the buffers' addresses
            entry = (graph, ops.tc_used)
        finally:
            ops.tc_used = was_used
        self._pass_graphs[key] = entry
        while len(self._pass_graphs) > PASS_GRAPHS_KEPT:
            self._pass_graphs.popitem(last=False)
        if len(self._pass_seen) > 4096:
            self._pass_seen.clear()
        return entry

    # ------------------------------------------------------------------ facts for reports
    def describe(self) -> str:
        p = torch.cuda.get_device_properties(self.device)
        return (f"{self.spec.architecture} {len(self.spec.layers)} layers hidden {self.spec.hidden_size} "
                f"vocab {self.spec.vocab_size} dtype {self.dtype} on {p.name} (sm_{p.major}{p.minor}, "
                f"{p.multi_processor_count} SMs); cache {self.cache.groups[0].n_pages if self.cache.groups else 0} "
                f"pages of {self.cache.page_size} tokens, {self.cache.bytes_per_token()} B/token")

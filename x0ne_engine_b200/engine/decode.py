"""A batch of sequences on the device: prompts in one step, then one token each per step.

Between two decode steps the token, the position and the draw counter of every sequence stay on
the device: the sampler kernel writes each pick where the next step reads it and advances the
position, and the step's launches read them from there.  So a decode step has no host-to-device
copy, and its launches are captured once per batch size into a CUDA graph and replayed, as the
library engine does for its single sequence (x0ne-core/runtime/src/engine.rs:484-501,
1095-1132).  Per step the host reads back one int32 per live sequence.

Because a step needs nothing from the host, the step after the one whose picks are being read is
already queued: `step(live)` returns the picks of the step it was asked for and leaves the next
one (for the same rows) running.  A row that the loop ends on those picks has then been stepped
once more than needed; the device has marked it finished where it could know (stop token, budget),
and either way its extra pick is dropped.  So the GPU never waits for the host's decisions.

When sequences finish, the live rows are compacted on the device and the graph of the smaller
batch size is used.  A graph also fixes how the decode attention divides its work, which depends
on how long the sequences are: graphs are kept per (batch size, context bucket), the bucket being
the longest live sequence rounded up to a power of two, so an engine sized for 40,000 positions
does not split a 500-token sequence as if it had 40,000 keys.

What a captured step reads lives at fixed device addresses for the life of the `DeviceBatch`: the
per-row arrays, and a stop-id list of fixed length (`STOP_IDS_ON_DEVICE` entries, unused ones -1)
that `start` refills for every batch, so a graph captured for one batch serves every later batch
whatever its stop tokens.  The int in which this library's tensor-core kernels report a wait that
ran out is copied by the sampler behind the step's picks and read with them; a step whose word is
not zero raises, naming the step.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache import CacheFull
from ..csrc import ops
from .engine import Engine, StepContext
from .generate import GenerationError, Row


# Stop tokens the device itself ends a row on (all rows of a batch must share them).  A batch with
# more, or with different ones per row, leaves them to the host, which decides every pick anyway.
STOP_IDS_ON_DEVICE = 16


# The smallest context bucket: below it the decode attention's division of work does not change.
DECODE_CONTEXT_BUCKET_MIN = 2048


def context_bucket(longest: int, limit: int) -> int:
    """The power of two (at least DECODE_CONTEXT_BUCKET_MIN, at most `limit`) that holds `longest` positions."""
    b = DECODE_CONTEXT_BUCKET_MIN
    while b < longest:
        b *= 2
    return min(b, limit)


def device_stop_ids(rows: Sequence[Row]) -> List[int]:
    """The stop-id list the device gets for a batch: the rows' common stop tokens padded with -1 to
    `STOP_IDS_ON_DEVICE`, or all -1 when the rows differ or have more than fit."""
    stops = {tuple(sorted(set(r.params.stop_token_ids))) for r in rows}
    common = stops.pop() if len(stops) == 1 else ()
    if len(common) > STOP_IDS_ON_DEVICE:
        common = ()
    return list(common) + [-1] * (STOP_IDS_ON_DEVICE - len(common))


class DeviceBatch:
    def __init__(self, engine: Engine, max_batch: int, cuda_graph: bool = True):
        self.engine = engine
        self.max_batch = max_batch
        self.cuda_graph = cuda_graph and engine.replayable      # a part that may not be replayed: every step is launched
        dev = engine.device
        i32 = dict(dtype=torch.int32, device=dev)
        self.tokens = torch.zeros(max_batch, **i32)
        self.row_slot = torch.zeros(max_batch, **i32)
        self.row_pos = torch.zeros(max_batch, **i32)
        self.counter = torch.zeros(max_batch, **i32)
        self.finished = torch.zeros(max_batch, **i32)
        self.budget = torch.zeros(max_batch, **i32)
        self.out_token = torch.zeros(max_batch + 1, **i32)      # picks, then the kernels' status word
        self.temperature = torch.zeros(max_batch, dtype=torch.float32, device=dev)
        self.top_p = torch.ones(max_batch, dtype=torch.float32, device=dev)
        self.seed = torch.zeros(max_batch, dtype=torch.int64, device=dev)
        self.row_best = torch.zeros(max_batch, dtype=torch.int64, device=dev)     # the sampler's scratch: zero between steps
        self.seq_first_row = torch.arange(max_batch + 1, **i32)
        self.want_rows = torch.arange(max_batch, **i32)
        self.logits = torch.empty((max_batch, engine.vocab_size), dtype=torch.float32, device=dev)
        self._out_host = [torch.zeros(max_batch + 1, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._out_event = [torch.cuda.Event(), torch.cuda.Event()]
        self._queued = 0                # steps queued so far (picks buffer = count % 2)
        self._batch_first = 0           # value of _queued when the current batch started
        # (the 32-bit path has no kernel that reports there: it gets a word of its own that stays zero)
        self.status = ops.gemm_tc_status(dev) if engine.dtype == torch.bfloat16 else torch.zeros(1, **i32)
        self._ahead: Optional[List[int]] = None    # rows of the step that is queued and not read yet
        self.run_ahead = True           # queue the next step before reading the current one's picks
        self._per_row = [self.tokens, self.row_slot, self.row_pos, self.counter, self.finished, self.budget,
                         self.temperature, self.top_p, self.seed]
        self.stop_ids = torch.full((STOP_IDS_ON_DEVICE,), -1, **i32)
        self.graphs: Dict[Tuple[int, int], torch.cuda.CUDAGraph] = {}     # by (rows, context bucket)
        self.last_graph: Optional[torch.cuda.CUDAGraph] = None            # the one the latest step replayed
        self.slots: List[int] = []
        self.rows: Sequence[Row] = ()
        self.live: List[int] = []
        self.graph_replays = 0
        self.launches_per_step = 0      # calls of this library's kernel entry points in one decode step
        self.eager_steps = 0
        if engine.ws.max_rows < max_batch:
            raise ValueError("the engine's largest pass is smaller than the batch")

    # ------------------------------------------------------------------ BatchRunner
    def start(self, rows: Sequence[Row]) -> List[int]:
        eng, n = self.engine, len(rows)
        if n > self.max_batch:
            raise GenerationError(f"{n} sequences in a batch of at most {self.max_batch}")
        self.slots = []
        try:
            for r in rows:
                self.slots.append(eng.new_sequence(len(r.prompt) + r.budget))
        except CacheFull:
            self.close()
            raise
        self.rows, self.live = rows, list(range(n))
        host = np.zeros((6, n), dtype=np.int64)
        host[0] = self.slots
        host[1] = [len(r.prompt) - 1 for r in rows]
        host[2] = [r.budget for r in rows]
        host[3] = [r.seed if r.seed < (1 << 63) else r.seed - (1 << 64) for r in rows]
        meta = torch.from_numpy(host).to(eng.device)
        self.row_slot[:n] = meta[0].to(torch.int32)
        self.row_pos[:n] = meta[1].to(torch.int32)
        self.budget[:n] = meta[2].to(torch.int32)
        self.seed[:n] = meta[3]
        self.counter[:n] = 0
        self.finished[:n] = 0
        fl = torch.tensor([[r.params.temperature if not r.params.greedy else 0.0 for r in rows],
                           [r.params.top_p for r in rows]], dtype=torch.float32).to(eng.device)
        self.temperature[:n] = fl[0]
        self.top_p[:n] = fl[1]
        self.stop_ids.copy_(torch.tensor(device_stop_ids(rows), dtype=torch.int32), non_blocking=False)
        logits = eng.step(self.slots, [r.prompt for r in rows])
        self._sample(logits, n)
        self._ahead = None
        self._batch_first = self._queued
        return self._read(self._queue_read(n), n)

    def step(self, live: Sequence[int]) -> List[int]:
        live = list(live)
        if self._ahead is None:
            self._queue_step(live)
        ahead, k = self._ahead, self._queued - 1           # the queued step, and where its picks go
        if ahead != live and not set(live) <= set(ahead):
            raise GenerationError("a decode step was asked for rows that are not in the batch any more")
        self._ahead = None
        if self.run_ahead:
            # rows whose budget the queued step uses up need no step after it
            nxt = [i for i in live if len(self.rows[i].generated) + 1 < self.rows[i].budget]
            if nxt:
                self._queue_step(nxt)                       # runs while the host reads and decides
        picks = self._read(k, len(ahead))
        if ahead == live:
            return picks
        where = {row: j for j, row in enumerate(ahead)}
        return [picks[where[i]] for i in live]

    def close(self) -> None:
        if self._ahead is not None:
            torch.cuda.current_stream().synchronize()       # a step is still running on these slots
            self._ahead = None
        for s in self.slots:
            self.engine.free_sequence(s)
        self.slots, self.rows, self.live = [], (), []

    # ------------------------------------------------------------------ pieces
    def _sample(self, logits: torch.Tensor, n: int) -> None:
        ops.sample(logits, n, self.out_token, temperature=self.temperature, top_p=self.top_p, seed=self.seed,
                   draw_counter=self.counter, stop_ids=self.stop_ids, finished=self.finished, budget=self.budget,
                   next_token=self.tokens, next_pos=self.row_pos, status=self.status, row_best=self.row_best)

    def _queue_step(self, live: List[int]) -> None:
        """Queues one decode step for `live` and the copy of its picks to the host."""
        if live != self.live:
            self._compact(live)
        n = len(live)
        lengths = self.engine.cache.lengths
        bucket = context_bucket(max(int(lengths[self.slots[i]]) for i in live) + 1, self.engine.max_seq_len)
        if self.cuda_graph:
            g = self.graphs.get((n, bucket))
            if g is None:
                g = self._capture(n, bucket)
            g.replay()
            self.last_graph = g
            self.graph_replays += 1
        else:
            self._launch(n, bucket)
            self.eager_steps += 1
        for i in live:
            self.engine.cache.lengths[self.slots[i]] += 1
        self._queue_read(n)
        self._ahead = live

    def _queue_read(self, n: int) -> int:
        k = self._queued
        self._queued += 1
        self._out_host[k % 2][:n + 1].copy_(self.out_token[:n + 1], non_blocking=True)
        self._out_event[k % 2].record()
        return k

    def _read(self, k: int, n: int) -> List[int]:
        """The picks of queued step `k` (n rows), once they have arrived.  The int behind them is the
        status word as it stood when that step's sampler ran; not zero means that a kernel of that
        step, or of an earlier one not yet reported, gave up a bounded wait, so the picks are not
        valid: the word is cleared and the step is named."""
        self._out_event[k % 2].synchronize()
        got = self._out_host[k % 2][:n + 1].tolist()
        if got[n] != 0:
            self.status.zero_()
            what = "the prompts' step" if k == self._batch_first else f"decode step {k - self._batch_first}"
            raise ops.KernelError(f"{what} of this batch: {ops.describe_tc_status(got[n])}")
        return got[:n]

    def _compact(self, live: List[int]) -> None:
        where = {row: k for k, row in enumerate(self.live)}
        idx = torch.tensor([where[i] for i in live], dtype=torch.int64, device=self.engine.device)
        n = len(live)
        for t in self._per_row:
            t[:n] = t[idx]
        self.live = live

    def _launch(self, n: int, max_context: int) -> None:
        eng = self.engine
        ctx = StepContext(n_rows=n, tokens=self.tokens, row_slot=self.row_slot, row_pos=self.row_pos,
                          dtype=eng.dtype, ws=eng.ws, cache=eng.cache, decode=True, n_seqs=n, max_seq_rows=1,
                          max_context=max_context, seq_first_row=self.seq_first_row, seq_slot=self.row_slot,
                          seq_pos0=self.row_pos, sm_count=eng.sm_count)
        eng.model.forward(ctx, self.want_rows, n, self.logits)
        self._sample(self.logits, n)

    def _capture(self, n: int, max_context: int) -> torch.cuda.CUDAGraph:
        """Captures the launches of one decode step of `n` rows whose sequences hold at most
        `max_context` positions (more would still be computed rightly, only divided less well).  The
        warm-up run before the capture would advance the sequences, so their state is saved and
        restored around it."""
        saved = [t[:n].clone() for t in self._per_row]
        saved_out = self.out_token[:n].clone()      # (the status word behind them is not touched)
        torch.cuda.synchronize()
        before = ops.LAUNCHES
        self._launch(n, max_context)            # lets libraries and the workspace finish their lazy set-up
        self.launches_per_step = ops.LAUNCHES - before
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._launch(n, max_context)
        for t, s in zip(self._per_row, saved):
            t[:n] = s
        self.out_token[:n] = saved_out
        torch.cuda.synchronize()
        self.engine.ws.frozen = True      # the graph holds the buffers' addresses
        self.graphs[(n, max_context)] = g
        return g

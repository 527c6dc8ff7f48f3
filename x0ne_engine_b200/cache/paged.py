"""The cache: a slot per sequence, keys and values per run-order entry in pages, per-sequence
state of fixed size beside them.

Run-order entries whose mixers need the same thing (kv heads, head size, window) form a GROUP
with storage of its own: one tensor [entries, pages, 2 (K, V), kv_heads, page_size, head_dim], a
pool of pages and a page table [slots, pages per sequence].  A sequence holds pages only for the
positions it has (all of them, or a ring that covers its window), so the cache is sized in
tokens, not in slots x longest sequence.  Entries whose mixers keep a fixed-size state get a
float32 tensor [slots, *state_shape], zeroed when a slot is taken.

The library engine has one sequence and one plane per layer and K/V,
[layer][k|v][max_ctx][kv_dim] (x0ne-core/runtime/src/engine.rs:83-84,191,747-748), and keeps
K after norm and rotation, V raw (x0ne-core/kernels/cuda/rope.cu:40-46); the latter is kept
here, the former becomes pages.  Reads are bounded by each sequence's length, so a reused page
needs no clearing for correctness.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..csrc.ops import PagedCacheArg
from ..parts.base import CacheNeed
from .slots import CacheFull, FreeList

PAGE_SIZE = 64


def pages_for(tokens: int, page_size: int = PAGE_SIZE) -> int:
    return (tokens + page_size - 1) // page_size


class KVGroup:
    """Storage of the run-order entries that share one kind of key/value need."""

    def __init__(self, need: CacheNeed, entries: List[int], n_pages: int, n_slots: int, max_seq_pages: int,
                 ring_pages: Optional[int], page_size: int, dtype: torch.dtype, device):
        self.need = need
        self.entries = list(entries)
        self.page_size = page_size
        self.n_pages = n_pages
        self.ring_pages = ring_pages if ring_pages is not None else max_seq_pages
        self.table_stride = self.ring_pages
        self.storage = torch.zeros((len(entries), n_pages, 2, need.kv_heads, page_size, need.head_dim),
                                   dtype=dtype, device=device)
        self.pool = FreeList(n_pages, "page")
        self.table_host = np.full((n_slots, self.table_stride), -1, dtype=np.int32)
        self.table = torch.full((n_slots, self.table_stride), -1, dtype=torch.int32, device=device)
        self.pages_of: Dict[int, List[int]] = {}
        self._views: Dict[int, PagedCacheArg] = {}
        page_stride = 2 * need.kv_heads * page_size * need.head_dim
        for i, e in enumerate(self.entries):
            self._views[e] = PagedCacheArg(self.storage[i].data_ptr(), self.table.data_ptr(), page_stride,
                                           self.table_stride, self.ring_pages, page_size, need.kv_heads,
                                           need.head_dim, n_pages)

    def bytes_per_token(self) -> int:
        return len(self.entries) * 2 * self.need.kv_heads * self.need.head_dim * self.storage.element_size()

    def view(self, entry: int) -> PagedCacheArg:
        return self._views[entry]

    def pages_needed(self, tokens: int) -> int:
        return min(pages_for(tokens, self.page_size), self.ring_pages)

    def ensure(self, slot: int, tokens: int) -> bool:
        """Makes the slot hold pages for positions 0..tokens-1 (or its ring).  True if the page
        table changed."""
        have = self.pages_of.setdefault(slot, [])
        want = self.pages_needed(tokens)
        if want <= len(have):
            return False
        new = self.pool.take(want - len(have))
        self.table_host[slot, len(have):want] = new
        have.extend(new)
        return True

    def push_row(self, slot: int) -> None:
        self.table[slot].copy_(torch.from_numpy(self.table_host[slot]))

    def release(self, slot: int) -> None:
        pages = self.pages_of.pop(slot, [])
        self.pool.give_back(pages)
        self.table_host[slot, :] = -1
        # The device row is rewritten when the slot is taken again; stale page numbers are
        # never read because no row of a step names a released slot.


class SequenceCache:
    """All groups and state areas of one model, and the slots that index them."""

    def __init__(self, needs: Sequence[CacheNeed], reads_cache_of: Sequence[Optional[int]], capacity_tokens: int,
                 max_seq_len: int, dtype: torch.dtype, device, max_slots: Optional[int] = None,
                 page_size: int = PAGE_SIZE, max_chunk: int = 1 << 30):
        self.page_size = page_size
        self.device = device
        self.max_seq_len = max_seq_len
        n_pages = max(1, pages_for(capacity_tokens, page_size))
        self.n_slots = max_slots if max_slots is not None else n_pages
        self.max_seq_pages = max(1, min(pages_for(max_seq_len, page_size), n_pages))
        self.slots = FreeList(self.n_slots, "slot")
        self.lengths = [0] * self.n_slots
        self.groups: List[KVGroup] = []
        self.states: Dict[int, torch.Tensor] = {}
        self._group_of: Dict[int, KVGroup] = {}
        self.max_chunk = max_chunk          # most tokens one sequence may bring to one pass
        by_key: Dict[Tuple, List[int]] = {}
        for e, need in enumerate(needs):
            if reads_cache_of[e] is not None:
                continue
            if need.kind == "kv":
                by_key.setdefault((need.kv_heads, need.head_dim, need.window), []).append(e)
            elif need.kind == "state":
                self.states[e] = torch.zeros((self.n_slots,) + tuple(need.state_shape), dtype=torch.float32,
                                             device=device)
            elif need.kind != "none":
                raise ValueError(f"run-order entry {e}: unknown cache need {need.kind!r}")
        for (kvh, hd, window), entries in by_key.items():
            ring = None
            if window is not None:
                # A pass of c tokens of one sequence writes c new keys before its queries read the
                # window of the first of them, so the ring must hold window + c - 1 positions.
                self.max_chunk = min(self.max_chunk, max(page_size, window))
                ring = min(self.max_seq_pages, pages_for(window + self.max_chunk - 1, page_size) + 1)
            g = KVGroup(needs[entries[0]], entries, n_pages if window is None else min(n_pages, ring * self.n_slots),
                        self.n_slots, self.max_seq_pages, ring, page_size, dtype, device)
            self.groups.append(g)
            for e in entries:
                self._group_of[e] = g
        for e, src in enumerate(reads_cache_of):
            if src is not None:
                if src in self._group_of:
                    self._group_of[e] = self._group_of[src]
                elif src in self.states:
                    self.states[e] = self.states[src]
        self._reads = list(reads_cache_of)

    # ---- what parts see
    def kv_view(self, entry: int) -> PagedCacheArg:
        src = self._reads[entry] if self._reads[entry] is not None else entry
        return self._group_of[src].view(src)

    def state(self, entry: int) -> torch.Tensor:
        return self.states[entry]

    # ---- slots
    def free_tokens(self) -> int:
        return min((g.pool.available() for g in self.groups if g.need.window is None), default=1 << 40) * self.page_size

    def acquire(self, reserve_tokens: int = 0) -> int:
        """Takes a free slot, zeroes its state, and reserves pages for `reserve_tokens` positions."""
        if reserve_tokens > self.max_seq_len:
            raise CacheFull(f"{reserve_tokens} tokens asked for, a sequence holds at most {self.max_seq_len}")
        (slot,) = self.slots.take(1)
        self.lengths[slot] = 0
        try:
            for g in self.groups:
                g.ensure(slot, reserve_tokens)
        except CacheFull:
            for g in self.groups:
                g.release(slot)
            self.slots.give_back([slot])
            raise
        for g in self.groups:
            g.push_row(slot)
        for t in {id(t): t for t in self.states.values()}.values():
            t[slot].zero_()
        return slot

    def ensure(self, slot: int, tokens: int) -> None:
        """Grows the slot's pages to hold `tokens` positions."""
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is not held")
        if tokens > self.max_seq_len:
            raise CacheFull(f"slot {slot}: {tokens} tokens, a sequence holds at most {self.max_seq_len}")
        for g in self.groups:
            if g.ensure(slot, tokens):
                g.push_row(slot)

    def ensure_all(self, requests) -> None:
        """`ensure` for several (slot, tokens) at once: either all get their pages or none does."""
        for g in self.groups:
            short = 0
            for slot, tokens in requests:
                if not self.slots.is_held(slot):
                    raise ValueError(f"slot {slot} is not held")
                if tokens > self.max_seq_len:
                    raise CacheFull(f"slot {slot}: {tokens} tokens, a sequence holds at most {self.max_seq_len}")
                short += max(0, g.pages_needed(tokens) - len(g.pages_of.get(slot, [])))
            if short > g.pool.available():
                raise CacheFull(f"{short} pages asked for, {g.pool.available()} of {g.n_pages} free")
        for slot, tokens in requests:
            self.ensure(slot, tokens)

    def release(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise ValueError(f"slot {slot} is freed twice (or was never held)")
        for g in self.groups:
            g.release(slot)
        self.lengths[slot] = 0
        self.slots.give_back([slot])

    def bytes_per_token(self) -> int:
        return sum(g.bytes_per_token() for g in self.groups)

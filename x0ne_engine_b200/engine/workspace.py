"""Activation buffers of a step, allocated once per name and reused by every layer."""
from __future__ import annotations

from typing import Dict, Tuple

import torch


class Workspace:
    """`buffer(name, shape, dtype)` returns the same tensor for the same name every time.

    Parts name their scratch generically ("attn.qkv", "ffn.act", "delta"), so layers of the same
    kind share it; a name asked for with a larger shape or another dtype is allocated anew.  Once
    a CUDA graph has been captured over the workspace (`frozen`), the graph holds the buffers'
    addresses: new names may still be added, but replacing a buffer that exists raises instead of
    leaving the graph with a pointer to freed memory.
    """

    def __init__(self, max_rows: int, device):
        self.max_rows = max_rows
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}
        self.frozen = False

    def buffer(self, name: str, shape: Tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        t = self._bufs.get(name)
        n = 1
        for s in shape:
            n *= s
        if t is None or t.dtype != dtype or t.numel() < n:
            if self.frozen and t is not None:
                raise RuntimeError(f"workspace buffer {name!r} ({t.numel()} x {t.dtype}) would be replaced by "
                                   f"{n} x {dtype} although a captured graph uses it")
            t = torch.empty(n, dtype=dtype, device=self.device)
            self._bufs[name] = t
        return t[:n].view(shape)

    def zeroed(self, name: str, nbytes: int) -> torch.Tensor:
        """A uint8 buffer that is zero when first handed out and whose user leaves it zero where it
        needs zeros (arrival counters); grown, and zeroed again, when a larger one is asked for."""
        t = self._bufs.get(name)
        if t is None or t.numel() < nbytes:
            if self.frozen and t is not None:
                raise RuntimeError(f"workspace buffer {name!r} would be replaced although a captured graph uses it")
            t = torch.zeros(max(nbytes, 1), dtype=torch.uint8, device=self.device)
            self._bufs[name] = t
        return t

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._bufs.values())

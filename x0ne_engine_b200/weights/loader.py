"""Weights by tensor name: what a model needs, checked against what a folder holds.

Every part declares its tensors as `TensorNeed`s.  `check` compares the whole set with a
folder before any byte is copied and before the GPU is touched, and raises ONE
`WeightsError` that lists every missing tensor, every unexpected tensor, every wrong shape
and every wrong dtype (x0ne-core/runtime/src/weights.rs:120-161 checks the same things;
x0ne-core/runtime/src/engine.rs:318-321 checks them before the device is opened).

Dtype policy.  `role="matrix"` tensors are held in the run's compute dtype: bfloat16 in a
bfloat16 run (a bfloat16 checkpoint is kept bit for bit), float32 in a 32-bit run (a
bfloat16 checkpoint is widened exactly).  `role="vector"` tensors (norm weights and other
small per-channel values) are always held in float32, so one stored in 32-bit stays so and a
bfloat16 one is widened exactly, which is what a kernel does with it anyway.
`role="stored"` keeps the stored floating dtype untouched.  Integer tensors of any width
become int32 (`role="table"`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, Mapping, Optional, Tuple

import torch

from .safetensors_io import SafetensorsError, TensorSource, open_folder

_FLOATS = {"BF16", "F16", "F32", "F64"}
_INTS = {"I64", "I32", "I16", "I8", "U8"}


@dataclass(frozen=True)
class TensorNeed:
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"          # matrix | vector | stored | table
    init: str = "linear"          # linear | embedding | norm : which random distribution


class WeightsError(ValueError):
    """A folder whose tensors do not match the model; lists every difference."""

    def __init__(self, missing, unexpected, wrong_shape, wrong_dtype, other=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
        self.other = list(other)
        lines = ["the checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n} is {list(got)}, the model needs {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtypes ({len(self.wrong_dtype)}): " + "; ".join(
                f"{n} is {got}, the model needs {want}" for n, got, want in self.wrong_dtype))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


def check(source: TensorSource, needs: Iterable[TensorNeed],
          same_as: Optional[Mapping[str, str]] = None) -> None:
    """Raises WeightsError unless the folder holds exactly the needed tensors.

    `same_as` maps a tensor name that MAY be present to the needed tensor it must equal byte
    for byte (a tied checkpoint that also carries its head,
    x0ne-core/runtime/src/weights.rs:154-159).
    """
    needs = list(needs)
    same_as = dict(same_as or {})
    want = {n.name: n for n in needs}
    have = set(source.names())
    missing = sorted(n for n in want if n not in have)
    unexpected = sorted(n for n in have if n not in want and n not in same_as)
    wrong_shape, wrong_dtype, other = [], [], []
    for name, need in want.items():
        if name not in have:
            continue
        meta = source.meta(name)
        if tuple(meta.shape) != tuple(need.shape):
            wrong_shape.append((name, meta.shape, need.shape))
        if need.role == "table":
            if meta.dtype not in _INTS:
                wrong_dtype.append((name, meta.dtype, "an integer type"))
        elif meta.dtype not in _FLOATS or meta.dtype in ("F16", "F64"):
            wrong_dtype.append((name, meta.dtype, "BF16 or F32"))
    for extra, base in same_as.items():
        if extra in have and base in have:
            if bytes(source.raw(extra)) != bytes(source.raw(base)) or \
                    source.meta(extra).dtype != source.meta(base).dtype:
                other.append(f"{extra} is present in a tied checkpoint but differs from {base}")
    if missing or unexpected or wrong_shape or wrong_dtype or other:
        raise WeightsError(missing, unexpected, wrong_shape, wrong_dtype, other)


def held_dtype(need: TensorNeed, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    """The dtype a tensor is held in on the device (the policy of this module's header)."""
    if need.role == "table":
        return torch.int32
    if need.role == "vector":
        return torch.float32
    if need.role == "stored":
        return stored
    return compute


def load(source: TensorSource, needs: Iterable[TensorNeed], compute: torch.dtype,
         device) -> Dict[str, torch.Tensor]:
    """Copies every needed tensor to the device in the dtype the policy gives it."""
    out: Dict[str, torch.Tensor] = {}
    for need in needs:
        t = source.tensor(need.name)
        dt = held_dtype(need, t.dtype, compute)
        if need.role == "table" and t.numel() and (int(t.max()) > 2**31 - 1 or int(t.min()) < -2**31):
            raise WeightsError([], [], [], [], [f"{need.name} holds values outside int32"])
        out[need.name] = t.to(device=device, dtype=dt, copy=True).contiguous()
    return out


def load_folder(folder: str, needs: Iterable[TensorNeed], compute: torch.dtype, device,
                same_as: Optional[Mapping[str, str]] = None) -> Dict[str, torch.Tensor]:
    needs = list(needs)
    source = open_folder(folder)
    try:
        check(source, needs, same_as)
        return load(source, needs, compute, device)
    finally:
        source.close()


__all__ = ["TensorNeed", "WeightsError", "SafetensorsError", "check", "load", "load_folder",
           "held_dtype"]

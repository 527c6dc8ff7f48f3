"""Random weights from a configuration and a seed.

Every value is a pure function of (seed, tensor name, element index): a splitmix64 hash
gives two uniforms per element and Box-Muller turns them into a normal deviate in float64,
which is then scaled and rounded to the stored dtype.  Because nothing depends on the order
of generation, a tensor can be made on any device, in pieces, and a model folder written on
the CPU holds the values a direct on-device initialisation would make (up to the last bit of
float64 `log`/`cos` between devices, which the rounding to float32 or bfloat16 hides in all
but vanishingly rare elements).

Distributions (the ones the benchmark configurations name): projections and embeddings
N(0, linear_std); norm weights 1 + N(0, norm_jitter), or exactly 1 when norm_jitter is 0.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Iterable, Iterator, Tuple

import torch

from .loader import TensorNeed
from .safetensors_io import write_file_streaming

_GOLDEN = 0x9E3779B97F4A7C15
_M1 = 0xBF58476D1CE4E5B9
_M2 = 0x94D049BB133111EB
_MASK = (1 << 64) - 1


def _signed(x: int) -> int:
    x &= _MASK
    return x - (1 << 64) if x >= (1 << 63) else x


def _lsr(z: torch.Tensor, s: int) -> torch.Tensor:
    return (z >> s) & ((1 << (64 - s)) - 1)


def _mix(z: torch.Tensor) -> torch.Tensor:
    z = (z ^ _lsr(z, 30)) * _signed(_M1)
    z = (z ^ _lsr(z, 27)) * _signed(_M2)
    return z ^ _lsr(z, 31)


def _mix_int(z: int) -> int:
    z &= _MASK
    z = ((z ^ (z >> 30)) * _M1) & _MASK
    z = ((z ^ (z >> 27)) * _M2) & _MASK
    return z ^ (z >> 31)


def tensor_key(seed: int, name: str) -> int:
    """A 64-bit key for one tensor: FNV-1a of its name, mixed with the seed."""
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & _MASK
    return _mix_int(h ^ _mix_int(seed & _MASK))


def standard_normal(key: int, start: int, count: int, device) -> torch.Tensor:
    """Elements [start, start + count) of the tensor's stream of N(0, 1) deviates, float64."""
    idx = torch.arange(start, start + count, dtype=torch.int64, device=device)
    a = _mix((idx * 2) * _signed(_GOLDEN) + _signed(key))
    b = _mix((idx * 2 + 1) * _signed(_GOLDEN) + _signed(key))
    u1 = (_lsr(a, 11).to(torch.float64) + 1.0) * (1.0 / (1 << 53))      # (0, 1]
    u2 = _lsr(b, 11).to(torch.float64) * (1.0 / (1 << 53))              # [0, 1)
    return torch.sqrt(-2.0 * torch.log(u1)) * torch.cos((2.0 * math.pi) * u2)


@dataclass(frozen=True)
class RandomInit:
    seed: int = 0
    linear_std: float = 0.02
    norm_jitter: float = 0.0


def make_tensor(need: TensorNeed, init: RandomInit, dtype: torch.dtype, device,
                chunk: int = 1 << 24) -> torch.Tensor:
    n = 1
    for s in need.shape:
        n *= s
    out = torch.empty(n, dtype=dtype, device=device)
    if need.role == "table":
        raise ValueError(f"{need.name}: integer tables have no random initialisation")
    if need.init == "norm" and init.norm_jitter == 0.0:
        out.fill_(1.0)
        return out.reshape(need.shape)
    key = tensor_key(init.seed, need.name)
    for start in range(0, n, chunk):
        c = min(chunk, n - start)
        z = standard_normal(key, start, c, device)
        if need.init == "norm":
            z = 1.0 + init.norm_jitter * z
        else:
            z = init.linear_std * z
        out[start:start + c] = z.to(dtype)
    return out.reshape(need.shape)


def make_tensors(needs: Iterable[TensorNeed], init: RandomInit, dtype: torch.dtype,
                 device) -> Iterator[Tuple[TensorNeed, torch.Tensor]]:
    for need in needs:
        yield need, make_tensor(need, init, dtype, device)


def write_model_folder(folder: str, config, init: RandomInit = RandomInit(), needs=None, device=None) -> None:
    """Writes config.json and model.safetensors of a randomly initialised model.

    `config` is an architecture's configuration object (`to_dict`, `to_spec`, `dtype`).  The
    tensors are stored in the config's dtype.
    """
    from ..engine.model import tensor_needs_of_spec
    os.makedirs(folder, exist_ok=True)
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[config.dtype]
    needs = list(needs if needs is not None else tensor_needs_of_spec(config.to_spec()))
    # The values depend on (seed, name, index) only, so they are made where that is fastest (an
    # 8B model takes a quarter of an hour on the host and seconds on a GPU) and written one tensor
    # at a time.
    device = device if device is not None else ("cuda" if torch.cuda.is_available() else "cpu")
    plan = [(n.name, dtype, n.shape) for n in needs]
    write_file_streaming(os.path.join(folder, "model.safetensors"), plan,
                         (t for _, t in make_tensors(needs, init, dtype, device)))
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config.to_dict(), f, indent=1)

"""Reading and writing safetensors files, by tensor name.

The format: 8 bytes little-endian header length, a JSON header mapping each tensor name to
{dtype, shape, data_offsets}, then the bytes.  A model folder holds either one
`model.safetensors` or `model.safetensors.index.json` with its shards, never both; shard
names must be plain file names; a tensor lives in exactly one shard and in the one the index
names (x0ne-core/runtime/src/st.rs:70-179).  Files are memory-mapped; a tensor is a view
until it is copied to the device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

_DTYPES = {
    "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4),
    "F64": (torch.float64, 8), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}

MAX_HEADER_BYTES = 100 << 20
SINGLE = "model.safetensors"
INDEX = "model.safetensors.index.json"


class SafetensorsError(ValueError):
    """A file that is not a well-formed safetensors file, or a folder that breaks the rules."""


@dataclass(frozen=True)
class TensorMeta:
    dtype: str
    shape: Tuple[int, ...]
    start: int        # byte offsets inside the data section
    end: int
    file: str

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][0]


def _numel(shape: Iterable[int]) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


def read_header(path: str) -> Tuple[Dict[str, TensorMeta], int]:
    """(name -> meta, offset of the data section) of one file, fully checked."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise SafetensorsError(f"{path}: shorter than a header length")
        (n,) = struct.unpack("<Q", head)
        if n > MAX_HEADER_BYTES or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file")
        raw = f.read(n)
    try:
        header = json.loads(raw)
    except (json.JSONDecodeError, UnicodeDecodeError) as e:
        raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
    if not isinstance(header, dict):
        raise SafetensorsError(f"{path}: header is not an object")
    data_len = size - 8 - n
    metas: Dict[str, TensorMeta] = {}
    spans: List[Tuple[int, int, str]] = []
    for name, m in header.items():
        if name == "__metadata__":
            continue
        try:
            dtype, shape, (a, b) = m["dtype"], tuple(m["shape"]), m["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"{path}: tensor {name!r} has a malformed entry") from None
        if dtype not in _DTYPES:
            raise SafetensorsError(f"{path}: tensor {name!r} has dtype {dtype!r}, not served")
        if any(isinstance(s, bool) or not isinstance(s, int) or s < 0 for s in shape):
            raise SafetensorsError(f"{path}: tensor {name!r} has a bad shape {shape}")
        if not (isinstance(a, int) and isinstance(b, int) and 0 <= a <= b <= data_len):
            raise SafetensorsError(f"{path}: tensor {name!r} lies outside the file")
        if b - a != _numel(shape) * _DTYPES[dtype][1]:
            raise SafetensorsError(f"{path}: tensor {name!r}: {b - a} bytes for shape {shape} {dtype}")
        metas[name] = TensorMeta(dtype, shape, a, b, path)
        spans.append((a, b, name))
    spans.sort()
    for (a0, b0, n0), (a1, b1, n1) in zip(spans, spans[1:]):
        if a1 < b0:
            raise SafetensorsError(f"{path}: tensors {n0!r} and {n1!r} overlap")
    return metas, 8 + n


class TensorSource:
    """The tensors of a model folder, by name."""

    def __init__(self, metas: Mapping[str, TensorMeta], data_offsets: Mapping[str, int]):
        self._metas = dict(metas)
        self._data_offsets = dict(data_offsets)
        self._maps: Dict[str, mmap.mmap] = {}

    def names(self) -> List[str]:
        return list(self._metas)

    def meta(self, name: str) -> TensorMeta:
        return self._metas[name]

    def __contains__(self, name: str) -> bool:
        return name in self._metas

    def _map(self, path: str) -> mmap.mmap:
        m = self._maps.get(path)
        if m is None:
            with open(path, "rb") as f:
                m = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
            self._maps[path] = m
        return m

    def raw(self, name: str) -> memoryview:
        meta = self._metas[name]
        base = self._data_offsets[meta.file]
        return memoryview(self._map(meta.file))[base + meta.start: base + meta.end]

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapped bytes (read-only: copy before writing)."""
        meta = self._metas[name]
        n = _numel(meta.shape)
        if n == 0:
            return torch.empty(meta.shape, dtype=meta.torch_dtype)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.frombuffer(self.raw(name), dtype=meta.torch_dtype, count=n)
        return t.reshape(meta.shape)

    def close(self) -> None:
        for m in self._maps.values():
            try:
                m.close()
            except BufferError:
                pass
        self._maps.clear()


def open_folder(folder: str) -> TensorSource:
    single = os.path.join(folder, SINGLE)
    index = os.path.join(folder, INDEX)
    has_single, has_index = os.path.isfile(single), os.path.isfile(index)
    if has_single and has_index:
        raise SafetensorsError(f"{folder}: both {SINGLE} and {INDEX} are present")
    if has_single:
        metas, off = read_header(single)
        return TensorSource(metas, {single: off})
    if not has_index:
        raise SafetensorsError(f"{folder}: neither {SINGLE} nor {INDEX} is present")
    try:
        with open(index) as f:
            weight_map = json.load(f)["weight_map"]
        assert isinstance(weight_map, dict)
    except Exception:
        raise SafetensorsError(f"{index}: no weight_map object") from None
    metas: Dict[str, TensorMeta] = {}
    offsets: Dict[str, int] = {}
    seen_in: Dict[str, str] = {}
    for shard in sorted(set(weight_map.values())):
        if not isinstance(shard, str) or os.path.basename(shard) != shard or shard in ("", ".", ".."):
            raise SafetensorsError(f"{index}: shard name {shard!r} is not a plain file name")
        path = os.path.join(folder, shard)
        shard_metas, off = read_header(path)
        offsets[path] = off
        for name, meta in shard_metas.items():
            if name in seen_in:
                raise SafetensorsError(f"{folder}: tensor {name!r} is in {seen_in[name]} and in {shard}")
            seen_in[name] = shard
            if weight_map.get(name) != shard:
                raise SafetensorsError(f"{folder}: tensor {name!r} is in {shard}, the index names "
                                       f"{weight_map.get(name)!r}")
            metas[name] = meta
    for name, shard in weight_map.items():
        if name not in metas:
            raise SafetensorsError(f"{folder}: the index names tensor {name!r} in {shard}, which lacks it")
    return TensorSource(metas, offsets)


def write_file_streaming(path: str, plan, tensors) -> None:
    """Writes one safetensors file without holding it in memory: `plan` lists (name, dtype, shape)
    in file order, which fixes the header; `tensors` then yields the tensors in that order (from
    any device), and each is written and dropped."""
    header, at = {}, 0
    plan = list(plan)
    for name, dtype, shape in plan:
        if dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {dtype} cannot be written")
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        header[name] = {"dtype": _NAMES[dtype], "shape": [int(d) for d in shape], "data_offsets": [at, at + nbytes]}
        at += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode()
    raw += b" " * (-len(raw) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for (name, dtype, shape), t in zip(plan, tensors):
            t = t.detach().to("cpu").contiguous()
            if t.dtype != dtype or tuple(t.shape) != tuple(int(d) for d in shape):
                raise SafetensorsError(f"tensor {name!r}: got {t.dtype} {tuple(t.shape)}, planned {dtype} {tuple(shape)}")
            f.write(memoryview(t.reshape(-1).view(torch.uint8).numpy()))
    os.replace(tmp, path)


def write_file(path: str, tensors: Mapping[str, torch.Tensor]) -> None:
    """Writes tensors (moved to the CPU) as one safetensors file, names in the given order."""
    header = {}
    blobs = []
    at = 0
    for name, t in tensors.items():
        t = t.detach().to("cpu").contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be written")
        b = t.reshape(-1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(b)]}
        at += len(b)
        blobs.append(b)
    raw = json.dumps(header, separators=(",", ":")).encode()
    raw += b" " * (-len(raw) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for b in blobs:
            f.write(b)
    os.replace(tmp, path)

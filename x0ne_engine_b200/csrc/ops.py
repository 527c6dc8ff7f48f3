"""Python entry points of the CUDA kernels: argument checks, then one C call each.

Tensors are torch CUDA tensors; a kernel gets raw device pointers and runs on torch's current
stream, so calls order themselves with torch work and can be captured into a CUDA graph.
Every function raises `KernelError` when the C entry point refuses its arguments or the launch
fails; nothing here computes on the CPU or through another library.
"""
from __future__ import annotations

import ctypes
from ctypes import Structure, c_float, c_int, c_int32, c_int64, c_void_p
from typing import Optional

import torch

from . import build as _build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_tag(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"no kernel for dtype {dtype}")


class PagedCacheArg(Structure):
    """Mirror of `struct PagedCache` in common.cuh."""
    _fields_ = [("base", c_void_p), ("page_table", c_void_p), ("page_stride", c_int64),
                ("table_stride", c_int32), ("ring_pages", c_int32), ("page_size", c_int32),
                ("kv_heads", c_int32), ("head_dim", c_int32), ("n_pages", c_int32)]


class SampleIOArg(Structure):
    """Mirror of `struct SampleIO` in sampling.cu."""
    _fields_ = [("logits", c_void_p), ("temperature", c_void_p), ("top_p", c_void_p), ("seed", c_void_p),
                ("draw_counter", c_void_p), ("stop_ids", c_void_p), ("finished", c_void_p), ("budget", c_void_p),
                ("out_token", c_void_p), ("next_token", c_void_p), ("next_pos", c_void_p),
                ("status", c_void_p), ("row_best", c_void_p), ("ld", c_int64), ("vocab", c_int32), ("n_stop", c_int32)]


_libs = {}


_P, _I, _F, _L = c_void_p, c_int, c_float, c_int64
# Argument types of the entry points, declared once per library: ctypes then converts plain Python
# numbers itself, which is about a third of the cost of building a c_int or c_void_p per argument
# and per call (1.4 us against 3.8 us for ten arguments).  Pointers are passed as integers.
_SIGNATURES = {
    "x0ne_embedding": [_P, _I, _P, _P, _I, _I, _I, _P],
    "x0ne_add_rmsnorm": [_P, _P, _P, _P, _I, _P, _I, _I, _F, _P],
    "x0ne_qk_norm_rope_kv_write": [_P, _I, _P, _P, _P, _I, _P, None, _P, _P, _I, _I, _F, _I, _P, _I, _P],
    "x0ne_swiglu": [_P, _P, _I, _I, _I, _P],
    "x0ne_attention_rows": [_P, _P, _I, None, _P, _P, _I, _I, _F, _I, _P],
    "x0ne_gemm_f32_nt": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "x0ne_attention_prefill_bf16": [_P, _P, None, _P, _P, _I, _P, _P, _P, _I, _F, _I, _P],
    "x0ne_attention_decode_bf16": [_P, _P, None, _P, _P, _I, _I, _F, _I, _I, _P, _L, _P],
    "x0ne_attention_decode_grouped_bf16": [_P, _P, None, _P, _P, _I, _I, _F, _I, _I, _I, _P, _L, _P],
    "x0ne_gemm_bf16_smallm": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P],
    "x0ne_attention_prefill_tcgen05": [_P, _P, _I, None, _P, _P, _I, _P, _P, _P, _I, _F, _I, _P, _P],
    "x0ne_gemm_bf16_tcgen05": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "x0ne_gemm_bf16_skinny_tcgen05": [_P, _P, _I, _P, _I, _I, _I, _I, _I, _P, _P],
    "x0ne_sample": ["io", _I, _P],
    "x0ne_plan_pass": [_I, _P, _P, _P, _P, _L, _L, _P, _I, _I, _I, _P, _L, _P],
}


def _lib(name: str) -> ctypes.CDLL:
    lib = _libs.get(name)
    if lib is None:
        lib = _build.load(name)
        lib.x0ne_last_error.restype = ctypes.c_char_p
        for fn_name, args in _SIGNATURES.items():
            fn = getattr(lib, fn_name, None)
            if fn is not None:
                # None: the cache view, by value; "io": the sampler's arguments, by value
                fn.argtypes = [PagedCacheArg if a is None else SampleIOArg if a == "io" else a for a in args]
                fn.restype = c_int
        _libs[name] = lib
    return lib


def loaded_libraries():
    """Paths of the kernel libraries this process has loaded."""
    return [lib._name for lib in _libs.values()]


LAUNCHES = 0   # kernel entry points called by this process (one or a few launches each)


def _check(lib, code: int, what: str) -> None:
    global LAUNCHES
    LAUNCHES += 1
    if code != 0:
        msg = lib.x0ne_last_error()
        raise KernelError(f"{what}: {msg.decode() if msg else 'error'} (code {code})")


def _stream() -> int:
    """The current stream of the current device, as a raw handle (the private accessor is some
    forty times cheaper than building a torch.cuda.Stream object for every launch)."""
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None:
        return raw(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, dtype, what: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} is not on the GPU")
    if t.dtype != dtype:
        raise KernelError(f"{what} is {t.dtype}, the kernel needs {dtype}")
    if not t.is_contiguous():
        raise KernelError(f"{what} is not contiguous")


def plan_pass(slots, starts, first_row, tokens, r0: int, r1: int, want_sorted, tile_rows: int, launch_rows: int,
              stage: torch.Tensor):
    """Fills the pinned staging table `stage` (int32 [9][stride]) for rows [r0, r1) of a step (native
    host code, step_plan.cu).  `slots`, `starts` (int32 per sequence), `first_row` (int64, one more
    than sequences), `tokens` (int32, all rows of the step) and `want_sorted` (int64) are contiguous
    NumPy arrays.  Returns (sequences in the pass, tiles, most rows of one sequence, one more than the
    largest position, lo, hi) with want_sorted[lo:hi] the wanted rows of the pass."""
    lib = _lib("core")
    out = (c_int32 * 6)()
    code = lib.x0ne_plan_pass(len(slots), slots.ctypes.data, starts.ctypes.data, first_row.ctypes.data,
                              tokens.ctypes.data, r0, r1, want_sorted.ctypes.data, len(want_sorted), tile_rows,
                              launch_rows, stage.data_ptr(), stage.stride(0), ctypes.addressof(out))
    if code != 0:
        msg = lib.x0ne_last_error()
        raise KernelError(f"plan_pass: {msg.decode() if msg else 'error'} (code {code})")
    return tuple(out)


def embedding(table: torch.Tensor, tokens: torch.Tensor, resid: torch.Tensor, n_rows: int) -> None:
    """resid[r] = float32(table[tokens[r]]); an id outside the table gives a zero row."""
    lib = _lib("core")
    _need(tokens, torch.int32, "tokens")
    _need(resid, torch.float32, "residual")
    _need(table, table.dtype, "embedding table")
    vocab, hidden = table.shape
    if resid.shape[-1] != hidden or resid.numel() < n_rows * hidden or tokens.numel() < n_rows:
        raise KernelError("embedding: buffers are smaller than the rows asked for")
    _check(lib, lib.x0ne_embedding(_ptr(table), dtype_tag(table.dtype), _ptr(tokens), _ptr(resid),
                                   n_rows, hidden, vocab, _stream()), "embedding")


def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                n_rows: int, eps: float, rows: Optional[torch.Tensor] = None) -> None:
    """resid += delta (if given); out = rmsnorm(resid) * weight.  `rows` gathers source rows."""
    lib = _lib("core")
    hidden = weight.numel()
    _need(resid, torch.float32, "residual")
    _need(weight, torch.float32, "norm weight")
    _need(out, out.dtype, "norm output")
    if delta is not None:
        _need(delta, out.dtype, "delta")
        if delta.shape[-1] != hidden:
            raise KernelError("add_rmsnorm: delta width differs from the norm's")
    if rows is not None:
        _need(rows, torch.int32, "row list")
        if rows.numel() < n_rows:
            raise KernelError("add_rmsnorm: row list shorter than the rows asked for")
    elif resid.numel() < n_rows * hidden:
        raise KernelError("add_rmsnorm: residual smaller than the rows asked for")
    if resid.shape[-1] != hidden or out.shape[-1] != hidden or out.numel() < n_rows * hidden:
        raise KernelError("add_rmsnorm: widths differ or output too small")
    _check(lib, lib.x0ne_add_rmsnorm(_ptr(resid), _ptr(delta), _ptr(weight), _ptr(out), dtype_tag(out.dtype),
                                     _ptr(rows), n_rows, hidden, eps, _stream()), "add_rmsnorm")


def qk_norm_rope_kv_write(qkv: torch.Tensor, q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor],
                          inv_freq: Optional[torch.Tensor], rotary_dim: int, q_out: torch.Tensor,
                          cache: PagedCacheArg, row_slot: torch.Tensor, row_pos: torch.Tensor, n_rows: int,
                          q_heads: int, eps: float, write_kv: bool = True,
                          rope_table: Optional[torch.Tensor] = None) -> None:
    """q/k head norm, rotation and cache write.  `rope_table` (float32 [positions, rotary_dim]: each
    row the cosines then the sines of position * inv_freq) replaces the on-the-fly sines and cosines
    for the positions it covers."""
    lib = _lib("core")
    _need(qkv, qkv.dtype, "qkv")
    _need(q_out, qkv.dtype, "q output")
    _need(row_slot, torch.int32, "row slots")
    _need(row_pos, torch.int32, "row positions")
    hd, kvh = cache.head_dim, cache.kv_heads
    if qkv.shape[-1] != (q_heads + 2 * kvh) * hd or q_out.shape[-1] != q_heads * hd:
        raise KernelError("rope: qkv or q widths do not match the head counts")
    if qkv.numel() < n_rows * qkv.shape[-1] or q_out.numel() < n_rows * q_out.shape[-1]:
        raise KernelError("rope: buffers smaller than the rows asked for")
    for w, what in ((q_norm, "q_norm"), (k_norm, "k_norm")):
        if w is not None:
            _need(w, torch.float32, what)
            if w.numel() != hd:
                raise KernelError(f"rope: {what} has {w.numel()} values, head_dim is {hd}")
    if inv_freq is not None:
        _need(inv_freq, torch.float32, "inv_freq")
        if inv_freq.numel() * 2 != rotary_dim:
            raise KernelError("rope: inv_freq length is not rotary_dim / 2")
    table_positions = 0
    if rope_table is not None:
        _need(rope_table, torch.float32, "rope table")
        if rope_table.dim() != 2 or rope_table.shape[1] != rotary_dim:
            raise KernelError("rope: the table is not [positions, rotary_dim]")
        table_positions = rope_table.shape[0]
    _check(lib, lib.x0ne_qk_norm_rope_kv_write(
        _ptr(qkv), dtype_tag(qkv.dtype), _ptr(q_norm), _ptr(k_norm), _ptr(inv_freq), rotary_dim,
        _ptr(q_out), cache, _ptr(row_slot), _ptr(row_pos), n_rows, q_heads, eps,
        1 if write_kv else 0, _ptr(rope_table), table_positions, _stream()), "qk_norm_rope_kv_write")


def attention_rows(q: torch.Tensor, out: torch.Tensor, cache: PagedCacheArg, row_slot: torch.Tensor,
                   row_pos: torch.Tensor, n_rows: int, q_heads: int, scale: float, window: int = 0) -> None:
    """The plain attention kernel: any head size up to 256, any window (0 = none)."""
    lib = _lib("core")
    _need(q, q.dtype, "q")
    _need(out, q.dtype, "attention output")
    _need(row_slot, torch.int32, "row slots")
    _need(row_pos, torch.int32, "row positions")
    width = q_heads * cache.head_dim
    if q.shape[-1] != width or out.shape[-1] != width or q.numel() < n_rows * width or out.numel() < n_rows * width:
        raise KernelError("attention: q or output do not match the head counts and rows")
    _check(lib, lib.x0ne_attention_rows(_ptr(q), _ptr(out), dtype_tag(q.dtype), cache, _ptr(row_slot),
                                        _ptr(row_pos), n_rows, q_heads, scale, window,
                                        _stream()), "attention_rows")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, n_rows: int) -> None:
    lib = _lib("core")
    _need(gate_up, gate_up.dtype, "gate_up")
    _need(out, gate_up.dtype, "swiglu output")
    inter = out.shape[-1]
    if gate_up.shape[-1] != 2 * inter or gate_up.numel() < n_rows * 2 * inter or out.numel() < n_rows * inter:
        raise KernelError("swiglu: widths or rows do not match")
    _check(lib, lib.x0ne_swiglu(_ptr(gate_up), _ptr(out), dtype_tag(out.dtype), n_rows, inter,
                                _stream()), "swiglu")


def gemm_f32_nt(a: torch.Tensor, w: torch.Tensor, c: torch.Tensor, m: int) -> None:
    """c[:m] = a[:m] @ w.T in true float32, one fixed-order FMA chain per output."""
    lib = _lib("core")
    _need(a, torch.float32, "gemm input")
    _need(w, torch.float32, "gemm weight")
    _need(c, torch.float32, "gemm output")
    n, k = w.shape
    if a.shape[-1] != k or c.shape[-1] != n or a.numel() < m * k or c.numel() < m * n:
        raise KernelError(f"gemm_f32: shapes a {tuple(a.shape)} w {tuple(w.shape)} c {tuple(c.shape)} m {m}")
    _check(lib, lib.x0ne_gemm_f32_nt(_ptr(a), _ptr(w), _ptr(c), m, n, k, k, k,
                                     n, _stream()), "gemm_f32_nt")


def sample(logits: torch.Tensor, n_rows: int, out_token: torch.Tensor, *, temperature=None, top_p=None, seed=None,
           draw_counter=None, stop_ids=None, finished=None, budget=None, next_token=None, next_pos=None,
           status=None, row_best=None) -> None:
    """Picks a token per logits row on the device (see sampling.cu for the rules).  `stop_ids` may
    be padded with -1 (no token has that id).  With `status` (one int32 on the device) the kernel
    also copies that int to out_token[n_rows], so it reaches the host with the picks.  With
    `row_best` (one int64 per row, zero; left zero) a launch of many blocks per row finds the rows'
    largest logits first, which one block per row takes 17 us for at a vocabulary of 151,936."""
    lib = _lib("core")
    _need(logits, torch.float32, "logits")
    _need(out_token, torch.int32, "token output")
    if logits.dim() != 2 or logits.shape[0] < n_rows or out_token.numel() < n_rows:
        raise KernelError("sample: logits or output smaller than the rows asked for")
    for t, dt, what in ((temperature, torch.float32, "temperature"), (top_p, torch.float32, "top_p"),
                        (seed, torch.int64, "seed"), (draw_counter, torch.int32, "draw counter"),
                        (finished, torch.int32, "finished flags"), (budget, torch.int32, "budget"),
                        (next_token, torch.int32, "next token"), (next_pos, torch.int32, "next position")):
        if t is not None:
            _need(t, dt, what)
            if t.numel() < n_rows:
                raise KernelError(f"sample: {what} shorter than the rows asked for")
    if status is not None:
        _need(status, torch.int32, "status word")
        if out_token.numel() < n_rows + 1:
            raise KernelError("sample: no room for the status word after the picks")
    if row_best is not None:
        _need(row_best, torch.int64, "largest-logit scratch")
        if row_best.numel() < n_rows:
            raise KernelError("sample: largest-logit scratch shorter than the rows asked for")
    n_stop = 0
    if stop_ids is not None and stop_ids.numel() > 0:
        _need(stop_ids, torch.int32, "stop ids")
        n_stop = stop_ids.numel()
    io = SampleIOArg(_ptr(logits), _ptr(temperature), _ptr(top_p), _ptr(seed), _ptr(draw_counter),
                     _ptr(stop_ids if n_stop else None), _ptr(finished), _ptr(budget), _ptr(out_token),
                     _ptr(next_token), _ptr(next_pos), _ptr(status), _ptr(row_best), logits.stride(0), logits.shape[1], n_stop)
    _check(lib, lib.x0ne_sample(io, n_rows, _stream()), "sample")
    if row_best is not None and n_rows > 0:
        global LAUNCHES
        LAUNCHES += 1        # that entry point launched two kernels


# ---------------------------------------------------------------------------------------------
# bfloat16 tensor-core attention (module `fast`)
# ---------------------------------------------------------------------------------------------
def fast_attention_takes(cache: PagedCacheArg, dtype: torch.dtype) -> bool:
    """Whether the tensor-core attention kernels take this shape; otherwise the plain kernel does."""
    return dtype == torch.bfloat16 and cache.page_size == 64 and cache.head_dim % 16 == 0 \
        and 16 <= cache.head_dim <= 128


def attention_prefill_bf16(q: torch.Tensor, out: torch.Tensor, cache: PagedCacheArg, tile_seq: torch.Tensor,
                           tile_row0: torch.Tensor, n_tiles: int, seq_first_row: torch.Tensor,
                           seq_slot: torch.Tensor, seq_pos0: torch.Tensor, q_heads: int, scale: float,
                           window: int = 0) -> None:
    """Causal flash attention of a pass whose sequences bring several rows; a tile is up to
    `attention_prefill_tile_rows()` consecutive rows of one sequence."""
    lib = _lib("fast")
    _need(q, torch.bfloat16, "q")
    _need(out, torch.bfloat16, "attention output")
    for t, what in ((tile_seq, "tile sequences"), (tile_row0, "tile rows"), (seq_first_row, "sequence rows"),
                    (seq_slot, "sequence slots"), (seq_pos0, "sequence positions")):
        _need(t, torch.int32, what)
    if tile_seq.numel() < n_tiles or tile_row0.numel() < n_tiles:
        raise KernelError("attention_prefill: tile tables shorter than the tiles asked for")
    if q.shape[-1] != q_heads * cache.head_dim or out.shape[-1] != q.shape[-1]:
        raise KernelError("attention_prefill: q or output width does not match the head counts")
    for first in range(0, n_tiles, 65535):
        n = min(65535, n_tiles - first)
        _check(lib, lib.x0ne_attention_prefill_bf16(
            _ptr(q), _ptr(out), cache, tile_seq.data_ptr() + 4 * first,
            tile_row0.data_ptr() + 4 * first, n, _ptr(seq_first_row), _ptr(seq_slot), _ptr(seq_pos0),
            q_heads, scale, window, _stream()), "attention_prefill_bf16")


def attention_prefill_tile_rows() -> int:
    """Rows of one tile of the prefill attention kernel (callers build their tile tables with it)."""
    return int(_lib("fast").x0ne_attention_prefill_tile_rows())


def attention_decode_blocks_per_sm() -> int:
    return int(_lib("fast").x0ne_attention_decode_blocks_per_sm())


_max_clusters = {}


def attention_decode_max_clusters(head_dim: int, splits: int) -> int:
    """Clusters of `splits` blocks of the decode kernel that run at once on this GPU (0: unknown)."""
    key = (torch.cuda.current_device(), head_dim, splits)
    if key not in _max_clusters:
        _max_clusters[key] = int(_lib("fast").x0ne_attention_decode_max_clusters(c_int(head_dim), c_int(splits)))
    return _max_clusters[key]


def attention_decode_scratch_bytes(n_rows: int, q_heads: int, kv_heads: int, head_dim: int, splits: int) -> int:
    lib = _lib("fast")
    lib.x0ne_attention_decode_scratch_bytes.restype = c_int64
    return int(lib.x0ne_attention_decode_scratch_bytes(c_int(n_rows), c_int(q_heads), c_int(kv_heads),
                                                       c_int(head_dim), c_int(splits)))


ATTENTION_DECODE_CLUSTER_SPLITS = 8     # splits that can merge inside one thread-block cluster
ATTENTION_DECODE_MAX_SPLITS = 64        # blocks per (sequence, kv head) the kernel takes


def attention_decode_bf16(q: torch.Tensor, out: torch.Tensor, cache: PagedCacheArg, row_slot: torch.Tensor,
                          row_pos: torch.Tensor, n_rows: int, q_heads: int, scale: float, window: int, splits: int,
                          scratch: Optional[torch.Tensor], groups: int = 1) -> None:
    """Split-KV flash decoding: one query row per sequence.  `scratch` (uint8, zero when first
    used; the kernel leaves its counters at zero) holds the partial results when splits > 1; without
    it (and with at most 8 splits) the splits merge inside a thread-block cluster instead.  With
    `groups` > 1 the splits are `groups` clusters of splits / groups blocks (2 to 8): each cluster
    merges in shared memory and the clusters' results meet in `scratch` (sized for `groups` parts)."""
    lib = _lib("fast")
    _need(q, torch.bfloat16, "q")
    _need(out, torch.bfloat16, "attention output")
    _need(row_slot, torch.int32, "row slots")
    _need(row_pos, torch.int32, "row positions")
    width = q_heads * cache.head_dim
    if q.shape[-1] != width or out.shape[-1] != width or q.numel() < n_rows * width or out.numel() < n_rows * width:
        raise KernelError("attention_decode: q or output do not match the head counts and rows")
    if row_slot.numel() < n_rows or row_pos.numel() < n_rows:
        raise KernelError("attention_decode: row tables shorter than the rows asked for")
    nbytes = 0
    if scratch is not None:
        _need(scratch, torch.uint8, "decode scratch")
        nbytes = scratch.numel()
    if groups > 1:
        _check(lib, lib.x0ne_attention_decode_grouped_bf16(
            _ptr(q), _ptr(out), cache, _ptr(row_slot), _ptr(row_pos), n_rows, q_heads, scale,
            window, splits, groups, _ptr(scratch), nbytes, _stream()), "attention_decode_grouped_bf16")
        return
    _check(lib, lib.x0ne_attention_decode_bf16(
        _ptr(q), _ptr(out), cache, _ptr(row_slot), _ptr(row_pos), n_rows, q_heads, scale,
        window, splits, _ptr(scratch), nbytes, _stream()), "attention_decode_bf16")


# ---------------------------------------------------------------------------------------------
# bfloat16 small-M weight-streaming product (module `fast`)
# ---------------------------------------------------------------------------------------------
SMALL_M_MAX_ROWS = 32       # rows the weight-streaming kernel takes (which products use it: routes.py)
_sm_count = {}


def _sms(device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    n = _sm_count.get(idx)
    if n is None:
        n = _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def gemm_smallm_takes(w: torch.Tensor, m: int, swiglu: bool = False) -> bool:
    """Whether the weight-streaming kernel takes this shape."""
    return w.dtype == torch.bfloat16 and 0 < m <= SMALL_M_MAX_ROWS and w.shape[1] % 8 == 0 and not (swiglu and w.shape[0] % 2)


def gemm_bf16_smallm(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, m: int, swiglu: bool = False) -> None:
    """y[:m] = x[:m] @ w.T for m <= 32 by streaming w once; y is bfloat16 or float32.  With
    `swiglu`, w is the packed [gate; up] weight and y[:m] = silu(x gate^T) * (x up^T)."""
    lib = _lib("fast")
    _need(x, torch.bfloat16, "gemm input")
    _need(w, torch.bfloat16, "gemm weight")
    _need(y, y.dtype, "gemm output")
    rows, k = w.shape
    n = rows // 2 if swiglu else rows
    if x.shape[-1] != k or y.shape[-1] != n or x.numel() < m * k or y.numel() < m * n or (swiglu and rows % 2):
        raise KernelError(f"gemm_smallm: shapes x {tuple(x.shape)} w {tuple(w.shape)} y {tuple(y.shape)} m {m}")
    if y.dtype == torch.float32 and not swiglu:
        kind = 1
    elif y.dtype == torch.bfloat16:
        kind = 2 if swiglu else 0
    else:
        raise KernelError(f"gemm_smallm: no output kind for {y.dtype} (swiglu={swiglu})")
    _check(lib, lib.x0ne_gemm_bf16_smallm(_ptr(w), _ptr(x), _ptr(y), m, n, k, n,
                                          kind, _sms(w.device), _stream()), "gemm_bf16_smallm")


# ---------------------------------------------------------------------------------------------
# bfloat16 product on tcgen05 tensor cores with TMA operands (module `tc`), for passes with many rows
# ---------------------------------------------------------------------------------------------
_tc_status = {}
tc_used = False          # set when a tcgen05 product was launched since the last check_tc_status()


def gemm_tc_takes(w: torch.Tensor, m: int) -> bool:
    """Whether the tcgen05 product for many rows takes this shape (from which row count it is used: routes.py)."""
    return w.dtype == torch.bfloat16 and m >= 1 and w.shape[1] % 8 == 0


def check_tc_status(device) -> None:
    """Raises if a tcgen05 kernel reported a barrier wait that ran out (reads one int back)."""
    global tc_used
    if not tc_used:
        return
    tc_used = False
    st = int(gemm_tc_status(device)[0])
    if st != 0:
        gemm_tc_status(device).zero_()
        raise KernelError(describe_tc_status(st))


def describe_tc_status(st: int) -> str:
    """The message for a status word that is not zero: one bit per kind of wait that ran out."""
    codes = [b for b in range(32) if st >> b & 1]
    return (f"a tcgen05 kernel gave up waiting on a barrier (codes {codes}; products: 1 copy, 2 MMA, "
            "3 epilogue, 4 accumulator; attention: 5 queries, 6 keys, 13 and 15 values, 7 probabilities, "
            "8, 11 and 14 output, 10, 12 and 17 scores, 16 and 18 the other half of the row; 9: misaligned "
            "shared memory); its output is not valid")


def gemm_tc_status(device) -> torch.Tensor:
    """The int the tcgen05 kernels report a timed-out barrier wait in (0 = all waits succeeded)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _tc_status.get(idx)
    if t is None:
        t = _tc_status[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return t


def gemm_bf16_tcgen05(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, m: int, swiglu: bool = False,
                      pair: bool = True) -> None:
    """y[:m] = x[:m] @ w.T on the tcgen05 tensor cores (128 x 256 tiles, TMA loads, accumulator in
    tensor memory; with `pair`, pairs of blocks on 256 x 256 tiles); y is bfloat16 or float32.  With `swiglu`, w is the packed [gate; up] weight and
    y[:m] = silu(x gate^T) * (x up^T).  Needs K % 8 == 0."""
    lib = _lib("tc")
    _need(x, torch.bfloat16, "gemm input")
    _need(w, torch.bfloat16, "gemm weight")
    _need(y, y.dtype, "gemm output")
    rows, k = w.shape
    n = rows // 2 if swiglu else rows
    if x.shape[-1] != k or y.shape[-1] != n or x.numel() < m * k or y.numel() < m * n or (swiglu and rows % 2):
        raise KernelError(f"gemm_tc: shapes x {tuple(x.shape)} w {tuple(w.shape)} y {tuple(y.shape)} m {m}")
    if y.dtype == torch.float32 and not swiglu:
        kind = 1
    elif y.dtype == torch.bfloat16:
        kind = 2 if swiglu else 0
    else:
        raise KernelError(f"gemm_tc: no output kind for {y.dtype} (swiglu={swiglu})")
    global tc_used
    tc_used = True
    _check(lib, lib.x0ne_gemm_bf16_tcgen05(_ptr(w), _ptr(x), _ptr(y), m, n, k, n,
                                           kind, 1 if pair else 0, _ptr(gemm_tc_status(w.device)),
                                           _stream()), "gemm_bf16_tcgen05")


SKINNY_MIN_ROWS, SKINNY_MAX_ROWS = 9, 64


def gemm_skinny_tc_takes(w: torch.Tensor, m: int) -> bool:
    """Whether the tcgen05 product for few rows takes this shape (more rows than the weight-streaming
    kernel is best at, few enough for one accumulator tile)."""
    return w.dtype == torch.bfloat16 and SKINNY_MIN_ROWS <= m <= SKINNY_MAX_ROWS and w.shape[1] % 8 == 0


def product_kernel(w: torch.Tensor, m: int, fused: bool = False) -> str:
    """The kernel the routing table names for m rows against w, or "library" where that kernel does not
    take the shape (a width that is no multiple of 8)."""
    from . import routes
    kernel = routes.kernel_for(m, w.shape[0], w.shape[1], fused=fused, sms=_sms(w.device))
    can = {"smallm": gemm_smallm_takes(w, m, fused), "skinny": gemm_skinny_tc_takes(w, m), "tc_pair": gemm_tc_takes(w, m),
           "library": True}[kernel]
    return kernel if can else "library"


def gemm_bf16_skinny_tcgen05(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, m: int, swiglu: bool = False) -> None:
    """y[:m] = x[:m] @ w.T for up to 64 rows on tcgen05, K cut over the blocks of a cluster that add
    their partial sums through shared memory; y is bfloat16 or float32.  With `swiglu`, w is the
    packed [gate; up] weight and y[:m] = silu(x gate^T) * (x up^T).  Failures of its bounded waits
    show in `gemm_tc_status`."""
    global tc_used
    lib = _lib("tc")
    _need(x, torch.bfloat16, "gemm input")
    _need(w, torch.bfloat16, "gemm weight")
    _need(y, y.dtype, "gemm output")
    rows, k = w.shape
    n = rows // 2 if swiglu else rows
    if x.shape[-1] != k or y.shape[-1] != n or x.numel() < m * k or y.numel() < m * n or (swiglu and rows % 2):
        raise KernelError(f"gemm_skinny_tc: shapes x {tuple(x.shape)} w {tuple(w.shape)} y {tuple(y.shape)} m {m}")
    if y.dtype == torch.float32 and not swiglu:
        kind = 1
    elif y.dtype == torch.bfloat16:
        kind = 2 if swiglu else 0
    else:
        raise KernelError(f"gemm_skinny_tc: no output kind for {y.dtype} (swiglu={swiglu})")
    tc_used = True
    x_rows = x.numel() // k      # rows really behind x: the copies may read them all (their results are not used)
    _check(lib, lib.x0ne_gemm_bf16_skinny_tcgen05(_ptr(w), _ptr(x), x_rows, _ptr(y), m, n, k, n, kind,
                                                  _ptr(gemm_tc_status(x.device)), _stream()), "gemm_bf16_skinny_tcgen05")


def attention_tc_takes(cache: PagedCacheArg, dtype: torch.dtype) -> bool:
    """Whether the tcgen05 prefill attention takes this shape."""
    return dtype == torch.bfloat16 and cache.page_size == 64 and cache.head_dim in (64, 128)


def attention_prefill_tcgen05(q: torch.Tensor, out: torch.Tensor, cache: PagedCacheArg, tile_seq: torch.Tensor,
                              tile_row0: torch.Tensor, n_tiles: int, seq_first_row: torch.Tensor,
                              seq_slot: torch.Tensor, seq_pos0: torch.Tensor, q_heads: int, scale: float,
                              window: int = 0) -> None:
    """Causal flash attention of a pass whose sequences bring several rows, on tcgen05 with TMA loads;
    tiles are up to 128 consecutive rows of one sequence (`attention_prefill_tile_rows()`)."""
    global tc_used
    lib = _lib("tc")
    _need(q, torch.bfloat16, "q")
    _need(out, torch.bfloat16, "attention output")
    for t, what in ((tile_seq, "tile sequences"), (tile_row0, "tile rows"), (seq_first_row, "sequence rows"),
                    (seq_slot, "sequence slots"), (seq_pos0, "sequence positions")):
        _need(t, torch.int32, what)
    if tile_seq.numel() < n_tiles or tile_row0.numel() < n_tiles:
        raise KernelError("attention_prefill_tc: tile tables shorter than the tiles asked for")
    if q.dim() != 2 or q.shape[-1] != q_heads * cache.head_dim or out.shape != q.shape:
        raise KernelError("attention_prefill_tc: q or output do not match the head counts")
    tc_used = True
    for first in range(0, n_tiles, 65535):
        n = min(65535, n_tiles - first)
        _check(lib, lib.x0ne_attention_prefill_tcgen05(
            _ptr(q), _ptr(out), q.shape[0], cache, tile_seq.data_ptr() + 4 * first,
            tile_row0.data_ptr() + 4 * first, n, _ptr(seq_first_row), _ptr(seq_slot), _ptr(seq_pos0),
            q_heads, scale, window, _ptr(gemm_tc_status(q.device)), _stream()),
            "attention_prefill_tcgen05")

"""The reference project's own CUDA kernels on this GPU, for timing beside this library's.

Nothing of the product path is here: `kernel-bench --impl reference` is the only caller.  The
reference's kernel sources are compiled UNCHANGED into one cubin, the way its build script does it
(x0ne-core/kernels/build.rs:59-77: `nvcc -cubin --gpu-architecture=sm_100a -O3 -std=c++17 -Icuda
cuda/x0ne_kernels.cu`), loaded through the CUDA driver API into the context torch uses, and
launched at the grids their definitions document (x0ne-core/kernels/cuda/*.cu; the split-K plan
of x0ne-core/runtime/src/gpu.rs:958-985 and its launch of x0ne-core/runtime/src/ops.rs:80-121).
Their interface is one sequence at a time (positions from one device word), a contiguous cache
[max_ctx][kv_heads][128] and head size 128, so they are timed at batch 1 only.

The sources are looked for in `$X0NE_REFERENCE_KERNELS`, else in `baseline/_ref/x0ne-core/kernels/cuda`
under the repository (an unmodified copy of the reference's folder).  Without them `load()` raises
`ReferenceUnavailable` with the reason.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
import tempfile
from ctypes import byref, c_char_p, c_float, c_int, c_uint, c_uint32, c_uint64, c_void_p
from typing import Dict, Optional, Sequence

import torch

from .csrc.build import find_nvcc

HEAD_DIM = 128
SPLIT_TILE = 128
SPLIT_STATE = HEAD_DIM + 4
SPLIT_BLOCK = 128


class ReferenceUnavailable(RuntimeError):
    pass


def sources_dir() -> str:
    env = os.environ.get("X0NE_REFERENCE_KERNELS")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for cand in (env, os.path.join(root, "baseline", "_ref", "x0ne-core", "kernels", "cuda")):
        if cand and os.path.isfile(os.path.join(cand, "x0ne_kernels.cu")):
            return cand
    raise ReferenceUnavailable("the reference's kernel sources (x0ne-core/kernels/cuda) are not under baseline/_ref "
                               "and X0NE_REFERENCE_KERNELS does not name them")


def build_cubin(src: Optional[str] = None) -> str:
    """The reference's single translation unit compiled for sm_100a with its own flags; the cubin is
    kept beside the sources (or in the temporary folder when that is read-only)."""
    src = src or sources_dir()
    out = os.path.join(os.path.dirname(src), "x0ne_kernels.sm_100a.cubin")
    try:
        with open(out + ".w", "w"):
            pass
        os.remove(out + ".w")
    except OSError:
        out = os.path.join(tempfile.gettempdir(), f"x0ne_reference_kernels_{os.getuid()}.sm_100a.cubin")
    newest = max(os.path.getmtime(os.path.join(src, f)) for f in os.listdir(src))
    if os.path.isfile(out) and os.path.getmtime(out) >= newest:
        return out
    cmd = [find_nvcc(), "-cubin", "--gpu-architecture=sm_100a", "-O3", "-std=c++17", "-Werror", "all-warnings",
           f"-I{src}", "-o", out, os.path.join(src, "x0ne_kernels.cu")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise ReferenceUnavailable(f"nvcc failed on the reference's kernels:\n{r.stdout}\n{r.stderr}")
    return out


class ReferenceKernels:
    """The loaded cubin; `launch(name, grid, block, args)` on torch's current stream."""

    def __init__(self, cubin: str):
        try:
            self.drv = ctypes.CDLL("libcuda.so.1")
        except OSError as e:
            raise ReferenceUnavailable(f"the CUDA driver library cannot be loaded: {e}") from None
        torch.cuda.init()
        torch.zeros(1, device="cuda")                    # makes the primary context current on this thread
        self.module = c_void_p()
        self._check(self.drv.cuModuleLoad(byref(self.module), c_char_p(cubin.encode())), "cuModuleLoad")
        self._functions: Dict[str, c_void_p] = {}

    def _check(self, code: int, what: str) -> None:
        if code != 0:
            msg = c_char_p()
            self.drv.cuGetErrorString(c_int(code), byref(msg))
            raise RuntimeError(f"{what}: CUDA driver error {code} ({(msg.value or b'?').decode()})")

    def function(self, name: str) -> c_void_p:
        f = self._functions.get(name)
        if f is None:
            f = c_void_p()
            self._check(self.drv.cuModuleGetFunction(byref(f), self.module, c_char_p(name.encode())),
                        f"cuModuleGetFunction({name})")
            self._functions[name] = f
        return f

    def blocks_per_sm(self, name: str, block: int) -> int:
        n = c_int(0)
        self._check(self.drv.cuOccupancyMaxActiveBlocksPerMultiprocessor(byref(n), self.function(name), c_int(block),
                                                                         ctypes.c_size_t(0)), "occupancy")
        return max(0, n.value)

    def launch(self, name: str, grid: Sequence[int], block: int, args: Sequence) -> None:
        """`args`: ctypes values in the kernel's parameter order (pointers as c_uint64)."""
        gx, gy = (list(grid) + [1])[:2]
        holders = list(args)
        params = (c_void_p * len(holders))(*[ctypes.cast(byref(a), c_void_p) for a in holders])
        stream = c_void_p(torch.cuda.current_stream().cuda_stream)
        self._check(self.drv.cuLaunchKernel(self.function(name), c_uint(gx), c_uint(gy), c_uint(1), c_uint(block),
                                            c_uint(1), c_uint(1), c_uint(0), stream, params, None), f"launch of {name}")


_loaded: Optional[ReferenceKernels] = None


def load() -> ReferenceKernels:
    global _loaded
    if _loaded is None:
        _loaded = ReferenceKernels(build_cubin())
    return _loaded


def _p(t: Optional[torch.Tensor]) -> c_uint64:
    return c_uint64(0 if t is None else t.data_ptr())


def _u(v: int) -> c_uint32:
    return c_uint32(v)


def split_plan(k: ReferenceKernels, q_heads: int, kv_heads: int, sms: int):
    """(kernel name, blocks along x, slices P): one wave of the grouped split-K kernel over the GPU
    (x0ne-core/runtime/src/gpu.rs:958-985); groups of 1, 2, 4 and 8 q heads have a kernel."""
    group = q_heads // kv_heads
    if group in (1, 2, 4, 8):
        name, grid_x = f"x0ne_attention_decode_split_g{group}_bf16", kv_heads
    else:
        name, grid_x = "x0ne_attention_decode_split_bf16", q_heads
    per_sm = k.blocks_per_sm(name, SPLIT_BLOCK)
    return name, grid_x, max(1, sms * per_sm // grid_x), group in (1, 2, 4, 8)


def attention_decode(k, q, k_cache, v_cache, state, counter, out, pos, q_heads, kv_heads, max_ctx, scale, plan):
    """Split-K decode with the last block merging (the loaded engine's default for grouped kernels)."""
    name, grid_x, splits, grouped = plan
    if grouped:
        k.launch(name, (grid_x, splits), SPLIT_BLOCK, [_p(q), _p(k_cache), _p(v_cache), _p(state), _p(counter), _p(out),
                                                      _p(pos), _u(q_heads), _u(kv_heads), _u(max_ctx), _u(splits),
                                                      c_float(scale)])
    else:
        k.launch(name, (grid_x, splits), SPLIT_BLOCK, [_p(q), _p(k_cache), _p(v_cache), _p(state), _p(pos), _u(q_heads),
                                                      _u(kv_heads), _u(max_ctx), _u(splits), c_float(scale)])
        k.launch("x0ne_attention_merge_bf16", (q_heads, 1), SPLIT_BLOCK, [_p(state), _p(out), _p(pos), _u(max_ctx),
                                                                          _u(splits)])


def attention_prefill(k, q, k_cache, v_cache, out, pos0, rows, q_heads, kv_heads, max_ctx, scale):
    """grid (q_heads, ceil(rows / 8)), block 256 (x0ne-core/kernels/cuda/attention.cu:83-85)."""
    k.launch("x0ne_attention_prefill_bf16", (q_heads, (rows + 7) // 8), 256,
             [_p(q), _p(k_cache), _p(v_cache), _p(out), _p(pos0), _u(rows), _u(q_heads), _u(kv_heads), _u(max_ctx),
              c_float(scale)])


def add_rmsnorm(k, residual, x, w, out, rows, hidden, eps):
    """grid (rows), block 256 (x0ne-core/kernels/cuda/rmsnorm.cu:4)."""
    k.launch("x0ne_add_rmsnorm_bf16", (rows, 1), 256, [_p(residual), _p(x), _p(w), _p(out), _u(hidden), c_float(eps)])


def qk_norm_rope_kv_write(k, qkv, q_norm, k_norm, inv_freq, q_out, k_cache, v_cache, pos0, rows, q_heads, kv_heads,
                          max_ctx, eps):
    """grid (q_heads + kv_heads, rows), block 64 (x0ne-core/kernels/cuda/rope.cu:4-6)."""
    k.launch("x0ne_qk_norm_rope_kv_write_bf16", (q_heads + kv_heads, rows), 64,
             [_p(qkv), _p(q_norm), _p(k_norm), _p(inv_freq), _p(q_out), _p(k_cache), _p(v_cache), _p(pos0), _u(q_heads),
              _u(kv_heads), _u(max_ctx), c_float(eps)])


def swiglu(k, gate_up, out, rows, inter):
    """grid (ceil(inter / 256), rows), block 256 (x0ne-core/kernels/cuda/swiglu.cu)."""
    k.launch("x0ne_swiglu_bf16", ((inter + 255) // 256, rows), 256, [_p(gate_up), _p(out), _u(inter)])


def embedding(k, table, tokens, out, rows, hidden, vocab):
    """grid (rows), block 128 (x0ne-core/kernels/cuda/embedding.cu)."""
    k.launch("x0ne_embedding_bf16", (rows, 1), 128, [_p(table), _p(tokens), _p(out), _u(hidden), _u(vocab)])


def argmax(k, logits, n, out, rows=1):
    """grid (rows), block 1024 (x0ne-core/kernels/cuda/argmax.cu)."""
    k.launch("x0ne_argmax_f32", (rows, 1), 1024, [_p(logits), _u(n), _p(out)])


def advance(k, pos):
    """grid (1), block 32 (x0ne-core/kernels/cuda/advance.cu)."""
    k.launch("x0ne_advance_u32", (1, 1), 32, [_p(pos)])


class DecodeStepInReferenceOrder:
    """One greedy decode step of one sequence made of the reference's kernels and cuBLAS products, in
    the order the reference engine launches them (x0ne-core/runtime/src/engine.rs:744-835: embedding,
    zeroed float32 residual, per layer add+RMSNorm / q|k|v product / q,k norm + RoPE + cache write /
    split-K attention with the last block merging / o product / add+RMSNorm / gate|up product / SwiGLU
    / down product, then the final norm, the float32 logits product, argmax and the position advance).

    It is this library's host code that launches them, so it is NOT the reference engine and no
    reference arm of a benchmark: it says what the reference's own device code costs per step on
    this GPU.  Random bfloat16 weights (every layer its own, so a step streams them from memory),
    a cache filled up to `context` positions."""

    def __init__(self, k: ReferenceKernels, layers: int, hidden: int, inter: int, q_heads: int, kv_heads: int, vocab: int,
                 context: int, device="cuda:0"):
        if hidden % 8 or context < 1:
            raise ValueError("hidden must be a multiple of 8 and the context at least 1")
        self.k, self.layers, self.h, self.inter, self.qh, self.kvh, self.vocab = k, layers, hidden, inter, q_heads, kv_heads, vocab
        self.max_ctx = context + 64
        hd = HEAD_DIM
        w = lambda r, c: torch.randn(r, c, device=device).mul_(0.02).bfloat16()      # noqa: E731
        ones = lambda n: torch.ones(n, device=device).bfloat16()                        # noqa: E731
        self.embed, self.lm_head, self.final_norm = w(vocab, hidden), w(vocab, hidden), ones(hidden)
        self.w = [dict(qkv=w((q_heads + 2 * kv_heads) * hd, hidden), o=w(hidden, q_heads * hd), gate_up=w(2 * inter, hidden),
                       down=w(hidden, inter), n1=ones(hidden), n2=ones(hidden), qn=ones(hd), kn=ones(hd)) for _ in range(layers)]
        self.kv = torch.randn(layers, 2, self.max_ctx, kv_heads * hd, device=device).bfloat16()
        self.inv_freq = (1e6 ** (-torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd)).contiguous()
        bf = lambda n: torch.zeros(1, n, device=device, dtype=torch.bfloat16)           # noqa: E731
        self.delta, self.normed, self.qkv, self.q, self.att = bf(hidden), bf(hidden), bf((q_heads + 2 * kv_heads) * hd), bf(q_heads * hd), bf(q_heads * hd)
        self.gate_up, self.act = bf(2 * inter), bf(inter)
        self.residual = torch.zeros(1, hidden, device=device)
        self.logits = torch.zeros(1, vocab, device=device)
        self.token = torch.tensor([17], dtype=torch.int32, device=device)
        self.pos = torch.tensor([context - 1], dtype=torch.int32, device=device)
        self.pos0 = context - 1
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        self.plan = split_plan(k, q_heads, kv_heads, sms)
        self.state = torch.zeros(q_heads * self.plan[2] * SPLIT_STATE, device=device)
        self.counter = torch.zeros(max(q_heads, kv_heads), dtype=torch.int32, device=device)
        self.scale = 1.0 / (hd ** 0.5)

    def weight_bytes(self) -> int:
        per_layer = sum(v.numel() for name, v in self.w[0].items() if name in ("qkv", "o", "gate_up", "down")) * 2
        return self.layers * per_layer + self.lm_head.numel() * 2

    def launch(self) -> None:
        k, h = self.k, self.h
        embedding(k, self.embed, self.token, self.delta, 1, h, self.vocab)
        self.residual.zero_()
        for l, w in enumerate(self.w):
            add_rmsnorm(k, self.residual, self.delta, w["n1"], self.normed, 1, h, 1e-6)
            torch.mm(self.normed, w["qkv"].t(), out=self.qkv)
            qk_norm_rope_kv_write(k, self.qkv, w["qn"], w["kn"], self.inv_freq, self.q, self.kv[l, 0], self.kv[l, 1], self.pos, 1,
                                  self.qh, self.kvh, self.max_ctx, 1e-6)
            attention_decode(k, self.q, self.kv[l, 0], self.kv[l, 1], self.state, self.counter, self.att, self.pos, self.qh, self.kvh,
                             self.max_ctx, self.scale, self.plan)
            torch.mm(self.att, w["o"].t(), out=self.delta)
            add_rmsnorm(k, self.residual, self.delta, w["n2"], self.normed, 1, h, 1e-6)
            torch.mm(self.normed, w["gate_up"].t(), out=self.gate_up)
            swiglu(k, self.gate_up, self.act, 1, self.inter)
            torch.mm(self.act, w["down"].t(), out=self.delta)
        add_rmsnorm(k, self.residual, self.delta, self.final_norm, self.normed, 1, h, 1e-6)
        torch.mm(self.normed, self.lm_head.t(), out_dtype=torch.float32, out=self.logits)
        argmax(k, self.logits, self.vocab, self.token)
        advance(k, self.pos)

    def reset(self) -> None:
        self.pos.fill_(self.pos0)
        self.token.fill_(17)

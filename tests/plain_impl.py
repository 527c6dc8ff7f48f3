"""Plain, slow Qwen3 dense forward in NumPy: whole sequences, no cache, one function per part.

This file is the tests' yardstick.  It shares no code with the package under test: it has
its own config reader, its own safetensors reader and its own arithmetic.  Everything is
computed in float64 unless `dtype=np.float32` is asked for.

It rests on the formulas of x0ne-labs/x0ne-Engine's x0ne-core (each function cites
file:line by the file's path inside that project).  The project's own model code is Rust
and its kernels are CUDA, neither of which can be compiled and run on a CPU-only machine
without a Rust toolchain, so there is no call into it; instead `tests/golden/` holds the
project's own tiny float32 Qwen3 checkpoint with the logits its upstream implementation
produced, and `tests/test_plain.py` checks this file against them.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np

# --------------------------------------------------------------------------------------
# reading a model folder
# --------------------------------------------------------------------------------------

_ST_DTYPES = {"F32": np.float32, "F64": np.float64, "I32": np.int32, "I64": np.int64,
              "F16": np.float16, "U8": np.uint8}


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """bfloat16 bit patterns (uint16) as the float32 values they stand for."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round float values to the nearest bfloat16 (ties to even), returned as float64/32.

    x0ne-core/oracle/src/bf16.rs:11-20 (round-to-nearest-even on the upper 16 bits).
    """
    f = np.asarray(x, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint32) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    out = np.where(np.isnan(f), f, out)
    return out.astype(np.asarray(x).dtype if np.asarray(x).dtype.kind == "f" else np.float32)


def read_safetensors(path: str) -> dict[str, np.ndarray]:
    """All tensors of one safetensors file, floating ones as float32 (bf16 widened exactly)."""
    with open(path, "rb") as f:
        raw = f.read()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + n])
    data = raw[8 + n:]
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        buf = data[a:b]
        if meta["dtype"] == "BF16":
            arr = bf16_bits_to_f32(np.frombuffer(buf, dtype=np.uint16))
        else:
            arr = np.frombuffer(buf, dtype=_ST_DTYPES[meta["dtype"]])
            if arr.dtype.kind == "f":
                arr = arr.astype(np.float32)
        out[name] = arr.reshape(meta["shape"]).copy()
    return out


def read_config(folder: str) -> dict:
    """The sizes and constants the forward needs, from config.json.

    Keys and their rules: x0ne-core/runtime/src/config.rs:65-118; `rope_theta` may sit
    under `rope_parameters` (x0ne-infer/src/core_backend.rs:28-55).
    """
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    theta = c.get("rope_theta")
    if theta is None:
        theta = c["rope_parameters"]["rope_theta"]
    return dict(
        hidden=c["hidden_size"], inter=c["intermediate_size"], layers=c["num_hidden_layers"],
        q_heads=c["num_attention_heads"], kv_heads=c["num_key_value_heads"],
        head_dim=c["head_dim"], vocab=c["vocab_size"], eps=c["rms_norm_eps"],
        theta=theta, tied=bool(c.get("tie_word_embeddings", False)),
        max_pos=c["max_position_embeddings"],
    )


def read_model(folder: str):
    """(config dict, tensors dict) of a folder with config.json and model.safetensors."""
    return read_config(folder), read_safetensors(os.path.join(folder, "model.safetensors"))


# --------------------------------------------------------------------------------------
# the parts, one function each
# --------------------------------------------------------------------------------------

def embedding(table: np.ndarray, ids) -> np.ndarray:
    """Rows of the table; an id outside the table gives a zero row.

    x0ne-core/kernels/cuda/embedding.cu:5-17, x0ne-core/oracle/src/lib.rs:39-46.
    """
    ids = np.asarray(ids, dtype=np.int64)
    out = np.zeros((len(ids), table.shape[1]), dtype=table.dtype)
    ok = (ids >= 0) & (ids < table.shape[0])
    out[ok] = table[ids[ok]]
    return out


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) * w over the last axis; eps inside the root.

    x0ne-core/kernels/cuda/rmsnorm.cu:11-20, x0ne-core/oracle/src/lib.rs:50-67.
    """
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return x * (1.0 / np.sqrt(ms + eps)) * w


def inv_freq(head_dim: int, theta: float) -> np.ndarray:
    """1 / theta^(2i/d), i < d/2, computed in float32 as the engine's host does.

    x0ne-core/runtime/src/ops.rs:210-214 (theta narrowed to f32 first,
    x0ne-core/runtime/src/engine.rs:351).
    """
    t = np.float32(theta)
    d = np.float32(head_dim)
    return np.array([np.float32(1.0) / np.power(t, np.float32(2 * i) / d, dtype=np.float32)
                     for i in range(head_dim // 2)], dtype=np.float32)


def rope(x: np.ndarray, positions: np.ndarray, freqs: np.ndarray) -> np.ndarray:
    """Rotate-half RoPE of x [n, heads, d]: the pair (i, i + d/2) turns by pos * inv_freq[i].

    The angle is the float32 product, as in x0ne-core/kernels/cuda/rope.cu:28-31 and
    x0ne-core/oracle/src/lib.rs:103-108.
    """
    half = x.shape[-1] // 2
    ang = (positions.astype(np.float32)[:, None] * freqs[None, :].astype(np.float32))
    ang = ang.astype(x.dtype)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * c - b * s, b * c + a * s], axis=-1)


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, window: int | None = None,
              return_probs: bool = False):
    """Causal grouped-query attention of one whole sequence.

    q [n, q_heads, d], k and v [n, kv_heads, d]; q head h reads kv head h // (q_heads //
    kv_heads); scale 1/sqrt(d); the query at position p sees keys 0..p (the last `window`
    of them if a window is given).  x0ne-core/oracle/src/lib.rs:150-174 (softmax in full),
    x0ne-core/kernels/cuda/attention.cu:20-28 (head mapping, causal by loop bound).
    """
    n, qh, d = q.shape
    kvh = k.shape[1]
    group = qh // kvh
    scale = 1.0 / math.sqrt(d)
    out = np.zeros_like(q)
    probs = np.zeros((qh, n, n), dtype=q.dtype)
    pos = np.arange(n)
    mask = pos[None, :] <= pos[:, None]
    if window is not None:
        mask &= pos[None, :] > pos[:, None] - window
    for h in range(qh):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale
        s = np.where(mask, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=-1, keepdims=True)
        probs[h] = p
        out[:, h, :] = p @ v[:, kh, :]
    return (out, probs) if return_probs else out


def attention_block(x, w, prefix, cfg, positions, round_fn=None, window=None,
                    return_probs=False):
    """Projections, per-head RMSNorm of q and k, RoPE, attention, output projection.

    x0ne-core/oracle/src/model.rs:218-244; q/k head norm x0ne-core/kernels/cuda/rope.cu:23-27
    (one weight of head_dim values shared by all heads, the block norms' eps).
    """
    r = round_fn or (lambda t: t)
    n = x.shape[0]
    qh, kvh, d = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"]
    dt = x.dtype
    q = r(x @ w[prefix + "q_proj.weight"].astype(dt).T).reshape(n, qh, d)
    k = r(x @ w[prefix + "k_proj.weight"].astype(dt).T).reshape(n, kvh, d)
    v = r(x @ w[prefix + "v_proj.weight"].astype(dt).T).reshape(n, kvh, d)
    q = rmsnorm(q, w[prefix + "q_norm.weight"].astype(dt), cfg["eps"])
    k = rmsnorm(k, w[prefix + "k_norm.weight"].astype(dt), cfg["eps"])
    freqs = inv_freq(d, cfg["theta"])
    q = r(rope(q, positions, freqs))
    k = r(rope(k, positions, freqs))
    res = attention(q, k, v, window=window, return_probs=return_probs)
    a, probs = res if return_probs else (res, None)
    a = r(a).reshape(n, qh * d)
    out = r(a @ w[prefix + "o_proj.weight"].astype(dt).T)
    return (out, probs) if return_probs else out


def swiglu_mlp(x, w, prefix, round_fn=None):
    """down( silu(gate(x)) * up(x) ), silu(g) = g / (1 + e^-g).

    x0ne-core/kernels/cuda/swiglu.cu:5-11, x0ne-core/oracle/src/lib.rs:199-209.
    """
    r = round_fn or (lambda t: t)
    dt = x.dtype
    g = r(x @ w[prefix + "gate_proj.weight"].astype(dt).T)
    u = r(x @ w[prefix + "up_proj.weight"].astype(dt).T)
    with np.errstate(over="ignore"):
        act = r(g / (1.0 + np.exp(-g)) * u)
    return r(act @ w[prefix + "down_proj.weight"].astype(dt).T)


def forward(cfg: dict, w: dict[str, np.ndarray], ids, dtype=np.float64, bf16_points=False,
            collect: dict | None = None) -> np.ndarray:
    """Logits [n, vocab] of one whole sequence that starts at position 0.

    Pre-norm residual blocks; the residual stream is never rounded; the final norm feeds the
    head, which is the embedding table when the model is tied
    (x0ne-core/oracle/src/model.rs:196-262, x0ne-core/runtime/src/engine.rs:744-835).
    With `bf16_points` every value the bf16 engine stores in bfloat16 is rounded to it
    (x0ne-core/oracle/src/model.rs:1-4); the weights are then expected to be bf16 values.
    `collect`, if given, receives per-layer hidden states and attention probabilities.
    """
    r = (lambda t: round_bf16(t).astype(dtype)) if bf16_points else None
    rr = r or (lambda t: t)
    ids = np.asarray(ids, dtype=np.int64)
    pos = np.arange(len(ids))
    x = embedding(w["model.embed_tokens.weight"].astype(dtype), ids)
    for l in range(cfg["layers"]):
        p = f"model.layers.{l}."
        normed = rr(rmsnorm(x, w[p + "input_layernorm.weight"].astype(dtype), cfg["eps"]))
        res = attention_block(normed, w, p + "self_attn.", cfg, pos, round_fn=r,
                              return_probs=collect is not None)
        if collect is not None:
            res, probs = res
            collect.setdefault("attentions", []).append(probs)
        x = x + res
        normed = rr(rmsnorm(x, w[p + "post_attention_layernorm.weight"].astype(dtype), cfg["eps"]))
        x = x + swiglu_mlp(normed, w, p + "mlp.", round_fn=r)
        if collect is not None:
            collect.setdefault("hidden", []).append(x.copy())
    normed = rr(rmsnorm(x, w["model.norm.weight"].astype(dtype), cfg["eps"]))
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return normed @ head.astype(dtype).T


# --------------------------------------------------------------------------------------
# picking tokens
# --------------------------------------------------------------------------------------

def argmax(row: np.ndarray):
    """Index of the largest value, lowest index on ties; None if the row holds a NaN.

    x0ne-core/kernels/cuda/argmax.cu:4-10, x0ne-core/oracle/src/lib.rs:213-227.
    """
    if len(row) == 0 or np.isnan(row).any():
        return None
    return int(np.argmax(row))


def greedy(cfg, w, prompt, n_new, dtype=np.float64, stop=()):
    """n_new greedy tokens after the prompt, recomputing the whole sequence each time.

    A stop token ends the sequence before it is fed or counted
    (x0ne-infer/src/stepped.rs:252-254).
    """
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        t = argmax(forward(cfg, w, ids, dtype=dtype)[-1])
        if t in stop:
            break
        out.append(t)
        ids.append(t)
    return out


def softmax_temperature(row: np.ndarray, temperature: float) -> np.ndarray:
    """Probabilities of logits / temperature (x0ne-infer/src/sampler.rs:120-136), in float64."""
    x = np.asarray(row, dtype=np.float64) * (1.0 / temperature)
    e = np.exp(x - x.max())
    return e / e.sum()


def nucleus_mask(p: np.ndarray, top_p: float) -> np.ndarray:
    """Which tokens top_p keeps: in the order (probability descending, index ascending) every
    token whose predecessors sum to less than top_p (x0ne-infer/src/sampler.rs:150-216)."""
    order = sorted(range(len(p)), key=lambda i: (-p[i], i))
    keep = np.zeros(len(p), dtype=bool)
    c = 0.0
    for i in order:
        if c >= top_p:
            break
        keep[i] = True
        c += p[i]
    return keep


def uniform_of(seed: int, counter: int) -> float:
    """The library's per-request draw stream: splitmix64 of (seed + counter * golden ratio),
    its top 24 bits as a float in [0, 1).  Restated here from the library's documentation,
    not imported (splitmix64 constants as in x0ne-core/oracle/examples/core-bench.rs:29-37)."""
    m = (1 << 64) - 1
    z = (seed + (counter + 1) * 0x9E3779B97F4A7C15) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def draw_interval(row, temperature, top_p, token):
    """[lo, hi): the range of u in [0,1) for which inverse-CDF sampling in index order over the
    kept tokens gives `token`, in float64.  Empty (lo == hi) if the token is not kept."""
    p = softmax_temperature(row, temperature)
    keep = nucleus_mask(p, top_p) if top_p < 1.0 else np.ones(len(p), dtype=bool)
    pk = np.where(keep, p, 0.0)
    c = np.cumsum(pk) / pk.sum()
    lo = 0.0 if token == 0 else float(c[token - 1])
    return lo, float(c[token])


def synthetic_ids(n: int, vocab: int, seed: int = 0x0C0E5EED):
    """n ids below vocab from splitmix64 (x0ne-core/oracle/examples/core-bench.rs:26-43)."""
    m = (1 << 64) - 1
    s = seed
    out = []
    for _ in range(n):
        s = (s + 0x9E3779B97F4A7C15) & m
        z = s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        out.append(int((z ^ (z >> 31)) % vocab))
    return out

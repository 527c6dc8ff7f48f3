"""Shared by the tests: the tiny configurations, model folders in temporary directories, and
the comparisons with their tolerances.

Tolerances (chosen before the first GPU run, never widened to pass):
  * 32-bit engine vs the plain float64 implementation: |got - want| <= 1e-4 * max|want row|.
  * 32-bit engine vs itself under another cut of the work (token by token, batched, reused
    slots): bit-identical.
  * bfloat16 engine vs the plain implementation run on the same bfloat16 weights: a logit within
    0.05 * max|want row| and KL(want || got) <= 0.02 nats per position, the model-level
    tolerances of x0ne-core/oracle/tests/gpu_engine.rs:29-115; bfloat16 vs itself under another
    cut: within 0.02 * max|row| (kernels may differ between prefill and decode).
"""
import os
import tempfile

import numpy as np

import plain_impl as P

F32_RTOL = 1e-4
BF16_LOGIT_TOL = 0.05
BF16_KL_TOL = 0.02
BF16_SELF_TOL = 0.02


def tiny_a(dtype="float32"):
    from x0ne_engine_b200 import Qwen3Config
    return Qwen3Config(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=16, vocab_size=256, max_position_embeddings=128,
                       rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True, dtype=dtype)


def tiny_b(dtype="float32"):
    from x0ne_engine_b200 import Qwen3Config
    return Qwen3Config(hidden_size=96, intermediate_size=160, num_hidden_layers=3, num_attention_heads=6,
                       num_key_value_heads=2, head_dim=32, vocab_size=384, max_position_embeddings=256,
                       rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False, dtype=dtype)


def tiny_c(dtype="float32"):
    """Sizes that are no power of two, head_dim 48, one kv head for five q heads, long context."""
    from x0ne_engine_b200 import Qwen3Config
    return Qwen3Config(hidden_size=120, intermediate_size=200, num_hidden_layers=2, num_attention_heads=5,
                       num_key_value_heads=1, head_dim=48, vocab_size=331, max_position_embeddings=2048,
                       rms_norm_eps=3e-6, rope_theta=50000.0, tie_word_embeddings=False, dtype=dtype)


TINY = {"A": (tiny_a, 0), "B": (tiny_b, 1), "C": (tiny_c, 2)}
_folders = {}


def model_folder(name: str, dtype: str = "float32", linear_std: float = 0.02):
    """A temporary folder with config.json and model.safetensors of a tiny model (made once)."""
    from x0ne_engine_b200 import RandomInit, write_model_folder
    key = (name, dtype, linear_std)
    if key not in _folders:
        make, seed = TINY[name]
        d = tempfile.mkdtemp(prefix=f"x0ne_tiny_{name}_{dtype}_")
        write_model_folder(d, make(dtype), RandomInit(seed=seed, linear_std=linear_std, norm_jitter=0.1))
        _folders[key] = d
    return _folders[key]


def golden_folder():
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qwen3_f32")


_plain = {}


def plain_model(folder, bf16_matrices=False):
    """(config, tensors).  With `bf16_matrices` every matrix is rounded to bfloat16 first: what a
    bfloat16 engine holds when the checkpoint stores float32 (vectors stay in 32-bit)."""
    key = (folder, bf16_matrices)
    if key not in _plain:
        cfg, w = P.read_model(folder)
        if bf16_matrices:
            w = {k: (P.round_bf16(v) if v.ndim == 2 else v) for k, v in w.items()}
        _plain[key] = (cfg, w)
    return _plain[key]


def plain_logits(folder, ids, bf16_matrices=False):
    cfg, w = plain_model(folder, bf16_matrices)
    return P.forward(cfg, w, ids)


def prompts_for(vocab, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, n).tolist() for n in lengths]


def assert_close_f32(got, want, what=""):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    scale = np.max(np.abs(want), axis=-1, keepdims=True) + 1e-30
    err = np.max(np.abs(got - want) / scale)
    assert err <= F32_RTOL, f"{what}: worst relative error {err:.3e} > {F32_RTOL}"


def kl_rows(want, got):
    def logsoftmax(x):
        x = x - x.max(axis=-1, keepdims=True)
        return x - np.log(np.exp(x).sum(axis=-1, keepdims=True))
    lw, lg = logsoftmax(np.asarray(want, np.float64)), logsoftmax(np.asarray(got, np.float64))
    return (np.exp(lw) * (lw - lg)).sum(axis=-1)


def assert_close_bf16(got, want, what="", logit_tol=BF16_LOGIT_TOL):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    scale = np.max(np.abs(want), axis=-1, keepdims=True) + 1e-30
    err = np.max(np.abs(got - want) / scale)
    assert err <= logit_tol, f"{what}: worst logit error {err:.3e} of the row's largest > {logit_tol}"
    kl = kl_rows(want, got).max()
    assert kl <= BF16_KL_TOL, f"{what}: worst KL {kl:.3e} > {BF16_KL_TOL}"


def first_difference(a, b):
    """(row, column) of the first differing element of two arrays, or None."""
    a, b = np.asarray(a), np.asarray(b)
    bad = np.argwhere(a != b)
    return tuple(bad[0]) if len(bad) else None

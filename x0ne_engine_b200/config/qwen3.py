"""Qwen3 dense: the typed configuration, read strictly from config.json, and its ModelSpec.

The reader follows x0ne-core/runtime/src/config.rs:65-118: every size is required, nothing
is derived (`head_dim` is read, never computed from hidden / heads), and an option this
library does not implement is refused by name rather than ignored.  `rope_theta` nested
under `rope_parameters` is lifted and any `rope_type` but "default" refused, as
x0ne-infer/src/core_backend.rs:28-55 does.  Differences from that reader, on purpose: the
checkpoint dtype may also be "float32" (or absent, which reads as bfloat16's rules with
the stored dtype kept), because this library has a true 32-bit path.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass
from typing import Any, Mapping

from .spec import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

ARCHITECTURE = "Qwen3ForCausalLM"
MODEL_TYPE = "qwen3"

_U32_MAX = (1 << 32) - 1


def _positive_int(d: Mapping[str, Any], key: str) -> int:
    if key not in d:
        raise ConfigError(f"config.json: missing {key}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {key} is not a positive integer")
    return v


def _positive_number(d: Mapping[str, Any], key: str) -> float:
    if key not in d:
        raise ConfigError(f"config.json: missing {key}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v <= 0:
        raise ConfigError(f"config.json: {key} is not a positive number")
    return float(v)


def _off(d: Mapping[str, Any], key: str) -> bool:
    return d.get(key) is None or d.get(key) is False


@dataclass(frozen=True)
class Qwen3Config:
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool = False
    dtype: str = "bfloat16"
    eos_token_ids: tuple = ()

    # ---- derived sizes (x0ne-core/runtime/src/config.rs:190-216)
    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def kv_bytes_per_position(self) -> int:
        """K and V bytes stored per cached position over all layers, bfloat16."""
        return self.num_hidden_layers * 2 * self.kv_dim * 2

    @property
    def linear_params_per_layer(self) -> int:
        h = self.hidden_size
        return h * (self.q_dim + 2 * self.kv_dim) + self.q_dim * h + 3 * h * self.intermediate_size

    def weight_params(self) -> int:
        per_layer = self.linear_params_per_layer + 2 * self.hidden_size + 2 * self.head_dim
        outer = self.vocab_size * self.hidden_size * (1 if self.tie_word_embeddings else 2)
        return self.num_hidden_layers * per_layer + outer + self.hidden_size

    # ---- reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        if not isinstance(d, Mapping):
            raise ConfigError("config.json: not a JSON object")
        mt = d.get("model_type")
        archs = d.get("architectures")
        if mt is None and not archs:
            raise ConfigError("config.json: missing model_type")
        if mt is not None and mt != MODEL_TYPE:
            raise ConfigError(f"config.json: model_type is {mt!r}, not {MODEL_TYPE!r}")
        if archs is not None:
            if not isinstance(archs, list) or len(archs) != 1 or archs[0] != ARCHITECTURE:
                raise ConfigError(f"config.json: architectures is {archs!r}, not [{ARCHITECTURE!r}]")
        dtype = d.get("dtype", d.get("torch_dtype"))
        if dtype is None:
            dtype = "bfloat16"
        if dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"config.json: dtype {dtype!r}; bfloat16 and float32 checkpoints are served")
        if d.get("hidden_act") != "silu":
            raise ConfigError("config.json: hidden_act is not silu")
        for key in ("attention_bias", "use_sliding_window", "rope_scaling"):
            if not _off(d, key):
                raise ConfigError(f"config.json: {key} is set, not implemented")
        tie = d.get("tie_word_embeddings", False)
        if not isinstance(tie, bool):
            raise ConfigError("config.json: tie_word_embeddings is not a boolean")

        src = dict(d)
        rp = d.get("rope_parameters")
        if rp is not None:
            if not isinstance(rp, Mapping):
                raise ConfigError("config.json: rope_parameters is not an object")
            if rp.get("rope_type", "default") != "default":
                raise ConfigError(f"config.json: rope_type {rp.get('rope_type')!r} is not implemented")
            extra = set(rp) - {"rope_type", "rope_theta"}
            if extra:
                raise ConfigError(f"config.json: rope_parameters has unknown keys {sorted(extra)}")
            if "rope_theta" in rp:
                if "rope_theta" in d and d["rope_theta"] != rp["rope_theta"]:
                    raise ConfigError("config.json: rope_theta is given twice with different values")
                src["rope_theta"] = rp["rope_theta"]

        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: tuple = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError("config.json: eos_token_id is neither an integer nor a list of integers")

        c = cls(
            hidden_size=_positive_int(src, "hidden_size"),
            intermediate_size=_positive_int(src, "intermediate_size"),
            num_hidden_layers=_positive_int(src, "num_hidden_layers"),
            num_attention_heads=_positive_int(src, "num_attention_heads"),
            num_key_value_heads=_positive_int(src, "num_key_value_heads"),
            head_dim=_positive_int(src, "head_dim"),
            vocab_size=_positive_int(src, "vocab_size"),
            max_position_embeddings=_positive_int(src, "max_position_embeddings"),
            rms_norm_eps=_positive_number(src, "rms_norm_eps"),
            rope_theta=_positive_number(src, "rope_theta"),
            tie_word_embeddings=tie,
            dtype=dtype,
            eos_token_ids=eos_ids,
        )
        c.check()
        return c

    def check(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError("config.json: attention heads are not a multiple of KV heads")
        if self.head_dim % 2 != 0:
            raise ConfigError("config.json: head_dim is odd, RoPE needs pairs")
        if self.vocab_size > _U32_MAX:
            raise ConfigError("config.json: vocab_size does not fit a 32-bit token id")
        for e in self.eos_token_ids:
            if not 0 <= e < self.vocab_size:
                raise ConfigError(f"config.json: eos_token_id {e} is outside the vocabulary")
        if self.weight_params() * 4 >= 1 << 62:
            raise ConfigError("config.json: a size derived from the config overflows")

    @classmethod
    def from_json(cls, text: str) -> "Qwen3Config":
        try:
            d = json.loads(text)
        except json.JSONDecodeError as e:
            raise ConfigError(f"config.json: {e}") from None
        return cls.from_dict(d)

    @classmethod
    def from_folder(cls, folder: str) -> "Qwen3Config":
        with open(os.path.join(folder, "config.json")) as f:
            return cls.from_json(f.read())

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = asdict(self)
        eos = d.pop("eos_token_ids")
        d["eos_token_id"] = None if not eos else (eos[0] if len(eos) == 1 else list(eos))
        d.update(model_type=MODEL_TYPE, architectures=[ARCHITECTURE], hidden_act="silu",
                 attention_bias=False, use_sliding_window=False)
        return d

    # ---- the model as data
    def to_spec(self) -> ModelSpec:
        """Pre-norm blocks of (RMSNorm, grouped-query attention with per-head q/k RMSNorm and
        rotate-half RoPE, RMSNorm, SwiGLU); final RMSNorm; a head that is the embedding table
        when tied.  Tensor names: x0ne-core/runtime/src/weights.rs:12-47."""
        h, eps = self.hidden_size, self.rms_norm_eps
        rope = PartSpec("rope", dict(head_dim=self.head_dim, rotary_dim=self.head_dim,
                                     theta=self.rope_theta))
        layers = []
        for l in range(self.num_hidden_layers):
            p = f"model.layers.{l}"
            attn = PartSpec("gqa_attention", dict(
                hidden_size=h, q_heads=self.num_attention_heads, kv_heads=self.num_key_value_heads,
                head_dim=self.head_dim, qk_norm_eps=eps, window=None, position="rope",
                scale=None,
                names=dict(q=f"{p}.self_attn.q_proj.weight", k=f"{p}.self_attn.k_proj.weight",
                           v=f"{p}.self_attn.v_proj.weight", o=f"{p}.self_attn.o_proj.weight",
                           q_norm=f"{p}.self_attn.q_norm.weight",
                           k_norm=f"{p}.self_attn.k_norm.weight")))
            mlp = PartSpec("swiglu", dict(
                hidden_size=h, intermediate_size=self.intermediate_size,
                names=dict(gate=f"{p}.mlp.gate_proj.weight", up=f"{p}.mlp.up_proj.weight",
                           down=f"{p}.mlp.down_proj.weight")))
            layers.append(LayerSpec(block="prenorm", parts=dict(
                mixer_norm=PartSpec("rmsnorm", dict(size=h, eps=eps,
                                                    names=dict(weight=f"{p}.input_layernorm.weight"))),
                mixer=attn,
                ffn_norm=PartSpec("rmsnorm", dict(size=h, eps=eps,
                                                  names=dict(weight=f"{p}.post_attention_layernorm.weight"))),
                ffn=mlp)))
        spec = ModelSpec(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab_size,
            hidden_size=h,
            max_position_embeddings=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", dict(
                vocab_size=self.vocab_size, hidden_size=h,
                names=dict(weight="model.embed_tokens.weight"))),
            positions={"rope": rope},
            layers=tuple(layers),
            run_order=tuple(RunEntry(l) for l in range(self.num_hidden_layers)),
            final_norm=PartSpec("rmsnorm", dict(size=h, eps=eps, names=dict(weight="model.norm.weight"))),
            head=PartSpec("lm_head", dict(
                vocab_size=self.vocab_size, hidden_size=h, tied=self.tie_word_embeddings,
                names=dict(weight="model.embed_tokens.weight" if self.tie_word_embeddings
                           else "lm_head.weight"))),
            stop_token_ids=tuple(self.eos_token_ids),
            checkpoint_dtype=self.dtype,
        )
        spec.validate()
        return spec

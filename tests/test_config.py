"""Configuration reading and the architecture registry (CPU)."""
import json

import pytest

from x0ne_engine_b200 import ConfigError, Qwen3Config
from x0ne_engine_b200.config import (architectures, config_from_dict, config_from_folder, detect,
                                     register_architecture, unregister_architecture)
from helpers import golden_folder, tiny_a, tiny_b


def good():
    return dict(model_type="qwen3", dtype="bfloat16", hidden_act="silu", attention_bias=False, hidden_size=64,
                intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                head_dim=16, vocab_size=256, max_position_embeddings=128, rms_norm_eps=1e-6, rope_theta=1e4,
                tie_word_embeddings=True)


def test_reads_every_size_from_its_own_key():
    c = Qwen3Config.from_dict(good())
    assert (c.hidden_size, c.intermediate_size, c.num_hidden_layers, c.num_attention_heads) == (64, 128, 2, 4)
    assert (c.num_key_value_heads, c.head_dim, c.vocab_size, c.max_position_embeddings) == (2, 16, 256, 128)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 1e4 and c.tie_word_embeddings
    assert c.q_dim == 64 and c.kv_dim == 32


def test_head_dim_is_read_not_derived():
    d = good()
    d["head_dim"] = 32                     # q width 128 != hidden 64
    assert Qwen3Config.from_dict(d).q_dim == 128
    del d["head_dim"]
    with pytest.raises(ConfigError, match="head_dim"):
        Qwen3Config.from_dict(d)


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                 "num_key_value_heads", "vocab_size", "max_position_embeddings", "rms_norm_eps",
                                 "rope_theta"])
def test_missing_key_is_named(key):
    d = good()
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(d)


@pytest.mark.parametrize("key,value", [("hidden_size", 0), ("hidden_size", -3), ("hidden_size", 2.5),
                                       ("hidden_size", True), ("rms_norm_eps", 0), ("rope_theta", float("inf")),
                                       ("rope_theta", "1e4"), ("tie_word_embeddings", 1)])
def test_bad_values_are_refused(key, value):
    d = good()
    d[key] = value
    with pytest.raises(ConfigError):
        Qwen3Config.from_dict(d)


@pytest.mark.parametrize("key,value", [("attention_bias", True), ("use_sliding_window", True),
                                       ("rope_scaling", {"rope_type": "yarn", "factor": 4.0}),
                                       ("hidden_act", "gelu"), ("dtype", "float16"), ("model_type", "llama")])
def test_unimplemented_options_are_refused_not_ignored(key, value):
    d = good()
    d[key] = value
    with pytest.raises(ConfigError):
        config_from_dict(d)


def test_heads_must_divide_and_head_dim_even():
    d = good()
    d["num_key_value_heads"] = 3
    with pytest.raises(ConfigError, match="multiple"):
        Qwen3Config.from_dict(d)
    d = good()
    d["head_dim"] = 15
    with pytest.raises(ConfigError, match="odd"):
        Qwen3Config.from_dict(d)


def test_rope_parameters_are_lifted_and_other_rope_types_refused():
    d = good()
    del d["rope_theta"]
    d["rope_parameters"] = {"rope_type": "default", "rope_theta": 5e5}
    assert Qwen3Config.from_dict(d).rope_theta == 5e5
    d["rope_parameters"]["rope_type"] = "yarn"
    with pytest.raises(ConfigError, match="rope_type"):
        Qwen3Config.from_dict(d)


def test_dtype_keys():
    d = good()
    del d["dtype"]
    d["torch_dtype"] = "float32"
    assert Qwen3Config.from_dict(d).dtype == "float32"


def test_round_trip_through_to_dict():
    for make in (tiny_a, tiny_b):
        c = make()
        assert Qwen3Config.from_dict(json.loads(json.dumps(c.to_dict()))) == c


def test_the_reference_projects_fixture_config_is_read():
    c = config_from_folder(golden_folder())
    assert (c.head_dim, c.num_attention_heads, c.num_key_value_heads, c.rope_theta) == (8, 3, 1, 10000.0)
    assert c.tie_word_embeddings


def test_registry_detects_by_class_and_by_model_type_and_refuses_disagreement():
    assert "Qwen3ForCausalLM" in architectures()
    assert detect({"architectures": ["Qwen3ForCausalLM"]}) == "Qwen3ForCausalLM"
    assert detect({"model_type": "qwen3"}) == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError, match="not served"):
        detect({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="neither"):
        detect({})

    class Other:
        @classmethod
        def from_dict(cls, d):
            return "other"
    register_architecture("OtherForCausalLM", "other", Other)
    try:
        assert config_from_dict({"architectures": ["OtherForCausalLM"]}) == "other"
        with pytest.raises(ConfigError, match="names"):
            detect({"architectures": ["OtherForCausalLM"], "model_type": "qwen3"})
        with pytest.raises(ValueError):
            register_architecture("OtherForCausalLM", "other2", Other)
    finally:
        unregister_architecture("OtherForCausalLM")
    assert "OtherForCausalLM" not in architectures()


def test_spec_is_data_with_one_entry_per_layer_and_all_sizes_as_parameters():
    spec = tiny_b().to_spec()
    assert len(spec.layers) == 3 and [e.layer for e in spec.run_order] == [0, 1, 2]
    m = spec.layers[1].part("mixer")
    assert m.kind == "gqa_attention" and m["q_heads"] == 6 and m["kv_heads"] == 2 and m["head_dim"] == 32
    assert m["qk_norm_eps"] == 1e-5 and m["names"]["q"] == "model.layers.1.self_attn.q_proj.weight"
    assert spec.layers[2].part("ffn")["intermediate_size"] == 160 and spec.positions["rope"]["theta"] == 1e6
    assert spec.head["tied"] is False and spec.head["names"]["weight"] == "lm_head.weight"
    assert tiny_a().to_spec().head["names"]["weight"] == "model.embed_tokens.weight"


def test_a_layer_s_roles_are_checked_against_its_arrangement():
    """A layer names its parts by role; which roles exist is the arrangement's business, and a
    layer that leaves one out or brings an unknown one is refused before anything is built."""
    import dataclasses
    from x0ne_engine_b200.config import ConfigError, LayerSpec
    from x0ne_engine_b200.engine import tensor_needs_of_spec
    from x0ne_engine_b200.engine.model import cache_need_of_layer, step_bytes_of_spec
    spec = tiny_b().to_spec()
    l0 = spec.layers[0]
    assert sorted(l0.parts) == ["ffn", "ffn_norm", "mixer", "mixer_norm"] and cache_need_of_layer(l0).kind == "kv"
    with pytest.raises(ConfigError, match="no part in the role 'router'"):
        l0.part("router")
    without_ffn = LayerSpec(l0.block, {k: v for k, v in l0.parts.items() if k != "ffn"})
    with pytest.raises(ConfigError, match=r"missing: \['ffn'\]"):
        tensor_needs_of_spec(dataclasses.replace(spec, layers=(without_ffn,) + spec.layers[1:]))
    extra = l0.with_part("post_norm", l0.part("ffn_norm"))
    with pytest.raises(ConfigError, match=r"unknown: \['post_norm'\]"):
        tensor_needs_of_spec(dataclasses.replace(spec, layers=(extra,) + spec.layers[1:]))
    # bytes a decode step reads and a position holds, from the spec alone
    c = tiny_b()
    weights, cache = step_bytes_of_spec(spec, 2)
    per_layer = (c.linear_params_per_layer) * 2 + (2 * c.hidden_size + 2 * c.head_dim) * 4
    assert weights == c.num_hidden_layers * per_layer + c.vocab_size * c.hidden_size * 2 + c.hidden_size * 4
    assert cache == c.kv_bytes_per_position

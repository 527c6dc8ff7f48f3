"""Safetensors by tensor name, the one error that lists every difference, random folders (CPU)."""
import json
import os
import struct

import numpy as np
import pytest
import torch

import plain_impl as P
from x0ne_engine_b200 import RandomInit, WeightsError, write_model_folder
from x0ne_engine_b200.engine.model import optional_duplicates_of_spec, tensor_needs_of_spec
from x0ne_engine_b200.weights import (SafetensorsError, TensorNeed, held_dtype, load_folder, make_tensor,
                                      open_folder, write_file)
from helpers import model_folder, tiny_a, tiny_b


def test_needs_list_every_tensor_of_the_architecture():
    names = [n.name for n in tensor_needs_of_spec(tiny_b().to_spec())]
    assert names[0] == "model.embed_tokens.weight" and names[-1] == "lm_head.weight"
    assert "model.layers.2.self_attn.k_norm.weight" in names and len(names) == 2 + 3 * 11 + 1
    tied = [n.name for n in tensor_needs_of_spec(tiny_a().to_spec())]
    assert "lm_head.weight" not in tied and len(tied) == 1 + 2 * 11 + 1


def test_written_folder_reads_back_and_matches_the_plain_reader(tmp_path):
    d = str(tmp_path / "m")
    write_model_folder(d, tiny_a("bfloat16"), RandomInit(seed=3, norm_jitter=0.1))
    needs = tensor_needs_of_spec(tiny_a().to_spec())
    got = load_folder(d, needs, torch.bfloat16, "cpu")
    _, plain = P.read_model(d)
    for n in needs:
        assert tuple(got[n.name].shape) == n.shape
        assert np.array_equal(got[n.name].float().numpy(), plain[n.name])
    assert got["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert got["model.norm.weight"].dtype == torch.float32          # per-channel vectors are held in 32-bit


def test_dtype_policy():
    m, v = TensorNeed("m", (2, 2)), TensorNeed("v", (2,), role="vector")
    s, t = TensorNeed("s", (2,), role="stored"), TensorNeed("t", (2,), role="table")
    assert held_dtype(m, torch.bfloat16, torch.bfloat16) == torch.bfloat16
    assert held_dtype(m, torch.bfloat16, torch.float32) == torch.float32
    assert held_dtype(v, torch.bfloat16, torch.bfloat16) == torch.float32
    assert held_dtype(s, torch.float32, torch.bfloat16) == torch.float32      # stored in 32-bit stays so
    assert held_dtype(s, torch.bfloat16, torch.bfloat16) == torch.bfloat16
    assert held_dtype(t, torch.int64, torch.bfloat16) == torch.int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = str(tmp_path / "m")
    write_model_folder(d, tiny_a(), RandomInit(seed=0))
    src = open_folder(d)
    tensors = {n: src.tensor(n).clone() for n in src.names()}
    src.close()
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.extra.weight"] = torch.zeros(3)
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32)
    tensors["model.layers.0.input_layernorm.weight"] = torch.zeros(64, dtype=torch.float16)
    write_file(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightsError) as e:
        load_folder(d, tensor_needs_of_spec(tiny_a().to_spec()), torch.float32, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.0.extra.weight"]
    assert [(n, tuple(g), tuple(w)) for n, g, w in err.wrong_shape] == \
        [("model.layers.0.self_attn.q_proj.weight", (64, 32), (64, 64))]
    assert err.wrong_dtype[0][0] == "model.layers.0.input_layernorm.weight"
    text = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)", "is [64, 32], the model needs [64, 64]"):
        assert piece in text


def test_tied_checkpoint_may_carry_an_identical_head_only(tmp_path):
    d = str(tmp_path / "m")
    cfg = tiny_a()
    write_model_folder(d, cfg, RandomInit(seed=0))
    spec = cfg.to_spec()
    src = open_folder(d)
    tensors = {n: src.tensor(n).clone() for n in src.names()}
    src.close()
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_file(os.path.join(d, "model.safetensors"), tensors)
    load_folder(d, tensor_needs_of_spec(spec), torch.float32, "cpu", same_as=optional_duplicates_of_spec(spec))
    tensors["lm_head.weight"][0, 0] += 1
    write_file(os.path.join(d, "model.safetensors"), tensors)
    with pytest.raises(WeightsError, match="differs"):
        load_folder(d, tensor_needs_of_spec(spec), torch.float32, "cpu", same_as=optional_duplicates_of_spec(spec))


def test_hostile_files(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    p = d / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(SafetensorsError, match="shorter"):
        open_folder(str(d))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        open_folder(str(d))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                      "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 12)
    with pytest.raises(SafetensorsError, match="overlap"):
        open_folder(str(d))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="bytes for shape"):
        open_folder(str(d))
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="outside"):
        open_folder(str(d))


def test_sharded_folder_rules(tmp_path):
    d = tmp_path / "m"
    d.mkdir()
    write_file(str(d / "s1.safetensors"), {"a": torch.ones(2)})
    write_file(str(d / "s2.safetensors"), {"b": torch.zeros(3)})
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    src = open_folder(str(d))
    assert sorted(src.names()) == ["a", "b"] and src.tensor("b").shape == (3,)
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "s2.safetensors", "b": "s2.safetensors"}}))
    with pytest.raises(SafetensorsError):
        open_folder(str(d))
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "../s1.safetensors"}}))
    with pytest.raises(SafetensorsError, match="plain file name"):
        open_folder(str(d))
    (d / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    write_file(str(d / "model.safetensors"), {"a": torch.ones(2)})
    with pytest.raises(SafetensorsError, match="both"):
        open_folder(str(d))


def test_random_values_depend_on_seed_name_and_index_only():
    need = TensorNeed("model.layers.0.mlp.up_proj.weight", (10, 7))
    whole = make_tensor(need, RandomInit(seed=4), torch.float32, "cpu")
    pieces = make_tensor(need, RandomInit(seed=4), torch.float32, "cpu", chunk=13)
    assert torch.equal(whole, pieces)
    assert not torch.equal(whole, make_tensor(need, RandomInit(seed=5), torch.float32, "cpu"))
    other = TensorNeed("model.layers.1.mlp.up_proj.weight", (10, 7))
    assert not torch.equal(whole, make_tensor(other, RandomInit(seed=4), torch.float32, "cpu"))
    big = make_tensor(TensorNeed("w", (400, 400)), RandomInit(seed=1, linear_std=0.02), torch.float32, "cpu")
    assert abs(float(big.std()) - 0.02) < 1e-3 and abs(float(big.mean())) < 1e-3
    norm = make_tensor(TensorNeed("n", (4096,), role="vector", init="norm"), RandomInit(seed=1, norm_jitter=0.1),
                       torch.float32, "cpu")
    assert abs(float(norm.mean()) - 1) < 0.01 and abs(float(norm.std()) - 0.1) < 0.01
    ones = make_tensor(TensorNeed("n", (8,), role="vector", init="norm"), RandomInit(seed=1), torch.float32, "cpu")
    assert torch.equal(ones, torch.ones(8))


def test_helper_folders_differ_in_every_size():
    a, b = P.read_config(model_folder("A")), P.read_config(model_folder("B"))
    assert all(a[k] != b[k] for k in a if k != "kv_heads")
    assert a["q_heads"] // a["kv_heads"] != b["q_heads"] // b["kv_heads"]


def test_a_file_written_tensor_by_tensor_reads_back_and_refuses_what_was_not_planned(tmp_path):
    """The streaming writer fixes the header from a plan and takes the tensors one at a time."""
    import torch
    from x0ne_engine_b200.weights import write_file_streaming
    a = torch.arange(12, dtype=torch.float32).reshape(3, 4)
    b = (torch.arange(10, dtype=torch.float32) / 3).bfloat16().reshape(2, 5)
    path = str(tmp_path / "model.safetensors")
    write_file_streaming(path, [("a", torch.float32, (3, 4)), ("b", torch.bfloat16, (2, 5))], iter([a, b]))
    got = P.read_safetensors(path)
    assert np.array_equal(got["a"], a.numpy()) and np.array_equal(got["b"], b.float().numpy())
    src = open_folder(str(tmp_path))
    assert sorted(src.names()) == ["a", "b"]
    with pytest.raises(SafetensorsError, match="planned"):
        write_file_streaming(path, [("a", torch.float32, (3, 4))], iter([b]))
    assert np.array_equal(P.read_safetensors(path)["a"], a.numpy())       # a failed write leaves the old file

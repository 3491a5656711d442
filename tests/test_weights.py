"""The safetensors reader and writer, the weight check with its one error, and the random-weights mode."""
import json
import os
import struct

import pytest
import torch

import kirai_b200
from kirai_b200.registry import config_from_dict, plan_for_config
from kirai_b200.weights import (ModelFiles, SafetensorsError, WeightError, open_checked, random_tensors,
                                write_random_model, write_safetensors)
from kirai_b200.weights.safetensors_io import SafetensorsFile
from tiny_configs import CONFIG_A, CONFIG_B


def test_round_trip_keeps_dtypes(tmp_path):
    tensors = {"w": torch.randn(5, 7).bfloat16(), "f": torch.randn(3), "t": torch.arange(6, dtype=torch.int64).reshape(2, 3)}
    write_safetensors(tmp_path / "model.safetensors", tensors)
    files = ModelFiles(tmp_path)
    assert set(files.names()) == set(tensors)
    for name, tensor in tensors.items():
        assert files.tensor(name).dtype == tensor.dtype and torch.equal(files.tensor(name), tensor)


def _write_raw(path, header: bytes, payload: bytes = b"", length=None):
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(header) if length is None else length))
        handle.write(header)
        handle.write(payload)


@pytest.mark.parametrize("case", ["short", "huge_header", "past_eof", "bad_json", "not_object", "no_tensors",
                                  "missing_dtype", "inverted", "past_payload", "bad_dtype", "shape_bytes"])
def test_malformed_files_are_refused(tmp_path, case):
    path = tmp_path / "model.safetensors"
    good = {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    if case == "short":
        path.write_bytes(b"\x01\x02")
    elif case == "huge_header":
        _write_raw(path, b"{}", length=65 * 1024 * 1024)
    elif case == "past_eof":
        _write_raw(path, b"{}", length=1000)
    elif case == "bad_json":
        _write_raw(path, b"{not json")
    elif case == "not_object":
        _write_raw(path, b"[1,2]")
    elif case == "no_tensors":
        _write_raw(path, json.dumps({"__metadata__": {}}).encode())
    else:
        entry = dict(good["a"])
        if case == "missing_dtype":
            del entry["dtype"]
        elif case == "inverted":
            entry["data_offsets"] = [8, 0]
        elif case == "past_payload":
            entry["data_offsets"] = [0, 16]
            entry["shape"] = [4]
        elif case == "bad_dtype":
            entry["dtype"] = "F8_E4M3"
        elif case == "shape_bytes":
            entry["shape"] = [3]
        _write_raw(path, json.dumps({"a": entry}).encode(), b"\0" * 8)
    with pytest.raises(SafetensorsError):
        SafetensorsFile(path)


def test_missing_folder_content_and_index(tmp_path):
    with pytest.raises(SafetensorsError) as err:
        ModelFiles(tmp_path)
    assert err.value.code == "model_artifact_missing"
    write_safetensors(tmp_path / "part-1.safetensors", {"a": torch.zeros(2)})
    write_safetensors(tmp_path / "part-2.safetensors", {"b": torch.ones(3)})
    index = {"metadata": {"total_size": 20}, "weight_map": {"a": "part-1.safetensors", "b": "part-2.safetensors"}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    files = ModelFiles(tmp_path)
    assert torch.equal(files.tensor("b"), torch.ones(3))
    index["weight_map"]["b"] = "../outside.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    with pytest.raises(SafetensorsError) as err:
        ModelFiles(tmp_path)
    assert "unsafe" in str(err.value) or "escapes" in str(err.value)


def test_one_error_lists_missing_unexpected_and_wrong(tmp_path):
    config = config_from_dict(CONFIG_B)
    specs = plan_for_config(config).weight_specs()
    tensors = random_tensors(specs, seed=3)
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(192).bfloat16()
    tensors["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(64, 90).bfloat16()
    tensors["model.norm.weight"] = torch.zeros(96, dtype=torch.int32)
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as err:
        open_checked(str(tmp_path), specs, "cpu")
    assert err.value.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert err.value.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    text = str(err.value)
    assert "model.layers.2.self_attn.k_proj.weight: shape [64, 90], expected [64, 96]" in text
    assert "model.norm.weight: dtype I32" in text


def test_dtype_policy_keeps_stored_width(tmp_path):
    config = config_from_dict(CONFIG_A)
    specs = plan_for_config(config).weight_specs()
    tensors = random_tensors(specs, seed=1)
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()  # one tensor stored in 32-bit
    write_safetensors(tmp_path / "model.safetensors", tensors)
    source = open_checked(str(tmp_path), specs, "cpu")
    assert source.stored("model.norm.weight").dtype == torch.float32
    assert source.stored("model.embed_tokens.weight").dtype == torch.bfloat16
    assert source.on_device("model.embed_tokens.weight") is source.on_device("model.embed_tokens.weight")


def test_random_model_folder_is_deterministic(tmp_path):
    config = config_from_dict(CONFIG_A)
    write_random_model(str(tmp_path / "one"), config, seed=0)
    write_random_model(str(tmp_path / "two"), config, seed=0)
    write_random_model(str(tmp_path / "three"), config, seed=1)
    one, two, three = (ModelFiles(tmp_path / n) for n in ("one", "two", "three"))
    assert sorted(os.listdir(tmp_path / "one")) == ["config.json", "model.safetensors"]
    name = "model.layers.1.mlp.down_proj.weight"
    assert torch.equal(one.tensor(name), two.tensor(name)) and not torch.equal(one.tensor(name), three.tensor(name))
    assert one.tensor(name).dtype == torch.bfloat16
    assert abs(float(one.tensor("model.layers.0.input_layernorm.weight").float().mean()) - 1.0) < 0.1
    assert json.loads((tmp_path / "one" / "config.json").read_text())["architectures"] == ["Qwen3ForCausalLM"]

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
                                  "missing_dtype", "inverted", "past_payload", "bad_dtype", "shape_bytes", "not_utf8"])
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
    elif case == "not_utf8":  # a tensor name with a broken multi-byte sequence
        _write_raw(path, json.dumps(good).encode().replace(b'"a"', b'"a\xc5\x22x"'), b"\0" * 8)
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
    codes = []
    for native in (True, False):  # the native reader and the Python one refuse the same files for the same reason
        with pytest.raises(SafetensorsError) as err:
            SafetensorsFile(path, native=native)
        codes.append(err.value.code)
    assert codes[0] == codes[1]


def test_native_reader_and_python_reader_agree(tmp_path):
    """Files with every dtype, empty and many-dimensional tensors, metadata, names that need escaping and padding
    after the header: the reader in native code (the default) and the Python reader give the same entries and bytes."""
    generator = torch.Generator().manual_seed(0)
    tensors = {
        "plain.weight": torch.randn(7, 5, generator=generator),
        "half": torch.randn(3, 4, generator=generator).to(torch.bfloat16),
        "sixteen": torch.randn(9, generator=generator).to(torch.float16),
        "double": torch.randn(2, 2, generator=generator).to(torch.float64),
        "ids": torch.arange(11, dtype=torch.int64),
        "table": torch.arange(6, dtype=torch.int32).view(2, 3),
        "small": torch.arange(5, dtype=torch.int16),
        "bytes": torch.arange(4, dtype=torch.uint8),
        "signed": torch.arange(-2, 2, dtype=torch.int8),
        "flags": torch.tensor([True, False, True]),
        "empty": torch.zeros(0, 3),
        "scalar": torch.tensor(2.5),
        "deep": torch.randn(2, 1, 3, 1, 2, generator=generator),
        'quoted "name" with \\ and \u00e9 \u4e2d': torch.ones(2),
    }
    path = tmp_path / "all.safetensors"
    write_safetensors(path, tensors, metadata={"format": "pt", "note": "{[\"nested\"]}"})
    native, python = SafetensorsFile(path), SafetensorsFile(path, native=False)
    assert native._native_handle is not None and python._native_handle is None
    assert dict(native.entries) == dict(python.entries) and set(native.names()) == set(tensors)
    for name, tensor in tensors.items():
        got = native.tensor(name)
        assert got.dtype == tensor.dtype and got.shape == tensor.shape
        assert torch.equal(got, tensor) and torch.equal(python.tensor(name), tensor)
    # a tensor outlives the reader object that handed it out
    kept = native.tensor("plain.weight")
    del native
    assert torch.equal(kept, tensors["plain.weight"])
    # a header written by hand: spaces, members in another order, an extra member, a repeated name
    header = (b'  { "__metadata__" : {"a": [1, 2.5e3, null, true]} ,\n "x":{"data_offsets":[0,8],"shape":[2],"extra":{"k":[]},'
              b'"dtype":"F32"}, "y": {"dtype":"U8","shape":[3],"data_offsets":[8,11]}, "y": {"dtype":"I8","shape":[1,3],'
              b'"data_offsets":[8,11]} }   ')
    _write_raw(tmp_path / "hand.safetensors", header, bytes(range(11)))
    native, python = SafetensorsFile(tmp_path / "hand.safetensors"), SafetensorsFile(tmp_path / "hand.safetensors", native=False)
    assert dict(native.entries) == dict(python.entries)
    assert native.entries["y"].dtype == "I8" and torch.equal(native.tensor("y"), python.tensor("y"))


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


def test_tied_folder_may_still_hold_the_output_head(tmp_path):
    """Some tied checkpoints ship lm_head.weight all the same; the reference loads them
    (crates/llm-models/src/qwen.rs:215-260 asks only for the names it needs).  Any other extra stays an error."""
    config = config_from_dict(CONFIG_A)  # tied
    plan = plan_for_config(config)
    specs = plan.weight_specs()
    assert "lm_head.weight" not in specs and plan.ignorable_weights == ["lm_head.weight"]
    tensors = random_tensors(specs, seed=1)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(tmp_path / "model.safetensors", tensors)
    source = open_checked(str(tmp_path), specs, "cpu", plan.ignorable_weights)
    assert source.stored("model.norm.weight").shape == (64,)
    with pytest.raises(WeightError) as err:
        open_checked(str(tmp_path), specs, "cpu")  # nothing declared ignorable: the extra is listed
    assert err.value.unexpected == ["lm_head.weight"]
    untied = plan_for_config(config_from_dict(CONFIG_B))
    assert untied.ignorable_weights == []


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

import json
import os
import struct

import numpy as np
import pytest
import torch

from quicknn_b200.config import GEMMA2, Gemma2Config, gemma2_spec
from quicknn_b200.parts import expected_tensors
from quicknn_b200.weights import (SafetensorsError, SafetensorsFile, TensorDirectory, WeightError,
                                  load_named_tensors, random_tensors, write_model_folder, write_safetensors)
from conftest import TINY_A, TINY_B


def _expected(raw):
    return {n: s for n, (s, _) in expected_tensors(gemma2_spec(Gemma2Config.from_dict(raw))).items()}


def test_random_folder_round_trip(tmp_path):
    cfg = Gemma2Config.from_dict(TINY_A)
    d = write_model_folder(str(tmp_path / "m"), GEMMA2, cfg, seed=3, dtype=torch.bfloat16, norm_std=0.1)
    assert sorted(os.listdir(d)) == ["config.json", "model.safetensors"]
    got = load_named_tensors(d, _expected(TINY_A), torch.bfloat16, "cpu")
    again = dict(random_tensors(GEMMA2, cfg, 3, torch.bfloat16, 0.1))
    for n, t in got.items():
        assert t.dtype == torch.bfloat16 and torch.equal(t, again[n]), n
    other = dict(random_tensors(GEMMA2, cfg, 4, torch.bfloat16, 0.1))
    assert not torch.equal(other["model.norm.weight"], again["model.norm.weight"])
    w = again["model.layers.0.mlp.up_proj.weight"].float()
    assert abs(float(w.std()) - 0.02) < 0.002
    assert abs(float(again["model.layers.0.input_layernorm.weight"].float().std()) - 0.1) < 0.03


def test_precision_policy(tmp_path):
    cfg = Gemma2Config.from_dict(TINY_A)
    tensors = dict(random_tensors(GEMMA2, cfg, 0, torch.bfloat16))
    tensors["model.norm.weight"] = tensors["model.norm.weight"].float()      # one tensor stored in 32-bit
    d = tmp_path / "mixed"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(cfg.to_dict()))
    write_safetensors(str(d / "model.safetensors"), tensors)
    bf = load_named_tensors(str(d), _expected(TINY_A), torch.bfloat16, "cpu")
    assert bf["model.norm.weight"].dtype == torch.float32                   # stays 32-bit
    assert bf["model.embed_tokens.weight"].dtype == torch.bfloat16          # stays bfloat16
    f32 = load_named_tensors(str(d), _expected(TINY_A), torch.float32, "cpu")
    assert all(t.dtype == torch.float32 for t in f32.values())
    assert torch.equal(f32["model.embed_tokens.weight"], tensors["model.embed_tokens.weight"].float())  # widened exactly


def test_one_error_lists_everything(tmp_path):
    cfg = Gemma2Config.from_dict(TINY_B)
    tensors = dict(random_tensors(GEMMA2, cfg, 0, torch.float32))
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(10, 96)
    tensors["lm_head.weight"] = torch.zeros(4, 4)
    tensors["model.layers.2.input_layernorm.weight"] = torch.zeros(96, dtype=torch.float16)
    d = tmp_path / "bad"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), tensors)
    with pytest.raises(WeightError) as e:
        load_named_tensors(str(d), _expected(TINY_B), torch.float32, "cpu")
    err = e.value
    assert sorted(err.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["lm_head.weight"]
    assert err.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (144, 96), (10, 96))]
    assert err.wrong_dtype == [("model.layers.2.input_layernorm.weight", "torch.float16")]
    msg = str(err)
    for piece in ("missing tensors (2)", "unexpected tensors (1)", "wrong shape", "[10, 96]", "[144, 96]", "float16"):
        assert piece in msg


def _raw_file(path, header, data=b""):
    blob = json.dumps(header).encode() if not isinstance(header, bytes) else header
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)) + blob + data)


def test_file_validation(tmp_path):
    p = str(tmp_path / "f.safetensors")
    ok = {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    _raw_file(p, ok, b"\0" * 8)
    assert SafetensorsFile(p).tensor("a").shape == (2,)
    cases = {
        "truncated": (ok, b"\0" * 4),
        "uncovered": (ok, b"\0" * 12),
        "bytes": ({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8),
        "dtype": ({"a": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8),
        "overlap": ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                     "b": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12),
        "gap": ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]},
                 "b": {"dtype": "F32", "shape": [1], "data_offsets": [8, 12]}}, b"\0" * 12),
        "metadata": ({"__metadata__": {"k": 1}}, b""),
        "notobject": (b"[1, 2]", b""),
        "duplicate": (b'{"a":{"dtype":"F32","shape":[1],"data_offsets":[0,4]},'
                      b'"a":{"dtype":"F32","shape":[1],"data_offsets":[4,8]}}', b"\0" * 8),
    }
    for name, (h, data) in cases.items():
        _raw_file(p, h, data)
        with pytest.raises(SafetensorsError):
            SafetensorsFile(p)
    with open(p, "wb") as fh:
        fh.write(struct.pack("<Q", 1 << 40))
    with pytest.raises(SafetensorsError):
        SafetensorsFile(p)


def test_shards_through_an_index(tmp_path):
    a = {"x": torch.arange(6, dtype=torch.float32).view(2, 3)}
    b = {"y": torch.ones(4, dtype=torch.bfloat16)}
    write_safetensors(str(tmp_path / "s1.safetensors"), a)
    write_safetensors(str(tmp_path / "s2.safetensors"), b)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"x": "s1.safetensors", "y": "s2.safetensors"}}))
    d = TensorDirectory.open(str(tmp_path))
    assert sorted(d.names()) == ["x", "y"]
    assert torch.equal(d.tensor("x"), a["x"]) and d.shape_dtype("y") == ((4,), torch.bfloat16)
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "s1.safetensors"}}))
    d = TensorDirectory.open(str(tmp_path))
    assert d.names() == ["x"]
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"z": "s1.safetensors"}}))
    with pytest.raises(SafetensorsError):
        TensorDirectory.open(str(tmp_path))


def test_sizes_the_kernels_do_not_take_are_refused_when_the_model_is_built():
    """A configuration may be valid and still ask for what the kernels refuse: a head size beyond the
    attention kernels' reach or one that is not made of whole 16-byte vectors.  The model says so when
    it is built, by name, and not at its first step (the checks are host functions of the kernel library)."""
    import torch
    from quicknn_b200.config import GEMMA2, Gemma2Config
    from quicknn_b200.engine import Model
    from quicknn_b200.weights import random_tensors
    from conftest import TINY_A

    def build(dtype, **over):
        cfg = Gemma2Config.from_dict(dict(TINY_A, **over))
        tensors = dict(random_tensors(GEMMA2, cfg, 0, dtype))
        return Model(GEMMA2, cfg, tensors, dtype, "cpu")
    build(torch.float32)                                                  # the sizes of tiny A are fine
    with pytest.raises(ValueError, match="head size 1152"):
        build(torch.bfloat16, head_dim=1152, num_attention_heads=1, num_key_value_heads=1)
    with pytest.raises(ValueError, match="head size 516"):
        build(torch.float32, head_dim=516, num_attention_heads=1, num_key_value_heads=1)
    with pytest.raises(ValueError, match="head size 20"):
        build(torch.bfloat16, head_dim=20)                                # 40 bytes: no whole 16-byte vectors
    build(torch.float32, head_dim=20)                                     # 80 bytes in float32: fine
    build(torch.bfloat16, hidden_size=68, intermediate_size=100)          # the products take any inner size
    build(torch.float32, hidden_size=67, intermediate_size=101)

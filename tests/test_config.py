import json
import os

import pytest

from quicknn_b200.config import (ConfigError, Gemma2Config, find_architecture, gemma2_spec, load_config,
                                 registered_architectures)
from quicknn_b200.parts import expected_tensors
from conftest import TINY_A, TINY_B


def test_registry_names():
    assert "Gemma2ForCausalLM" in registered_architectures()
    assert find_architecture({"architectures": ["Gemma2ForCausalLM"]}).name == "Gemma2ForCausalLM"
    assert find_architecture({"model_type": "gemma2"}).name == "Gemma2ForCausalLM"
    with pytest.raises(ConfigError) as e:
        find_architecture({"architectures": ["NoSuchModel"], "model_type": "nope"})
    assert "NoSuchModel" in str(e.value) and "Gemma2ForCausalLM" in str(e.value)


def test_typed_values_and_defaults():
    c = Gemma2Config.from_dict(TINY_A)
    assert (c.hidden_size, c.num_hidden_layers, c.head_dim, c.sliding_window) == (64, 2, 16, 8)
    assert c.eos_token_id == (1,)
    assert abs(c.attention_scale - 0.25) < 1e-12
    b = Gemma2Config.from_dict(TINY_B)
    assert b.attn_logit_softcapping is None and b.eos_token_id == (1, 7)
    assert abs(b.attention_scale - 32 ** -0.5) < 1e-12
    # the reference's defaults (Gemma2.pas:82-88)
    d = {k: v for k, v in TINY_A.items() if k not in ("rope_theta", "rms_norm_eps", "sliding_window",
                                                      "attn_logit_softcapping", "final_logit_softcapping",
                                                      "query_pre_attn_scalar")}
    c = Gemma2Config.from_dict(d)
    assert (c.rope_theta, c.rms_norm_eps, c.sliding_window) == (10000.0, 1e-6, 4096)
    assert (c.attn_logit_softcapping, c.final_logit_softcapping) == (50.0, 30.0)
    assert abs(c.attention_scale - 16 ** -0.5) < 1e-12          # defaults to head_dim


def test_every_violated_rule_is_named():
    bad = dict(TINY_A, num_attention_heads=3, num_key_value_heads=2, head_dim=15, num_hidden_layers=0,
               rms_norm_eps=0.0, tie_word_embeddings=False, attention_bias=True, hidden_activation="relu",
               eos_token_id=99999)
    with pytest.raises(ConfigError) as e:
        Gemma2Config.from_dict(bad)
    msg = str(e.value)
    for piece in ("num_key_value_heads", "head_dim", "num_hidden_layers", "rms_norm_eps", "tie_word_embeddings",
                  "attention_bias", "hidden_activation", "eos_token_id"):
        assert piece in msg, piece
    with pytest.raises(ConfigError) as e:
        Gemma2Config.from_dict({k: v for k, v in TINY_A.items() if k not in ("hidden_size", "vocab_size")})
    assert "hidden_size" in str(e.value) and "vocab_size" in str(e.value)
    with pytest.raises(ConfigError):
        Gemma2Config.from_dict(dict(TINY_A, hidden_size="64"))


def test_layer_pattern_and_spec():
    c = Gemma2Config.from_dict(TINY_B)
    spec = gemma2_spec(c)
    windows = [l.mixer.params["window"] for l in spec.layers]
    assert windows == [5, None, 5]                              # even layers local (Gemma2.pas:177)
    c2 = Gemma2Config.from_dict(dict(TINY_B, layer_types=["full_attention", "sliding_attention", "full_attention"]))
    assert [l.mixer.params["window"] for l in gemma2_spec(c2).layers] == [None, 5, None]
    with pytest.raises(ConfigError):
        Gemma2Config.from_dict(dict(TINY_B, layer_types=["full_attention"]))
    names = expected_tensors(spec)
    assert names["model.layers.2.mlp.down_proj.weight"][0] == (96, 200)
    assert names["model.layers.0.self_attn.k_proj.weight"][0] == (24, 96)
    assert names["model.embed_tokens.weight"][0] == (1000, 96)
    assert len(names) == 2 + 11 * 3
    assert [e.layer for e in spec.schedule] == [0, 1, 2] and spec.stop_ids == (1, 7)


def test_round_trip_through_a_file(tmp_path):
    c = Gemma2Config.from_dict(TINY_B)
    p = tmp_path / "config.json"
    p.write_text(json.dumps(c.to_dict()))
    arch, c2 = load_config(str(tmp_path))
    assert arch.name == "Gemma2ForCausalLM" and c2 == c


def test_stop_ids_of_a_folder(tmp_path):
    """eos_token_id of generation_config.json joins the ids of config.json: an integer or a list, each id once,
    an id outside the vocabulary or a file that is no JSON object is an error."""
    import json
    from quicknn_b200.config.generation import stop_ids_of_folder
    d = str(tmp_path)
    assert stop_ids_of_folder(d, 100, [1]) == [1]                     # no file: the configuration's ids
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [1, 7, [9, 7]], "top_k": 5}))
    assert stop_ids_of_folder(d, 100, [1, 3, 1]) == [1, 3, 7, 9]
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 42}))
    assert stop_ids_of_folder(d, 100, []) == [42]
    (tmp_path / "generation_config.json").write_text(json.dumps({"temperature": 1.0}))
    assert stop_ids_of_folder(d, 100, [2]) == [2]
    for bad in ({"eos_token_id": 100}, {"eos_token_id": -1}, {"eos_token_id": "1"}, {"eos_token_id": True}, [1]):
        (tmp_path / "generation_config.json").write_text(json.dumps(bad))
        with pytest.raises(ValueError):
            stop_ids_of_folder(d, 100, [1])
    (tmp_path / "generation_config.json").write_text("{not json")
    with pytest.raises(ValueError):
        stop_ids_of_folder(d, 100, [1])


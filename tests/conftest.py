"""Shared fixtures: two tiny Gemma 2 configurations that differ in every size and option,
model folders with random weights in temporary directories, and the plain implementation."""
import os
import sys
import warnings

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

warnings.filterwarnings("ignore", message="The given buffer is not writable")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


# Tiny A: 2 layers, GQA 4/2, head_dim = hidden/heads, both softcaps on, window 8.
TINY_A = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2",
    hidden_size=64, intermediate_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    vocab_size=512, num_hidden_layers=2, max_position_embeddings=1024, rope_theta=10000.0,
    rms_norm_eps=1e-6, sliding_window=8, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
    query_pre_attn_scalar=16, eos_token_id=1, bos_token_id=2, initializer_range=0.02,
    hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True)
TINY_A_SEED, TINY_A_NORM_STD = 0, 0.1

# Tiny B: 3 layers, MQA 6/1, head_dim 24 decoupled from hidden/heads, sizes that are no power
# of two, attention softcap off, window 5, another eps, theta, scale factor and vocabulary.
TINY_B = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2",
    hidden_size=96, intermediate_size=200, num_attention_heads=6, num_key_value_heads=1, head_dim=24,
    vocab_size=1000, num_hidden_layers=3, max_position_embeddings=1024, rope_theta=1e6,
    rms_norm_eps=1e-5, sliding_window=5, attn_logit_softcapping=None, final_logit_softcapping=15.0,
    query_pre_attn_scalar=32, eos_token_id=[1, 7], bos_token_id=2, initializer_range=0.05,
    hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True)
TINY_B_SEED, TINY_B_NORM_STD = 1, 0.2

# Small C: head size 64 and a window of 96, so that the engine's bfloat16 path runs the tensor-core
# attention kernels (head sizes 64/128/256) and the tcgen05 product, not only the generic ones.
TINY_C = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2",
    hidden_size=192, intermediate_size=320, num_attention_heads=6, num_key_value_heads=2, head_dim=64,
    vocab_size=1536, num_hidden_layers=3, max_position_embeddings=1024, rope_theta=50000.0,
    rms_norm_eps=1e-6, sliding_window=96, attn_logit_softcapping=30.0, final_logit_softcapping=20.0,
    query_pre_attn_scalar=48, eos_token_id=1, bos_token_id=2, initializer_range=0.04,
    hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True)

# Small D: head size 256 (the benchmark's), two query heads on one kv head, so that the engine runs the
# tcgen05 prefill attention and the head-256 decode attention end to end.
TINY_D = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2",
    hidden_size=256, intermediate_size=384, num_attention_heads=2, num_key_value_heads=1, head_dim=256,
    vocab_size=1280, num_hidden_layers=2, max_position_embeddings=1024, rope_theta=10000.0,
    rms_norm_eps=1e-6, sliding_window=80, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
    query_pre_attn_scalar=256, eos_token_id=1, bos_token_id=2, initializer_range=0.03,
    hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True)

# Tiny E: a width, a feed-forward width and a vocabulary that are no multiple of 8 (bfloat16 rows that do not
# start on 16 bytes), five query heads on five kv heads, one layer more than a local/global pair.
TINY_E = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2",
    hidden_size=100, intermediate_size=70, num_attention_heads=5, num_key_value_heads=5, head_dim=16,
    vocab_size=301, num_hidden_layers=3, max_position_embeddings=1024, rope_theta=20000.0,
    rms_norm_eps=1e-4, sliding_window=11, attn_logit_softcapping=40.0, final_logit_softcapping=None,
    query_pre_attn_scalar=20, eos_token_id=1, bos_token_id=2, initializer_range=0.05,
    hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True)

TINY = {"E": (TINY_E, 4, 0.15), "A": (TINY_A, TINY_A_SEED, TINY_A_NORM_STD), "B": (TINY_B, TINY_B_SEED, TINY_B_NORM_STD),
        "C": (TINY_C, 2, 0.15), "D": (TINY_D, 3, 0.1)}


def make_folder(tmp, name, storage, peaky=False):
    """Write the tiny model `name` with weights stored as `storage` ("float32"/"bfloat16").
    `peaky` multiplies the query and key projections by 6 so that attention concentrates on
    few keys and any fault in masking, windows or cache addressing shows in the logits."""
    import torch
    from quicknn_b200.config import GEMMA2, Gemma2Config
    from quicknn_b200.weights import random_tensors, write_safetensors
    import json
    raw, seed, nstd = TINY[name]
    cfg = Gemma2Config.from_dict(raw)
    dt = torch.float32 if storage == "float32" else torch.bfloat16
    d = os.path.join(str(tmp), f"tiny{name}_{storage}{'_peaky' if peaky else ''}")
    os.makedirs(d, exist_ok=True)
    tensors = dict(random_tensors(GEMMA2, cfg, seed, torch.float32, nstd))
    if peaky:
        for k in tensors:
            if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
                tensors[k] = tensors[k] * 6.0
    tensors = {k: v.to(dt) for k, v in tensors.items()}
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(cfg.to_dict(), fh)
    write_safetensors(os.path.join(d, "model.safetensors"), tensors)
    return d


@pytest.fixture(scope="session")
def folders(tmp_path_factory):
    """Lazily written model folders, keyed by (name, storage, peaky)."""
    base = tmp_path_factory.mktemp("models")
    made = {}

    def get(name, storage="float32", peaky=False):
        key = (name, storage, peaky)
        if key not in made:
            made[key] = make_folder(base, name, storage, peaky)
        return made[key]
    return get


@pytest.fixture(scope="session")
def plain_models(folders):
    from plain.gemma2_plain import PlainGemma2
    made = {}

    def get(name, storage="float32", peaky=False):
        key = (name, storage, peaky)
        if key not in made:
            made[key] = PlainGemma2(folders(name, storage, peaky))
        return made[key]
    return get


def prompts_for(name, lengths, seed=None):
    raw, s, _ = TINY[name]
    rng = np.random.default_rng(s if seed is None else seed)
    return [rng.integers(1, raw["vocab_size"], n).tolist() for n in lengths]


def close(got, ref, dtype):
    """Tolerance of the comparisons with the plain implementation, relative to the size of
    the logits: float32 2e-5, bfloat16 (same bf16 weights on both sides, so only the
    rounding of activations differs) 3e-2."""
    ref = np.asarray(ref, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    scale = max(1.0, float(np.abs(ref).max()))
    tol = (2e-5 if dtype == "float32" else 3e-2) * scale
    err = float(np.abs(got - ref).max()) if got.size else 0.0
    return err <= tol, err, tol

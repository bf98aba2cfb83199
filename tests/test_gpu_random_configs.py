"""Random tiny configurations of the architecture: every size and option drawn at random (head counts and groups,
head sizes in steps of 8 and 16, widths and vocabularies that are no power of two, one to four layers, windows shorter
and longer than the prompts, softcaps on and off, eps, theta, the scale of the scores), written to a folder with
random weights, and run through whole prompts, single tokens and portions against the plain implementation."""
import json
import os

import numpy as np
import pytest
import torch

from conftest import close


def same(got, ref, dtype, what):
    ok, err, tol = close(got, ref, dtype)
    assert ok, f"{what}: error {err:.3g} above {tol:.3g}"

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def random_config(rng, dtype):
    hd = int(rng.choice([16, 32, 48, 64, 80, 128] if dtype == "bfloat16" else [8, 16, 24, 40, 64]))
    nkv = int(rng.choice([1, 2, 3, 4]))
    group = int(rng.choice([1, 2, 3, 4, 8]))
    hidden = int(rng.choice([36, 40, 50, 72, 96, 100, 136, 200]))
    return dict(
        architectures=["Gemma2ForCausalLM"], model_type="gemma2", hidden_size=hidden,
        intermediate_size=int(rng.choice([64, 70, 88, 100, 160, 264])), num_attention_heads=nkv * group, num_key_value_heads=nkv,
        head_dim=hd, vocab_size=int(rng.integers(100, 1200)), num_hidden_layers=int(rng.integers(1, 5)),
        max_position_embeddings=512, rope_theta=float(rng.choice([1e4, 5e4, 1e6])),
        rms_norm_eps=float(rng.choice([1e-6, 1e-5, 1e-4])), sliding_window=int(rng.choice([4, 9, 33, 64, 100, 400])),
        attn_logit_softcapping=[None, 20.0, 50.0, 80.0][int(rng.integers(0, 4))],
        final_logit_softcapping=[None, 15.0, 30.0][int(rng.integers(0, 3))],
        query_pre_attn_scalar=int(rng.choice([hd, 2 * hd, 100, 144])), eos_token_id=1, bos_token_id=2,
        initializer_range=0.05, hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True)


@pytest.mark.parametrize("seed,dtype", [(s, "float32") for s in range(6)] + [(s, "bfloat16") for s in range(6, 14)])
def test_a_random_configuration_gives_the_plain_logits(tmp_path, seed, dtype):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from plain.gemma2_plain import PlainGemma2
    from quicknn_b200.config import GEMMA2, Gemma2Config
    from quicknn_b200.engine import Engine, Model
    from quicknn_b200.weights import random_tensors, write_safetensors
    rng = np.random.default_rng(1000 + seed)
    raw = random_config(rng, dtype)
    cfg = Gemma2Config.from_dict(raw)
    folder = str(tmp_path / "model")
    os.makedirs(folder)
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = {k: v.to(dt) for k, v in random_tensors(GEMMA2, cfg, seed, torch.float32, 0.15)}
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(cfg.to_dict(), fh)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    plain = PlainGemma2(folder)
    eng = Engine(Model.from_folder(folder, dtype, DEV), max_tokens=64 * 12, max_slots=4, max_seq=160)
    lens = [int(n) for n in rng.integers(2, 150, 3)]
    seqs = [rng.integers(1, raw["vocab_size"], n).tolist() for n in lens]
    ref = [plain.logits(s) for s in seqs]
    what = json.dumps({k: raw[k] for k in ("hidden_size", "num_attention_heads", "num_key_value_heads", "head_dim",
                                           "num_hidden_layers", "sliding_window", "attn_logit_softcapping",
                                           "final_logit_softcapping", "vocab_size")})
    slots = [eng.new_sequence() for _ in seqs]
    # whole prompts but for each sequence's tail: a portion of it, then its last tokens one by one
    cut = [max(1, n - int(rng.integers(1, min(n, 12) + 1))) for n in lens]
    mid = [max(1, c - int(rng.integers(0, min(c, 40) + 1))) for c in cut]
    got = eng.step([(s, q[:m]) for s, q, m in zip(slots, seqs, mid)], [[m - 1] for m in mid]).cpu().numpy()
    for i in range(3):
        same(got[i], ref[i][mid[i] - 1], dtype, what + " prompt")
    going = [i for i in range(3) if cut[i] > mid[i]]
    if going:
        got = eng.step([(slots[i], seqs[i][mid[i]:cut[i]]) for i in going],
                       [[0, cut[i] - mid[i] - 1] for i in going]).cpu().numpy()
        for j, i in enumerate(going):
            same(got[2 * j], ref[i][mid[i]], dtype, what + " portion")
            same(got[2 * j + 1], ref[i][cut[i] - 1], dtype, what + " portion")
    pos = list(cut)
    while any(p < n for p, n in zip(pos, lens)):
        live = [i for i in range(3) if pos[i] < lens[i]]
        got = eng.step([(slots[i], [seqs[i][pos[i]]]) for i in live], [[0]] * len(live)).cpu().numpy()
        for j, i in enumerate(live):
            same(got[j], ref[i][pos[i]], dtype, what + f" token {pos[i]} of {lens[i]}")
            pos[i] += 1
    for s in slots:
        eng.release(s)
    eng.cache.audit()

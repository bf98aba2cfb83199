"""The plain implementation checked against itself: each part against an independent
restatement of its formula or a property that the formula implies."""
import math

import numpy as np
import pytest

from plain import gemma2_plain as P
from conftest import prompts_for


def test_gelu_softcap_values():
    assert abs(float(P.gelu_tanh(np.array([0.7]))[0]) - 0.530570149) < 1e-7    # the float32 value of the shader line compiled as C++
    x = np.array([-1e4, -3.0, 0.0, 3.0, 1e4])
    y = P.softcap(x, 30.0)
    assert np.all(np.abs(y) <= 30.0) and abs(y[3] - 30 * math.tanh(0.1)) < 1e-12
    assert P.softcap(x, None) is x and P.softcap(x, 0.0) is x


def test_rmsnorm_formula():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(3, 10))
    w = rng.normal(size=10) * 0.1
    y = P.rmsnorm(x, w, 1e-6)
    for r in range(3):
        inv = 1.0 / math.sqrt(sum(v * v for v in x[r]) / 10 + 1e-6)
        assert np.allclose(y[r], [x[r, j] * inv * (1 + w[j]) for j in range(10)], atol=1e-12)


def test_rope_is_a_rotation_by_relative_position():
    rng = np.random.default_rng(1)
    q = rng.normal(size=(1, 1, 8))
    k = rng.normal(size=(1, 1, 8))
    def dot(pq, pk):
        a = P.rope(q, np.array([pq]), 10000.0)[0, 0]
        b = P.rope(k, np.array([pk]), 10000.0)[0, 0]
        return float(a @ b)
    assert abs(dot(7, 3) - dot(14, 10)) < 1e-5
    assert abs(np.linalg.norm(P.rope(q, np.array([55]), 10000.0)) - np.linalg.norm(q)) < 1e-6
    # pair j is (x_j, x_{j + hd/2}) and its frequency theta^(-2j/hd)
    x = np.zeros((1, 1, 8)); x[0, 0, 1] = 1.0
    y = P.rope(x, np.array([3]), 100.0)[0, 0]
    ang = 3 * 100.0 ** (-2 * 1 / 8)
    assert abs(y[1] - math.cos(ang)) < 1e-6 and abs(y[5] - math.sin(ang)) < 1e-6


def _attention_dense(q, k, v, scale, cap, window):
    T, nq, hd = q.shape
    g = nq // k.shape[1]
    out = np.zeros_like(q)
    for h in range(nq):
        s = np.einsum("td,sd->ts", q[:, h], k[:, h // g]) * scale
        if cap:
            s = cap * np.tanh(s / cap)
        i, j = np.arange(T)[:, None], np.arange(T)[None, :]
        mask = (j <= i) & ((i - j < window) if window else True)
        s = np.where(mask, s, -np.inf)
        w = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h] = (w / w.sum(axis=1, keepdims=True)) @ v[:, h // g]
    return out


@pytest.mark.parametrize("window,cap", [(None, 50.0), (4, None), (1, 20.0), (30, None)])
def test_attention_against_a_dense_mask(window, cap):
    rng = np.random.default_rng(2)
    q, k, v = rng.normal(size=(13, 6, 8)), rng.normal(size=(13, 2, 8)), rng.normal(size=(13, 2, 8))
    a = P.attention(q, k, v, 0.3, cap, window)
    assert np.allclose(a, _attention_dense(q, k, v, 0.3, cap, window), atol=1e-12)


def test_window_edge_is_exact():
    """A query sees itself and the window-1 tokens before it, nothing earlier."""
    T, W = 12, 5
    q = np.ones((T, 1, 4)); k = np.ones((T, 1, 4)); v = np.zeros((T, 1, 4))
    v[:, 0, 0] = np.arange(T)
    a = P.attention(q, k, v, 1.0, None, W)
    for p in range(T):
        lo = max(0, p - W + 1)
        assert abs(a[p, 0, 0] - np.mean(np.arange(lo, p + 1))) < 1e-12


def test_causality_and_precisions(plain_models, folders):
    m = plain_models("B")
    ids = prompts_for("B", [20])[0]
    full = m.logits(ids)
    assert np.allclose(m.logits(ids[:9]), full[:9], atol=1e-10)
    m32 = P.PlainGemma2(folders("B"), np.float32)
    assert np.abs(m32.logits(ids) - full).max() < 5e-5
    assert full.shape == (20, 1000) and np.abs(full).max() <= 15.0


def test_layer_pattern_of_the_model(plain_models):
    m = plain_models("A")
    assert [m.layer_window(i) for i in range(2)] == [8, None]
    assert abs(m.scale - 0.25) < 1e-12


def test_sampler_follows_the_shader():
    assert P.argmax_lowest(np.array([1.0, 3.0, 3.0, 2.0])) == 1
    s, u = P.xorshift32(42)
    assert s == 11355432 and abs(float(u) - (11355432 + 0.5) / 2 ** 32) < 1e-9
    row = np.array([0.0, 2.0, 1.0, -5.0, 2.0], dtype=np.float32)
    assert P.sample(row, 0.0, 20, 0.95, 1.0, None, 0.9) == 1                 # greedy, lowest id on ties
    assert P.sample(row, 1.0, 1, 1.0, 1.0, None, 0.9) == 1                   # k = 1
    # k = 3 keeps ids 1, 4, 2 with p = 1, 1, e^-1; u picks by the running sum
    picks = [P.sample(row, 1.0, 3, 1.0, 1.0, None, u) for u in (0.0, 0.4, 0.5, 0.9)]
    assert picks == [1, 1, 4, 2]
    assert P.sample(row, 1.0, 3, 0.5, 1.0, None, 0.99) == 4                  # nucleus keeps two
    seen = np.array([0, 1, 0, 0, 1])
    assert P.sample(row, 0.0, 20, 1.0, 4.0, seen, 0.0) == 2                  # 2/4 < 1
    counts = np.zeros(5)
    st = P.seed_state(7)
    for _ in range(4000):
        st, u = P.xorshift32(st)
        counts[P.sample(row, 1.0, 5, 1.0, 1.0, None, u)] += 1
    p = np.exp(row - 2.0); p /= p.sum()
    assert np.abs(counts / 4000 - p).max() < 0.03


@pytest.mark.parametrize("name", ["A", "B"])
def test_the_torch_plain_implementation_agrees_with_the_numpy_one(plain_models, folders, name):
    """The second plain implementation (torch operations; it runs the large layer sizes on the GPU
    and is the timed baseline of the benchmark) gives the logits of the first at every position,
    for prompts longer than the windows of both tiny models."""
    import torch
    from plain.gemma2_torch import TorchGemma2
    ids = prompts_for(name, [29])[0]
    ref = plain_models(name).logits(ids)
    t64 = TorchGemma2(folders(name), "cpu", torch.float64)
    assert np.abs(t64.logits(ids) - ref).max() < 1e-10
    assert np.abs(t64.logits(ids, [0, 28]) - ref[[0, 28]]).max() < 1e-10
    t32 = TorchGemma2(folders(name), "cpu", torch.float32)
    assert np.abs(t32.logits(ids) - ref).max() < 5e-5
    assert t64.greedy(ids[:7], 4) == plain_models(name).greedy(ids[:7], 4)
    assert [t64.layer_window(i) for i in range(2)] == [plain_models(name).layer_window(i) for i in range(2)]


def test_the_timed_baseline_decodes_what_the_plain_model_computes(plain_models, folders):
    """baseline/torch_ops_decode.py (torch operations with a contiguous cache; what the benchmark's
    vs_baseline is measured against) fed a sequence token by token picks, at every position, the
    plain model's best token: it is a correct implementation, not only a timed one."""
    import json
    import os
    import sys
    import torch
    from conftest import ROOT
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    from torch_ops_decode import CachedTorchGemma2
    from plain.gemma2_torch import read_safetensors
    for name in ("A", "B"):
        folder = folders(name)
        with open(os.path.join(folder, "config.json")) as fh:
            cfg = json.load(fh)
        w = read_safetensors(os.path.join(folder, "model.safetensors"), "cpu", torch.float64)
        seqs = prompts_for(name, [20, 20])
        ref = [plain_models(name).logits(s) for s in seqs]
        m = CachedTorchGemma2(cfg, w, batch=2, max_len=32, device="cpu", dtype=torch.float64)
        for t in range(20):
            got = m.decode(torch.tensor([s[t] for s in seqs])).tolist()
            assert got == [int(np.argmax(r[t])) for r in ref], t

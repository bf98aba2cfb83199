"""The layer sizes of Gemma 2 2B, 9B and 27B under every cutting, through bin/trace_run, in
float32 and in bfloat16, against the plain implementation in torch operations (float64, on the
GPU).

Each model has two layers, one local with the real window of 4096 and one global (fewer layers
is no smaller layer), random weights, and for the 2B sizes the real vocabulary of 256,000 (the
head and its 1 MB rows of logits at full size).  Two requests are longer than the window, so the
ring of the local layer wraps, once inside a prompt and once while decoding, and decode attention
walks more key ranges than fit one thread-block cluster.  The cuttings are those of the tiny
models: each request alone and whole; its last 32 tokens one by one; two batches of unequal
lengths whose shorter requests end earlier, the second batch in the slots and pages of the first.
"""
import json
import os

import numpy as np
import pytest
import torch

from conftest import close
from test_gpu_replay import Replay

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

SIZES = {
    "2b": dict(hidden_size=2304, intermediate_size=9216, num_attention_heads=8, num_key_value_heads=4, head_dim=256,
               query_pre_attn_scalar=256, vocab_size=256000),
    "9b": dict(hidden_size=3584, intermediate_size=14336, num_attention_heads=16, num_key_value_heads=8, head_dim=256,
               query_pre_attn_scalar=256, vocab_size=2048),
    "27b": dict(hidden_size=4608, intermediate_size=36864, num_attention_heads=32, num_key_value_heads=16,
                head_dim=128, query_pre_attn_scalar=144, vocab_size=2048),
}
SEEDS = {"2b": 2, "9b": 3, "27b": 4}
WINDOW = 4096
LENGTHS = [4200, 130, 700, 40, 4120]
# (requests, tokens of each that go in as the prompt); the rest is decoded one by one
BATCHES = (([0, 1, 2], [4170, 100, 690]), ([3, 4, 1], [1, 4090, 120]))
MAX_TOKENS = 4224 + 192 + 704


@pytest.fixture(scope="module")
def large(tmp_path_factory):
    """name -> (folder, requests, plain model, residual streams of the requests), made once."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from plain.gemma2_torch import TorchGemma2
    from quicknn_b200.config import GEMMA2, Gemma2Config
    from quicknn_b200.weights import write_model_folder
    base = tmp_path_factory.mktemp("large")
    made = {}

    def get(name):
        if name not in made:
            made.clear()                                  # one model's float64 weights at a time
            torch.cuda.empty_cache()
            raw = dict(architectures=["Gemma2ForCausalLM"], model_type="gemma2", num_hidden_layers=2,
                       max_position_embeddings=8192, rope_theta=10000.0, rms_norm_eps=1e-6, sliding_window=WINDOW,
                       attn_logit_softcapping=50.0, final_logit_softcapping=30.0, eos_token_id=1,
                       initializer_range=0.02, **SIZES[name])
            folder = os.path.join(str(base), name)
            if not os.path.isdir(folder):
                write_model_folder(folder, GEMMA2, Gemma2Config.from_dict(raw), SEEDS[name], torch.bfloat16, 0.1,
                                   device=DEV)
            rng = np.random.default_rng(SEEDS[name])
            requests = [rng.integers(1, raw["vocab_size"], n).tolist() for n in LENGTHS]
            plain = TorchGemma2(folder, DEV, torch.float64)
            hidden = [plain.hidden_states(t) for t in requests]
            made[name] = (folder, requests, plain, hidden)
        return made[name]
    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["2b", "9b", "27b"])
def test_model_sizes_under_every_cutting(large, tmp_path, name, dtype):
    folder, requests, plain, hidden = large(name)
    worst = 0.0

    def check(got, i, rows, what):
        nonlocal worst
        ok, err, tol = close(got, plain.logits_of_hidden(hidden[i], rows), dtype)
        worst = max(worst, err / tol)
        assert ok, f"{name} {dtype} {what}: error {err:.3g} > {tol:.3g}"

    replay = Replay(folder, dtype, tmp_path, max_tokens=MAX_TOKENS)
    try:
        # 1. whole: the first rows, both sides of a page edge and of the window's edge, the last row
        for i, toks in enumerate(requests):
            rows = sorted({r for r in (0, 1, 63, 64, WINDOW - 2, WINDOW - 1, WINDOW, WINDOW + 1, len(toks) - 1)
                           if r < len(toks)})
            check(replay.step([(f"w{i}", toks, rows)], end=[f"w{i}"]), i, rows, f"request {i} whole")
        # 2. the last 32 tokens one by one (request 4 crosses position 4096 while decoding)
        for i, toks in enumerate(requests):
            cut = len(toks) - 32
            check(replay.step([(f"s{i}", toks[:cut], [cut - 1])]), i, [cut - 1], f"request {i} prefix")
            for p in range(cut, len(toks)):
                got = replay.step([(f"s{i}", [toks[p]], [0])], end=[f"s{i}"] if p == len(toks) - 1 else [])
                check(got, i, [p], f"request {i} position {p} decoded alone")
        # 3. unequal batches, the second in what the first gave back
        for batch, cuts in BATCHES:
            ids = {i: f"b{batch[0]}_{i}" for i in batch}
            got = replay.step([(ids[i], requests[i][:n], [0, n - 1] if n > 1 else [0]) for i, n in zip(batch, cuts)])
            r = 0
            for i, n in zip(batch, cuts):
                rows = [0, n - 1] if n > 1 else [0]
                check(got[r:r + len(rows)], i, rows, f"batch {batch} prompt of request {i}")
                r += len(rows)
            pos = dict(zip(batch, cuts))
            while pos:
                live = sorted(pos)
                ended = [ids[i] for i in live if pos[i] + 1 == len(requests[i])]
                got = replay.step([(ids[i], [requests[i][pos[i]]], [0]) for i in live], end=ended)
                for r, i in enumerate(live):
                    check(got[r:r + 1], i, [pos[i]], f"batch {batch} request {i} position {pos[i]}")
                    pos[i] += 1
                    if pos[i] == len(requests[i]):
                        del pos[i]
        # 4. a prompt in portions: 4000 + 100 + 20 tokens of request 4, beside request 1 that starts with the
        #    second portion.  That portion crosses position 4096, where the ring of the local layer (exactly as
        #    long as the window) begins to be overwritten by the portion's own later rows
        toks, p0 = requests[4], 0
        for n, other in ((4000, None), (100, 1), (20, None)):
            rows = sorted({0, 1, n // 2, n - 2, n - 1})
            entries = [("p4", toks[p0:p0 + n], rows)]
            if other is not None:
                entries.append(("p1", requests[other][:50], [0, 49]))
            got = replay.step(entries, end=["p1"] if other is not None else [])
            check(got[:len(rows)], 4, [p0 + r for r in rows], f"portion of request 4 at {p0}")
            if other is not None:
                check(got[len(rows):], other, [0, 49], "the request that joined")
            p0 += n
        replay.step([], end=["p4"])
    finally:
        replay.close()
    print(f"{name} {dtype}: largest error {worst:.3g} of the tolerance")


def _follows_the_plain_model(plain, prompt, tokens, dtype, what):
    """Every generated token is, at its place, within the tolerance of the plain model's best."""
    seq = list(prompt) + list(tokens)
    rows = list(range(len(prompt) - 1, len(seq) - 1))
    ref = plain.logits_of_hidden(plain.hidden_states(seq), rows)
    for j, t in enumerate(tokens):
        tol = (2e-5 if dtype == "float32" else 3e-2) * max(1.0, float(np.abs(ref[j]).max()))
        assert ref[j][t] >= ref[j].max() - tol, f"{what}: token {j} ({t}) is {ref[j].max() - ref[j][t]:.3g} below the best"


@pytest.mark.parametrize("ahead", [True, False])
def test_a_batch_of_twelve_shrinks_to_seven_while_generating(large, ahead):
    """The schedules of the benchmark inside a test, at the 2B layer sizes: with 9 to 16 rows the big
    matrices (gate|up, down, the head of 256,000) take the tcgen05 decode product inside the captured
    step, with 8 or fewer the mma.sync one; requests that reach the end of their context leave the
    batch one by one, so the family of kernels and the graph change in mid-generation, with and
    without a step running ahead of the host."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    folder, _, plain, _ = large("2b")
    rng = np.random.default_rng(12)
    lens = [94, 93, 92, 91, 90, 30, 31, 32, 33, 34, 35, 36]
    prompts = [rng.integers(1, 256000, n).tolist() for n in lens]
    llm = LLM(folder, max_context=96, max_batch=12, dtype="bfloat16")
    llm.run_ahead = ahead
    out = llm.generate(prompts, GenerationOptions.greedy(8), stop_ids=[])
    assert [len(r.tokens) for r in out] == [min(8, 96 - n) for n in lens]
    assert [r.finish_reason for r in out] == ["context_full"] * 5 + ["max_tokens"] * 7
    assert sorted({k[0] for k in llm.engine._decode_state}) == [7, 8, 10, 12]   # row counts of the padded steps: 9 and 11 sequences run as 10 and 12 rows
    for r, p in zip(out, prompts):
        _follows_the_plain_model(plain, p, r.tokens, "bfloat16", f"request {r.index}")
    assert llm.engine.cache.slots.live() == []
    llm.engine.cache.audit()


def test_decode_steps_of_forty_rows_give_the_plain_logits(large):
    """33 rows and more: every product of the step, the small q|k|v and o matrices too, is the tcgen05
    decode product.  Logits of every row against the plain model, eagerly and through the graph."""
    from quicknn_b200.engine import Engine, Model
    folder, _, plain, _ = large("9b")
    rng = np.random.default_rng(40)
    B = 40
    seqs = [rng.integers(1, 2048, 3 + (7 * i) % 70 + 4).tolist() for i in range(B)]
    hidden = [plain.hidden_states(s) for s in seqs]
    eng = Engine(Model.from_folder(folder, "bfloat16", DEV), max_tokens=B * 128, max_slots=B, max_seq=128)
    slots = [eng.new_sequence() for _ in seqs]
    pos = [len(s) - 4 for s in seqs]
    eng.step([(sl, s[:p]) for sl, s, p in zip(slots, seqs, pos)], want=[[] for _ in seqs])
    for step in range(4):
        toks = torch.tensor([s[p] for s, p in zip(seqs, pos)], dtype=torch.int32, device=DEV)
        got = eng.decode(slots, toks, use_graph=step > 0).cpu().numpy()
        eng.check()
        for r in range(B):
            ok, err, tol = close(got[r], plain.logits_of_hidden(hidden[r], [pos[r]])[0], "bfloat16")
            assert ok, (step, r, err, tol)
            pos[r] += 1

"""The engine in process: long decoding, the first tokens of a sequence, padding, captured
decode steps, greedy and sampled generation through the Python entry point."""
import numpy as np
import pytest
import torch

from plain import gemma2_plain as P
from conftest import TINY, close, prompts_for

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module", autouse=True)
def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


def build(folder, dtype, **kw):
    from quicknn_b200.engine import Engine, Model
    return Engine(Model.from_folder(folder, dtype, DEV), **kw)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16")])
def test_long_decoding_matches_whole_sequences(folders, plain_models, name, dtype):
    """400 tokens decoded one by one (pages fill and new ones are taken, the window slides over
    the ring several times), eager and through the captured graph, against one plain pass."""
    eng = build(folders(name, dtype), dtype, max_tokens=1024, decode_splits=3)
    seqs = prompts_for(name, [420, 401])
    ref = [plain_models(name, dtype).logits(s) for s in seqs]
    slots = [eng.new_sequence(), eng.new_sequence()]
    starts = [20, 1]
    got = eng.step([(s, q[:n]) for s, q, n in zip(slots, seqs, starts)], "last").cpu().numpy()
    for r in range(2):
        ok, err, tol = close(got[r], ref[r][starts[r] - 1], dtype)
        assert ok, ("prompt", r, err, tol)
    worst = 0.0
    for step in range(400):
        toks = torch.tensor([seqs[r][starts[r] + step] for r in range(2)], dtype=torch.int32, device=DEV)
        got = eng.decode(slots, toks, use_graph=(step % 2 == 0)).cpu().numpy()
        for r in range(2):
            ok, err, tol = close(got[r], ref[r][starts[r] + step], dtype)
            worst = max(worst, err)
            assert ok, (f"step {step} row {r}", err, tol)
    for s in slots:
        eng.release(s)
    eng.cache.audit()
    print(f"long decoding tiny {name} {dtype}: largest error {worst:.3g}")


@pytest.mark.parametrize("name,dtype", [("A", "bfloat16"), ("B", "float32")])
def test_first_tokens_of_a_sequence(folders, plain_models, name, dtype):
    """Prompts of one, two and three tokens, then the first decoded tokens: the places where a
    sequence has fewer keys than a window, a page or a split."""
    eng = build(folders(name, dtype), dtype, max_tokens=512, decode_splits=4)
    plain = plain_models(name, dtype)
    seqs = prompts_for(name, [12, 12, 12], seed=5)
    slots = [eng.new_sequence() for _ in seqs]
    got = eng.step([(s, q[:n]) for s, q, n in zip(slots, seqs, (1, 2, 3))], "all").cpu().numpy()
    ref = [plain.logits(q) for q in seqs]
    want = np.concatenate([ref[0][:1], ref[1][:2], ref[2][:3]])
    ok, err, tol = close(got, want, dtype)
    assert ok, (err, tol)
    pos = [1, 2, 3]
    for _ in range(8):
        got = eng.step([(s, [q[p]]) for s, q, p in zip(slots, seqs, pos)]).cpu().numpy()
        for r in range(3):
            ok, err, tol = close(got[r], ref[r][pos[r]], dtype)
            assert ok, (r, pos[r], err, tol)
            pos[r] += 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_padding_rows_change_no_result(folders, dtype):
    """The same decode step with and without padding rows (negative slot) in the batch."""
    from quicknn_b200.engine.batch import StepBatch
    eng = build(folders("B", dtype), dtype, max_tokens=512, decode_splits=2)
    seqs = prompts_for("B", [30, 9])
    slots = [eng.new_sequence(), eng.new_sequence()]
    eng.step(list(zip(slots, seqs)))
    nxt = [11, 12]
    base = eng.step([(s, [t]) for s, t in zip(slots, nxt)]).cpu().numpy()
    # run the same step again by hand, with padding rows around the real ones: the cache already
    # holds these positions, the rewrite stores identical values
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)  # noqa: E731
    step = StepBatch("decode", 5, 5, i32([3, nxt[0], 4, nxt[1], 5]), i32([0, 30, 0, 9, 0]),
                     i32([-1, slots[0], -1, slots[1], -1]), i32([0, 1, 2, 3, 4]),
                     i32([-1, slots[0], -1, slots[1], -1]), i32([1, 3]), eng.model.dtype, max_seq=eng.max_seq,
                     tuning=eng.tuning)
    eng._give_scratch(step)
    again = eng.model.forward(step, eng.cache).cpu().numpy()
    assert np.array_equal(again, base)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("A", "bfloat16"), ("E", "bfloat16")])
def test_greedy_generation_through_the_entry_point(folders, plain_models, name, dtype):
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    plain = plain_models(name, dtype)
    llm = LLM(folders(name, dtype), max_context=128, max_batch=3, dtype=dtype)
    lens = [5, 11, 17] if name == "A" else [1, 6, 13, 29]
    prompts = prompts_for(name, lens)
    steps = 8 if name == "A" else 12
    streamed = {}
    res = llm.generate(prompts, GenerationOptions.greedy(steps), stop_ids=[],
                       on_token=lambda i, t: streamed.setdefault(i, []).append(t))
    for r, p in zip(res, prompts):
        assert r.finish_reason == "max_tokens" and r.generated_tokens == steps
        assert streamed[r.index] == r.tokens
        if dtype == "float32":
            assert r.tokens == plain.greedy(p, steps), f"request {r.index}"
        else:
            # bfloat16 may break a near-tie differently; every chosen token must be the plain model's
            # best or within the tolerance of it, given the same history
            seq = list(p)
            for t in r.tokens:
                row = plain.logits(seq)[-1]
                assert row[t] >= row.max() - 0.06 * max(1.0, np.abs(row).max()), (r.index, len(seq))
                seq.append(t)
    # stop tokens: the token that the plain model generates third ends request 0 after two tokens
    ref0 = plain.greedy(prompts[0], steps)
    if dtype == "float32" and ref0[2] not in ref0[:2]:
        res = llm.generate(prompts[:2], GenerationOptions.greedy(steps), stop_ids=[ref0[2]])
        assert res[0].tokens == ref0[:2] and res[0].finish_reason == "eos"
        ref1 = plain.greedy(prompts[1], steps, stop_ids=[ref0[2]])
        assert res[1].tokens == ref1
    assert llm.engine.cache.slots.live() == []
    llm.engine.cache.audit()
    assert np.abs(llm.evaluate_tokens(prompts[1]) - plain.logits(prompts[1])[-1]).max() < (1e-4 if dtype == "float32" else 0.1)


def test_stop_ids_of_generation_config_json_end_a_request(folders, plain_models, tmp_path):
    """A folder's generation_config.json adds its eos_token_id to the stop ids of config.json (LLM.pas:260-271)."""
    import json
    import shutil
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    plain = plain_models("A", "float32")
    prompt = prompts_for("A", [9], seed=3)[0]
    ref = plain.greedy(prompt, 8)
    stop = next(t for t in ref[2:] if t not in ref[:2])
    folder = tmp_path / "model"
    shutil.copytree(folders("A", "float32"), folder)
    (folder / "generation_config.json").write_text(json.dumps({"eos_token_id": [stop]}))
    llm = LLM(str(folder), max_context=64, max_batch=1, dtype="float32")
    assert stop in llm.stop_ids and set(llm.model.spec.stop_ids) <= set(llm.stop_ids)
    res = llm.generate([prompt], GenerationOptions.greedy(8))[0]
    assert res.finish_reason == "eos" and res.tokens == ref[:ref.index(stop)]


def test_warm_up_captures_the_graphs_that_generation_then_finds(folders, plain_models):
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    plain = plain_models("A", "float32")
    llm = LLM(folders("A", "float32"), max_context=64, max_batch=6, dtype="float32")
    opts = GenerationOptions.greedy(5)
    states = llm.warm_up(opts, context=40)
    assert states == 6 and sorted({k[0] for k in llm.engine._decode_state}) == [1, 2, 3, 4, 5, 6]
    assert llm.memory_status()["live_sequences"] == 0
    llm.engine.cache.audit()
    prompts = prompts_for("A", [30, 12, 33, 20], seed=4)
    res = llm.generate(prompts, opts, stop_ids=[])
    for r, p in zip(res, prompts):
        assert r.tokens == plain.greedy(p, 5)
    assert len(llm.engine._decode_state) == states                    # nothing new had to be captured
    assert llm.warm_up(opts, batch_sizes=[2, 3], context=40) == states


def test_more_requests_than_slots_reuse_them(folders, plain_models):
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    plain = plain_models("B", "float32")
    llm = LLM(folders("B", "float32"), max_context=64, max_batch=2, dtype="float32")
    prompts = prompts_for("B", [3, 20, 7, 1, 15], seed=9)
    res = llm.generate(prompts, GenerationOptions.greedy(6), stop_ids=[])
    for r, p in zip(res, prompts):
        assert r.tokens == plain.greedy(p, 6)
    assert llm.memory_status()["live_sequences"] == 0


def test_decode_graphs_are_kept_per_length_class_and_the_oldest_goes(folders, plain_models, monkeypatch):
    """A decode graph belongs to a batch size and to classes of the sequences' lengths (they decide the number of
    key ranges).  A batch that grows from 250 to 270 tokens changes class on the way, batches of other sizes and
    spreads bring more states than the engine keeps (2 here): generation goes on with the same tokens as the
    plain implementation, and graphs that were dropped are captured again when their class comes back."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.engine import engine as engine_module
    from quicknn_b200.sampling import GenerationOptions
    monkeypatch.setattr(engine_module, "MAX_DECODE_GRAPHS", 2)
    plain = plain_models("B", "float32")
    llm = LLM(folders("B", "float32"), max_context=300, max_batch=3, dtype="float32")
    for lens in ([250, 40, 3], [250, 245], [30], [250, 40, 3]):
        prompts = prompts_for("B", lens, seed=sum(lens))
        res = llm.generate(prompts, GenerationOptions.greedy(20), stop_ids=[])
        for r, p in zip(res, prompts):
            assert r.tokens == plain.greedy(p, 20)
        assert len(llm.engine._decode_state) <= 2
    assert llm.memory_status()["live_sequences"] == 0


@pytest.mark.parametrize("name,dtype,ahead", [("A", "float32", True), ("B", "float32", False), ("A", "bfloat16", True)])
def test_a_conversation_reuses_the_common_prefix(folders, plain_models, name, dtype, ahead):
    """Successive prompts through one ``Conversation``: a next turn (old prompt + reply + new text) runs only the new
    tokens; a prompt that departs a little way back shortens the cache; one that departs further back than the ring
    of the windowed layers still has, or at once, starts over; a repeated prompt recomputes its last token.  Every
    reply is what the plain implementation generates for the whole prompt."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    plain = plain_models(name, dtype)
    llm = LLM(folders(name, dtype), max_context=400, max_batch=2, dtype=dtype)
    llm.run_ahead = ahead
    window = TINY[name][0]["sliding_window"]
    greedy = GenerationOptions.greedy(6)

    def same(res, prompt, n=6):
        if dtype == "float32":
            assert res.tokens == plain.greedy(prompt, n)
            return
        seq = list(prompt)                        # bfloat16: a near tie may fall the other way
        for t in res.tokens:
            row = plain.logits(seq)[-1]
            assert row[t] >= row.max() - 0.06 * max(1.0, np.abs(row).max()), len(seq)
            seq.append(t)

    with llm.conversation() as conv:
        p1 = prompts_for(name, [20], seed=5)[0]
        r1 = conv.generate(p1, greedy, stop_ids=[])
        assert r1.reused_tokens == 0
        same(r1, p1)
        # the next turn
        p2 = p1 + r1.tokens + prompts_for(name, [5], seed=6)[0]
        r2 = conv.generate(p2, greedy, stop_ids=[])
        assert r2.reused_tokens in (len(p1) + 5, len(p1) + 6)           # the last reply token was fed only by a step ahead
        same(r2, p2)
        # the same prompt again: everything but its last token is there
        r2b = conv.generate(p2, greedy, stop_ids=[])
        assert r2b.reused_tokens == len(p2) - 1 and r2b.tokens == r2.tokens
        # departs 4 tokens back: the ring (64 positions) still holds what the window needs
        p3 = p2[:-4] + prompts_for(name, [7], seed=7)[0]
        r3 = conv.generate(p3, greedy, stop_ids=[])
        assert r3.reused_tokens == len(p2) - 4
        same(r3, p3)
        # a long turn, so that the rings have wrapped; then a prompt that departs further back than they reach
        p4 = p3 + r3.tokens[:5] + prompts_for(name, [150], seed=8)[0]
        r4 = conv.generate(p4, greedy, stop_ids=[])
        assert r4.reused_tokens >= len(p3)
        same(r4, p4)
        back = 64 - window + 10
        p5 = p4[:-back] + prompts_for(name, [3], seed=9)[0]
        r5 = conv.generate(p5, greedy, stop_ids=[])
        assert r5.reused_tokens == 0
        same(r5, p5)
        # within reach of the rings: kept
        p6 = p5[:-3] + prompts_for(name, [2], seed=10)[0]
        r6 = conv.generate(p6, greedy, stop_ids=[])
        assert r6.reused_tokens == len(p5) - 3
        same(r6, p6)
        # a reply continued after it stopped is the reply that never stopped
        r6b = conv.continue_generation(greedy, stop_ids=[])
        assert r6b.reused_tokens == len(p6) + len(r6.tokens) - 1
        same(r6b, p6 + r6.tokens)
        if dtype == "float32":
            assert r6.tokens + r6b.tokens == plain.greedy(p6, 12)
        # an unrelated prompt starts over; and a batch beside the conversation leaves it alone
        p7 = prompts_for(name, [9], seed=11)[0]
        others = llm.generate([p1], greedy, stop_ids=[])
        same(others[0], p1)
        r7 = conv.generate(p7, greedy, stop_ids=[])
        assert r7.reused_tokens == 0
        same(r7, p7)
        assert llm.memory_status()["live_sequences"] == 1
    assert llm.memory_status()["live_sequences"] == 0


@pytest.mark.parametrize("name,dtype,seed", [("A", "float32", 1), ("B", "float32", 2), ("C", "bfloat16", 3),
                                             ("D", "bfloat16", 4), ("A", "float32", 5)])
def test_random_schedules_of_steps_give_the_plain_logits(folders, plain_models, name, dtype, seed):
    """Sequences of random lengths fed in random portions: in every step a random subset of the live sequences goes
    on by a random number of tokens (one token each, several, whole prompts of sequences that start, all mixed),
    logits are wanted at random places, finished sequences give their slots and pages back and new ones take
    them.  Every logit equals the plain model's for the whole sequence, whatever the cutting and the company."""
    rng = np.random.default_rng(seed)
    plain = plain_models(name, dtype)
    eng = build(folders(name, dtype), dtype, max_tokens=64 * 16, max_slots=5, max_seq=200)
    todo = [rng.integers(1, TINY[name][0]["vocab_size"], int(n)).tolist() for n in rng.integers(1, 190, 14)]
    ref = {}
    live = {}                                          # slot -> [tokens, fed]
    steps = checked = 0
    modes = set()
    while todo or live:
        while todo and len(live) < 5 and (not live or rng.random() < 0.5):
            live[eng.new_sequence()] = [todo.pop(), 0]
        chosen = [s for s in live if rng.random() < 0.7] or [next(iter(live))]
        kind = rng.integers(0, 3)
        entries, want = [], []
        for s in chosen:
            toks, fed = live[s]
            n = 1 if kind == 0 else int(rng.integers(1, 1 + min(len(toks) - fed, 3 if kind == 1 else 80)))
            entries.append((s, toks[fed:fed + n]))
            want.append(sorted(set(rng.integers(0, n, int(rng.integers(0, 3))).tolist())))
        starts = [live[s][1] for s in chosen]
        modes.add("prefill" if all(p == 0 for p in starts) else ("decode" if all(len(t) == 1 for _, t in entries) else "extend"))
        logits = eng.step(entries, want).cpu().numpy()
        row = 0
        for (s, t), w in zip(entries, want):
            toks, fed = live[s]
            if id(toks) not in ref:
                ref[id(toks)] = plain.logits(toks)
            for place in w:
                ok, err, tol = close(logits[row], ref[id(toks)][fed + place], dtype)
                assert ok, f"step {steps}, place {fed + place} of {len(toks)}: error {err:.3g} above {tol:.3g}"
                row += 1
                checked += 1
            live[s][1] = fed + len(t)
            if live[s][1] == len(toks):
                eng.release(s)
                del live[s]
        assert row == logits.shape[0]
        if steps % 7 == 0:
            eng.cache.verify_device()              # the page tables and lengths on the device are the host's
        steps += 1
    assert modes == {"prefill", "decode", "extend"} and checked > 50 and steps > 30
    assert eng.cache.slots.live() == []
    eng.cache.audit()


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("D", "bfloat16")])
def test_padded_decode_steps_give_the_sequences_rows(folders, name, dtype):
    """``Engine.decode(..., pad=True)`` runs 9 sequences as 10 rows and 13 as 14 (rows of no sequence at the end);
    the logits of the sequences' rows are those of the unpadded step, and the cache holds what it would."""
    eng_a = build(folders(name, dtype), dtype, max_tokens=64 * 24, max_slots=16, max_seq=64)
    eng_b = build(folders(name, dtype), dtype, max_tokens=64 * 24, max_slots=16, max_seq=64)
    assert [eng_a.decode_rows(n) for n in (1, 7, 8, 9, 10, 13, 15, 16)] == [1, 7, 8, 10, 10, 14, 16, 16]
    for n in (9, 13):
        prompts = prompts_for(name, [3 + (5 * i) % 11 for i in range(n)], seed=n)
        slots_a = [eng_a.new_sequence() for _ in prompts]
        slots_b = [eng_b.new_sequence() for _ in prompts]
        eng_a.step(list(zip(slots_a, prompts)), "last")
        eng_b.step(list(zip(slots_b, prompts)), "last")
        tok = torch.tensor([p[0] for p in prompts], dtype=torch.int32, device=DEV)
        for t in range(4):
            la = eng_a.decode(slots_a, tok, pad=True)
            lb = eng_b.decode(slots_b, tok)
            assert la.shape == lb.shape == (n, TINY[name][0]["vocab_size"])
            ok, err, tol = close(la.cpu().numpy(), lb.cpu().numpy(), dtype)
            assert ok, f"{n} sequences, token {t}: error {err:.3g} above {tol:.3g}"
            tok = lb.argmax(dim=-1).to(torch.int32)
        assert [eng_a.length(s) for s in slots_a] == [eng_b.length(s) for s in slots_b]
        for s in slots_a:
            eng_a.release(s)
        for s in slots_b:
            eng_b.release(s)
    assert sorted({k[0] for k in eng_a._decode_state}) == [10, 14] and sorted({k[0] for k in eng_b._decode_state}) == [9, 13]


def test_running_one_step_ahead_changes_no_token(folders, plain_models):
    """The entry point queues each decode step before it reads the ids of the one before; rows
    that end (stop token, budget, full context) are dropped a step late and their extra token is
    thrown away.  Same tokens, same finish reasons, no slot or page lost, with and without."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    plain = plain_models("B", "float32")
    llm = LLM(folders("B", "float32"), max_context=40, max_batch=3, dtype="float32")
    prompts = prompts_for("B", [3, 30, 9, 1, 22], seed=4)         # 30 and 22 run into the context of 40
    ref = [plain.greedy(p, 14) for p in prompts]
    stop = [ref[2][4]]                                            # request 2 ends early; others may too
    runs = {}
    for ahead in (True, False):
        llm.run_ahead = ahead
        out = llm.generate(prompts, GenerationOptions.greedy(14), stop_ids=stop)
        runs[ahead] = [(r.tokens, r.finish_reason) for r in out]
        assert llm.engine.cache.slots.live() == []
        llm.engine.cache.audit()
        assert llm.last_io["decode_steps"] > 0
    assert runs[True] == runs[False]
    for (toks, why), p, full in zip(runs[True], prompts, ref):
        want = plain.greedy(p, min(14, 40 - len(p)), stop_ids=stop)
        assert toks == want, (len(p), why)
    assert runs[True][1][1] == "context_full" and runs[True][2][1] == "eos"
    # sampling with a repetition penalty: the generator and the table of seen ids advance alike
    opt = GenerationOptions(max_new_tokens=10, temperature=0.9, top_k=8, repetition_penalty=1.3, seed=7)
    llm.run_ahead = True
    a = [r.tokens for r in llm.generate(prompts, opt, stop_ids=stop)]
    llm.run_ahead = False
    b = [r.tokens for r in llm.generate(prompts, opt, stop_ids=stop)]
    assert a == b


def test_temperature_sampling_is_seeded_and_follows_the_plain_sampler(folders, plain_models):
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    llm = LLM(folders("B", "float32"), max_context=64, max_batch=4, dtype="float32")
    prompts = prompts_for("B", [1, 6, 13, 29])
    opt = GenerationOptions(max_new_tokens=12, temperature=0.8, seed=1234)
    a = llm.generate(prompts, opt, stop_ids=[])
    b = llm.generate(prompts, opt, stop_ids=[])
    assert [r.tokens for r in a] == [r.tokens for r in b]
    c = llm.generate(prompts, GenerationOptions(max_new_tokens=12, temperature=0.8, seed=99), stop_ids=[])
    assert [r.tokens for r in a] != [r.tokens for r in c]
    # the same draws with the plain model and the plain sampler: request i uses seed + i
    plain = plain_models("B", "float32")
    for i, (r, p) in enumerate(zip(a, prompts)):
        st = P.seed_state(1234 + i)
        seq = list(p)
        for t in r.tokens:
            st, u = P.xorshift32(st)
            row = plain.logits(seq)[-1]
            info = {}
            ref = P.sample(row.astype(np.float32), 0.8, 20, 0.95, 1.0, None, u, info)
            if ref != t:
                # the engine's float32 logits differ from the float64 ones by rounding; only a draw that
                # falls within that distance of the boundary between two candidates may land on the neighbour
                assert info["margin"] < 1e-4, (i, len(seq), ref, t, info["margin"])
            seq.append(t)
    # repetition penalty and top-k 1 run and stay reproducible
    o2 = GenerationOptions(max_new_tokens=8, temperature=1.0, top_k=5, repetition_penalty=1.5, seed=3)
    d1 = llm.generate(prompts[:2], o2, stop_ids=[])
    d2 = llm.generate(prompts[:2], o2, stop_ids=[])
    assert [r.tokens for r in d1] == [r.tokens for r in d2]


def test_step_rules_and_loud_failures(folders):
    from quicknn_b200.cache import CacheFull
    from quicknn_b200.engine import StepError
    eng = build(folders("A", "float32"), "float32", max_tokens=128)
    a, b = eng.new_sequence(), eng.new_sequence()
    eng.step([(a, [5, 6, 7])])
    with pytest.raises(StepError):
        eng.step([(a, [8]), (a, [9])])              # a sequence twice in one step
    with pytest.raises(StepError):
        eng.step([(a, [])])                         # nothing to run
    with pytest.raises(StepError):
        eng.step([(b, [600])])                      # outside the vocabulary
    with pytest.raises(StepError):
        eng.step([(b, [5])], want=[[1]])            # a wanted place that the step does not bring
    with pytest.raises(CacheFull):
        eng.step([(b, list(range(1, 100)))])        # 64 (held by a) + 128 > 128 tokens
    assert eng.length(a) == 3 and eng.length(b) == 0
    eng.cache.audit()
    with pytest.raises(Exception):
        from quicknn_b200.engine import Model
        Model.from_folder(folders("A", "float32"), "float32", "cpu").forward(None, None)


def test_many_option_sets_do_not_pile_up_graphs(folders):
    """Every distinct option set gets a sampler and decode graphs of its own; the entry point keeps a
    handful and lets the engine drop the graphs of those it forgets."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions
    llm = LLM(folders("A", "bfloat16"), max_context=64, max_batch=2, dtype="bfloat16")
    prompts = prompts_for("A", [4, 7])
    first = None
    for seed in range(8):
        out = llm.generate(prompts, GenerationOptions(max_new_tokens=4, temperature=0.7, seed=seed), stop_ids=[])
        first = first or [r.tokens for r in out]
        assert len(llm._samplers) <= 5
        assert len({k[1] for k in llm.engine._decode_state}) <= 5
    again = llm.generate(prompts, GenerationOptions(max_new_tokens=4, temperature=0.7, seed=0), stop_ids=[])
    assert [r.tokens for r in again] == first
    assert len(llm._samplers) == 1                      # calls that differ in the seed alone share a sampler and its graphs
    for k in (3, 5, 7, 9, 11, 13):
        llm.generate(prompts, GenerationOptions(max_new_tokens=2, temperature=0.7, top_k=k), stop_ids=[])
        assert len(llm._samplers) <= 5 and len({key[1] for key in llm.engine._decode_state}) <= 5
    for k in (3, 5, 7):                                 # greedy is greedy whatever top_k says
        llm.generate(prompts, GenerationOptions(max_new_tokens=2, temperature=0.0, top_k=k), stop_ids=[])
    assert sum(1 for key in llm._samplers if key[0] == "greedy") == 1
    assert llm.engine.cache.slots.live() == []


def test_non_finite_logits_raise_after_every_forward(folders):
    """NaN planted in the embedding table (which is the head as well, so every forward meets it): a
    prompt, a single token, evaluate_tokens, generate and a decode step without a sampler all raise;
    with the value put back everything runs again."""
    from quicknn_b200.engine import LLM, NonFiniteLogits
    from quicknn_b200.sampling import GenerationOptions
    llm = LLM(folders("A", "float32"), max_context=64, max_batch=2, dtype="float32")
    eng = llm.engine
    a = eng.new_sequence()
    eng.step([(a, [5, 6, 7])])
    good = float(llm.model.embedding[77, 3])
    llm.model.embedding[77, 3] = float("nan")
    with pytest.raises(NonFiniteLogits):
        eng.step([(a, [8])])
    with pytest.raises(NonFiniteLogits):
        eng.step([(a, [9, 4])], "all")
    eng.decode([a], torch.tensor([8], dtype=torch.int32, device=DEV))      # no sampler: the caller asks
    with pytest.raises(NonFiniteLogits):
        eng.check()
    eng.check()                                                            # the word was cleared
    eng.release(a)
    b = eng.new_sequence()
    with pytest.raises(NonFiniteLogits):
        eng.step([(b, [9, 77, 4])], "all")
    eng.release(b)
    with pytest.raises(NonFiniteLogits):
        llm.evaluate_tokens([5, 6])
    with pytest.raises(NonFiniteLogits):
        llm.generate([[5, 6], [8, 9]], GenerationOptions.greedy(4), stop_ids=[])
    with pytest.raises(NonFiniteLogits):
        llm.generate([[5, 6]], GenerationOptions(max_new_tokens=4, temperature=0.7, seed=1), stop_ids=[])
    assert eng.cache.slots.live() == []
    llm.model.embedding[77, 3] = good
    assert np.isfinite(llm.evaluate_tokens([5, 6])).all()
    out = llm.generate([[5, 6]], GenerationOptions.greedy(4), stop_ids=[])
    assert len(out[0].tokens) == 4


def test_a_wait_that_ran_out_is_seen_in_decode_too(folders):
    """The status word of the bounded waits, set here from the host (no kernel is made to hang): the
    next decode step of a generation raises, through the error word that comes back with the ids."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.kernels import ops
    from quicknn_b200.kernels.lib import KernelError
    from quicknn_b200.sampling import GenerationOptions
    llm = LLM(folders("A", "bfloat16"), max_context=64, max_batch=2, dtype="bfloat16")
    seen = []

    def on_token(i, tok):
        seen.append(tok)
        if len(seen) == 3:
            ops.status_words(DEV)[0:1].fill_(4)
    with pytest.raises(KernelError, match="gave up waiting"):
        llm.generate([[5, 6, 7]], GenerationOptions.greedy(20), on_token=on_token, stop_ids=[])
    assert len(seen) < 8 and llm.engine.cache.slots.live() == []
    assert ops.status_words(DEV).tolist() == [0, 0]
    out = llm.generate([[5, 6, 7]], GenerationOptions.greedy(5), stop_ids=[])
    assert len(out[0].tokens) == 5
    ops.status_words(DEV)[0:1].fill_(2)             # and behind a prompt
    s = llm.engine.new_sequence()
    with pytest.raises(KernelError):
        llm.engine.step([(s, [5, 6])])
    llm.engine.release(s)


def test_a_step_that_cannot_be_launched_leaves_the_cache_as_it_was(folders, monkeypatch):
    from quicknn_b200.kernels.lib import KernelError
    eng = build(folders("A", "float32"), "float32", max_tokens=256)
    a, b = eng.new_sequence(), eng.new_sequence()
    eng.step([(a, list(range(1, 70))), (b, [3, 4])])
    held = eng.cache.tokens_held()

    def broken(step, cache):
        raise KernelError("refused")
    good = eng.model.forward
    monkeypatch.setattr(eng.model, "forward", broken)
    c = eng.new_sequence()
    with pytest.raises(KernelError):
        eng.step([(c, list(range(1, 31)))])
    with pytest.raises(KernelError):
        eng.step([(a, [5]), (b, [6])])
    with pytest.raises(KernelError):
        eng.decode([a, b], torch.tensor([5, 6], dtype=torch.int32, device=DEV), use_graph=False)
    assert (eng.length(a), eng.length(b), eng.length(c)) == (69, 2, 0) and eng.cache.tokens_held() == held
    eng.cache.audit()
    monkeypatch.setattr(eng.model, "forward", good)
    eng.step([(a, [5]), (b, [6])])
    assert (eng.length(a), eng.length(b)) == (70, 3)
    eng.cache.audit()


def test_greedy_ids_without_logits_are_those_with_logits(folders, monkeypatch):
    """bfloat16 greedy generation takes its ids from the head product's arg-max epilogue; with that
    switched off (logits written, then the sampler's two kernels) the same ids come out."""
    from quicknn_b200.engine import LLM
    from quicknn_b200.sampling import GenerationOptions, Sampler
    prompts = prompts_for("C", [40, 3, 77, 9, 120], seed=8)
    llm = LLM(folders("C", "bfloat16"), max_context=160, max_batch=5, dtype="bfloat16")
    used = []
    real = Sampler.head

    def spy(self, hidden, weight, cap):
        out = real(self, hidden, weight, cap)
        used.append(out is not None)
        return out
    monkeypatch.setattr(Sampler, "head", spy)
    fused = [r.tokens for r in llm.generate(prompts, GenerationOptions.greedy(24), stop_ids=[])]
    assert used and all(used)
    monkeypatch.setattr(Sampler, "head", lambda self, hidden, weight, cap: None)
    llm2 = LLM(model=llm.model, max_context=160, max_batch=5, dtype="bfloat16")
    plain = [r.tokens for r in llm2.generate(prompts, GenerationOptions.greedy(24), stop_ids=[])]
    assert fused == plain
    monkeypatch.setattr(Sampler, "head", spy)
    del used[:]
    llm.generate(prompts[:2], GenerationOptions(max_new_tokens=4, temperature=0.5, seed=1), stop_ids=[])
    llm.generate(prompts[:2], GenerationOptions(max_new_tokens=4, temperature=0.0, repetition_penalty=1.2), stop_ids=[])
    assert used and not any(used)            # sampling and penalties need the logits


def test_the_profile_table_accounts_for_every_step_and_puts_everything_back(folders):
    from quicknn_b200.engine import LLM, StepProfiler
    from quicknn_b200.parts.norm import RMSNorm
    from quicknn_b200.sampling import GenerationOptions
    llm = LLM(folders("C", "bfloat16"), max_context=64, max_batch=2, dtype="bfloat16")
    prompts = prompts_for("C", [20, 7])
    opts = GenerationOptions.greedy(6)
    before = [r.tokens for r in llm.generate(prompts, opts, stop_ids=[])]
    norm_call = RMSNorm.__call__
    with StepProfiler(llm.engine) as prof:
        during = [r.tokens for r in llm.generate(prompts, opts, stop_ids=[])]
    assert during == before and llm.engine.use_graphs and RMSNorm.__call__ is norm_call
    assert "forward" not in vars(llm.model.blocks[0].mixer) and "step" not in vars(llm.engine)
    steps = prof.steps()
    assert steps["prompt"][:2] == (1, 27) and steps["decode"][0] >= 5 and steps["decode"][1] == 2 * steps["decode"][0]
    kinds = prof.by_kind()
    assert all(kinds[k] > 0 for k in ("embedding", "norms and residual", "mixer", "feed-forward", "head", "sampling"))
    inside = sum(kinds.values())
    outside = sum(ms for _, _, ms in steps.values())
    assert 0 < inside <= outside * 1.05                        # the parts' time lies inside the steps' (whose events also span the host's gaps)
    table = prof.table()
    assert "feed-forward" in table and "tokens/s" in table
    assert [r.tokens for r in llm.generate(prompts, opts, stop_ids=[])] == before
    with StepProfiler(llm.engine, nvtx=True) as prof2:           # NVTX ranges around the same calls change nothing
        assert [r.tokens for r in llm.generate(prompts, opts, stop_ids=[])] == before
    assert prof2.by_kind()["mixer"] > 0

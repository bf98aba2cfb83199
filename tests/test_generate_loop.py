"""Decisions of the generation loop, with a backend that needs no GPU."""
import numpy as np
import pytest

from quicknn_b200.engine.generate import (CANCELLED, CONTEXT_FULL, EOS, HARD_LIMIT, MAX_TOKENS, GenerationBackend,
                                          PromptError, generate, plan_batches)
from quicknn_b200.sampling import GenerationOptions, OptionsError, seed_state


class Script(GenerationBackend):
    """Request i emits the tokens of script[i] one after another."""

    def __init__(self, script, max_batch=4, max_tokens=4096, max_seq=512, vocab_size=100):
        self.script, self.max_batch, self.max_tokens = script, max_batch, max_tokens
        self.max_seq, self.vocab_size = max_seq, vocab_size
        self.log, self.rows, self.pos, self.open = [], [], {}, False

    def _next(self):
        out = []
        for i in self.rows:
            k = self.pos.get(i, 0)
            self.pos[i] = k + 1
            out.append(self.script[i][min(k, len(self.script[i]) - 1)])
        return np.asarray(out)

    def begin(self, first_index, prompts):
        assert not self.open
        self.open = True
        self.rows = list(range(first_index, first_index + len(prompts)))
        self.log.append(("begin", list(self.rows)))
        return self._next()

    def advance(self, keep_rows):
        self.rows = [self.rows[r] for r in keep_rows]
        self.log.append(("advance", list(self.rows)))
        return self._next()

    def finish(self):
        self.open = False
        self.log.append(("finish",))


def test_options_follow_the_reference():
    o = GenerationOptions()
    assert (o.max_new_tokens, o.hard_max_new_tokens, o.top_k, o.temperature, o.top_p, o.repetition_penalty,
            o.seed, o.auto_continue) == (256, 4096, 20, 0.6, 0.95, 1.0, 42, False)
    o.validate()
    for bad in (dict(max_new_tokens=0), dict(top_k=0), dict(top_k=65), dict(temperature=-1.0),
                dict(temperature=float("nan")), dict(top_p=0.0), dict(top_p=1.5), dict(repetition_penalty=0.0),
                dict(auto_continue=True, hard_max_new_tokens=10, max_new_tokens=20), dict(enable_thinking=True)):
        with pytest.raises(OptionsError):
            GenerationOptions(**bad).validate()
    assert seed_state(42) == 42 and seed_state(0) == 0x9E3779B9 and seed_state((7 << 32) | 7) == 0x9E3779B9
    assert seed_state(42, 3) == 45


def test_stop_tokens_and_early_finishers():
    b = Script({0: [5, 6, 9], 1: [9], 2: [5, 5, 5, 5, 5, 5, 9]})
    res = generate(b, [[1, 2], [3], [4, 5, 6]], GenerationOptions.greedy(5), stop_ids=[9])
    assert [r.tokens for r in res] == [[5, 6], [], [5, 5, 5, 5, 5]]
    assert [r.finish_reason for r in res] == [EOS, EOS, MAX_TOKENS]
    # request 1 left after the first step, request 0 after the third; the last sampled token is never fed
    assert b.log == [("begin", [0, 1, 2]), ("advance", [0, 2]), ("advance", [0, 2]), ("advance", [2]),
                     ("advance", [2]), ("finish",)]
    assert res[2].prompt_tokens == 3 and res[2].generated_tokens == 5


def test_batches_one_after_another():
    b = Script({i: [5, 9] for i in range(5)}, max_batch=2)
    res = generate(b, [[1]] * 5, GenerationOptions.greedy(4), stop_ids=[9])
    begins = [e[1] for e in b.log if e[0] == "begin"]
    assert begins == [[0, 1], [2, 3], [4]]
    assert sum(1 for e in b.log if e[0] == "finish") == 3
    assert all(r.tokens == [5] and r.finish_reason == EOS for r in res)


def test_plan_respects_the_token_budget():
    o = GenerationOptions.greedy(16)
    assert plan_batches([10, 10, 10], o, max_batch=8, max_tokens=128, max_seq=512) == [[0, 1], [2]]
    assert plan_batches([120, 10], o, max_batch=8, max_tokens=192, max_seq=512) == [[0], [1]]
    with pytest.raises(PromptError):
        plan_batches([600], o, 8, 4096, 512)       # the prompt fills the context
    with pytest.raises(PromptError):
        plan_batches([0], o, 8, 4096, 512)
    with pytest.raises(PromptError):
        plan_batches([300], o, 8, 256, 512)        # does not fit the cache at all


def test_context_full_and_hard_limit():
    b = Script({0: [5] * 100}, max_seq=20)
    res = generate(b, [[1] * 15], GenerationOptions.greedy(50), stop_ids=[])
    assert res[0].finish_reason == CONTEXT_FULL and res[0].generated_tokens == 5
    b = Script({0: [5] * 100})
    res = generate(b, [[1]], GenerationOptions(max_new_tokens=3, hard_max_new_tokens=7, auto_continue=True,
                                               temperature=0.0), stop_ids=[])
    assert res[0].finish_reason == HARD_LIMIT and res[0].generated_tokens == 7


def test_cancel_from_the_callback_and_from_the_probe():
    b = Script({0: [5] * 100, 1: [6] * 100})
    seen = []

    def on_token(i, t):
        seen.append((i, t))
        return len(seen) >= 3

    res = generate(b, [[1], [2]], GenerationOptions.greedy(50), on_token=on_token)
    assert [r.finish_reason for r in res] == [CANCELLED, CANCELLED]
    assert seen[:2] == [(0, 5), (1, 6)] and not b.open
    b = Script({0: [5] * 100}, max_batch=1)
    calls = []
    res = generate(b, [[1], [2]], GenerationOptions.greedy(50),
                   should_cancel=lambda: (calls.append(1) or len(calls) > 3))
    assert res[0].finish_reason == CANCELLED and res[1].finish_reason == CANCELLED and res[1].tokens == []


def test_out_of_vocabulary_prompt():
    with pytest.raises(PromptError):
        generate(Script({0: [1]}), [[1, 100]], GenerationOptions.greedy(2))


def test_backend_is_released_on_errors():
    class Boom(Script):
        def advance(self, keep_rows):
            raise RuntimeError("boom")
    b = Boom({0: [5] * 10})
    with pytest.raises(RuntimeError):
        generate(b, [[1]], GenerationOptions.greedy(5))
    assert not b.open

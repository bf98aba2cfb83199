"""The generation loop: batches of unequal prompts, stop tokens, early finishers, and as
many batches one after another as there are requests.

Per sequence the order is the reference's (``TQNNLLM.Decode``,
src/models/QuickNN.Models.LLM.pas:796-834): sample from the current logits; a stop token
ends the sequence and is not emitted; otherwise the token is emitted and becomes the
pending input of the next step; the last sampled token is never fed.  The budget is
``min(Budget, Capacity - Position)`` (:790-795) and the finish reasons are those of
``TLLMFinishReason`` (src/models/QuickNN.Models.LLM.Types.pas:77).  What the reference
does for one sequence is done here for every sequence of a batch; a sequence that ends
leaves the batch and gives its slot back at once.

The loop is host logic over a small backend interface, so its decisions can be tested
without a GPU.
"""
from __future__ import annotations

import dataclasses
import time
from typing import Callable, List, Optional, Sequence

import numpy as np

from ..sampling.options import GenerationOptions

from ..cache.pages import PAGE

EOS, MAX_TOKENS, CANCELLED, CONTEXT_FULL, HARD_LIMIT = "eos", "max_tokens", "cancelled", "context_full", "hard_limit"


class PromptError(ValueError):
    pass


@dataclasses.dataclass
class GenerationResult:
    """``TLLMGenerationResult`` (LLM.Types.pas:91-98) without the text fields."""

    index: int
    prompt_tokens: int
    tokens: List[int] = dataclasses.field(default_factory=list)
    finish_reason: str = CANCELLED
    time_to_first_token_seconds: float = 0.0
    decode_seconds: float = 0.0
    total_seconds: float = 0.0
    reused_tokens: int = 0          # tokens of the prompt that a conversation found in its cache (ReusedTokens)

    @property
    def generated_tokens(self) -> int:
        return len(self.tokens)

    def decode_tokens_per_second(self) -> float:
        """(generated - 1) / decode seconds (LLM.Types.pas:129-135)."""
        if self.generated_tokens > 1 and self.decode_seconds > 0:
            return (self.generated_tokens - 1) / self.decode_seconds
        return 0.0


class GenerationBackend:
    """What the loop needs from the engine."""

    max_batch: int
    max_tokens: int
    max_seq: int
    vocab_size: int

    def begin(self, first_index: int, prompts: Sequence[Sequence[int]]) -> np.ndarray:
        """Take a slot per prompt, run all prompts in one step, sample; returns one id per prompt."""
        raise NotImplementedError

    def advance(self, keep_rows: Sequence[int]) -> np.ndarray:
        """Release the rows that are not kept; feed each kept row its last sampled id, one
        step, sample; returns one id per kept row, in order."""
        raise NotImplementedError

    def finish(self) -> None:
        """Release whatever the batch still holds."""
        raise NotImplementedError


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


def token_limit(prompt_len: int, options: GenerationOptions, max_seq: int) -> int:
    """New tokens this request may get: min(budget, capacity - position)."""
    return min(options.budget(), max_seq - prompt_len)


def plan_batches(prompt_lens: Sequence[int], options: GenerationOptions, max_batch: int, max_tokens: int,
                 max_seq: int) -> List[List[int]]:
    """Cut the requests, in order, into batches that fit the cache at their largest.

    A request holds at most ``prompt + limit`` tokens, rounded up to a page.  A prompt must
    have at least one token and leave room for one more ("Chat prompt fills context",
    LLM.pas:963-964)."""
    batches: List[List[int]] = []
    cur: List[int] = []
    held = 0
    for i, n in enumerate(prompt_lens):
        if n < 1:
            raise PromptError(f"request {i}: an empty prompt")
        if n >= max_seq:
            raise PromptError(f"request {i}: the prompt of {n} tokens fills the context of {max_seq}")
        need = _round_up(n + token_limit(n, options, max_seq), PAGE)
        if need > max_tokens:
            raise PromptError(f"request {i}: {need} tokens do not fit a cache of {max_tokens}")
        if cur and (len(cur) >= max_batch or held + need > max_tokens):
            batches.append(cur)
            cur, held = [], 0
        cur.append(i)
        held += need
    if cur:
        batches.append(cur)
    return batches


TokenCallback = Callable[[int, int], Optional[bool]]


def generate(backend: GenerationBackend, prompts: Sequence[Sequence[int]], options: GenerationOptions,
             stop_ids: Sequence[int] = (), on_token: Optional[TokenCallback] = None,
             should_cancel: Optional[Callable[[], bool]] = None) -> List[GenerationResult]:
    """Generate for every prompt.  ``on_token(request index, token id)`` is called for each
    emitted token in step order and may return True to cancel everything;
    ``should_cancel()`` is probed before every step (the reference probes its callback
    with an empty text, LLM.pas:798-801)."""
    options.validate()
    stop = set(int(s) for s in stop_ids)
    for i, p in enumerate(prompts):
        a = np.asarray(p, dtype=np.int64).reshape(-1)
        if a.size and (int(a.min()) < 0 or int(a.max()) >= backend.vocab_size):
            bad = a[(a < 0) | (a >= backend.vocab_size)][0]
            raise PromptError(f"request {i}: token id {int(bad)} is outside the vocabulary")
    lens = [len(p) for p in prompts]
    batches = plan_batches(lens, options, backend.max_batch, backend.max_tokens, backend.max_seq)
    results = [GenerationResult(i, lens[i]) for i in range(len(prompts))]
    cancelled = False

    for batch in batches:
        if cancelled:
            break
        t0 = time.perf_counter()
        limits = [token_limit(lens[i], options, backend.max_seq) for i in batch]
        live = list(range(len(batch)))           # rows of the current step -> position in `batch`
        first_at = [0.0] * len(batch)
        last_at = [0.0] * len(batch)
        try:
            if should_cancel is not None and should_cancel():
                cancelled = True
                break
            sampled = backend.begin(batch[0], [prompts[i] for i in batch])
            while True:
                now = time.perf_counter()
                keep_rows: List[int] = []
                next_live: List[int] = []
                for row, b in enumerate(live):
                    res = results[batch[b]]
                    tok = int(sampled[row])
                    if tok in stop:
                        res.finish_reason = EOS
                        continue
                    res.tokens.append(tok)
                    if not first_at[b]:
                        first_at[b] = now
                    last_at[b] = now
                    if on_token is not None and on_token(batch[b], tok):
                        cancelled = True
                    if len(res.tokens) >= limits[b]:
                        if backend.max_seq - lens[batch[b]] <= options.budget():
                            res.finish_reason = CONTEXT_FULL     # Available <= Budget (LLM.pas:840-841)
                        elif options.auto_continue:
                            res.finish_reason = HARD_LIMIT
                        else:
                            res.finish_reason = MAX_TOKENS
                        continue
                    keep_rows.append(row)
                    next_live.append(b)
                if should_cancel is not None and should_cancel():
                    cancelled = True
                if cancelled:
                    for b in next_live:
                        results[batch[b]].finish_reason = CANCELLED
                    break
                if not keep_rows:
                    break
                sampled = backend.advance(keep_rows)
                live = next_live
        finally:
            backend.finish()
        end = time.perf_counter()
        for b, i in enumerate(batch):
            r = results[i]
            r.total_seconds = end - t0
            if first_at[b]:
                r.time_to_first_token_seconds = first_at[b] - t0
            if r.generated_tokens > 1:
                r.decode_seconds = last_at[b] - first_at[b]
    return results

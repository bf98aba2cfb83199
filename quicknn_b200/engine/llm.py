"""The Python entry point, in the manner of the reference's ``TQNNLLM``
(src/models/QuickNN.Models.LLM.pas:55-77): ``Create(ModelDir, ..., MaxContext)``,
``Generate(..., Options, OnToken)``, ``EvaluateTokens(Ids)``, ``ResetContext``,
``MemoryStatus``.  The interface is token ids; there is no tokenizer.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import numpy as np
import torch

from ..config.base import Architecture, ModelConfig, find_architecture
from ..config.generation import stop_ids_of_folder
from ..cache.pages import PAGE, CacheFull
from ..sampling import GenerationOptions, Sampler
from ..weights.random_init import random_tensors
from .engine import Engine
from .generate import GenerationBackend, GenerationResult, generate
from .model import Model, as_dtype

class _Backend(GenerationBackend):
    """The engine and the sampler behind the generation loop.

    One step ahead: before the host waits for the ids of a step, the next step (for the same
    rows, fed those ids on the device) is already queued, so the device does not idle while
    the host reads ids, looks for stop tokens and prepares the next launch.  If the loop then
    drops a row, the step that ran ahead has computed one token too many for it; that token
    is thrown away with the row's slot, and the other rows' ids do not depend on it.  A step
    runs ahead only if every row has room for one more token."""

    def __init__(self, engine: Engine, sampler: Sampler, max_batch: int, run_ahead: bool = True,
                 seed: Optional[int] = None):
        self.engine, self.sampler = engine, sampler
        self.seed = seed
        self.max_batch = max_batch
        self.max_tokens = engine.cache.max_tokens
        self.max_seq = engine.max_seq
        self.vocab_size = engine.model.spec.embedding.vocab_size
        self.run_ahead = run_ahead
        self.slots: List[int] = []
        self.cur: Optional[torch.Tensor] = None      # ids of the step last returned to the loop, rows = slots
        self.ahead: Optional[torch.Tensor] = None    # ids of the step after it, if that step already runs
        self.decode_steps = 0                        # decode steps launched, and the bytes they sent and read
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    def _decode(self, tokens: torch.Tensor) -> torch.Tensor:
        up = self.engine.cache.uploader
        before = up.bytes_sent
        # the sampler runs inside the step's graph; its ids stay valid until the next step of this batch
        # size is launched, and everything that reads them is queued before that
        ids = self.engine.decode(self.slots, tokens, tail=self.sampler, pad=True)    # few row counts, few graphs
        self.h2d_bytes += up.bytes_sent - before
        self.d2h_bytes += 4 * (len(self.slots) + 1)
        self.decode_steps += 1
        return ids

    def _launch_ahead(self) -> Optional[torch.Tensor]:
        eng = self.engine
        if not self.run_ahead or any(eng.cache.length(s) + 1 > self.max_seq for s in self.slots):
            return None
        try:
            return self._decode(self.cur)
        except CacheFull:
            return None

    def begin(self, first_index: int, prompts: Sequence[Sequence[int]]) -> np.ndarray:
        eng = self.engine
        self.slots = [eng.new_sequence() for _ in prompts]
        self.sampler.start(first_index, len(prompts), self.seed)
        if self.sampler.penalised:
            toks = torch.tensor([t for p in prompts for t in p], dtype=torch.int32, device=eng.device)
            rows = torch.tensor([r for r, p in enumerate(prompts) for _ in p], dtype=torch.int32, device=eng.device)
            self.sampler.mark_prompt(toks, rows)
        logits = eng.step(list(zip(self.slots, prompts)), "last")
        self.cur = self.sampler(logits).clone()
        self.sampler.post(self.cur)
        self.ahead = self._launch_ahead()
        return self.sampler.collect()

    def advance(self, keep_rows: Sequence[int]) -> np.ndarray:
        eng = self.engine
        keep = list(keep_rows)
        idx = None
        if len(keep) != len(self.slots):
            for r, s in enumerate(self.slots):
                if r not in keep:
                    eng.release(s)
            self.slots = [self.slots[r] for r in keep]
            idx = torch.tensor(keep, dtype=torch.long, device=eng.device)
            self.sampler.compact(keep)
        if self.ahead is not None:
            self.cur = self.ahead if idx is None else self.ahead[idx].contiguous()
        else:
            tokens = self.cur if idx is None else self.cur[idx].contiguous()
            self.cur = self._decode(tokens)
        self.sampler.post(self.cur)
        self.ahead = self._launch_ahead()
        return self.sampler.collect()

    def finish(self) -> None:
        for s in self.slots:
            self.engine.release(s)
        self.slots = []
        self.cur = None
        self.ahead = None


class _ConversationBackend(_Backend):
    """The backend of a ``Conversation``: one sequence whose slot outlives the call.  ``begin`` keeps what
    the cache holds of the new prompt and runs only the rest; ``finish`` releases nothing."""

    def __init__(self, engine: Engine, sampler: Sampler, run_ahead: bool, conv: "Conversation", seed: Optional[int] = None):
        super().__init__(engine, sampler, 1, run_ahead, seed)
        self.conv = conv

    def begin(self, first_index: int, prompts: Sequence[Sequence[int]]) -> np.ndarray:
        eng, conv = self.engine, self.conv
        prompt = list(prompts[0])
        common = conv.keep_common_prefix(prompt)
        self.slots = [conv.slot]
        self.sampler.start(first_index, 1, self.seed)
        if self.sampler.penalised:                 # the whole prompt counts as seen, reused or not (LLM.pas:737-744)
            toks = torch.tensor(prompt, dtype=torch.int32, device=eng.device)
            self.sampler.mark_prompt(toks, torch.zeros(len(prompt), dtype=torch.int32, device=eng.device))
        logits = eng.step([(conv.slot, prompt[common:])], "last")
        self.cur = self.sampler(logits).clone()
        self.sampler.post(self.cur)
        self.ahead = self._launch_ahead()
        return self.sampler.collect()

    def finish(self) -> None:
        self.slots = []
        self.cur = None
        self.ahead = None


class Conversation:
    """One sequence that keeps its cache between calls, as the reference's engine keeps its history
    (``FHistory``, src/models/QuickNN.Models.LLM.pas:24,715-745): a call whose prompt begins with what the cache
    already holds (the usual next turn: old prompt + old reply + new text) runs only the new tokens, and
    ``GenerationResult.reused_tokens`` says how many were found.  Where the prompt departs from the history the
    cache is shortened to the common part, if the model can go back that far (rings of windowed layers have
    lost what later tokens overwrote, fixed-size state cannot go back at all: ``KVCache.rewind_limit``);
    otherwise the sequence starts again from its first token.  A conversation holds one of the engine's
    ``max_batch`` slots until ``close`` (or the ``with`` block's end)."""

    def __init__(self, llm: "LLM"):
        self.llm = llm
        self.slot: Optional[int] = None
        self.history: List[int] = []               # the tokens whose keys and values the cache holds
        self.reused = 0
        self.said: List[int] = []                  # the last call's prompt and reply

    def __enter__(self) -> "Conversation":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def reset(self) -> None:
        """Forget the history (``ResetContext``, LLM.pas:436-449); the next call starts at the first token."""
        if self.slot is not None:
            self.llm.engine.release(self.slot)
        self.slot, self.history = None, []

    close = reset

    def keep_common_prefix(self, prompt: Sequence[int]) -> int:
        """Shorten the cache to what it shares with ``prompt`` and return that many tokens; the last token of
        the prompt is never taken from the cache, since its logits are wanted (LLM.pas:719-721)."""
        eng = self.llm.engine
        common = 0
        while common < len(prompt) and common < len(self.history) and prompt[common] == self.history[common]:
            common += 1
        if common == len(prompt):
            common -= 1
        if self.slot is not None and (common <= 0 or common < eng.cache.rewind_limit(self.slot)):
            self.reset()
        if self.slot is None:
            self.slot, common = eng.new_sequence(), 0
        elif common < eng.length(self.slot):
            eng.cache.truncate([(self.slot, common)])
        self.history = list(prompt[:common])
        self.reused = common
        return common

    def generate(self, prompt: Sequence[int], options: Optional[GenerationOptions] = None,
                 on_token: Optional[Callable[[int, int], Optional[bool]]] = None,
                 stop_ids: Optional[Sequence[int]] = None,
                 should_cancel: Optional[Callable[[], bool]] = None) -> GenerationResult:
        llm = self.llm
        options = options or GenerationOptions()
        options.validate()
        backend = _ConversationBackend(llm.engine, llm._sampler(options), llm.run_ahead, self, options.seed)
        stops = llm.stop_ids if stop_ids is None else list(stop_ids)
        self.reused = 0
        try:
            res = generate(backend, [list(prompt)], options, stops, on_token, should_cancel)[0]
        except Exception:
            self.reset()                           # what the cache holds is no longer known
            raise
        res.reused_tokens = self.reused
        self.said = list(prompt) + list(res.tokens)
        if self.slot is not None:
            # the cache holds the prompt and every generated token that was fed back (the step that runs ahead
            # may have fed one that the loop then dropped: a stop token)
            known = list(prompt) + list(res.tokens)
            held = llm.engine.length(self.slot)
            if held > len(known) and llm.engine.cache.rewind_limit(self.slot) <= len(known):
                llm.engine.cache.truncate([(self.slot, len(known))])
                held = len(known)
            # (state that cannot go back keeps the dropped token: no later prompt matches beyond it)
            self.history = (known + [-1] * max(0, held - len(known)))[:held]
        return res


    def continue_generation(self, options: Optional[GenerationOptions] = None, **kw) -> GenerationResult:
        """Go on from where the last call stopped (``ContinueGeneration``, LLM.pas:1029-1047): the prompt is
        everything said so far, all of which but the last token the cache still holds.  Greedy replies continue
        as if they had never stopped; sampled ones draw from freshly seeded generators."""
        if not self.said:
            raise ValueError("nothing to continue: generate first")
        return self.generate(self.said, options, **kw)


class LLM:
    """A loaded model with its cache, ready to generate.

    ``LLM(model_dir, max_context=...)`` loads a folder with ``config.json`` and
    ``model.safetensors``; ``LLM.random(config, seed)`` builds random weights on the
    device.  ``max_context`` is the reference's ``MaxContext``: the longest sequence
    (prompt plus generated) a request may reach."""

    def __init__(self, model_dir: Optional[str] = None, *, max_context: int = 2048, max_batch: int = 8,
                 max_tokens: Optional[int] = None, dtype="bfloat16", device="cuda:0", model: Optional[Model] = None,
                 decode_splits: Optional[int] = None):
        if model is None:
            if model_dir is None:
                raise ValueError("give a model folder or a Model")
            model = Model.from_folder(model_dir, dtype, device)
        self.model = model
        stops = list(model.spec.stop_ids)
        if model_dir is not None:              # the folder's generation_config.json may add stop ids (LLM.pas:260-271)
            stops = stop_ids_of_folder(model_dir, model.spec.embedding.vocab_size, stops)
        self._stop_ids = stops
        if max_context > model.spec.max_positions:
            raise ValueError(f"max_context {max_context} exceeds max_position_embeddings {model.spec.max_positions}")
        if max_tokens is None:
            max_tokens = max_batch * ((max_context + PAGE - 1) // PAGE * PAGE)
        self.max_batch = max_batch
        self.engine = Engine(model, max_tokens=max_tokens, max_slots=max(max_batch, 1), max_seq=max_context,
                             decode_splits=decode_splits)
        self.run_ahead = True            # queue each decode step before the host reads the ids of the one before
        self.last_io: Dict[str, float] = {}
        self._samplers: Dict[tuple, Sampler] = {}

    @classmethod
    def random(cls, config: Dict, seed: int = 0, *, dtype="bfloat16", device="cuda:0", norm_std: Optional[float] = None,
               **kw) -> "LLM":
        arch = find_architecture(config)
        cfg = arch.config_cls.from_dict(config)
        cd = as_dtype(dtype)
        tensors = dict(random_tensors(arch, cfg, seed, cd, norm_std, device=device))
        model = Model(arch, cfg, tensors, cd, device)
        return cls(model=model, dtype=dtype, device=device, **kw)

    @property
    def stop_ids(self) -> List[int]:
        """Stop ids from the configuration's ``eos_token_id`` (LLM.pas:166) and, for a model folder, from its
        generation_config.json as well."""
        return list(self._stop_ids)

    def _sampler(self, options: GenerationOptions) -> Sampler:
        # what the captured decode steps bake in; the seed is not part of it (it only sets the generators' states)
        key = (options.top_k, options.temperature, options.top_p, options.repetition_penalty)
        if options.temperature <= 0:
            key = ("greedy", options.repetition_penalty)          # an arg-max whatever top_k and top_p say
        s = self._samplers.get(key)
        if s is None:
            if len(self._samplers) > 4:
                for old in self._samplers.values():
                    self.engine.forget_tail(old)          # and the decode graphs that embed them
                self._samplers.clear()
            s = Sampler(self.model.spec.embedding.vocab_size, self.max_batch, options, self.engine.device)
            self._samplers[key] = s
        return s

    def generate(self, prompts: Sequence[Sequence[int]], options: Optional[GenerationOptions] = None,
                 on_token: Optional[Callable[[int, int], Optional[bool]]] = None,
                 stop_ids: Optional[Sequence[int]] = None,
                 should_cancel: Optional[Callable[[], bool]] = None) -> List[GenerationResult]:
        """Generate for a list of prompts (lists of token ids).  Requests are run in batches of
        up to ``max_batch``, one batch after another."""
        options = options or GenerationOptions()
        options.validate()
        backend = _Backend(self.engine, self._sampler(options), self.max_batch, self.run_ahead, options.seed)
        stops = self.stop_ids if stop_ids is None else list(stop_ids)
        try:
            return generate(backend, prompts, options, stops, on_token, should_cancel)
        finally:
            n = max(backend.decode_steps, 1)
            self.last_io = {"decode_steps": backend.decode_steps, "h2d_bytes_per_step": backend.h2d_bytes / n,
                            "d2h_bytes_per_step": backend.d2h_bytes / n}

    def warm_up(self, options: Optional[GenerationOptions] = None, batch_sizes: Optional[Sequence[int]] = None,
                context: Optional[int] = None) -> int:
        """Capture the decode graphs that ``generate`` with these options would otherwise capture on the way (about
        10 ms each, in the middle of a reply): for every row count that batches of ``batch_sizes`` (default: all up
        to ``max_batch``) pass through, at sequences of ``context`` tokens (default: the longest allowed; the
        schedule of a step depends on the lengths' class).  The cache contents of the dummy sequences are whatever
        the pages held; their tokens are thrown away.  Returns the number of decode states held afterwards."""
        opts = options or GenerationOptions()
        opts.validate()
        eng, sampler = self.engine, self._sampler(opts)
        sizes = sorted({b for b in (batch_sizes or range(1, self.max_batch + 1)) if 1 <= b <= self.max_batch})
        length = max(1, min(context or eng.max_seq, eng.max_seq) - 3)
        done = set()
        for b in sizes:
            rows = eng.decode_rows(b)
            if rows in done or b * (length + 3) > eng.cache.max_tokens:
                continue
            done.add(rows)
            slots = [eng.new_sequence() for _ in range(b)]
            try:
                eng.cache.extend([(s, length) for s in slots])
                sampler.start(0, b, opts.seed)
                tok = torch.ones(b, dtype=torch.int32, device=eng.device)
                for _ in range(2):                                  # the eager pass with the capture, then a replay
                    tok = eng.decode(slots, tok, tail=sampler, pad=True)
                try:
                    sampler.read(tok)
                except Exception:                                   # whatever the stale pages gave: nothing is kept
                    pass
            finally:
                for s in slots:
                    eng.release(s)
        return len(eng._decode_state)

    def conversation(self) -> Conversation:
        """A sequence that keeps its cache between calls and reuses the common prefix of successive prompts."""
        return Conversation(self)

    def evaluate_tokens(self, ids: Sequence[int]) -> np.ndarray:
        """Logits after the last of ``ids`` as a host array (``EvaluateTokens``, LLM.pas:1064-1088)."""
        slot = self.engine.new_sequence()
        try:
            return self.engine.step([(slot, list(ids))], "last")[0].cpu().numpy()
        finally:
            self.engine.release(slot)

    def memory_status(self) -> Dict[str, int]:
        return self.engine.stats()

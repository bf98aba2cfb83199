"""The step function: a batch of sequences that start together, from the cache.

One ``Engine`` owns a model, its cache and the scratch of the kernels.  ``step``
runs exactly the tokens it is given as one batch and returns the logits at the
wanted places.  The reference's counterpart is ``ForwardRows`` for one sequence in
128-row chunks, returning the last row's logits
(src/models/QuickNN.Models.LLM.pas:459-493); here a step takes several sequences of
unequal length, whole prompts at once, then one token each; a step may also continue
sequences by several tokens (the reference's prompts cut into portions and its reused prefix,
LLM.pas:459-493, 715-745), or start some sequences beside others that go on.
"""
from __future__ import annotations

from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..cache import PAGE, CacheFull, KVCache
from ..kernels import lib as _klib
from ..kernels import ops as _kops
from .batch import StepBatch, WholeSequences
from .model import Model

MAX_DECODE_GRAPHS = 256       # decode states (graph, buffers, scratch) kept at a time, over batch sizes, samplers and schedules


class StepError(ValueError):
    pass


class Engine:
    def __init__(self, model: Model, max_tokens: int, max_slots: Optional[int] = None,
                 max_seq: Optional[int] = None, decode_splits: Optional[int] = None,
                 tuning: Optional[Mapping[str, Any]] = None):
        """``tuning``: options by name that the parts may look up in a step (``decode_splits`` fixes
        the number of key ranges of decode attention; the argument of that name is a shorthand)."""
        self.model = model
        self.device = model.device
        if self.device.type != "cuda":
            raise RuntimeError("quicknn_b200 runs on a CUDA device only; there is no CPU path")
        max_tokens = (int(max_tokens) + PAGE - 1) // PAGE * PAGE
        if max_seq is None:
            max_seq = min(max_tokens, model.spec.max_positions)
        if max_seq > model.spec.max_positions:
            raise ValueError(f"max_seq {max_seq} exceeds the model's max positions {model.spec.max_positions}")
        if max_slots is None:
            max_slots = max(1, min(max_tokens // PAGE, 256))
        needs, states = model.cache_needs()
        self.cache = KVCache(needs, states, max_tokens, max_slots, max_seq, model.dtype, self.device)
        self.max_seq, self.max_slots = max_seq, max_slots
        self.tuning: Dict[str, Any] = dict(tuning or {})
        if decode_splits:
            self.tuning["decode_splits"] = int(decode_splits)
        self._scratch_other: Optional[torch.Tensor] = None   # steps outside decode graphs: one buffer that grows
        self._decode_state: Dict[tuple, dict] = {}
        self._schedules: Dict[tuple, int] = {}               # (batch, longest, spread) -> hash of the model's schedule
        self.use_graphs = True
        self.graph_kernels_replayed = 0
        self.steps_run = 0

    # ---- sequences -------------------------------------------------------------------
    def new_sequence(self) -> int:
        return self.cache.allocate()

    def release(self, slot: int) -> None:
        self.cache.free(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step ----------------------------------------------------------------------
    def _give_scratch(self, step: StepBatch) -> None:
        """Ask the parts what scratch a step of this shape needs and hand it over as ``step.scratch``."""
        need = (int(self.model.scratch_need(step)) + 255) // 256 * 256
        if need <= 0:
            step.scratch = None
        elif step.mode == "decode" and step.want_every_row:
            # a decode state of its own (its graph keeps the address): never shared, never replaced
            step.scratch = torch.empty(need, dtype=torch.uint8, device=self.device)
        else:
            if self._scratch_other is None or self._scratch_other.numel() < need:
                self._scratch_other = torch.empty(need, dtype=torch.uint8, device=self.device)
            step.scratch = self._scratch_other

    def plan(self, entries: Sequence[Tuple[int, Sequence[int]]],
             want: Union[str, Sequence[Sequence[int]]] = "last"):
        """Host-side half of a step: checks, cache growth, packed metadata (numpy)."""
        if not entries:
            raise StepError("a step needs at least one sequence")
        slots = [int(s) for s, _ in entries]
        if len(set(slots)) != len(slots):
            raise StepError("a sequence appears twice in one step")
        lens = [len(t) for _, t in entries]
        if min(lens) < 1:
            raise StepError("every sequence of a step brings at least one token")
        starts = [self.cache.length(s) for s in slots]
        if all(p == 0 for p in starts):
            mode = "prefill"          # whole prompts: attention over the step's own rows
        elif all(n == 1 for n in lens):
            mode = "decode"           # one token each: attention over the cache
        else:
            mode = "extend"           # anything else: cached keys first, then the step's own rows
        V = self.model.spec.embedding.vocab_size
        arrays = [np.asarray(t, dtype=np.int64).reshape(-1) for _, t in entries]
        for a in arrays:
            if a.size and (int(a.min()) < 0 or int(a.max()) >= V):
                bad = a[(a < 0) | (a >= V)][0]
                raise StepError(f"token id {int(bad)} is outside the vocabulary of {V}")
        if want == "last":
            want = [[n - 1] for n in lens]
        elif want == "all":
            want = [range(n) for n in lens]
        if len(want) != len(entries):
            raise StepError("`want` needs one list per sequence")
        T, B = sum(lens), len(entries)
        lens_a = np.asarray(lens, np.int32)
        row0 = (np.cumsum(lens_a) - lens_a).astype(np.int32)
        tokens = np.concatenate(arrays).astype(np.int32)
        tok_row0 = np.repeat(row0, lens_a)
        tok_pos = (np.arange(T, dtype=np.int32) - tok_row0 + np.repeat(np.asarray(starts, np.int32), lens_a)).astype(np.int32)
        tok_slot = np.repeat(np.asarray(slots, np.int32), lens_a)
        rows: List[np.ndarray] = []
        for r0, n, w in zip(row0, lens, want):
            w = np.asarray(list(w) if not isinstance(w, range) else w, dtype=np.int64).reshape(-1)
            if w.size and (int(w.min()) < 0 or int(w.max()) >= n):
                bad = w[(w < 0) | (w >= n)][0]
                raise StepError(f"wanted place {int(bad)} is outside the {n} tokens the sequence brings")
            rows.append(w + int(r0))
        rows_a = np.concatenate(rows).astype(np.int32) if rows else np.zeros(0, np.int32)
        # only now, with everything checked, does the cache change
        self.cache.extend([(s, p + n) for s, p, n in zip(slots, starts, lens)])
        return (mode, T, B, tokens, tok_pos, tok_slot, tok_row0, np.asarray(slots, np.int32), rows_a, row0, lens_a,
                list(zip(slots, starts)))

    def step(self, entries: Sequence[Tuple[int, Sequence[int]]],
             want: Union[str, Sequence[Sequence[int]]] = "last") -> torch.Tensor:
        """Run the given tokens as one batch; return float32 logits ``[wanted, vocab]`` in the
        order of the entries and of their wanted places.  Raises ``NonFiniteLogits`` if they hold
        NaN or Inf.  If the step cannot be launched, the sequences keep their earlier lengths."""
        mode, T, B, tokens, tok_pos, tok_slot, tok_row0, slots, rows, row0, lens, before = self.plan(entries, want)
        try:
            logits = self._launch_step(mode, T, B, (tokens, tok_pos, tok_slot, tok_row0, slots, rows, row0, lens))
        except Exception:
            self.cache.truncate(before)
            raise
        self.steps_run += 1
        self.check()
        return logits

    def _launch_step(self, mode, T, B, arrays) -> torch.Tensor:
        self.cache.sync()
        extra = ()
        if mode == "extend":
            tok_pos, row0, lens = arrays[1], arrays[6], arrays[7]
            start = tok_pos[row0]                                   # a sequence's first row stands at its cached length
            length = start + lens
            whole_row0 = (np.cumsum(length) - length).astype(np.int32)
            tok_row = (np.repeat(whole_row0, lens) + tok_pos).astype(np.int32)  # position p of sequence b is row whole_row0[b] + p
            extra = (start.astype(np.int32), whole_row0, length.astype(np.int32), tok_row)
            arrays = tuple(arrays) + extra
        packed = np.concatenate(arrays).astype(np.int32, copy=False)
        dev = torch.empty(packed.size, dtype=torch.int32, device=self.device)
        self.cache.uploader.send(dev, packed)
        o = 0
        views = []
        for a in arrays:
            views.append(dev[o:o + a.size])
            o += a.size
        longest, spread = self.length_classes((arrays[1] + 1).tolist()) if mode == "decode" else (0, 0.0)
        whole = None
        if extra:
            whole = WholeSequences(views[4], views[8], views[6], views[7], views[9], views[10], views[11],
                                   total=int(extra[2].sum()), longest=int(extra[2].max()), most_new=int(arrays[7].max()))
        step = StepBatch(mode, T, B, views[0], views[1], views[2], views[3], views[4], views[5],
                         self.model.dtype, max_q_len=int(arrays[7].max()), seq_row0=views[6], seq_len=views[7],
                         max_seq=self.max_seq, tuning=self.tuning, longest=longest, spread=spread, whole=whole)
        self._give_scratch(step)
        logits = self.model.forward(step, self.cache)
        if logits.numel():
            _kops.check_finite(logits)
        return logits

    def check(self) -> None:
        """Raise ``NonFiniteLogits`` if a forward pass since the last check gave NaN or Inf
        (the reference flags them after every forward, src/models/QuickNN.Models.Gemma2.pas:196, and raises at
        the next readback, QuickNN.Vulkan.Context.Implementation.inc:732-756), ``KernelError`` if a
        bounded wait inside a tcgen05 kernel ran out.  One 8-byte read that waits for the device;
        ``step`` calls it itself, ``decode`` leaves it to the caller (or to the sampler's error word)."""
        _kops.raise_on_status(self.device)

    # ---- decode with ids that are already on the device -------------------------------
    def decode(self, slots: Sequence[int], tokens_dev: torch.Tensor, use_graph: Optional[bool] = None,
               tail=None, pad: bool = False) -> torch.Tensor:
        """One token for each sequence in ``slots``; ``tokens_dev`` ([B] int32) stays on the
        device (the reference feeds the sampled id from device memory too,
        src/models/QuickNN.Models.LLM.pas:802-807).  Returns the logits of every row, or, with
        ``tail`` (a callable on the logits that launches device work only, such as a sampler),
        what ``tail`` returns: it then runs as part of the same graph, and its result lives in a
        buffer that the next step replayed from the same graph overwrites.

        The launch sequence is captured in a CUDA graph the first time it runs and replayed
        afterwards; lengths, page tables and ids are read from device memory by the kernels, so
        one graph serves every step of the same row count, ``tail`` and schedule (what the parts
        decide from the lengths' classes, ``Part.schedule``).

        ``pad``: run the step with a few more rows than sequences (rows of no sequence, which attend to nothing
        and write nothing) so that a batch that shrinks one sequence at a time passes through few row counts
        (``decode_rows``) and so needs few graphs, each of which takes about 10 ms to capture; the result is
        that of the sequences' rows.  ``tail`` then sees the padded rows too and must have room for them."""
        B = len(slots)
        if B < 1:
            raise StepError("a step needs at least one sequence")
        if len(set(slots)) != B:
            raise StepError("a sequence appears twice in one step")
        starts = [self.cache.length(s) for s in slots]
        if min(starts) < 1:
            raise StepError("decode continues sequences that have at least one token")
        if tokens_dev.dtype != torch.int32 or tokens_dev.numel() != B or not tokens_dev.is_cuda:
            raise StepError("decode needs one int32 id per sequence on the device")
        self.cache.extend([(s, p + 1) for s, p in zip(slots, starts)])
        try:
            return self._decode(slots, starts, tokens_dev, use_graph, tail, self.decode_rows(B) if pad else B)
        except Exception:
            self.cache.truncate(list(zip(slots, starts)))
            raise

    def decode_rows(self, n_seqs: int) -> int:
        """Rows of a padded decode step for this many sequences: every count up to 8, then steps of 2 up to 16,
        of 4 up to 32, of 8 up to 64, of 16 beyond; never more than the cache has slots."""
        step = 1 if n_seqs <= 8 else (2 if n_seqs <= 16 else (4 if n_seqs <= 32 else (8 if n_seqs <= 64 else 16)))
        return max(n_seqs, min((n_seqs + step - 1) // step * step, self.max_slots))

    @staticmethod
    def length_classes(lengths: Sequence[int]) -> Tuple[int, float]:
        """(longest, spread) of ``StepBatch`` for sequences of these lengths: the longest rounded up to a power
        of two (at least 256), and longest / mean as one of four classes.  Coarse on purpose: a decode graph is
        captured per class, and a batch changes class a few times in its life."""
        longest = max(lengths)
        bound = 256
        while bound < longest:
            bound *= 2
        ratio = longest * len(lengths) / max(1, sum(lengths))
        return bound, (1.0 if ratio < 1.1 else (1.25 if ratio < 1.4 else (1.6 if ratio < 1.9 else 2.2)))

    def _decode(self, slots, starts, tokens_dev, use_graph, tail, rows):
        n_seqs, B = len(slots), rows                 # B rows, of which the last B - n_seqs belong to no sequence
        self.cache.sync()
        use_graph = self.use_graphs if use_graph is None else use_graph
        longest, spread = self.length_classes([p + 1 for p in starts])
        # a graph per batch size, sampler and schedule that the parts derive from the length classes (classes
        # that lead to the same decisions share one); the schedule of a class is asked once
        shape = (B, longest, spread, tuple(sorted(self.tuning.items())))
        sched = self._schedules.get(shape)
        if sched is None:
            probe = StepBatch("decode", B, B, None, None, None, None, None, None, self.model.dtype, max_seq=self.max_seq,
                              tuning=self.tuning, want_every_row=True, longest=longest, spread=spread)
            sched = self._schedules[shape] = hash(self.model.schedule(probe))
        key = (B, id(tail) if tail is not None else None, sched)
        st = self._decode_state.pop(key, None)
        if st is not None:
            self._decode_state[key] = st                          # most recently used last
        else:
            if len(self._decode_state) >= MAX_DECODE_GRAPHS:     # the least recently used goes (graph, buffers, scratch)
                del self._decode_state[next(iter(self._decode_state))]
            meta = torch.zeros(2 * B, dtype=torch.int32, device=self.device)
            ar = torch.arange(B, dtype=torch.int32, device=self.device)
            tokens = torch.zeros(B, dtype=torch.int32, device=self.device)
            step = StepBatch("decode", B, B, tokens, meta[:B], meta[B:], ar, meta[B:], ar, self.model.dtype,
                             max_seq=self.max_seq, tuning=self.tuning, want_every_row=True, longest=longest,
                             spread=spread)
            self._give_scratch(step)
            st = {"meta": meta, "step": step, "graph": None, "logits": None, "tail": tail}    # holds `tail` alive: its id is the key
            self._decode_state[key] = st
        pad_rows = B - n_seqs
        self.cache.uploader.send(st["meta"], np.concatenate([np.asarray(list(starts) + [0] * pad_rows, np.int32),
                                                             np.asarray(list(slots) + [-1] * pad_rows, np.int32)]))
        st["step"].tokens[:n_seqs].copy_(tokens_dev.reshape(-1))
        self.steps_run += 1
        if pad_rows:
            inner = self._replay_or_capture(st, tail, use_graph)
            return inner[:n_seqs]
        return self._replay_or_capture(st, tail, use_graph)

    def _replay_or_capture(self, st, tail, use_graph):
        def run():
            if tail is not None:
                return self.model.forward(st["step"], self.cache, reduce=tail)    # a sampler has its own error word
            logits = self.model.forward(st["step"], self.cache)
            _kops.check_finite(logits)                # read by check()
            return logits

        if not use_graph:
            return run()
        if st["graph"] is None:
            logits = run()                                            # eager: also warms everything up
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            before = _klib.launches
            with torch.cuda.graph(g):
                st["logits"] = run()
            st["kernels"] = _klib.launches - before      # our kernels in one replay of this graph
            _klib.launches = before
            st["graph"] = g
            return logits
        st["graph"].replay()
        self.graph_kernels_replayed += st["kernels"]
        return st["logits"]

    def forget_tail(self, tail) -> None:
        """Drop the graphs that were captured with ``tail`` (a sampler that is no longer used)."""
        for key in [k for k in self._decode_state if k[1] == id(tail)]:
            del self._decode_state[key]

    def kernels_launched(self) -> int:
        """Kernels of this library launched so far, eagerly or inside replayed graphs."""
        return _klib.launches + self.graph_kernels_replayed

    def stats(self) -> Dict[str, int]:
        return {"weight_bytes": self.model.weight_bytes(), "cache_bytes": self.cache.bytes(),
                "tokens_held": self.cache.tokens_held(), "max_tokens": self.cache.max_tokens,
                "live_sequences": len(self.cache.slots.live()), "steps": self.steps_run}

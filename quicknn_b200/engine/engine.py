"""The step function: a batch of sequences that start together, from the cache.

One ``Engine`` owns a model, its cache and the scratch of the kernels.  ``step``
runs exactly the tokens it is given as one batch and returns the logits at the
wanted places.  The reference's counterpart is ``ForwardRows`` for one sequence in
128-row chunks, returning the last row's logits
(src/models/QuickNN.Models.LLM.pas:459-493); here a step takes several sequences of
unequal length, whole prompts at once, then one token each.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ..cache import PAGE, CacheFull, KVCache
from ..kernels import lib as _klib
from ..kernels import ops as _kops
from .batch import StepBatch
from .model import Model


class StepError(ValueError):
    pass


class Engine:
    def __init__(self, model: Model, max_tokens: int, max_slots: Optional[int] = None,
                 max_seq: Optional[int] = None, decode_splits: Optional[int] = None):
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
        # Key ranges per sequence in decode attention.  A fixed number when given; else chosen per
        # batch size so that one wave of CTAs covers the GPU (results then differ between batch
        # sizes by rounding only: the ranges are summed in a fixed order either way).
        self._fixed_splits = int(decode_splits) if decode_splits else None
        self._max_splits = max(1, min(64, max_seq // 128))
        self._kv_groups = max([getattr(b.mixer, "n_kv", 1) for b in model.blocks] or [1])
        # blocks of the decode attention kernel that the device holds at once: its shared
        # memory is 384 bytes per element of a head, so two fit on an SM at head size 256,
        # four at 128, eight at 64
        head = max([getattr(b.mixer, "head_dim", 256) for b in model.blocks] or [256])
        sms = torch.cuda.get_device_properties(self.device).multi_processor_count if self.device.type == "cuda" else 148
        self._resident = sms * max(1, min(8, 512 // max(1, head)))
        self.decode_splits = self._fixed_splits or self._max_splits
        self._scratch: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._decode_state: Dict[tuple, dict] = {}
        self.use_graphs = True
        self.graph_kernels_replayed = 0
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.steps_run = 0

    # ---- sequences -------------------------------------------------------------------
    def new_sequence(self) -> int:
        return self.cache.allocate()

    def release(self, slot: int) -> None:
        self.cache.free(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step ----------------------------------------------------------------------
    def splits_for(self, batch: int) -> int:
        if self._fixed_splits:
            return self._fixed_splits
        pairs = batch * self._kv_groups
        # as many key ranges as keep one wave of blocks on the device (measured at head size 256, context
        # 8192: batch 64 one range 9.48 ms against two 9.69; batch 32 two ranges; batch 16 four; batch 8 nine)
        return max(1, min(self._max_splits, self._resident // max(1, pairs)))

    def _scratch_for(self, batch: int) -> Tuple[torch.Tensor, torch.Tensor]:
        key = 1
        while key < batch:
            key *= 2
        if key not in self._scratch:
            po, pm = self.model.decode_scratch(key, max(self._max_splits, self.decode_splits))
            self._scratch[key] = (torch.empty(max(po, 1), dtype=torch.float32, device=self.device),
                                  torch.empty(max(pm, 1), dtype=torch.float32, device=self.device))
        return self._scratch[key]

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
            mode = "prefill"
        elif all(n == 1 for n in lens):
            mode = "decode"
        else:
            raise StepError("the sequences of a step either all start at their first token or all go on "
                            "by one token")
        V = self.model.spec.embedding.vocab_size
        for _, toks in entries:
            for t in toks:
                if not (0 <= int(t) < V):
                    raise StepError(f"token id {t} is outside the vocabulary of {V}")
        if want == "last":
            want = [[n - 1] for n in lens]
        elif want == "all":
            want = [list(range(n)) for n in lens]
        if len(want) != len(entries):
            raise StepError("`want` needs one list per sequence")
        T, B = sum(lens), len(entries)
        tokens = np.empty(T, np.int32)
        tok_pos = np.empty(T, np.int32)
        tok_slot = np.empty(T, np.int32)
        tok_row0 = np.empty(T, np.int32)
        rows: List[int] = []
        r = 0
        for (s, toks), p0, n, w in zip(entries, starts, lens, want):
            tokens[r:r + n] = np.asarray(toks, dtype=np.int64)
            tok_pos[r:r + n] = np.arange(p0, p0 + n)
            tok_slot[r:r + n] = s
            tok_row0[r:r + n] = r
            for i in w:
                if not (0 <= int(i) < n):
                    raise StepError(f"wanted place {i} is outside the {n} tokens the sequence brings")
                rows.append(r + int(i))
            r += n
        # only now, with everything checked, does the cache change
        self.cache.extend([(s, p + n) for s, p, n in zip(slots, starts, lens)])
        return mode, T, B, tokens, tok_pos, tok_slot, tok_row0, np.asarray(slots, np.int32), np.asarray(rows, np.int32)

    def step(self, entries: Sequence[Tuple[int, Sequence[int]]],
             want: Union[str, Sequence[Sequence[int]]] = "last") -> torch.Tensor:
        """Run the given tokens as one batch; return float32 logits ``[wanted, vocab]`` in the
        order of the entries and of their wanted places."""
        mode, T, B, tokens, tok_pos, tok_slot, tok_row0, slots, rows = self.plan(entries, want)
        self.cache.sync()
        lens = np.asarray([len(t) for _, t in entries], np.int32)
        starts = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
        packed = np.concatenate([tokens, tok_pos, tok_slot, tok_row0, slots, rows, starts, lens])
        dev = torch.empty(packed.size, dtype=torch.int32, device=self.device)
        self.cache.uploader.send(dev, packed.astype(np.int32, copy=False))
        o = 0
        views = []
        for n in (T, T, T, T, B, len(rows), B, B):
            views.append(dev[o:o + n])
            o += n
        part_o, part_ml = self._scratch_for(B) if mode == "decode" else (None, None)
        step = StepBatch(mode, T, B, views[0], views[1], views[2], views[3], views[4], views[5],
                         self.model.dtype, self.splits_for(B), part_o, part_ml, max_q_len=int(lens.max()),
                         seq_row0=views[6], seq_len=views[7])
        logits = self.model.forward(step, self.cache)
        self.steps_run += 1
        if mode == "prefill":
            _kops.check_gemm_status(self.device)      # a bounded wait of the tcgen05 product ran out?
        return logits

    # ---- decode with ids that are already on the device -------------------------------
    def decode(self, slots: Sequence[int], tokens_dev: torch.Tensor, use_graph: Optional[bool] = None,
               tail=None) -> torch.Tensor:
        """One token for each sequence in ``slots``; ``tokens_dev`` ([B] int32) stays on the
        device (the reference feeds the sampled id from device memory too,
        src/models/QuickNN.Models.LLM.pas:802-807).  Returns the logits of every row, or, with
        ``tail`` (a callable on the logits that launches device work only, such as a sampler),
        what ``tail`` returns: it then runs as part of the same graph, and its result lives in a
        buffer that the next step of this batch size overwrites.

        The launch sequence of a batch size is captured in a CUDA graph the first time it
        runs and replayed afterwards; lengths, page tables and ids are read from device
        memory by the kernels, so one graph serves every step of that batch size."""
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
        self.cache.sync()
        use_graph = self.use_graphs if use_graph is None else use_graph
        key = (B, id(tail) if tail is not None else None)
        st = self._decode_state.get(key)
        if st is None:
            meta = torch.zeros(2 * B, dtype=torch.int32, device=self.device)
            ar = torch.arange(B, dtype=torch.int32, device=self.device)
            part_o, part_ml = self._scratch_for(B)
            tokens = torch.zeros(B, dtype=torch.int32, device=self.device)
            step = StepBatch("decode", B, B, tokens, meta[:B], meta[B:], ar, meta[B:], ar, self.model.dtype,
                             self.splits_for(B), part_o, part_ml)
            st = {"meta": meta, "step": step, "graph": None, "logits": None, "tail": tail}    # holds `tail` alive: its id is the key
            self._decode_state[key] = st
        self.cache.uploader.send(st["meta"], np.concatenate([np.asarray(starts, np.int32), np.asarray(slots, np.int32)]))
        st["step"].tokens.copy_(tokens_dev.reshape(-1))
        self.steps_run += 1
        def run():
            logits = self.model.forward(st["step"], self.cache)
            return logits if tail is None else tail(logits)

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

    def fill_synthetic(self, slots: Sequence[int], lengths: Sequence[int], seed: int = 0) -> None:
        """Give sequences a history of the given lengths without computing it: pages are taken
        as a prompt of that length would take them and every cache line is filled with random
        keys and values.  For timing decode steps at a chosen context; the logits mean nothing."""
        self.cache.extend(list(zip(slots, lengths)))
        self.cache.sync()
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        for grp in self.cache.groups:
            for t in (grp.k, grp.v):
                for li in range(t.shape[0]):
                    t[li].normal_(0.0, 1.0, generator=g)

    def stats(self) -> Dict[str, int]:
        return {"weight_bytes": self.model.weight_bytes(), "cache_bytes": self.cache.bytes(),
                "tokens_held": self.cache.tokens_held(), "max_tokens": self.cache.max_tokens,
                "live_sequences": len(self.cache.slots.live()), "steps": self.steps_run}

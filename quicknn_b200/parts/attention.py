"""The attention mixer: grouped-query attention over the paged cache, with the window,
the softcap and the scale as parameters.

Order of operations as in the reference's layer body
(src/models/QuickNN.Models.Gemma2.pas:167-180): Q, K, V projections; rotation of Q and K;
append K, V to the cache; attention with scale 1/sqrt(query_pre_attn_scalar), softcap
and window; output projection.  The three projections are one product against the
stacked matrix; rotation and append belong to the position part (one kernel, or, for the
few rows of a decode step, the epilogue of that product).

Decode attention cuts each sequence's keys into ranges that run as separate blocks and are
merged afterwards; how many ranges, and the scratch that the partial results need, are
decided here (``tuning["decode_splits"]`` fixes the number).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .base import MIXERS, POSITIONS, CacheNeed, HeadShape, Mixer
from .linear import project, stack_rows
from .spec import PartSpec


BLOCK_COST = 64.0        # a decode-attention block's fixed cost, in keys of its walk
MERGE_COST = 100.0       # the kernel that merges more than four ranges, in the same unit


@MIXERS.register("attention")
class AttentionMixer(Mixer):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.n_heads = int(p["n_heads"])
        self.n_kv = int(p["n_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.scale = float(p["scale"])
        self.softcap = p.get("softcap")
        self.window = p.get("window")
        if self.n_heads % self.n_kv:
            raise ValueError(f"{self.n_kv} kv heads do not divide {self.n_heads} heads")
        self.heads = HeadShape(self.n_heads, self.n_kv, self.head_dim)
        pos: PartSpec = p["position"]
        self.position = POSITIONS.get(pos.kind)(pos)
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self._resident = 148

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        p = spec.params
        H, nq, nkv, hd = int(p["hidden_size"]), int(p["n_heads"]), int(p["n_kv_heads"]), int(p["head_dim"])
        M = cls.PARAM_ROLE_MATRIX
        return {"q_proj": ((nq * hd, H), M), "k_proj": ((nkv * hd, H), M), "v_proj": ((nkv * hd, H), M),
                "o_proj": ((H, nq * hd), M)}

    def load(self, tensors, compute_dtype, device) -> None:
        self.w_qkv = stack_rows([tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]])
        self.w_o = tensors["o_proj"].contiguous()
        self.position.prepare(device)
        # sizes that the kernels do not take are refused here, when the model is built, not at its first step
        why = (ops.attention_refusal(compute_dtype, self.n_heads, self.n_kv, self.head_dim)
               or ops.linear_refusal(self.w_qkv.dtype, self.hidden)
               or ops.linear_refusal(self.w_o.dtype, self.n_heads * self.head_dim))
        if why:
            raise ValueError(f"attention mixer: {why}")
        # blocks of the decode attention kernel that the device holds at once: its shared memory is
        # 384 bytes per element of a head, so two fit on an SM at head size 256, four at 128, eight at 64
        dev = torch.device(device)
        sms = torch.cuda.get_device_properties(dev).multi_processor_count if dev.type == "cuda" else 148
        self._resident = sms * max(1, min(8, 512 // max(1, self.head_dim)))

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_qkv, self.w_o))

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(self.n_kv, self.head_dim, self.window)

    def decode_splits(self, step) -> int:
        """Key ranges per sequence in a decode step: a fixed number when the engine's owner gave one, else the
        number with the shortest estimated time for the step's length classes (``step.longest``, ``step.spread``).

        A sequence's keys are cut into equal ranges, a block per (range, kv head, sequence).  While all blocks
        fit the device at once the step takes as long as the longest sequence's range.  With more blocks than
        that they run in turns: blocks of one length (sequences of nearly equal lengths) in whole rounds, each as
        long as a block; blocks of unequal lengths fill the device evenly, and the time is the work of all blocks
        spread over the device plus about half a block at the end.  A block costs about as much as 64 keys before
        its first key, and more than four ranges are merged by a kernel of its own, which costs about as much as a
        hundred.  Measured at head size 256, context 8192, equal lengths, 6 layers, ms per step by ranges: batch 24:
        2: 1.32, 3: 1.08, 4: 1.34, 5: 1.20, 6: 1.11, 8: 1.18 (one round of 288 blocks, then 2, 2, 2 and 3 rounds);
        batch 28: 2: 1.34, 3: 1.60, 5: 1.23, 6: 1.39; batch 12: 4: 0.91, 5: 0.85, 6: 0.81, 8: 0.94; batch 64 one
        range 9.48 ms (26 layers) against two 9.69 and eight 8.42; batch 64 with prompts of 512 to 2048 tokens one
        range 4.20 ms, four 4.03, six 3.90, nine 4.12 (the longest sequence no longer sets the pace).  Results
        differ between these choices by rounding only: ranges are summed in a fixed order."""
        fixed = step.tuning.get("decode_splits")
        if fixed:
            return int(fixed)
        tiles = max(1, step.n_seqs * self.n_kv)
        longest = step.longest or step.max_seq
        if self.window:
            longest = min(longest, self.window)
        most = max(1, min(64, longest // 32))
        mean = longest / (step.spread or 1.0)
        best, best_time = 1, float("inf")
        equal = (step.spread or 1.0) <= 1.0
        for s in range(1, most + 1):                 # times in keys of one block's walk
            if s * tiles <= self._resident:
                t = longest / s + BLOCK_COST
            elif equal:                              # blocks of one length run in rounds
                t = -(-s * tiles // self._resident) * (longest / s + BLOCK_COST)
            else:
                t = tiles * (mean + s * BLOCK_COST) / self._resident + longest / (2 * s)
            if s > 4:
                t += MERGE_COST
            if t < best_time * 0.999:
                best, best_time = s, t
        return best

    def schedule(self, step) -> tuple:
        return (self.decode_splits(step),) if step.mode == "decode" else ()

    def scratch_need(self, step) -> int:
        """Partial (maximum, sum, output) of every key range: float32, [rows, heads, ranges, head_dim + 2]."""
        if step.mode != "decode":
            return 0
        return step.n_seqs * self.n_heads * self.decode_splits(step) * (self.head_dim + 2) * 4

    def forward(self, x: torch.Tensor, step, line) -> torch.Tensor:
        h = self.heads
        extend = step.mode == "extend"
        qkv = None if extend else self.position.project_and_place(x, self.w_qkv, h, step, line)
        if qkv is None:
            qkv = project(x, self.w_qkv)
            self.position.place(qkv, h, step, line, append=not extend)
        if extend and line.writes:
            # cached keys from before this step, this step's own rows from there on; the append comes last,
            # so that the first rows still find the ring cells that the last rows overwrite
            a = ops.attn_extend(qkv, h.n_heads, h.n_kv_heads, h.head_dim, line.k, line.v, line.page_table,
                                line.page_size, line.ring, step.tok_pos, step.tok_row0, step.tok_slot, self.scale,
                                self.softcap, self.window, whole=getattr(step, "whole", None))
            ops.cache_append(qkv, h.n_heads, h.n_kv_heads, h.head_dim, step.tok_pos, step.tok_slot, line)
        elif step.mode != "decode" and not line.writes:
            # the keys of this line were written by another layer earlier in this step; in a ring the last
            # rows of the step have by then overwritten cells: whole prompts may fill the ring, a step that
            # continues a sequence may bring only as many rows as the ring has cells beyond the window
            room = line.ring - ((self.window or line.ring) - 1 if extend else 0)
            if line.ring and step.max_q_len > room:
                raise ValueError(f"a step of {step.max_q_len} tokens overruns the ring of {line.ring} "
                                 f"positions that this layer reads from another layer's cache line")
            a = ops.attn_prefill_paged(qkv, self.n_heads, self.n_kv, self.head_dim, line.k, line.v,
                                       line.page_table, line.page_size, line.ring, step.tok_pos, step.tok_slot,
                                       self.scale, self.softcap, self.window)
        elif step.mode == "prefill":
            a = ops.attn_prefill(qkv, self.n_heads, self.n_kv, self.head_dim, step.tok_pos, step.tok_row0,
                                 self.scale, self.softcap, self.window, step.seq_row0, step.seq_len, step.max_q_len)
        else:
            splits = self.decode_splits(step)
            n = step.n_seqs * self.n_heads * splits
            part = step.scratch.view(torch.float32)
            a = ops.attn_decode(qkv, self.n_heads, self.n_kv, self.head_dim, line.k, line.v, line.page_table,
                                line.page_size, line.ring, step.slots, line.slot_len, self.scale, self.softcap,
                                self.window, splits, part[:n * self.head_dim], part[n * self.head_dim:n * (self.head_dim + 2)])
        return project(a, self.w_o)

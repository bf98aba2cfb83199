"""The attention mixer: grouped-query attention over the paged cache, with the window,
the softcap and the scale as parameters.

Order of operations as in the reference's layer body
(src/models/QuickNN.Models.Gemma2.pas:167-180): Q, K, V projections; rotation of Q and K;
append K, V to the cache; attention with scale 1/sqrt(query_pre_attn_scalar), softcap
and window; output projection.  The three projections are one product against the
stacked matrix; rotation and append are one kernel, or, for the few rows of a decode
step, the epilogue of that product.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .base import MIXERS, POSITIONS, CacheNeed, Mixer
from .linear import project, stack_rows
from .spec import PartSpec


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
        pos: PartSpec = p["position"]
        self.position = POSITIONS.get(pos.kind)(pos)
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

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
        elem = 4 if compute_dtype == torch.float32 else 2
        if (self.head_dim * elem) % 16:
            raise ValueError(f"head_dim {self.head_dim} is not a whole number of 16-byte vectors in "
                             f"{compute_dtype}: the attention kernels refuse it")

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_qkv, self.w_o))

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(self.n_kv, self.head_dim, self.window)

    def forward(self, x: torch.Tensor, step, line) -> torch.Tensor:
        if step.mode == "decode" and ops.qkv_rope_cache_fusable(x, self.w_qkv, self.head_dim,
                                                                self.position.rotary_dim):
            # few rows: rotation and append ride in the product's epilogue
            qkv = ops.qkv_rope_cache(x, self.w_qkv, self.n_heads, self.n_kv, self.head_dim,
                                     self.position.inv_freq, step.tok_pos, step.tok_slot, line.k, line.v,
                                     line.page_table, line.page_size, line.ring, line.slot_len, line.writes)
        else:
            qkv = project(x, self.w_qkv)
            ops.rope_cache_write(qkv, self.n_heads, self.n_kv, self.head_dim, self.position.rotary_dim,
                                 self.position.inv_freq, step.tok_pos, step.tok_slot, line.k, line.v,
                                 line.page_table, line.page_size, line.ring, line.slot_len, line.writes)
        if step.mode == "prefill" and not line.writes:
            # the keys of this line were written by another layer earlier in this step
            if line.ring and step.max_q_len > line.ring:
                raise ValueError(f"a prompt of {step.max_q_len} tokens has overrun the ring of {line.ring} "
                                 f"positions that this layer reads from another layer's cache line")
            a = ops.attn_prefill_paged(qkv, self.n_heads, self.n_kv, self.head_dim, line.k, line.v,
                                       line.page_table, line.page_size, line.ring, step.tok_pos, step.tok_slot,
                                       self.scale, self.softcap, self.window)
        elif step.mode == "prefill":
            a = ops.attn_prefill(qkv, self.n_heads, self.n_kv, self.head_dim, step.tok_pos, step.tok_row0,
                                 self.scale, self.softcap, self.window, step.seq_row0, step.seq_len, step.max_q_len)
        else:
            a = ops.attn_decode(qkv, self.n_heads, self.n_kv, self.head_dim, line.k, line.v, line.page_table,
                                line.page_size, line.ring, step.slots, line.slot_len, self.scale, self.softcap,
                                self.window, step.decode_splits, step.part_o, step.part_ml)
        return project(a, self.w_o)

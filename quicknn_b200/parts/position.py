"""Position encodings.  A position part places a step's tokens: it changes the queries and keys
of the packed q|k|v rows according to their positions and appends keys and values to the cache
(one kernel does both, so the two belong to one call).

Reference: GO_LLM_ROPE, angle = position * exp(-ln(theta) * 2j / head_dim), half-split
rotation of the whole head (src/backends/vulkan/shaders/tensor.comp:318-327).  The
frequencies are computed once on the host in float64 and rounded to float32; the
angle itself is formed in float32 on the device.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..kernels import ops
from .base import POSITIONS, HeadShape, Positions
from .spec import PartSpec


@POSITIONS.register("rotary")
class Rotary(Positions):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.head_dim = int(spec.params["head_dim"])
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or not (0 <= self.rotary_dim <= self.head_dim):
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.inv_freq: Optional[torch.Tensor] = None

    def prepare(self, device) -> None:
        j = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        f = torch.exp(-math.log(self.theta) * 2.0 * j / self.rotary_dim)
        self.inv_freq = f.to(torch.float32).to(device)

    def place(self, qkv, heads: HeadShape, step, line, append: bool = True) -> None:
        ops.rope_cache_write(qkv, heads.n_heads, heads.n_kv_heads, heads.head_dim, self.rotary_dim, self.inv_freq,
                             step.tok_pos, step.tok_slot, line.k, line.v, line.page_table, line.page_size, line.ring,
                             line.slot_len, bool(append and line.writes))

    def project_and_place(self, x, w_qkv, heads: HeadShape, step, line):
        """For the few rows of a decode step, rotation and append ride in the product's epilogue."""
        if step.mode != "decode" or not ops.qkv_rope_cache_fusable(x, w_qkv, heads.head_dim, self.rotary_dim):
            return None
        return ops.qkv_rope_cache(x, w_qkv, heads.n_heads, heads.n_kv_heads, heads.head_dim, self.inv_freq,
                                  step.tok_pos, step.tok_slot, line.k, line.v, line.page_table, line.page_size,
                                  line.ring, line.slot_len, line.writes)


@POSITIONS.register("none")
class NoPositions(Positions):
    """Keys and queries are used as projected (rotated width 0)."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.head_dim = int(spec.get("head_dim", 0))
        self.rotary_dim = 0
        self.inv_freq: Optional[torch.Tensor] = None

    def prepare(self, device) -> None:
        self.inv_freq = torch.zeros(0, dtype=torch.float32, device=device)

    def place(self, qkv, heads: HeadShape, step, line, append: bool = True) -> None:
        if append and line.writes:
            ops.cache_append(qkv, heads.n_heads, heads.n_kv_heads, heads.head_dim, step.tok_pos, step.tok_slot, line)

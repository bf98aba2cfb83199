"""Position encodings.  A position part hands the mixer's kernels what they need to
place a token: for ``rotary`` the table of frequencies and the rotated width.

Reference: GO_LLM_ROPE, angle = position * exp(-ln(theta) * 2j / head_dim), half-split
rotation of the whole head (src/backends/vulkan/shaders/tensor.comp:318-327).  The
frequencies are computed once on the host in float64 and rounded to float32; the
angle itself is formed in float32 on the device.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import POSITIONS, Positions
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

"""Feed-forward parts.  ``gated_mlp``: down(act(gate(x)) * up(x)).

Reference: two products and a GO_GEGLU dispatch, then the down product
(src/models/QuickNN.Models.Gemma2.pas:184-187; gelu_tanh at shaders/tensor.comp:23).
Gate and up are one product against the stacked matrix; for up to 64 rows the
activation is the product's epilogue.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .base import FEED_FORWARDS, FeedForward
from .linear import project, stack_rows
from .spec import PartSpec


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.activation = str(spec.get("activation", "gelu_tanh"))
        if self.activation not in ops.ACT_CODES:
            raise ValueError(f"activation {self.activation!r} is not one of {sorted(ops.ACT_CODES)}")
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        H, I = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        M = cls.PARAM_ROLE_MATRIX
        return {"gate_proj": ((I, H), M), "up_proj": ((I, H), M), "down_proj": ((H, I), M)}

    def load(self, tensors, compute_dtype, device) -> None:
        self.w_gate_up = stack_rows([tensors["gate_proj"], tensors["up_proj"]])
        self.w_down = tensors["down_proj"].contiguous()
        why = ops.linear_refusal(self.w_gate_up.dtype, self.hidden) or ops.linear_refusal(self.w_down.dtype, self.inter)
        if why:
            raise ValueError(f"gated feed-forward: {why}")

    def weight_bytes(self) -> int:
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def forward(self, x: torch.Tensor, step) -> torch.Tensor:
        h = project(x, self.w_gate_up, epilogue=ops.EPI_GATED, activation=self.activation)
        return project(h, self.w_down)

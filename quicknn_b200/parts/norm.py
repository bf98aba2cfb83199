"""Norms.  ``rmsnorm``: y = x / sqrt(mean(x^2) + eps) * (w + offset), offset 1 for the
"(1 + w)" flavour.  Reference: GO_NORM without centring and bias
(src/backends/vulkan/shaders/tensor.comp:63-72; Operations.pas:129-149); the
reference's files hold 1 + w already (src/models/QuickNN.Models.Gemma2.pas:58), the
checkpoints read here hold w.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..kernels import ops
from .base import NORMS, Norm
from .spec import PartSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.unit_offset = bool(spec.get("unit_offset", False))
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        return {"weight": ((int(spec.params["size"]),), cls.PARAM_ROLE_NORM)}

    def load(self, tensors, compute_dtype, device) -> None:
        self.weight = tensors["weight"].contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def __call__(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, self.unit_offset, out_dtype)

    def of_embedding(self, tokens: torch.Tensor, table: torch.Tensor, scale: float, out_dtype: torch.dtype):
        """(embedded rows, self(embedded rows)) in one kernel: the first norm of a model's first layer."""
        return ops.embed_rmsnorm(tokens, table, scale, self.weight, self.eps, self.unit_offset, out_dtype)

    def add_to(self, resid: torch.Tensor, y: torch.Tensor, then: Optional["RMSNorm"] = None,
               out_dtype: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
        """resid += self(y); returns then(resid) when ``then`` is given, in one kernel."""
        if then is None:
            return ops.add_rmsnorm(resid, y, self.weight, self.eps, self.unit_offset)
        return ops.add_rmsnorm(resid, y, self.weight, self.eps, self.unit_offset,
                               then.weight, then.eps, then.unit_offset, out_dtype)

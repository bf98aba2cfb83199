"""Weights of matrix products and the precision rule that goes with them."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from ..kernels import ops


def stack_rows(ws: Sequence[torch.Tensor]) -> torch.Tensor:
    """Stack [n_i, K] matrices into one [sum n_i, K] matrix (q|k|v, gate|up).  If the
    stored precisions differ, the wider one wins."""
    dt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
    return torch.cat([w.to(dt) for w in ws], dim=0).contiguous()


def project(x: torch.Tensor, w: torch.Tensor, *, epilogue: int = ops.EPI_NONE, cap: Optional[float] = None,
            activation: str = "gelu_tanh", out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """x w^T.  A matrix that was stored in 32-bit is multiplied in 32-bit even when the
    activations are bfloat16: x is widened, the result narrowed again."""
    if w.dtype == x.dtype:
        return ops.linear(x, w, epilogue=epilogue, cap=cap, activation=activation, out_dtype=out_dtype)
    if w.dtype == torch.float32 and x.dtype == torch.bfloat16:
        y = ops.linear(ops.cast(x, torch.float32), w, epilogue=epilogue, cap=cap, activation=activation)
        want = out_dtype or (torch.float32 if epilogue == ops.EPI_SOFTCAP else x.dtype)
        return ops.cast(y, want)
    if w.dtype == torch.bfloat16 and x.dtype == torch.float32:
        raise TypeError("a bfloat16 matrix in the float32 path: weights must be widened at load")
    raise TypeError(f"cannot multiply {x.dtype} activations with a {w.dtype} matrix")

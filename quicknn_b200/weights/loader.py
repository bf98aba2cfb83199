"""Checkpoint -> named device tensors, with one error that names every fault.

The reference looks each tensor up by name and raises on the first fault:
"Missing Gemma 2 tensor", "Invalid Gemma 2 normalization", "Invalid Gemma 2 matrix"
(src/models/QuickNN.Models.Gemma2.pas:50-66).  Here all missing names, unexpected
names, wrong shapes and unusable dtypes are collected and raised together.

Precision policy: in ``bfloat16`` mode a tensor keeps the precision it was stored
in (bf16 stays bf16, a tensor stored in 32-bit stays 32-bit); in ``float32`` mode
bf16 is widened exactly.  Integer tables become int32.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from .safetensors_io import TensorDirectory

_FLOATS = (torch.bfloat16, torch.float32)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightError(ValueError):
    def __init__(self, missing: Sequence[str], unexpected: Sequence[str],
                 wrong_shape: Sequence[Tuple[str, Tuple[int, ...], Tuple[int, ...]]],
                 wrong_dtype: Sequence[Tuple[str, str]], where: str = ""):
        self.missing, self.unexpected = list(missing), list(unexpected)
        self.wrong_shape, self.wrong_dtype = list(wrong_shape), list(wrong_dtype)
        lines = [f"checkpoint {where} does not fit the model:" if where
                 else "checkpoint does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for n, want, got in self.wrong_shape:
            lines.append(f"  wrong shape: {n} is {list(got)}, the model needs {list(want)}")
        for n, got in self.wrong_dtype:
            lines.append(f"  unusable dtype: {n} is {got} (bfloat16, float32 or an integer table expected)")
        super().__init__("\n".join(lines))


def check_names_and_shapes(expected: Mapping[str, Tuple[int, ...]],
                           found: Mapping[str, Tuple[Tuple[int, ...], torch.dtype]],
                           where: str = "") -> None:
    missing = [n for n in expected if n not in found]
    unexpected = [n for n in found if n not in expected]
    wrong_shape, wrong_dtype = [], []
    for n, want in expected.items():
        if n in found:
            shape, dt = found[n]
            if tuple(shape) != tuple(want):
                wrong_shape.append((n, tuple(want), tuple(shape)))
            if dt not in _FLOATS and dt not in _INTS:
                wrong_dtype.append((n, str(dt)))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(missing, unexpected, wrong_shape, wrong_dtype, where)


def place(t: torch.Tensor, compute_dtype: torch.dtype, device) -> torch.Tensor:
    """Apply the precision policy and move to the device."""
    if t.dtype in _INTS:
        return t.to(device=device, dtype=torch.int32)
    if compute_dtype == torch.float32:
        return t.to(device=device, dtype=torch.float32)
    # bfloat16 mode: keep the stored precision
    return t.to(device=device).contiguous()


def load_named_tensors(model_dir: str, expected: Mapping[str, Tuple[int, ...]],
                       compute_dtype: torch.dtype, device) -> Dict[str, torch.Tensor]:
    d = TensorDirectory.open(model_dir)
    try:
        found = {n: d.shape_dtype(n) for n in d.names()}
        check_names_and_shapes(expected, found, where=model_dir)
        out: Dict[str, torch.Tensor] = {}
        for n in expected:
            out[n] = place(d.tensor(n), compute_dtype, device)
        return out
    finally:
        d.close()


def check_state_dict(expected: Mapping[str, Tuple[int, ...]],
                     tensors: Mapping[str, torch.Tensor]) -> None:
    check_names_and_shapes(expected, {n: (tuple(t.shape), t.dtype) for n, t in tensors.items()},
                           where="(in memory)")

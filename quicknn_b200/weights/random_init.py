"""Random weights from a configuration and a seed; optionally written as a model folder.

The reference has no such mode.  Matrices are drawn from N(0, init_std) (the
configuration's ``initializer_range``), norm weights from N(0, norm_std); each tensor
has a generator of its own, seeded from the seed and the tensor's name, so a tensor's
values do not depend on which other tensors exist.  Values are drawn in float32 and
rounded to the stored dtype.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Optional, Tuple

import torch

from ..config.base import Architecture, ModelConfig
from ..parts.base import Part
from ..parts.layout import expected_tensors
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensors(arch: Architecture, cfg: ModelConfig, seed: int, dtype: torch.dtype = torch.bfloat16,
                   norm_std: Optional[float] = None, device="cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    spec = arch.build_spec(cfg)
    nstd = spec.init_norm_std if norm_std is None else norm_std
    for name, (shape, role) in expected_tensors(spec).items():
        g = torch.Generator(device=device)
        g.manual_seed(_tensor_seed(seed, name))
        std = nstd if role == Part.PARAM_ROLE_NORM else spec.init_std
        t = torch.empty(shape, dtype=torch.float32, device=device)
        t.normal_(0.0, std, generator=g)
        yield name, t.to(dtype)


def write_model_folder(path: str, arch: Architecture, cfg: ModelConfig, seed: int,
                       dtype: torch.dtype = torch.bfloat16, norm_std: Optional[float] = None,
                       device="cpu") -> str:
    """Write ``config.json`` and ``model.safetensors`` for a random model.  ``device`` is where
    the values are drawn (a CUDA device draws a large model in seconds; its generator gives
    other values than the host's for the same seed)."""
    os.makedirs(path, exist_ok=True)
    raw = cfg.to_dict()
    if not raw.get("architectures"):
        raw["architectures"] = [arch.name]        # the registry finds the model class by this name
    raw["torch_dtype"] = "bfloat16" if dtype == torch.bfloat16 else "float32"
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(raw, fh, indent=1)
    tensors: Dict[str, torch.Tensor] = {n: t.cpu() for n, t in random_tensors(arch, cfg, seed, dtype, norm_std, device)}
    write_safetensors(os.path.join(path, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": str(seed)})
    return path

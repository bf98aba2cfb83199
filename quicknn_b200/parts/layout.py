"""From a model's layout to the list of checkpoint tensors it needs (no GPU involved)."""
from __future__ import annotations

from typing import Dict, Tuple

from .base import BLOCKS, NORMS, Part
from .spec import ModelSpec


def expected_tensors(spec: ModelSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
    """checkpoint name -> (shape, role)."""
    out: Dict[str, Tuple[Tuple[int, ...], str]] = {}

    def put(name, shape, role):
        if name in out and out[name][0] != tuple(shape):
            raise ValueError(f"tensor {name} is asked for with two shapes: {out[name][0]} and {tuple(shape)}")
        out[name] = (tuple(shape), role)

    put(spec.embedding.tensor, (spec.embedding.vocab_size, spec.embedding.hidden_size), Part.PARAM_ROLE_MATRIX)
    for li, layer in enumerate(spec.layers):
        shapes = BLOCKS.get(layer.block.kind).layer_param_shapes(layer)
        for local, (shape, role) in shapes.items():
            if local not in layer.tensors:
                raise ValueError(f"layer {li}: the architecture names no checkpoint tensor for '{local}'")
            put(layer.tensors[local], shape, role)
        extra = sorted(set(layer.tensors) - set(shapes))
        if extra:
            raise ValueError(f"layer {li}: the architecture names tensors that no part takes: {extra}")
    for k, (shape, role) in NORMS.get(spec.head.norm.kind).param_shapes(spec.head.norm).items():
        put(spec.head.norm_tensor if k == "weight" else f"{spec.head.norm_tensor}.{k}", shape, role)
    if not spec.head.tied:
        put(spec.head.tensor, (spec.head.vocab_size, spec.head.hidden_size), Part.PARAM_ROLE_MATRIX)
    return out

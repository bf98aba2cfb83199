"""Plain-data description of a model: which parts, with which sizes, in which order.

An architecture turns its typed configuration into a ``ModelSpec``.  Everything
below the architecture (parts, cache, step function, loader) works from these
records only, so no part knows which model it is in.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Mapping, Optional, Tuple


@dataclasses.dataclass(frozen=True)
class PartSpec:
    """A part named by ``kind`` (a key of one of the part registries) and its parameters."""

    kind: str
    params: Mapping[str, Any] = dataclasses.field(default_factory=dict)

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    """One layer = one block arrangement around a mixer and a feed-forward.

    ``tensors`` maps the local parameter names that the parts declare
    (for instance ``"mixer.q_proj"``) to tensor names in the checkpoint.
    """

    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norms: Mapping[str, PartSpec]
    tensors: Mapping[str, str]


@dataclasses.dataclass(frozen=True)
class ScheduleEntry:
    """One executed layer.  ``layer`` indexes ``ModelSpec.layers`` (weights);
    ``cache`` names the cache line that this execution reads; ``writes_cache``
    is False when it only reads a line another entry wrote."""

    layer: int
    cache: int
    writes_cache: bool = True


@dataclasses.dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    hidden_size: int
    scale: float                      # multiplies the looked-up row (fp32 scalar)
    tensor: str                       # checkpoint name of the table


@dataclasses.dataclass(frozen=True)
class HeadSpec:
    vocab_size: int
    hidden_size: int
    tied: bool                        # use the embedding table as the output matrix
    tensor: Optional[str]             # checkpoint name when not tied
    softcap: Optional[float]          # cap * tanh(logit / cap), None = off
    norm: PartSpec = None             # final norm
    norm_tensor: str = ""


@dataclasses.dataclass(frozen=True)
class ModelSpec:
    name: str
    hidden_size: int
    embedding: EmbeddingSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    head: HeadSpec
    max_positions: int
    stop_ids: Tuple[int, ...] = ()
    # standard deviations that the random-weights mode uses: matrices, norm weights
    init_std: float = 0.02
    init_norm_std: float = 0.1

    def n_cache_lines(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(n_layers))

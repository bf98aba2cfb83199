"""Interfaces of the parts and the registries that name them.

A model is put together from five kinds of part.  Each is chosen by a
``PartSpec`` (kind + parameters) that the architecture wrote into the model's
layout, layer by layer; no part knows which model it is in.

=============  ==============================================================
kind of part   interface
=============  ==============================================================
Norm           ``param_shapes(spec)``; ``load(tensors)``; ``__call__(x, out_dtype)``
Positions      ``param_shapes`` (usually none); ``prepare(device)``;
               ``place(qkv, heads, step, line, append)`` puts the step's
               positions into its queries and keys and appends keys and
               values to the cache line; ``project_and_place`` may fuse that
               with the q|k|v product
Mixer          ``param_shapes``; ``load``; ``cache_need()`` (growing keys/values,
               possibly windowed), ``state_need()`` (fixed-size per-sequence
               state), ``scratch_need(step)`` (bytes of scratch for one step),
               ``schedule(step)`` (what it decides from a step's shape that a
               captured decode graph bakes in); ``forward(x, step, cache_line)``
FeedForward    ``param_shapes``; ``load``; ``forward(x, step)``
Block          arrangement of the four above around the residual stream:
               ``forward(resid, step, cache_line)``
=============  ==============================================================

``param_shapes`` is a classmethod over the spec so that the expected tensor list
(and random weights) can be produced without a GPU.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, Mapping, Optional, Tuple, Type

from .spec import PartSpec


class PartRegistry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: Dict[str, type] = {}

    def register(self, kind: str, cls: Optional[type] = None, *, replace: bool = False):
        def deco(c):
            if kind in self._kinds and not replace and self._kinds[kind] is not c:
                raise KeyError(f"{self.what} kind '{kind}' is already registered")
            self._kinds[kind] = c
            return c
        return deco(cls) if cls is not None else deco

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def get(self, kind: str) -> type:
        try:
            return self._kinds[kind]
        except KeyError:
            raise KeyError(f"unknown {self.what} kind '{kind}'; registered: {sorted(self._kinds)}") from None

    def kinds(self):
        return sorted(self._kinds)


NORMS = PartRegistry("norm")
POSITIONS = PartRegistry("position encoding")
MIXERS = PartRegistry("mixer")
FEED_FORWARDS = PartRegistry("feed-forward")
BLOCKS = PartRegistry("block")


# ---- what a mixer asks of the cache ------------------------------------------------

@dataclasses.dataclass(frozen=True)
class CacheNeed:
    """Keys and values that grow with the sequence.  ``window`` = None keeps every
    position; an integer keeps the last ``window`` positions (a ring)."""

    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def group_key(self) -> Tuple:
        return (self.n_kv_heads, self.head_dim, self.window)


@dataclasses.dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-sequence state: ``shape`` elements of ``dtype`` ("float32",
    "bfloat16" or "compute"), zeroed when a slot is handed out, never rewound."""

    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclasses.dataclass(frozen=True)
class HeadShape:
    """How the columns of a packed q|k|v row are cut: ``n_heads`` query heads, then ``n_kv_heads``
    key heads, then as many value heads, ``head_dim`` columns each."""

    n_heads: int
    n_kv_heads: int
    head_dim: int

    @property
    def width(self) -> int:
        return (self.n_heads + 2 * self.n_kv_heads) * self.head_dim


class Part:
    """Common base: parameters by local name."""

    PARAM_ROLE_MATRIX = "matrix"
    PARAM_ROLE_NORM = "norm"

    def __init__(self, spec: PartSpec):
        self.spec = spec

    @classmethod
    def param_shapes(cls, spec: PartSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        """local name -> (shape, role).  The role picks the standard deviation that the
        random-weights mode draws with."""
        return {}

    def load(self, tensors: Mapping[str, Any], compute_dtype, device) -> None:
        """Take the tensors named in ``param_shapes`` (already on the device)."""

    def weight_bytes(self) -> int:
        return 0

    def schedule(self, step) -> tuple:
        """What this part decides from the step's shape and length classes that a captured launch sequence
        would bake in (grid sizes, kernels chosen), as a hashable value; ``()`` when nothing.  The engine keeps
        one decode graph per batch size and distinct schedule of the model, so two length classes that lead to
        the same decisions share a graph."""
        return ()

    def scratch_need(self, step) -> int:
        """Bytes of scratch (global memory beyond inputs and outputs) that this part wants for a
        step of this shape: ``step.mode``, ``step.n_seqs``, ``step.n_tokens``, ``step.max_seq`` and
        ``step.tuning`` are set when this is asked.  The engine allocates the largest need of all
        parts once per shape and hands it to every part as ``step.scratch`` (uint8, 256-byte
        aligned); parts run one after another, so they share it."""
        return 0


class Norm(Part):
    def __call__(self, x, out_dtype=None):  # pragma: no cover - interface
        raise NotImplementedError


class Positions(Part):
    """A position encoding owns what it does to queries and keys.  The mixer hands it the packed
    q|k|v rows of the step and never looks inside."""

    def prepare(self, device) -> None:
        pass

    def place(self, qkv, heads: HeadShape, step, line, append: bool = True) -> None:  # pragma: no cover - interface
        """Put the positions ``step.tok_pos`` into the queries and keys of ``qkv``
        ([tokens, heads.width], in place) and, with ``append``, write the keys and values of the
        rows whose slot is not negative to the cache line (``line.writes`` permitting)."""
        raise NotImplementedError

    def project_and_place(self, x, w_qkv, heads: HeadShape, step, line):
        """``x w_qkv^T`` with ``place(..., append=True)`` done in the same kernel, or None when this
        encoding (or these sizes) has no such kernel; the mixer then projects and calls ``place``."""
        return None


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, x, step, line):  # pragma: no cover - interface
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x, step):  # pragma: no cover - interface
        raise NotImplementedError


class Block(Part):
    def first_norm(self):
        """The norm that this block applies to its input first, or None.  When it gives one,
        the block that runs before it may apply it (fused with its own last add) and hand
        the result over as ``normed``."""
        return None

    def forward(self, resid, step, line, normed=None, next_norm=None):  # pragma: no cover - interface
        """Update the float32 residual stream in place.  Returns it, or the pair
        (residual stream, next_norm(residual stream)) when ``next_norm`` is given."""
        raise NotImplementedError

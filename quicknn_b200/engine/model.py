"""A model: embedding, the layers in the order of the schedule, final norm and head.

Built from a ``ModelSpec`` only; which architecture wrote the spec is not known here.
Forward order as in the reference (src/models/QuickNN.Models.Gemma2.pas:158-196):
gather and scale the embedding rows; the layers; then, for the rows whose logits are
wanted only (the reference: the last row), final norm, the tied head and the softcap.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ..config.base import Architecture, ModelConfig, load_config
from ..kernels import ops
from ..parts.base import BLOCKS, NORMS, CacheNeed, StateNeed
from ..parts.layout import expected_tensors
from ..parts.linear import project
from ..parts.spec import ModelSpec
from ..weights.loader import check_state_dict, load_named_tensors, place
from .batch import StepBatch

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def as_dtype(d) -> torch.dtype:
    if isinstance(d, torch.dtype):
        if d not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype must be bfloat16 or float32, got {d}")
        return d
    try:
        return DTYPES[str(d)]
    except KeyError:
        raise ValueError(f"compute dtype must be one of {sorted(DTYPES)}, got {d!r}") from None


class Model:
    def __init__(self, arch: Architecture, config: ModelConfig, tensors: Mapping[str, torch.Tensor],
                 dtype, device):
        self.arch, self.config = arch, config
        self.spec: ModelSpec = arch.build_spec(config)
        self.dtype = as_dtype(dtype)
        self.device = torch.device(device)
        spec = self.spec
        self.blocks = []
        for layer in spec.layers:
            blk = BLOCKS.get(layer.block.kind)(layer)
            local = {ln: tensors[cn] for ln, cn in layer.tensors.items()}
            blk.load(local, self.dtype, self.device)
            self.blocks.append(blk)
        self.embedding = tensors[spec.embedding.tensor].contiguous()
        self.final_norm = NORMS.get(spec.head.norm.kind)(spec.head.norm)
        self.final_norm.load({"weight": tensors[spec.head.norm_tensor]}, self.dtype, self.device)
        self.head = self.embedding if spec.head.tied else tensors[spec.head.tensor].contiguous()
        why = ops.linear_refusal(self.head.dtype, spec.hidden_size)
        if why:
            raise ValueError(f"output head: {why}")
        self._check_schedule()

    # ---- construction --------------------------------------------------------------
    @classmethod
    def from_folder(cls, model_dir: str, dtype="bfloat16", device="cuda:0") -> "Model":
        arch, cfg = load_config(model_dir)
        spec = arch.build_spec(cfg)
        want = {n: s for n, (s, _) in expected_tensors(spec).items()}
        tensors = load_named_tensors(model_dir, want, as_dtype(dtype), device)
        return cls(arch, cfg, tensors, dtype, device)

    @classmethod
    def from_tensors(cls, arch: Architecture, cfg: ModelConfig, tensors: Mapping[str, torch.Tensor],
                     dtype="bfloat16", device="cuda:0") -> "Model":
        spec = arch.build_spec(cfg)
        check_state_dict({n: s for n, (s, _) in expected_tensors(spec).items()}, tensors)
        placed = {n: place(t, as_dtype(dtype), device) for n, t in tensors.items()}
        return cls(arch, cfg, placed, dtype, device)

    # ---- what the cache has to provide ------------------------------------------------
    def _check_schedule(self) -> None:
        spec = self.spec
        writers: Dict[int, int] = {}
        for e in spec.schedule:
            if not (0 <= e.layer < len(self.blocks)):
                raise ValueError(f"schedule names layer {e.layer}, the model has {len(self.blocks)}")
            if e.writes_cache:
                if e.cache in writers:
                    raise ValueError(f"cache line {e.cache} is written by two schedule entries")
                writers[e.cache] = e.layer
        for e in spec.schedule:
            if not e.writes_cache:
                if e.cache not in writers:
                    raise ValueError(f"schedule entry of layer {e.layer} reads cache line {e.cache} that nobody writes")
                a = self.blocks[e.layer].mixer.cache_need()
                b = self.blocks[writers[e.cache]].mixer.cache_need()
                if a is None or b is None or (a.n_kv_heads, a.head_dim) != (b.n_kv_heads, b.head_dim):
                    raise ValueError(f"layer {e.layer} cannot read cache line {e.cache}: its keys have another shape")

    def cache_needs(self) -> Tuple[List[Optional[CacheNeed]], List[Optional[StateNeed]]]:
        n = self.spec.n_cache_lines()
        needs: List[Optional[CacheNeed]] = [None] * n
        states: List[Optional[StateNeed]] = [None] * n
        for e in self.spec.schedule:
            if e.writes_cache:
                needs[e.cache] = self.blocks[e.layer].mixer.cache_need()
                states[e.cache] = self.blocks[e.layer].mixer.state_need()
        return needs, states

    def scratch_need(self, step) -> int:
        """Bytes of scratch that a step of this shape needs: the largest need of the layers that run
        (they run one after another and share it)."""
        return max([self.blocks[e.layer].scratch_need(step) for e in self.spec.schedule] or [0])

    def schedule(self, step) -> tuple:
        """The decisions of the layers that run, in order (see ``Part.schedule``)."""
        return tuple(self.blocks[e.layer].schedule(step) for e in self.spec.schedule)

    def weight_bytes(self) -> int:
        n = self.embedding.numel() * self.embedding.element_size()
        if self.head is not self.embedding:
            n += self.head.numel() * self.head.element_size()
        return n + self.final_norm.weight_bytes() + sum(b.weight_bytes() for b in self.blocks)

    def step_weight_bytes(self) -> int:
        """Bytes of weights that one decode step reads: every scheduled layer's matrices and
        norms once, the head once (the embedding rows it gathers are negligible)."""
        n = self.head.numel() * self.head.element_size() + self.final_norm.weight_bytes()
        return n + sum(self.blocks[e.layer].weight_bytes() for e in self.spec.schedule)

    # ---- forward ----------------------------------------------------------------------
    def forward(self, step: StepBatch, cache, reduce=None):
        """Logits (float32, [wanted rows, vocab]) of the rows in ``step.want_rows``; with ``reduce`` (a
        callable on the logits that launches device work only, such as a sampler) what it returns.  If
        ``reduce`` has a method ``head(rows, weight, softcap)`` it is offered the rows that go into the
        output head first and may return its result without the logits ever being written."""
        spec = self.spec
        sched = spec.schedule
        first = self.blocks[sched[0].layer].first_norm() if sched else None
        if hasattr(first, "of_embedding"):
            # the first layer's first norm in the embedding's kernel; the layer is handed its input normed
            x, normed = first.of_embedding(step.tokens, self.embedding, spec.embedding.scale, step.act_dtype)
        else:
            x, normed = ops.embed(step.tokens, self.embedding, spec.embedding.scale), None
        for i, e in enumerate(sched):
            line = cache.line(e.cache, writes=e.writes_cache)
            # the first norm of the layer that runs next is applied by this one, in the kernel
            # that adds this layer's last sublayer to the residual stream
            nxt = self.blocks[sched[i + 1].layer].first_norm() if i + 1 < len(sched) else None
            out = self.blocks[e.layer].forward(x, step, line, normed=normed, next_norm=nxt)
            x, normed = out if nxt is not None else (out, None)
        return self.logits_of_rows(x, None if step.want_every_row else step.want_rows, step.act_dtype, reduce)

    def logits_of_rows(self, x: torch.Tensor, rows: Optional[torch.Tensor], act_dtype: torch.dtype, reduce=None):
        """Final norm, head and softcap of the rows ``rows`` of the residual stream (None: every row)."""
        if rows is not None and rows.numel() == 0:
            empty = torch.empty((0, self.spec.head.vocab_size), dtype=torch.float32, device=x.device)
            return empty if reduce is None else reduce(empty)
        picked = x if rows is None else ops.gather_rows(x, rows, torch.float32)
        n = self.final_norm(picked, act_dtype)
        cap = self.spec.head.softcap
        if reduce is not None and hasattr(reduce, "head"):
            out = reduce.head(n, self.head, cap)
            if out is not None:
                return out
        logits = project(n, self.head, epilogue=ops.EPI_SOFTCAP, cap=cap, out_dtype=torch.float32)
        return logits if reduce is None else reduce(logits)

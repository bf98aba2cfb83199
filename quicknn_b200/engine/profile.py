"""Where a step's time goes: CUDA events per step and per kind of part.

The reference can put timestamp queries around its command buffer
(src/backends/vulkan/QuickNN.Vulkan.Context.Implementation.inc:221-225) and reports time to the
first token, decode seconds and tokens per second for every reply
(src/models/QuickNN.Models.LLM.pas:851-857).  Here a ``StepProfiler`` wraps an engine for the
length of a ``with`` block: every step is bracketed by two events, and inside it every call of a
mixer, a feed-forward, a norm, the embedding, the output head and the sampler.  Steps run eagerly
meanwhile (events cannot be recorded inside a captured graph), so the per-step figures are those of
eager launches; the shares between the kinds of part are what the table is for.

    with StepProfiler(llm.engine) as prof:
        llm.generate(prompts, options)
    print(prof.table())

``StepProfiler(engine, nvtx=True)`` also opens an NVTX range of the part's kind around every call.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..kernels import ops
from ..parts.norm import RMSNorm
from ..sampling.sampler import Sampler

KINDS = ("embedding", "norms and residual", "mixer", "feed-forward", "head", "sampling")


class StepProfiler:
    def __init__(self, engine, nvtx: bool = False):
        self.engine = engine
        self.nvtx = nvtx                         # also an NVTX range around every call of a part, for a timeline tool
        self._undo: List[Tuple[object, str, object]] = []
        self._open: List[list] = []            # the calls that are running: [kind, start, stop, time of the calls inside]
        self._calls: List[list] = []
        self._steps: List[Tuple[str, int, int, torch.cuda.Event, torch.cuda.Event]] = []
        self._graphs: Optional[bool] = None

    # ---- wrapping ------------------------------------------------------------------------------
    def _timed(self, kind: str, fn):
        def call(*a, **kw):
            rec = [kind, torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), []]
            if self._open:
                self._open[-1][3].append(rec)
            else:
                self._calls.append(rec)
            self._open.append(rec)
            if self.nvtx:
                torch.cuda.nvtx.range_push(kind)
            rec[1].record()
            try:
                return fn(*a, **kw)
            finally:
                rec[2].record()
                if self.nvtx:
                    torch.cuda.nvtx.range_pop()
                self._open.pop()
        return call

    def _patch(self, owner, name: str, kind: str) -> None:
        old = getattr(owner, name)
        self._undo.append((owner, name, owner.__dict__.get(name, _MISSING) if not isinstance(owner, type) else old))
        setattr(owner, name, self._timed(kind, old))

    def __enter__(self) -> "StepProfiler":
        eng, model = self.engine, self.engine.model
        self._graphs, eng.use_graphs = eng.use_graphs, False
        for blk in model.blocks:
            self._patch(blk.mixer, "forward", "mixer")
            self._patch(blk.ff, "forward", "feed-forward")
        self._patch(RMSNorm, "__call__", "norms and residual")
        self._patch(RMSNorm, "add_to", "norms and residual")
        self._patch(ops, "add_", "norms and residual")
        self._patch(ops, "embed", "embedding")
        self._patch(ops, "embed_rmsnorm", "embedding")
        self._patch(model, "logits_of_rows", "head")
        self._patch(Sampler, "__call__", "sampling")
        self._patch(Sampler, "head", "sampling")
        for name in ("step", "decode"):
            old = getattr(eng, name)
            self._undo.append((eng, name, _MISSING))

            def stepped(*a, _old=old, _name=name, **kw):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                try:
                    return _old(*a, **kw)
                finally:
                    e1.record()
                    entries = a[0]
                    rows = len(entries)
                    toks = rows if _name == "decode" else sum(len(t) for _, t in entries)
                    mode = "decode" if toks == rows and _name == "decode" else ("prompt" if toks > rows else "single")
                    self._steps.append((mode, rows, toks, e0, e1))
            setattr(eng, name, stepped)
        return self

    def __exit__(self, *exc) -> None:
        for owner, name, old in reversed(self._undo):
            if old is _MISSING:
                try:
                    delattr(owner, name)
                except AttributeError:
                    pass
            else:
                setattr(owner, name, old)
        self._undo.clear()
        self.engine.use_graphs = self._graphs
        torch.cuda.synchronize(self.engine.device)

    # ---- results -------------------------------------------------------------------------------
    def by_kind(self) -> Dict[str, float]:
        """Milliseconds per kind of part, each call counted without the calls inside it."""
        out = {k: 0.0 for k in KINDS}

        def walk(rec) -> float:
            total = rec[1].elapsed_time(rec[2])
            inner = sum(walk(r) for r in rec[3])
            out[rec[0]] = out.get(rec[0], 0.0) + max(0.0, total - inner)
            return total
        for rec in self._calls:
            walk(rec)
        return out

    def steps(self) -> Dict[str, Tuple[int, int, float]]:
        """mode -> (steps, tokens, milliseconds)."""
        out: Dict[str, List[float]] = {}
        for mode, rows, toks, e0, e1 in self._steps:
            s = out.setdefault(mode, [0, 0, 0.0])
            s[0] += 1
            s[1] += toks
            s[2] += e0.elapsed_time(e1)
        return {k: (int(v[0]), int(v[1]), float(v[2])) for k, v in out.items()}

    def table(self) -> str:
        torch.cuda.synchronize(self.engine.device)
        lines = ["steps (launched eagerly while profiling):"]
        for mode, (n, toks, ms) in sorted(self.steps().items()):
            lines.append(f"  {mode:8s} {n:6d} steps {toks:9d} tokens {ms:10.3f} ms {toks / max(ms, 1e-9) * 1e3:12.1f} tokens/s")
        kinds = self.by_kind()
        total = sum(kinds.values()) or 1.0
        lines.append("time on the device by kind of part:")
        for k in KINDS:
            lines.append(f"  {k:20s} {kinds[k]:10.3f} ms {100.0 * kinds[k] / total:6.1f} %")
        return "\n".join(lines)


class _Missing:
    pass


_MISSING = _Missing()

"""Blocks: how norms, mixer and feed-forward sit around the residual stream.

``sandwich`` (Gemma 2, src/models/QuickNN.Models.Gemma2.pas:166-189): a norm before
and after each sublayer, the post-norm applied to the sublayer's output before it
is added:  x += post(mixer(pre(x)));  x += post(ff(pre(x))).
``prenorm``: x += mixer(pre(x));  x += ff(pre(x)).

The residual stream is float32 in both precisions.  When the norms are RMSNorm the
post-norm, the add and the next pre-norm run as one kernel; that also holds across the
border of two layers: ``forward`` may be handed its input already normed (``normed``) and
may be asked to apply the first norm of the layer that runs next (``next_norm``).
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from ..kernels import ops
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block
from .norm import RMSNorm
from .spec import LayerSpec, PartSpec


class _LayerParts(Block):
    NORM_NAMES: Tuple[str, ...] = ()

    def __init__(self, layer: LayerSpec):
        super().__init__(layer.block)
        self.layer = layer
        self.mixer = MIXERS.get(layer.mixer.kind)(layer.mixer)
        self.ff = FEED_FORWARDS.get(layer.feed_forward.kind)(layer.feed_forward)
        missing = [n for n in self.NORM_NAMES if n not in layer.norms]
        if missing:
            raise ValueError(f"block '{layer.block.kind}' needs the norms {missing}")
        self.norms = {n: NORMS.get(layer.norms[n].kind)(layer.norms[n]) for n in self.NORM_NAMES}

    @classmethod
    def layer_param_shapes(cls, layer: LayerSpec) -> Dict[str, Tuple[Tuple[int, ...], str]]:
        out: Dict[str, Tuple[Tuple[int, ...], str]] = {}
        for k, v in MIXERS.get(layer.mixer.kind).param_shapes(layer.mixer).items():
            out["mixer." + k] = v
        for k, v in FEED_FORWARDS.get(layer.feed_forward.kind).param_shapes(layer.feed_forward).items():
            out["ff." + k] = v
        for n in cls.NORM_NAMES:
            for k, v in NORMS.get(layer.norms[n].kind).param_shapes(layer.norms[n]).items():
                out[f"norms.{n}.{k}"] = v
        return out

    def load(self, tensors, compute_dtype, device) -> None:
        def sub(prefix):
            return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}
        self.mixer.load(sub("mixer."), compute_dtype, device)
        self.ff.load(sub("ff."), compute_dtype, device)
        for n, part in self.norms.items():
            part.load(sub(f"norms.{n}."), compute_dtype, device)

    def weight_bytes(self) -> int:
        return self.mixer.weight_bytes() + self.ff.weight_bytes() + sum(n.weight_bytes() for n in self.norms.values())

    def scratch_need(self, step) -> int:
        return max(self.mixer.scratch_need(step), self.ff.scratch_need(step))

    def schedule(self, step) -> tuple:
        return self.mixer.schedule(step) + self.ff.schedule(step)


@BLOCKS.register("sandwich")
class SandwichBlock(_LayerParts):
    NORM_NAMES = ("pre_mixer", "post_mixer", "pre_ff", "post_ff")

    def first_norm(self):
        return self.norms["pre_mixer"]

    def forward(self, resid: torch.Tensor, step, line, normed=None, next_norm=None):
        """Returns the residual stream, or (residual stream, next_norm(residual stream)) when
        ``next_norm`` (an RMSNorm) is given."""
        nm = self.norms
        act = step.act_dtype
        n = normed if normed is not None else nm["pre_mixer"](resid, act)
        y = self.mixer.forward(n, step, line)
        if isinstance(nm["post_mixer"], RMSNorm) and isinstance(nm["pre_ff"], RMSNorm):
            n = nm["post_mixer"].add_to(resid, y, then=nm["pre_ff"], out_dtype=act)
        else:
            ops.add_(resid, nm["post_mixer"](y, act))
            n = nm["pre_ff"](resid, act)
        y = self.ff.forward(n, step)
        if isinstance(nm["post_ff"], RMSNorm):
            if isinstance(next_norm, RMSNorm):
                return resid, nm["post_ff"].add_to(resid, y, then=next_norm, out_dtype=act)
            nm["post_ff"].add_to(resid, y)
        else:
            ops.add_(resid, nm["post_ff"](y, act))
        if next_norm is not None:
            return resid, next_norm(resid, act)
        return resid


@BLOCKS.register("prenorm")
class PreNormBlock(_LayerParts):
    NORM_NAMES = ("pre_mixer", "pre_ff")

    def first_norm(self):
        return self.norms["pre_mixer"]

    def forward(self, resid: torch.Tensor, step, line, normed=None, next_norm=None):
        act = step.act_dtype
        n = normed if normed is not None else self.norms["pre_mixer"](resid, act)
        ops.add_(resid, self.mixer.forward(n, step, line))
        ops.add_(resid, self.ff.forward(self.norms["pre_ff"](resid, act), step))
        if next_norm is not None:
            return resid, next_norm(resid, act)
        return resid

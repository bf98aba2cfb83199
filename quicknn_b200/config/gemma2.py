"""Gemma 2: typed configuration and its layout as parts.

Keys, defaults and validity rules follow the reference's constructor
(src/models/QuickNN.Models.Gemma2.pas:76-96): ``rope_theta`` 10000,
``rms_norm_eps`` 1e-6, ``sliding_window`` 4096, ``attn_logit_softcapping`` 50,
``final_logit_softcapping`` 30, ``query_pre_attn_scalar`` = ``head_dim``.
Differences, on purpose: a softcap of ``null`` switches it off (the shader already
treats cap <= 0 as off, shaders/attention.comp:27, while the host check forbids
it, Gemma2.pas:93); checkpoint tensors carry Hugging Face names and norm weights
are stored as ``w`` and applied as ``1 + w`` (the reference's GGUF files store
``1 + w``, Gemma2.pas:58).

Layer pattern: even layer indices attend through the sliding window, odd ones
see every key (``if not Odd(I) then Window := FWindow``, Gemma2.pas:177).  An
optional ``layer_types`` list overrides the pattern layer by layer.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, List, Optional, Tuple

from ..parts.spec import (EmbeddingSpec, HeadSpec, LayerSpec, ModelSpec, PartSpec,
                          default_schedule)
from .base import (Architecture, ModelConfig, as_bool, as_float, as_id_tuple, as_int,
                   as_opt_float, as_str_tuple, register_architecture)

_GELU_TANH_NAMES = ("gelu_pytorch_tanh", "gelu_tanh", "gelu_new")
LOCAL, GLOBAL = "sliding_attention", "full_attention"


def _f(conv, **kw):
    md = {"convert": conv}
    md.update({k: v for k, v in kw.items() if k in ("key", "required")})
    if "default" in kw:
        return dataclasses.field(default=kw["default"], metadata=md)
    md["required"] = True
    return dataclasses.field(default=None, metadata=md)


@dataclasses.dataclass(frozen=True)
class Gemma2Config(ModelConfig):
    hidden_size: int = _f(as_int)
    intermediate_size: int = _f(as_int)
    num_attention_heads: int = _f(as_int)
    num_key_value_heads: int = _f(as_int)
    head_dim: int = _f(as_int)
    vocab_size: int = _f(as_int)
    num_hidden_layers: int = _f(as_int)
    max_position_embeddings: int = _f(as_int)
    rope_theta: float = _f(as_float, default=10000.0)
    rms_norm_eps: float = _f(as_float, default=1e-6)
    sliding_window: int = _f(as_int, default=4096)
    attn_logit_softcapping: Optional[float] = _f(as_opt_float, default=50.0)
    final_logit_softcapping: Optional[float] = _f(as_opt_float, default=30.0)
    # None stands for "head_dim" (Gemma2.pas:88)
    query_pre_attn_scalar: Optional[float] = _f(as_opt_float, default=None)
    eos_token_id: Tuple[int, ...] = _f(as_id_tuple, default=())
    bos_token_id: Optional[int] = _f(lambda v: None if v is None else as_int(v), default=None)
    pad_token_id: Optional[int] = _f(lambda v: None if v is None else as_int(v), default=None)
    hidden_activation: str = _f(str, default="gelu_pytorch_tanh")
    hidden_act: str = _f(str, default="gelu_pytorch_tanh")
    tie_word_embeddings: bool = _f(as_bool, default=True)
    attention_bias: bool = _f(as_bool, default=False)
    layer_types: Tuple[str, ...] = _f(as_str_tuple, default=())
    initializer_range: float = _f(as_float, default=0.02)
    model_type: str = _f(str, default="gemma2")
    architectures: Tuple[str, ...] = _f(as_str_tuple, default=("Gemma2ForCausalLM",))
    torch_dtype: str = _f(str, default="bfloat16")

    @classmethod
    def architecture_names(cls) -> Tuple[str, ...]:
        return ("Gemma2ForCausalLM", "gemma2")

    # ---- derived -----------------------------------------------------------------
    @property
    def attention_scale(self) -> float:
        """1/sqrt(query_pre_attn_scalar) (``FScale := 1 / Sqrt(QueryScale)``, Gemma2.pas:96)."""
        q = self.query_pre_attn_scalar
        return 1.0 / math.sqrt(float(self.head_dim) if q is None else q)

    def layer_is_local(self, index: int) -> bool:
        if self.layer_types:
            return self.layer_types[index] == LOCAL
        return index % 2 == 0

    # ---- rules -------------------------------------------------------------------
    def problems(self) -> List[str]:
        p: List[str] = []
        pos = lambda name: getattr(self, name) is not None and getattr(self, name) >= 1  # noqa: E731
        for name in ("hidden_size", "intermediate_size", "num_attention_heads",
                     "num_key_value_heads", "vocab_size", "sliding_window"):
            if not pos(name):
                p.append(f"{name} must be >= 1 (got {getattr(self, name)})")
        if not (1 <= (self.num_hidden_layers or 0) <= 256):
            p.append(f"num_hidden_layers must be in 1..256 (got {self.num_hidden_layers})")
        if pos("num_attention_heads") and pos("num_key_value_heads") and \
                self.num_attention_heads % self.num_key_value_heads != 0:
            p.append(f"num_key_value_heads ({self.num_key_value_heads}) must divide "
                     f"num_attention_heads ({self.num_attention_heads})")
        if self.head_dim is None or self.head_dim < 2 or self.head_dim > 1152 or self.head_dim % 2:
            p.append(f"head_dim must be even and in 2..1152 (got {self.head_dim})")
        if (self.max_position_embeddings or 0) < 2:
            p.append(f"max_position_embeddings must be >= 2 (got {self.max_position_embeddings})")
        if not (self.rms_norm_eps > 0):
            p.append(f"rms_norm_eps must be > 0 (got {self.rms_norm_eps})")
        if not (self.rope_theta > 0):
            p.append(f"rope_theta must be > 0 (got {self.rope_theta})")
        for name in ("attn_logit_softcapping", "final_logit_softcapping", "query_pre_attn_scalar"):
            v = getattr(self, name)
            if v is not None and not (v > 0 and math.isfinite(v)):
                p.append(f"{name} must be > 0 or null (got {v})")
        act = self.hidden_activation if self.hidden_activation is not None else self.hidden_act
        if act not in _GELU_TANH_NAMES or self.hidden_act not in _GELU_TANH_NAMES:
            p.append(f"hidden_activation must be one of {_GELU_TANH_NAMES} "
                     f"(got {self.hidden_activation!r}/{self.hidden_act!r})")
        if not self.tie_word_embeddings:
            p.append("tie_word_embeddings must be true: the output head is the embedding table")
        if self.attention_bias:
            p.append("attention_bias must be false: projections have no bias")
        if self.layer_types:
            if len(self.layer_types) != self.num_hidden_layers:
                p.append(f"layer_types has {len(self.layer_types)} entries for "
                         f"{self.num_hidden_layers} layers")
            bad = sorted({t for t in self.layer_types if t not in (LOCAL, GLOBAL)})
            if bad:
                p.append(f"layer_types entries must be '{LOCAL}' or '{GLOBAL}' (got {bad})")
        for i in self.eos_token_id:
            if not (0 <= i < (self.vocab_size or 0)):
                p.append(f"eos_token_id {i} is outside the vocabulary")
        if not (self.initializer_range > 0):
            p.append(f"initializer_range must be > 0 (got {self.initializer_range})")
        return p


def gemma2_spec(cfg: Gemma2Config) -> ModelSpec:
    """Lay Gemma 2 out as parts, in the order of Gemma2.pas:161-196."""
    H, L = cfg.hidden_size, cfg.num_hidden_layers
    norm = PartSpec("rmsnorm", {"size": H, "eps": cfg.rms_norm_eps, "unit_offset": True})
    rotary = PartSpec("rotary", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                 "rotary_dim": cfg.head_dim})
    layers = []
    for i in range(L):
        window = cfg.sliding_window if cfg.layer_is_local(i) else None
        mixer = PartSpec("attention", {
            "hidden_size": H, "n_heads": cfg.num_attention_heads,
            "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
            "scale": cfg.attention_scale, "softcap": cfg.attn_logit_softcapping,
            "window": window, "position": rotary})
        ff = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": cfg.intermediate_size,
                                    "activation": "gelu_tanh"})
        pre = f"model.layers.{i}."
        tensors = {
            "norms.pre_mixer.weight": pre + "input_layernorm.weight",
            "norms.post_mixer.weight": pre + "post_attention_layernorm.weight",
            "norms.pre_ff.weight": pre + "pre_feedforward_layernorm.weight",
            "norms.post_ff.weight": pre + "post_feedforward_layernorm.weight",
            "mixer.q_proj": pre + "self_attn.q_proj.weight",
            "mixer.k_proj": pre + "self_attn.k_proj.weight",
            "mixer.v_proj": pre + "self_attn.v_proj.weight",
            "mixer.o_proj": pre + "self_attn.o_proj.weight",
            "ff.gate_proj": pre + "mlp.gate_proj.weight",
            "ff.up_proj": pre + "mlp.up_proj.weight",
            "ff.down_proj": pre + "mlp.down_proj.weight",
        }
        layers.append(LayerSpec(
            block=PartSpec("sandwich", {}), mixer=mixer, feed_forward=ff,
            norms={"pre_mixer": norm, "post_mixer": norm, "pre_ff": norm, "post_ff": norm},
            tensors=tensors))
    return ModelSpec(
        name="Gemma2ForCausalLM",
        hidden_size=H,
        embedding=EmbeddingSpec(cfg.vocab_size, H, math.sqrt(H), "model.embed_tokens.weight"),
        layers=tuple(layers),
        schedule=default_schedule(L),
        head=HeadSpec(cfg.vocab_size, H, tied=True, tensor=None,
                      softcap=cfg.final_logit_softcapping, norm=norm,
                      norm_tensor="model.norm.weight"),
        max_positions=cfg.max_position_embeddings,
        stop_ids=tuple(cfg.eos_token_id),
        init_std=cfg.initializer_range,
    )


GEMMA2 = register_architecture(Architecture(
    name="Gemma2ForCausalLM", config_cls=Gemma2Config, build_spec=gemma2_spec,
    aliases=("gemma2",)))

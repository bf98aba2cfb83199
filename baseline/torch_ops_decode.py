"""The timed baseline of the benchmark: Gemma 2 decoding written with plain PyTorch tensor
operations and a contiguous key/value cache, nothing of this library in it.

HemulGM/QuickNN publishes no Gemma 2 figure and cannot run here (Delphi + Vulkan), so the
benchmark's ``vs_baseline`` is taken against what a user would write first on this GPU: the
formulas of ``tests/plain/gemma2_torch.py`` (whose part functions this file imports), eager
PyTorch kernels and cuBLAS products in the precision that is timed, one ``[batch, kv heads,
context, head]`` cache tensor per layer and side.  All sequences of the batch have the same
length, as in the benchmark; a windowed layer reads the last ``window`` positions as a slice.
"""
from __future__ import annotations

import math
import os
import sys
from typing import Dict

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "tests"))
from plain.gemma2_torch import gelu_tanh, rmsnorm, rope, softcap  # noqa: E402


class CachedTorchGemma2:
    def __init__(self, config: Dict, weights: Dict[str, torch.Tensor], batch: int, max_len: int, device,
                 dtype: torch.dtype = torch.bfloat16):
        c = self.cfg = dict(config)
        self.device, self.dtype = torch.device(device), dtype
        self.w = {k: v.to(device=device, dtype=dtype) for k, v in weights.items()}
        self.H, self.L = c["hidden_size"], c["num_hidden_layers"]
        self.nq, self.nkv, self.hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        self.theta, self.eps = c.get("rope_theta", 10000.0), c.get("rms_norm_eps", 1e-6)
        self.window = c.get("sliding_window", 4096)
        self.attn_cap, self.final_cap = c.get("attn_logit_softcapping", 50.0), c.get("final_logit_softcapping", 30.0)
        qpas = c.get("query_pre_attn_scalar")
        self.scale = 1.0 / math.sqrt(self.hd if qpas is None else qpas)
        shape = (batch, self.nkv, max_len, self.hd)
        self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(self.L)]
        self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(self.L)]
        self.length = 0

    def fill_random(self, length: int, seed: int = 0) -> None:
        """A history of ``length`` positions without computing it (a decode step's time does not
        depend on the values)."""
        g = torch.Generator(device=self.device)
        g.manual_seed(seed)
        for t in self.k + self.v:
            t[:, :, :length].normal_(0.0, 1.0, generator=g)
        self.length = length

    @torch.no_grad()
    def decode(self, tokens: torch.Tensor) -> torch.Tensor:
        """One token for every sequence ([batch] int64); returns the next ids (greedy)."""
        w, B, p = self.w, tokens.shape[0], self.length
        pos = torch.full((1,), p, device=self.device)
        x = w["model.embed_tokens.weight"][tokens] * math.sqrt(self.H)
        g = self.nq // self.nkv
        for i in range(self.L):
            n = f"model.layers.{i}."
            h = rmsnorm(x, w[n + "input_layernorm.weight"], self.eps)
            q = (h @ w[n + "self_attn.q_proj.weight"].T).view(B, self.nq, self.hd)
            k = (h @ w[n + "self_attn.k_proj.weight"].T).view(B, self.nkv, self.hd)
            v = (h @ w[n + "self_attn.v_proj.weight"].T).view(B, self.nkv, self.hd)
            # rope() rotates [tokens, heads, head]: every row of the batch stands at position p
            q = rope(q.reshape(1, B * self.nq, self.hd), pos, self.theta).view(B, self.nkv, g, self.hd)
            k = rope(k.reshape(1, B * self.nkv, self.hd), pos, self.theta).view(B, self.nkv, self.hd)
            self.k[i][:, :, p] = k
            self.v[i][:, :, p] = v
            lo = max(0, p + 1 - self.window) if i % 2 == 0 else 0          # even layers are local
            keys, vals = self.k[i][:, :, lo:p + 1], self.v[i][:, :, lo:p + 1]
            s = softcap((q @ keys.transpose(2, 3)).float() * self.scale, self.attn_cap)
            a = (torch.softmax(s, dim=-1).to(self.dtype) @ vals).reshape(B, self.nq * self.hd)
            x = x + rmsnorm(a @ w[n + "self_attn.o_proj.weight"].T, w[n + "post_attention_layernorm.weight"], self.eps)
            h = rmsnorm(x, w[n + "pre_feedforward_layernorm.weight"], self.eps)
            y = (gelu_tanh(h @ w[n + "mlp.gate_proj.weight"].T) * (h @ w[n + "mlp.up_proj.weight"].T)) \
                @ w[n + "mlp.down_proj.weight"].T
            x = x + rmsnorm(y, w[n + "post_feedforward_layernorm.weight"], self.eps)
        h = rmsnorm(x, w["model.norm.weight"], self.eps)
        logits = softcap((h @ w["model.embed_tokens.weight"].T).float(), self.final_cap)
        self.length = p + 1
        return logits.argmax(dim=-1)

"""Plain Gemma 2 in PyTorch tensor operations: whole sequences, no cache, one function per
part, on any device.

The second plain implementation.  ``gemma2_plain.py`` (NumPy, float64) is the oracle of the
tiny models; this one states the same formulas with torch operations so that it can run on
the GPU at the layer sizes of the 2B, 9B and 27B models, where NumPy would take minutes, and
so that it can be timed as the "plain tensor operations" baseline of the benchmark.  Like
the NumPy file it rests on the reference's formulas (the reference is Delphi + Vulkan and
can be neither compiled nor imported here), cites the lines it restates, shares no code with
the library (own safetensors reader, own reading of ``config.json``) and works on one whole
sequence at a time.  ``tests/test_plain.py`` shows that the two plain implementations agree.

Precision: ``dtype`` is the working precision of everything (float64 by default; float32
gives the reference's own).  Matrix products in reduced precision are switched off for the
calling process while a model of this file computes (`allow_tf32 = False`), so float32 means
float32.  Rotation angles are formed in float32, ``float32(position) * float32(inv_freq)``,
as the shader does (shaders/tensor.comp:318-327), and only then widened.
"""
from __future__ import annotations

import json
import math
import mmap
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# ---- files ---------------------------------------------------------------------

def read_safetensors(path: str, device, dtype: torch.dtype) -> Dict[str, torch.Tensor]:
    """Tensor by tensor from a memory map to ``device`` in ``dtype``; bf16 widens exactly
    (a 16-bit shift, shaders/gemm.comp:39-42)."""
    out: Dict[str, torch.Tensor] = {}
    with open(path, "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(n).decode("utf-8"))
        mm = mmap.mmap(fh.fileno(), 0, access=mmap.ACCESS_READ)
        base = 8 + n
        for name, info in header.items():
            if name == "__metadata__":
                continue
            b, e = info["data_offsets"]
            if info["dtype"] == "BF16":
                raw = np.frombuffer(mm, dtype="<i2", count=(e - b) // 2, offset=base + b)
                t = torch.from_numpy(raw.copy()).view(torch.bfloat16)
            elif info["dtype"] == "F32":
                raw = np.frombuffer(mm, dtype="<f4", count=(e - b) // 4, offset=base + b)
                t = torch.from_numpy(raw.copy())
            else:
                raise ValueError(f"plain reader: dtype {info['dtype']} of {name}")
            out[name] = t.reshape(info["shape"]).to(device).to(dtype)
            del raw
        mm.close()
    return out


# ---- parts ---------------------------------------------------------------------

def embed(table: torch.Tensor, ids: Sequence[int], hidden: int) -> torch.Tensor:
    """X[r,:] = E[id_r,:] * sqrt(H), the factor rounded to float32 first; an id outside the
    table gives zeros (Gemma2.pas:159-160; tensor.comp:237-242, op 43 at :309)."""
    idx = torch.as_tensor(list(ids), dtype=torch.long, device=table.device)
    ok = (idx >= 0) & (idx < table.shape[0])
    x = table[idx.clamp(0, table.shape[0] - 1)] * ok[:, None].to(table.dtype)
    return x * float(np.float32(math.sqrt(hidden)))


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """inv = 1/sqrt(mean(x^2) + eps); y = x * inv * (1 + w): no centring, no bias
    (tensor.comp:63-72 with Center=False, Operations.pas:139-148).  The reference's files
    store 1+w (Gemma2.pas:58); checkpoints here store w."""
    inv = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * inv * (1.0 + w)


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x: [T, heads, hd].  angle[p, j] = p * exp(-ln(theta) * 2j / hd) in float32
    (tensor.comp:320); half-split rotation of the whole head (tensor.comp:318-327):
    a' = a cos - b sin, b' = a sin + b cos with a = x[..., :hd/2], b = x[..., hd/2:]."""
    hd = x.shape[-1]
    j = torch.arange(hd // 2, dtype=torch.float64)
    inv_freq = torch.exp(-math.log(theta) * 2.0 * j / hd).to(torch.float32).to(x.device)
    ang = (positions.to(torch.float32)[:, None] * inv_freq[None, :]).to(torch.float64)
    c = torch.cos(ang).to(x.dtype)[:, None, :]
    s = torch.sin(ang).to(x.dtype)[:, None, :]
    a, b = x[..., : hd // 2], x[..., hd // 2:]
    return torch.cat([a * c - b * s, a * s + b * c], dim=-1)


def softcap(x: torch.Tensor, cap: Optional[float]) -> torch.Tensor:
    """cap * tanh(clamp(x / cap, -20, 20)); off when cap is None or <= 0
    (attention.comp:27; tensor.comp:308)."""
    if cap is None or cap <= 0:
        return x
    return cap * torch.tanh(torch.clamp(x / cap, -20.0, 20.0))


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, cap: Optional[float],
              window: Optional[int], rows_per_block: int = 1024) -> torch.Tensor:
    """q: [T, nq, hd]; k, v: [T, nkv, hd] -> [T, nq, hd].  Head h reads kv head h // (nq/nkv)
    (attention.comp:14); score = softcap((q.k) * scale); query p sees the keys j with
    keyStart <= j <= p, keyStart = p + 1 - window if window > 0 and p + 1 > window, else 0
    (attention.comp:21-27); softmax and the weighted sum of the values (:28-37).  Query rows
    are taken in blocks only to bound the size of the score matrix."""
    T, nq, hd = q.shape
    g = nq // k.shape[1]
    out = torch.empty_like(q)
    keys = torch.arange(T, device=q.device)
    for h in range(nq):
        kh = h // g
        for r0 in range(0, T, rows_per_block):
            r1 = min(T, r0 + rows_per_block)
            s = softcap((q[r0:r1, h, :] @ k[:r1, kh, :].T) * scale, cap)
            p = torch.arange(r0, r1, device=q.device)[:, None]
            seen = keys[None, :r1] <= p
            if window and window > 0:
                seen &= keys[None, :r1] >= p + 1 - window
            s = s.masked_fill(~seen, float("-inf"))
            w = torch.exp(s - s.max(dim=-1, keepdim=True).values)
            out[r0:r1, h, :] = (w @ v[:r1, kh, :]) / w.sum(dim=-1, keepdim=True)
    return out


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    """0.5 x (1 + tanh(0.7978845608028654 (x + 0.044715 x^3)))  (tensor.comp:23)."""
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x * x * x)))


def geglu_mlp(n: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """G = n Wgate^T, U = n Wup^T, Y = (gelu_tanh(G) * U) Wdown^T  (Gemma2.pas:184-187)."""
    return (gelu_tanh(n @ w_gate.T) * (n @ w_up.T)) @ w_down.T


# ---- the model -----------------------------------------------------------------

class TorchGemma2:
    def __init__(self, model_dir: str, device="cpu", dtype: torch.dtype = torch.float64):
        with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
            c = json.load(fh)
        self._setup(c, read_safetensors(os.path.join(model_dir, "model.safetensors"), torch.device(device), dtype),
                    device, dtype)

    @classmethod
    def from_tensors(cls, config: Dict, weights: Dict[str, torch.Tensor], device, dtype: torch.dtype) -> "TorchGemma2":
        """A model over tensors that are already in memory (checkpoint names -> tensors), for timing at
        sizes whose files would take gigabytes."""
        self = cls.__new__(cls)
        self._setup(dict(config), {k: v.to(device=device, dtype=dtype) for k, v in weights.items()}, device, dtype)
        return self

    def _setup(self, c: Dict, weights: Dict[str, torch.Tensor], device, dtype: torch.dtype) -> None:
        self.cfg, self.device, self.dtype = c, torch.device(device), dtype
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        self.w = weights
        self.H, self.L = c["hidden_size"], c["num_hidden_layers"]
        self.nq, self.nkv, self.hd = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
        self.V = c["vocab_size"]
        self.theta = c.get("rope_theta", 10000.0)
        self.eps = c.get("rms_norm_eps", 1e-6)
        self.window = c.get("sliding_window", 4096)
        self.attn_cap = c.get("attn_logit_softcapping", 50.0)
        self.final_cap = c.get("final_logit_softcapping", 30.0)
        qpas = c.get("query_pre_attn_scalar")
        self.scale = 1.0 / math.sqrt(self.hd if qpas is None else qpas)     # Gemma2.pas:88,96
        self.layer_types = c.get("layer_types")

    def layer_window(self, i: int) -> Optional[int]:
        """Even layers are local, odd ones global (Gemma2.pas:177)."""
        if self.layer_types:
            return self.window if self.layer_types[i] == "sliding_attention" else None
        return self.window if i % 2 == 0 else None

    @torch.no_grad()
    def hidden_states(self, ids: Sequence[int]) -> torch.Tensor:
        """Residual stream after the last layer, [T, H]  (Gemma2.pas:158-191)."""
        w, T = self.w, len(ids)
        pos = torch.arange(T, device=self.device)
        x = embed(w["model.embed_tokens.weight"], ids, self.H)
        for i in range(self.L):
            p = f"model.layers.{i}."
            n = rmsnorm(x, w[p + "input_layernorm.weight"], self.eps)
            q = (n @ w[p + "self_attn.q_proj.weight"].T).reshape(T, self.nq, self.hd)
            k = (n @ w[p + "self_attn.k_proj.weight"].T).reshape(T, self.nkv, self.hd)
            v = (n @ w[p + "self_attn.v_proj.weight"].T).reshape(T, self.nkv, self.hd)
            a = attention(rope(q, pos, self.theta), rope(k, pos, self.theta), v, self.scale, self.attn_cap,
                          self.layer_window(i))
            y = a.reshape(T, self.nq * self.hd) @ w[p + "self_attn.o_proj.weight"].T
            x = x + rmsnorm(y, w[p + "post_attention_layernorm.weight"], self.eps)
            n = rmsnorm(x, w[p + "pre_feedforward_layernorm.weight"], self.eps)
            y = geglu_mlp(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
            x = x + rmsnorm(y, w[p + "post_feedforward_layernorm.weight"], self.eps)
        return x

    @torch.no_grad()
    def logits(self, ids: Sequence[int], rows: Optional[Sequence[int]] = None) -> np.ndarray:
        """Logits [rows, V] (every position when ``rows`` is None): final norm, tied head, final
        softcap (Gemma2.pas:192-195; the reference keeps only the last row)."""
        return self.logits_of_hidden(self.hidden_states(ids), rows)

    @torch.no_grad()
    def logits_of_hidden(self, x: torch.Tensor, rows: Optional[Sequence[int]] = None) -> np.ndarray:
        """The head alone, on rows of a residual stream that ``hidden_states`` returned."""
        if rows is not None:
            x = x[torch.as_tensor(list(rows), dtype=torch.long, device=self.device)]
        n = rmsnorm(x, self.w["model.norm.weight"], self.eps)
        out = softcap(n @ self.w["model.embed_tokens.weight"].T, self.final_cap)
        return (out.float() if out.dtype == torch.bfloat16 else out).cpu().numpy()    # NumPy has no bfloat16

    def greedy(self, ids: Sequence[int], steps: int, stop_ids: Sequence[int] = ()) -> List[int]:
        """Greedy continuation by recomputing the whole sequence each step; the largest score
        wins, the lowest id on ties (tensor.comp:136)."""
        ids, out = list(ids), []
        for _ in range(steps):
            row = self.logits(ids, [len(ids) - 1])[0]
            t = int(np.flatnonzero(row == row.max())[0])
            if t in stop_ids:
                break
            out.append(t)
            ids.append(t)
        return out

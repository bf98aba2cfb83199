"""Plain, slow Gemma 2: whole sequences, no cache, one function per part, NumPy only.

This file rests on the reference's formulas, not on running it: HemulGM/QuickNN is
Delphi-only Object Pascal whose Gemma 2 path needs a Vulkan device
(src/models/QuickNN.Models.Gemma2.pas:35), and neither a Pascal compiler nor a
Vulkan loader exists where this is developed, so its model code can be neither
imported nor compiled.  Each function cites the lines it restates.

It shares no code with the library: it has its own safetensors reader, reads
``config.json`` keys itself and works on one whole sequence at a time.  Arithmetic
is float64 by default (an oracle that is more exact than either engine path);
``dtype=np.float32`` gives the reference's own working precision.  Rotation
angles are always formed in float32, ``float32(position) * float32(inv_freq)``,
as the shader does (shaders/tensor.comp:318-327), and only then widened.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np


# ---- files ---------------------------------------------------------------------

def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    """Minimal reader: bf16 is widened by a 16-bit shift (shaders/gemm.comp:39-42)."""
    with open(path, "rb") as fh:
        (n,) = struct.unpack("<Q", fh.read(8))
        header = json.loads(fh.read(n).decode("utf-8"))
        data = fh.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        raw = data[b:e]
        dt = info["dtype"]
        if dt == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32)
        elif dt == "F32":
            arr = np.frombuffer(raw, dtype="<f4")
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = arr.reshape(info["shape"]).copy()
    return out


def read_model(model_dir: str):
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as fh:
        cfg = json.load(fh)
    weights = read_safetensors(os.path.join(model_dir, "model.safetensors"))
    return cfg, weights


# ---- parts ---------------------------------------------------------------------

def embed(table: np.ndarray, ids: Sequence[int], hidden: int, dtype) -> np.ndarray:
    """X[r,:] = E[id_r,:] * sqrt(H); an id outside the table gives zeros
    (Gemma2.pas:159-160; tensor.comp:237-242, op 43 at :309)."""
    x = np.zeros((len(ids), hidden), dtype=dtype)
    for r, t in enumerate(ids):
        if 0 <= t < table.shape[0]:
            x[r] = table[t].astype(dtype)
    return x * dtype(np.float32(math.sqrt(hidden)))


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """inv = 1/sqrt(mean(x^2) + eps); y = x * inv * (1 + w).  No centring, no bias
    (tensor.comp:63-72 with Center=False, Operations.pas:139-148).  The reference's
    files store 1+w (Gemma2.pas:58); checkpoints here store w, so 1 is added here."""
    dt = x.dtype.type
    inv = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + dt(eps))
    return x * inv * (dt(1.0) + w.astype(x.dtype))


def rope_angles(positions: np.ndarray, head_dim: int, theta: float) -> np.ndarray:
    """angle[p, j] = p * exp(-ln(theta) * 2j / head_dim), j in [0, head_dim/2), in float32
    (tensor.comp:320).  The frequency is rounded to float32 once, then multiplied by
    the float32 position."""
    j = np.arange(head_dim // 2, dtype=np.float64)
    inv_freq = np.exp(-math.log(theta) * 2.0 * j / head_dim).astype(np.float32)
    return positions.astype(np.float32)[:, None] * inv_freq[None, :]


def rope(x: np.ndarray, positions: np.ndarray, theta: float) -> np.ndarray:
    """x: [T, heads, head_dim]; half-split rotation of the whole head
    (tensor.comp:318-327): x' = x_j cos - x_{j+hd/2} sin, y' = x_j sin + x_{j+hd/2} cos."""
    hd = x.shape[-1]
    ang = rope_angles(positions, hd, theta).astype(np.float64)
    c = np.cos(ang).astype(x.dtype)[:, None, :]
    s = np.sin(ang).astype(x.dtype)[:, None, :]
    a, b = x[..., : hd // 2], x[..., hd // 2:]
    return np.concatenate([a * c - b * s, a * s + b * c], axis=-1)


def softcap(x: np.ndarray, cap: Optional[float]) -> np.ndarray:
    """cap * tanh(clamp(x / cap, -20, 20)); off when cap is None or <= 0
    (attention.comp:27; tensor.comp:308)."""
    if cap is None or cap <= 0:
        return x
    dt = x.dtype.type
    return dt(cap) * np.tanh(np.clip(x / dt(cap), -20.0, 20.0))


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float,
              cap: Optional[float], window: Optional[int]) -> np.ndarray:
    """q: [T, nq, hd]; k, v: [T, nkv, hd] -> [T, nq, hd].
    Query row p of head h uses kv head h // (nq/nkv) (attention.comp:14), scores
    (q.k) * scale, then the softcap, over keys j in [keyStart, p] with
    keyStart = p + 1 - window when window > 0 and p + 1 > window, else 0
    (attention.comp:21-27), softmax and the weighted sum of values (:28-37)."""
    T, nq, hd = q.shape
    nkv = k.shape[1]
    g = nq // nkv
    out = np.zeros_like(q)
    dt = q.dtype.type
    for h in range(nq):
        kh = h // g
        s = (q[:, h, :] @ k[:, kh, :].T) * dt(scale)            # [T, T]
        s = softcap(s, cap)
        for p in range(T):
            end = p + 1
            start = end - window if (window and window > 0 and end > window) else 0
            row = s[p, start:end]
            w = np.exp(row - row.max())
            out[p, h, :] = (w[:, None] * v[start:end, kh, :]).sum(axis=0) / w.sum()
    return out


def gelu_tanh(x: np.ndarray) -> np.ndarray:
    """0.5 x (1 + tanh(0.7978845608028654 (x + 0.044715 x^3)))  (tensor.comp:23)."""
    dt = x.dtype.type
    return dt(0.5) * x * (dt(1.0) + np.tanh(dt(0.7978845608028654) * (x + dt(0.044715) * x * x * x)))


def geglu_mlp(n: np.ndarray, w_gate: np.ndarray, w_up: np.ndarray, w_down: np.ndarray) -> np.ndarray:
    """G = n Wgate^T, U = n Wup^T, Y = (gelu_tanh(G) * U) Wdown^T  (Gemma2.pas:184-187)."""
    dt = n.dtype
    g = n @ w_gate.astype(dt).T
    u = n @ w_up.astype(dt).T
    return (gelu_tanh(g) * u) @ w_down.astype(dt).T


# ---- the model -----------------------------------------------------------------

class PlainGemma2:
    def __init__(self, model_dir: str, dtype=np.float64):
        self.cfg, self.w = read_model(model_dir)
        self.dtype = dtype
        c = self.cfg
        self.H = c["hidden_size"]
        self.L = c["num_hidden_layers"]
        self.nq = c["num_attention_heads"]
        self.nkv = c["num_key_value_heads"]
        self.hd = c["head_dim"]
        self.V = c["vocab_size"]
        self.theta = c.get("rope_theta", 10000.0)
        self.eps = c.get("rms_norm_eps", 1e-6)
        self.window = c.get("sliding_window", 4096)
        self.attn_cap = c.get("attn_logit_softcapping", 50.0)
        self.final_cap = c.get("final_logit_softcapping", 30.0)
        qpas = c.get("query_pre_attn_scalar")
        self.scale = 1.0 / math.sqrt(self.hd if qpas is None else qpas)   # Gemma2.pas:88,96
        self.layer_types = c.get("layer_types")

    def layer_window(self, i: int) -> Optional[int]:
        """Even layers are local, odd ones global (Gemma2.pas:177)."""
        if self.layer_types:
            return self.window if self.layer_types[i] == "sliding_attention" else None
        return self.window if i % 2 == 0 else None

    def hidden_states(self, ids: Sequence[int]) -> np.ndarray:
        """Residual stream after the last layer, [T, H]  (Gemma2.pas:158-191)."""
        dt = self.dtype
        w = self.w
        T = len(ids)
        pos = np.arange(T)
        x = embed(w["model.embed_tokens.weight"], ids, self.H, dt)
        for i in range(self.L):
            p = f"model.layers.{i}."
            n = rmsnorm(x, w[p + "input_layernorm.weight"], self.eps)
            q = (n @ w[p + "self_attn.q_proj.weight"].astype(dt).T).reshape(T, self.nq, self.hd)
            k = (n @ w[p + "self_attn.k_proj.weight"].astype(dt).T).reshape(T, self.nkv, self.hd)
            v = (n @ w[p + "self_attn.v_proj.weight"].astype(dt).T).reshape(T, self.nkv, self.hd)
            q = rope(q, pos, self.theta)
            k = rope(k, pos, self.theta)
            a = attention(q, k, v, self.scale, self.attn_cap, self.layer_window(i))
            y = a.reshape(T, self.nq * self.hd) @ w[p + "self_attn.o_proj.weight"].astype(dt).T
            x = x + rmsnorm(y, w[p + "post_attention_layernorm.weight"], self.eps)
            n = rmsnorm(x, w[p + "pre_feedforward_layernorm.weight"], self.eps)
            y = geglu_mlp(n, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                          w[p + "mlp.down_proj.weight"])
            x = x + rmsnorm(y, w[p + "post_feedforward_layernorm.weight"], self.eps)
        return x

    def logits(self, ids: Sequence[int]) -> np.ndarray:
        """Logits at every position, [T, V]: final norm, tied head, final softcap
        (Gemma2.pas:192-195; the reference keeps only the last row)."""
        x = self.hidden_states(ids)
        n = rmsnorm(x, self.w["model.norm.weight"], self.eps)
        lg = n @ self.w["model.embed_tokens.weight"].astype(self.dtype).T
        return softcap(lg, self.final_cap)

    def greedy(self, ids: Sequence[int], steps: int, stop_ids: Sequence[int] = ()) -> List[int]:
        """Greedy continuation by recomputing the whole sequence each step."""
        ids = list(ids)
        out: List[int] = []
        for _ in range(steps):
            t = argmax_lowest(self.logits(ids)[-1])
            if t in stop_ids:
                break
            out.append(t)
            ids.append(t)
        return out


# ---- sampling ------------------------------------------------------------------

def argmax_lowest(row: np.ndarray) -> int:
    """Largest score, lowest id on ties (tensor.comp:136)."""
    return int(np.flatnonzero(row == row.max())[0])


def xorshift32(state: int):
    """x ^= x<<13; x ^= x>>17; x ^= x<<5; u = min(0.99999994, (x + 0.5) / 2^32)
    (src/models/QuickNN.Models.LLM.pas:625-628)."""
    x = state & 0xFFFFFFFF
    x ^= (x << 13) & 0xFFFFFFFF
    x ^= x >> 17
    x ^= (x << 5) & 0xFFFFFFFF
    u = min(float(np.float32(0.99999994)), (x + 0.5) / 4294967296.0)
    return x, np.float32(u)


def seed_state(seed: int) -> int:
    """lo xor hi of the 64-bit seed, 0 replaced by 0x9E3779B9 (LLM.pas:976-978)."""
    s = (seed & 0xFFFFFFFF) ^ ((seed >> 32) & 0xFFFFFFFF)
    return s if s else 0x9E3779B9


def sample(row: np.ndarray, temperature: float, top_k: int, top_p: float, penalty: float,
           seen: Optional[np.ndarray], uniform: float, info: Optional[dict] = None) -> int:
    """Top-k, temperature softmax over the kept, nucleus cut, inverse CDF
    (tensor.comp:164-197): repetition penalty s<0 ? s*pen : s/pen on seen ids (:172);
    k = 1 when temperature <= 0 (:168); candidates ordered by score, lowest id first on
    ties (:173); p_j = exp((s_j - s_0)/T); keep the shortest prefix whose mass reaches
    top_p * total (:190-191); draw target = u * retained, pick the first j whose running
    sum exceeds it, else the last kept (:192-194).  Sums run in float32 as in the shader.
    ``info`` (if given) receives ``margin``: the distance of the draw from the nearest boundary
    between two candidates, as a fraction of the retained mass (1.0 for a greedy pick)."""
    s = row.astype(np.float32).copy()
    if seen is not None and penalty != 1.0:
        m = seen.astype(bool)
        s[m] = np.where(s[m] < 0, s[m] * np.float32(penalty), s[m] / np.float32(penalty))
    k = min(len(s), max(1, min(top_k, 64)))
    if temperature <= 0:
        k = 1
    order = np.lexsort((np.arange(len(s)), -s))[:k]
    if info is not None:
        info["margin"] = 1.0
    if k == 1:
        return int(order[0])
    vals = s[order]
    probs = np.exp((vals - vals[0]) / np.float32(temperature)).astype(np.float32)
    total = np.float32(0)
    for p in probs:
        total = np.float32(total + p)
    retained = np.float32(0)
    count = 0
    while True:
        retained = np.float32(retained + probs[count])
        count += 1
        if not (count < k and retained < np.float32(top_p) * total):
            break
    target = np.float32(uniform) * retained
    acc = np.float32(0)
    chosen = int(order[count - 1])
    for j in range(count):
        acc = np.float32(acc + probs[j])
        if target < acc:
            chosen = int(order[j])
            break
    if info is not None:
        sums = np.cumsum(probs[:count].astype(np.float64))
        info["margin"] = float(np.abs(sums - float(target)).min() / float(retained))
    return chosen

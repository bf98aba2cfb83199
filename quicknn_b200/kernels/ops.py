"""Tensor-level wrappers of the CUDA launchers.

Each function checks devices, dtypes, shapes and contiguity on the host, then
calls the C entry point on the current CUDA stream.  Outputs are allocated by the
caller or here with ``torch.empty`` (the caching allocator, so that a step can be
captured in a CUDA graph).  Library matrix products (cuBLAS through
``torch.matmul``) are used for bfloat16 products of more than 64 rows only.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import lib as _lib

F32, BF16 = 0, 1
EPI_NONE, EPI_SOFTCAP, EPI_GATED = 0, 1, 2
ACT_CODES = {"gelu_tanh": 0, "silu": 1}
SKINNY_MAX_ROWS = 64


def dt_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise TypeError(f"unsupported dtype {t.dtype} (float32 or bfloat16 expected)")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _req(t: torch.Tensor, name: str, dtype=None, dim=None) -> None:
    if not t.is_cuda:
        raise _lib.KernelError(f"{name} must be a CUDA tensor: quicknn_b200 has no CPU path")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise ValueError(f"{name} must have {dim} dimensions, got {tuple(t.shape)}")


def embed(tokens: torch.Tensor, table: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None):
    _req(tokens, "tokens", torch.int32, 1)
    _req(table, "table", None, 2)
    T, (V, H) = tokens.numel(), table.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=tokens.device)
    _req(out, "out", torch.float32, 2)
    L = _lib.load()
    _lib.check(L.qnn_embed(_p(tokens), _p(table), dt_code(table), float(scale), _p(out), T, H, V, _stream()),
               "embed")
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, unit_offset: bool, out_dtype: torch.dtype,
            out: Optional[torch.Tensor] = None):
    _req(x, "x", None, 2)
    _req(weight, "weight", None, 1)
    T, H = x.shape
    if weight.numel() != H:
        raise ValueError(f"norm weight has {weight.numel()} elements for width {H}")
    if out is None:
        out = torch.empty((T, H), dtype=out_dtype, device=x.device)
    _req(out, "out", out_dtype, 2)
    L = _lib.load()
    _lib.check(L.qnn_rmsnorm(_p(x), dt_code(x), _p(weight), dt_code(weight), float(eps), int(unit_offset),
                             _p(out), dt_code(out), T, H, _stream()), "rmsnorm")
    return out


def add_rmsnorm(resid: torch.Tensor, y: torch.Tensor, w_post: torch.Tensor, eps_post: float, unit_post: bool,
                w_next: Optional[torch.Tensor] = None, eps_next: float = 0.0, unit_next: bool = False,
                out_dtype: Optional[torch.dtype] = None):
    """resid += rmsnorm(y, w_post); returns rmsnorm(resid, w_next) when w_next is given."""
    _req(resid, "resid", torch.float32, 2)
    _req(y, "y", None, 2)
    T, H = resid.shape
    if tuple(y.shape) != (T, H) or w_post.numel() != H or (w_next is not None and w_next.numel() != H):
        raise ValueError("add_rmsnorm: shapes do not agree")
    out = None
    if w_next is not None:
        out = torch.empty((T, H), dtype=out_dtype, device=resid.device)
    L = _lib.load()
    _lib.check(L.qnn_add_rmsnorm(_p(resid), _p(y), dt_code(y), _p(w_post), dt_code(w_post), float(eps_post),
                                 int(unit_post), _p(w_next), dt_code(w_next) if w_next is not None else 0,
                                 float(eps_next), int(unit_next), _p(out), dt_code(out) if out is not None else 0,
                                 T, H, _stream()), "add_rmsnorm")
    return out


def add_(resid: torch.Tensor, y: torch.Tensor):
    _req(resid, "resid", torch.float32)
    _req(y, "y")
    if resid.numel() != y.numel():
        raise ValueError("add_: sizes differ")
    L = _lib.load()
    _lib.check(L.qnn_add(_p(resid), _p(y), dt_code(y), resid.numel(), _stream()), "add")
    return resid


def gated_act(gu: torch.Tensor, activation: str):
    _req(gu, "gate_up", None, 2)
    T, I2 = gu.shape
    out = torch.empty((T, I2 // 2), dtype=gu.dtype, device=gu.device)
    L = _lib.load()
    _lib.check(L.qnn_gated_act(_p(gu), _p(out), dt_code(gu), T, I2 // 2, ACT_CODES[activation], _stream()),
               "gated_act")
    return out


def softcap(x: torch.Tensor, cap: Optional[float]):
    _req(x, "x")
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    L = _lib.load()
    _lib.check(L.qnn_softcap(_p(x), dt_code(x), _p(out), float(cap or 0.0), x.numel(), _stream()), "softcap")
    return out


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out_dtype: torch.dtype):
    _req(src, "src", None, 2)
    _req(rows, "rows", torch.int32, 1)
    out = torch.empty((rows.numel(), src.shape[1]), dtype=out_dtype, device=src.device)
    L = _lib.load()
    _lib.check(L.qnn_gather_rows(_p(src), dt_code(src), _p(rows), _p(out), dt_code(out), rows.numel(),
                                 src.shape[1], _stream()), "gather_rows")
    return out


def cast(x: torch.Tensor, dtype: torch.dtype):
    if x.dtype == dtype:
        return x
    _req(x, "x")
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    L = _lib.load()
    _lib.check(L.qnn_cast(_p(x), dt_code(x), _p(out), dt_code(out), x.numel(), _stream()), "cast")
    return out


def check_finite(x: torch.Tensor, flag: torch.Tensor):
    _req(x, "x", torch.float32)
    _req(flag, "flag", torch.int32)
    L = _lib.load()
    _lib.check(L.qnn_check_finite(_p(x), x.numel(), _p(flag), _stream()), "check_finite")


def rope_cache_write(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, rot_dim: int,
                     inv_freq: torch.Tensor, tok_pos: torch.Tensor, tok_slot: torch.Tensor,
                     k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                     page_table: Optional[torch.Tensor], page_size: int, ring: int,
                     slot_len: Optional[torch.Tensor], write_cache: bool):
    _req(qkv, "qkv", None, 2)
    T = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv) * head_dim:
        raise ValueError("rope_cache_write: qkv width does not match the head counts")
    _req(inv_freq, "inv_freq", torch.float32, 1)
    if inv_freq.numel() != rot_dim // 2:
        raise ValueError("rope_cache_write: inv_freq has the wrong length")
    _req(tok_pos, "tok_pos", torch.int32, 1)
    _req(tok_slot, "tok_slot", torch.int32, 1)
    if write_cache:
        for n, t in (("k_pool", k_pool), ("v_pool", v_pool)):
            _req(t, n, qkv.dtype, 4)
            if tuple(t.shape[1:]) != (n_kv, page_size, head_dim):
                raise ValueError(f"{n} has shape {tuple(t.shape)}, expected [pages, {n_kv}, {page_size}, {head_dim}]")
        _req(page_table, "page_table", torch.int32, 2)
        _req(slot_len, "slot_len", torch.int32, 1)
    L = _lib.load()
    _lib.check(L.qnn_rope_cache_write(
        _p(qkv), dt_code(qkv), T, n_heads, n_kv, head_dim, rot_dim, _p(inv_freq), _p(tok_pos), _p(tok_slot),
        _p(k_pool), _p(v_pool), _p(page_table), page_table.shape[1] if page_table is not None else 0,
        page_size, ring, _p(slot_len), int(write_cache), _stream()), "rope_cache_write")


FUSE_ROPE = os.environ.get("QNN_FUSE_ROPE", "1") != "0"


def qkv_rope_cache_fusable(x: torch.Tensor, w: torch.Tensor, head_dim: int, rot_dim: int) -> bool:
    """Whether qkv_rope_cache takes this product: bfloat16 on both sides, few rows, a matrix
    that the small-M kernel would multiply anyway, a rotation over the whole head."""
    M, K = x.shape
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not FUSE_ROPE:
        return False
    if M > SKINNY_MAX_ROWS or K % 8 or head_dim % 16 or rot_dim != head_dim:
        return False
    return not _takes_skinny_tcgen05(M, w.shape[0], K)


def qkv_rope_cache(x: torch.Tensor, w: torch.Tensor, n_heads: int, n_kv: int, head_dim: int,
                   inv_freq: torch.Tensor, tok_pos: torch.Tensor, tok_slot: torch.Tensor,
                   k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                   page_table: Optional[torch.Tensor], page_size: int, ring: int,
                   slot_len: Optional[torch.Tensor], write_cache: bool) -> torch.Tensor:
    """linear(x, w) followed by rope_cache_write(...) as one kernel: the stacked q|k|v product
    with Q and K rotated and K, V appended to the cache in its epilogue.  Returns qkv."""
    _req(x, "x", torch.bfloat16, 2)
    _req(w, "w", torch.bfloat16, 2)
    M, K = x.shape
    N = (n_heads + 2 * n_kv) * head_dim
    if tuple(w.shape) != (N, K):
        raise ValueError(f"qkv_rope_cache: w is {tuple(w.shape)}, expected {(N, K)}")
    _req(inv_freq, "inv_freq", torch.float32, 1)
    if inv_freq.numel() != head_dim // 2:
        raise ValueError("qkv_rope_cache: inv_freq has the wrong length")
    _req(tok_pos, "tok_pos", torch.int32, 1)
    _req(tok_slot, "tok_slot", torch.int32, 1)
    if tok_pos.numel() < M or tok_slot.numel() < M:
        raise ValueError("qkv_rope_cache: fewer positions than rows")
    if write_cache:
        for n, t in (("k_pool", k_pool), ("v_pool", v_pool)):
            _req(t, n, torch.bfloat16, 4)
            if tuple(t.shape[1:]) != (n_kv, page_size, head_dim):
                raise ValueError(f"{n} has shape {tuple(t.shape)}, expected [pages, {n_kv}, {page_size}, {head_dim}]")
        _req(page_table, "page_table", torch.int32, 2)
        _req(slot_len, "slot_len", torch.int32, 1)
    qkv = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    L = _lib.load()
    _lib.check(L.qnn_skinny_qkv_rope(
        _p(x), _p(w), _p(qkv), M, K, n_heads, n_kv, head_dim, _p(inv_freq), _p(tok_pos), _p(tok_slot),
        _p(k_pool), _p(v_pool), _p(page_table), page_table.shape[1] if page_table is not None else 0,
        page_size, ring, _p(slot_len), int(write_cache), _stream()), "skinny_qkv_rope")
    return qkv


_gemm_status = {}


def _status_word(device) -> torch.Tensor:
    t = _gemm_status.get(device)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _gemm_status[device] = t
    return t


def check_gemm_status(device) -> None:
    """Raise if a bounded wait inside the tcgen05 product ran out since the last check (one
    4-byte read; call it where the host synchronises anyway)."""
    t = _gemm_status.get(torch.device(device))
    if t is None:
        return
    v = int(t.item())
    if v:
        t.zero_()
        raise _lib.KernelError(f"the tcgen05 matrix product gave up waiting (status {v}: 1 loads, 2 tensor-core "
                               f"issue, 4 epilogue); its result is not valid")


GEMM_2CTA = os.environ.get("QNN_GEMM_2CTA", "1") != "0"


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, *, epilogue: int = EPI_NONE, activation: str = "gelu_tanh",
                 pair: Optional[bool] = None):
    """x w^T for whole prompts on the 5th-generation tensor cores (bfloat16, any M; K a multiple of 8).
    Epilogues: none, or gated (w = [gate; up] stacked).  With more than 128 rows pairs of CTAs
    compute 256 x 256 tiles (``pair``; QNN_GEMM_2CTA=0 keeps one CTA per tile).  Returns None when
    the sizes are refused."""
    _req(x, "x", torch.bfloat16, 2)
    _req(w, "w", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if epilogue not in (EPI_NONE, EPI_GATED) or K % 8 or w.shape[1] != K:
        return None
    n_out = N // 2 if epilogue == EPI_GATED else N
    out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
    L = _lib.load()
    if pair is None:
        pair = GEMM_2CTA and M > 128
    if pair:
        code = L.qnn_gemm_tcgen05_2cta(_p(x), _p(w), _p(out), M, N, K, epilogue, ACT_CODES[activation],
                                       _p(_status_word(x.device)), _stream())
        if code != _lib.ERR_UNSUPPORTED:
            _lib.check(code, "gemm_tcgen05_2cta")
            return out
    code = L.qnn_gemm_tcgen05(_p(x), _p(w), _p(out), M, N, K, epilogue, ACT_CODES[activation],
                              _p(_status_word(x.device)), _stream())
    if code == _lib.ERR_UNSUPPORTED:
        return None
    _lib.check(code, "gemm_tcgen05")
    return out


def gemm_skinny_tcgen05(x: torch.Tensor, w: torch.Tensor, *, epilogue: int = EPI_NONE, cap: Optional[float] = None,
                        activation: str = "gelu_tanh"):
    """x w^T for up to 128 rows: TMA + tcgen05 with K split over a thread-block cluster and summed
    through distributed shared memory.  Epilogues: none (bfloat16), softcap (float32), gated.
    Returns None when the sizes are refused."""
    _req(x, "x", torch.bfloat16, 2)
    _req(w, "w", torch.bfloat16, 2)
    M, K = x.shape
    N = w.shape[0]
    if M > 128 or K % 8 or w.shape[1] != K:
        return None
    n_out = N // 2 if epilogue == EPI_GATED else N
    out = torch.empty((M, n_out), dtype=torch.float32 if epilogue == EPI_SOFTCAP else torch.bfloat16, device=x.device)
    L = _lib.load()
    code = L.qnn_gemm_skinny_tcgen05(_p(x), _p(w), _p(out), M, N, K, epilogue, float(cap or 0.0),
                                     ACT_CODES[activation], _p(_status_word(x.device)), _stream())
    if code == _lib.ERR_UNSUPPORTED:
        return None
    _lib.check(code, "gemm_skinny_tcgen05")
    return out


USE_TCGEN05 = os.environ.get("QNN_GEMM", "tcgen05") != "cublas"
# From this many rows on, products against big matrices (>= 2^24 weights) take the cluster split-K
# tcgen05 kernel instead of the mma.sync small-M kernel (measured on B200: up to 8 rows, one 8-row
# tile of mma.sync, and for the small q/k/v and o matrices up to about 30 rows, the mma.sync kernel is
# the faster one; at 12 and 16 rows the step gains 8-9 % with the tcgen05 kernel for the big matrices).
SKINNY_TCGEN05_FROM = int(os.environ.get("QNN_SKINNY_TCGEN05_FROM", "9"))
SKINNY_TCGEN05_MIN_WEIGHTS = 1 << 24
SKINNY_TCGEN05_ANY_FROM = 32          # from this many rows on, the small matrices too (q|k|v at 32 rows: 10.7 against 13.0 us)


def _takes_skinny_tcgen05(M: int, N: int, K: int) -> bool:
    return USE_TCGEN05 and SKINNY_TCGEN05_FROM <= M <= 128 and (M >= SKINNY_TCGEN05_ANY_FROM or
                                                                N * K >= SKINNY_TCGEN05_MIN_WEIGHTS)


def linear(x: torch.Tensor, w: torch.Tensor, *, epilogue: int = EPI_NONE, cap: Optional[float] = None,
           activation: str = "gelu_tanh", out_dtype: Optional[torch.dtype] = None):
    """y = x w^T with an optional epilogue.  x: [M, K]; w: [N, K] (gated: [2*N_out, K]).

    float32: FFMA kernels only.  bfloat16: the tensor-core small-M kernel up to 64 rows, the
    tcgen05/TMA kernel above that (a library product, cuBLAS, only for the softcap epilogue of
    many rows, for sizes the kernel refuses, or when QNN_GEMM=cublas is set)."""
    _req(x, "x", None, 2)
    _req(w, "w", None, 2)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError(f"linear: x is [*, {K}] but w is [*, {w.shape[1]}]")
    if x.dtype != w.dtype:
        raise TypeError(f"linear: x is {x.dtype} but w is {w.dtype}")
    n_out = N // 2 if epilogue == EPI_GATED else N
    if out_dtype is None:
        out_dtype = torch.float32 if epilogue == EPI_SOFTCAP else x.dtype
    L = _lib.load()
    capv = float(cap or 0.0)
    act = ACT_CODES[activation]
    if x.dtype == torch.float32:
        if out_dtype != torch.float32:
            raise TypeError("float32 products give float32")
        out = torch.empty((M, n_out), dtype=torch.float32, device=x.device)
        if M <= 8:
            _lib.check(L.qnn_gemv_f32(_p(x), _p(w), _p(out), M, N, K, epilogue, capv, act, _stream()), "gemv_f32")
        elif epilogue == EPI_GATED:
            gu = torch.empty((M, N), dtype=torch.float32, device=x.device)
            _lib.check(L.qnn_sgemm_f32(_p(x), _p(w), _p(gu), M, N, K, EPI_NONE, 0.0, _stream()), "sgemm_f32")
            out = gated_act(gu, activation)
        else:
            _lib.check(L.qnn_sgemm_f32(_p(x), _p(w), _p(out), M, N, K, epilogue, capv, _stream()), "sgemm_f32")
        return out
    # bfloat16
    if K % 8:
        raise _lib.KernelError(f"bfloat16 products need an inner size that is a multiple of 8 (got {K})")
    if _takes_skinny_tcgen05(M, N, K) and out_dtype == (torch.float32 if epilogue == EPI_SOFTCAP else torch.bfloat16):
        y = gemm_skinny_tcgen05(x, w, epilogue=epilogue, cap=cap, activation=activation)
        if y is not None:
            return y
    if M <= SKINNY_MAX_ROWS:
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        _lib.check(L.qnn_skinny_bf16(_p(x), _p(w), _p(out), dt_code(out), M, N, K, epilogue, capv, act, _stream()),
                   "skinny_bf16")
        return out
    if USE_TCGEN05 and epilogue in (EPI_NONE, EPI_GATED) and out_dtype == torch.bfloat16:
        y = gemm_tcgen05(x, w, epilogue=epilogue, activation=activation)
        if y is not None:
            return y
    y = torch.matmul(x, w.t())
    if epilogue == EPI_GATED:
        return gated_act(y, activation)
    if epilogue == EPI_SOFTCAP:
        return softcap(y, cap)
    return y if out_dtype == y.dtype else cast(y, out_dtype)


ATTN_TCGEN05 = os.environ.get("QNN_ATTN", "tcgen05") != "mma"


def attn_prefill(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, tok_pos: torch.Tensor,
                 tok_row0: torch.Tensor, scale: float, cap: Optional[float], window: Optional[int],
                 seq_row0: Optional[torch.Tensor] = None, seq_len: Optional[torch.Tensor] = None,
                 max_len: int = 0):
    """Causal (optionally windowed) attention of this step's own rows.  qkv: [T, (nq+2nkv)*hd]
    after rotation; returns [T, nq*hd].  bfloat16 with head sizes 64/128/256 runs on the tensor
    cores when the per-sequence arrays (first row, length) are given; everything else takes the
    generic kernel."""
    _req(qkv, "qkv", None, 2)
    T = qkv.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    es = qkv.element_size()
    q_ptr = qkv.data_ptr()
    k_ptr = q_ptr + n_heads * head_dim * es
    v_ptr = k_ptr + n_kv * head_dim * es
    L = _lib.load()
    if (qkv.dtype == torch.bfloat16 and seq_row0 is not None and seq_len is not None and max_len > 0
            and head_dim in (64, 128, 256)):
        _req(seq_row0, "seq_row0", torch.int32, 1)
        _req(seq_len, "seq_len", torch.int32, 1)
        if ATTN_TCGEN05:
            code = L.qnn_attn_prefill_tcgen05(
                _p(qkv), T, _p(out), out.shape[1], _p(seq_row0), _p(seq_len), seq_row0.numel(), int(max_len),
                n_heads, n_kv, head_dim, float(scale), float(cap or 0.0), int(window or 0),
                _p(_status_word(qkv.device)), _stream())
            if code != _lib.ERR_UNSUPPORTED:
                _lib.check(code, "attn_prefill_tcgen05")
                return out
        code = L.qnn_attn_prefill_mma(
            ctypes.c_void_p(q_ptr), ctypes.c_void_p(k_ptr), ctypes.c_void_p(v_ptr), qkv.shape[1], _p(out),
            out.shape[1], _p(seq_row0), _p(seq_len), seq_row0.numel(), int(max_len), n_heads, n_kv, head_dim,
            float(scale), float(cap or 0.0), int(window or 0), _stream())
        if code != _lib.ERR_UNSUPPORTED:
            _lib.check(code, "attn_prefill_mma")
            return out
    _lib.check(L.qnn_attn_prefill_generic(
        ctypes.c_void_p(q_ptr), ctypes.c_void_p(k_ptr), ctypes.c_void_p(v_ptr), qkv.shape[1], dt_code(qkv),
        _p(out), out.shape[1], _p(tok_pos), _p(tok_row0), T, n_heads, n_kv, head_dim, float(scale),
        float(cap or 0.0), int(window or 0), _stream()), "attn_prefill")
    return out


def attn_prefill_paged(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, k_pool: torch.Tensor,
                       v_pool: torch.Tensor, page_table: torch.Tensor, page_size: int, ring: int,
                       tok_pos: torch.Tensor, tok_slot: torch.Tensor, scale: float, cap: Optional[float],
                       window: Optional[int]):
    """Several query rows per sequence against the paged cache (keys written earlier in the
    same step by the layer that owns the line).  q = the first nq*hd columns of qkv."""
    _req(qkv, "qkv", None, 2)
    _req(k_pool, "k_pool", qkv.dtype, 4)
    _req(v_pool, "v_pool", qkv.dtype, 4)
    T = qkv.shape[0]
    out = torch.empty((T, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    L = _lib.load()
    _lib.check(L.qnn_attn_prefill_paged(
        _p(qkv), qkv.shape[1], dt_code(qkv), _p(k_pool), _p(v_pool), _p(page_table), page_table.shape[1],
        page_size, ring, _p(out), out.shape[1], _p(tok_pos), _p(tok_slot), T, n_heads, n_kv, head_dim,
        float(scale), float(cap or 0.0), int(window or 0), _stream()), "attn_prefill_paged")
    return out


def attn_decode(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, k_pool: torch.Tensor,
                v_pool: torch.Tensor, page_table: torch.Tensor, page_size: int, ring: int,
                slots: torch.Tensor, slot_len: torch.Tensor, scale: float, cap: Optional[float],
                window: Optional[int], n_splits: int, part_o: torch.Tensor, part_ml: torch.Tensor):
    """One query row per sequence against the paged cache.  q = the first nq*hd columns of qkv.
    ``slots``, ``slot_len`` and ``page_table`` must be complete before the kernel that runs just before
    this one on the stream starts (host copies and earlier kernels are): the tensor-core kernel reads
    them while that kernel may still run."""
    _req(qkv, "qkv", None, 2)
    B = qkv.shape[0]
    _req(k_pool, "k_pool", qkv.dtype, 4)
    _req(v_pool, "v_pool", qkv.dtype, 4)
    _req(page_table, "page_table", torch.int32, 2)
    _req(slots, "slots", torch.int32, 1)
    _req(slot_len, "slot_len", torch.int32, 1)
    need = B * n_heads * n_splits
    if part_o.numel() < need * head_dim or part_ml.numel() < need * 2:
        raise ValueError("attn_decode: scratch is too small")
    out = torch.empty((B, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    L = _lib.load()
    _lib.check(L.qnn_attn_decode(
        _p(qkv), qkv.shape[1], dt_code(qkv), _p(k_pool), _p(v_pool), _p(page_table), page_table.shape[1],
        page_size, ring, _p(slots), _p(slot_len), B, n_heads, n_kv, head_dim, float(scale), float(cap or 0.0),
        int(window or 0), _p(part_o), _p(part_ml), n_splits, _p(out), out.shape[1], _stream()), "attn_decode", 2)
    return out


def sample_scratch_bytes(rows: int, vocab: int, top_k: int) -> int:
    L = _lib.load()
    return int(L.qnn_sample_scratch_bytes(rows, vocab, top_k))


def sample(logits: torch.Tensor, top_k: int, temperature: float, top_p: float, penalty: float,
           rng_state: torch.Tensor, seen: Optional[torch.Tensor], seen_rows: Optional[torch.Tensor],
           scratch: torch.Tensor, out_tokens: torch.Tensor, error_flag: Optional[torch.Tensor]):
    _req(logits, "logits", torch.float32, 2)
    R, V = logits.shape
    _req(out_tokens, "out_tokens", torch.int32, 1)
    _req(rng_state, "rng_state", torch.int32, 1)
    if out_tokens.numel() < R or rng_state.numel() < R:
        raise ValueError("sample: out_tokens / rng_state are shorter than the batch")
    if scratch.numel() * scratch.element_size() < sample_scratch_bytes(R, V, top_k):
        raise ValueError("sample: scratch is too small")
    L = _lib.load()
    _lib.check(L.qnn_sample(_p(logits), R, V, int(top_k), float(temperature), float(top_p), float(penalty),
                            _p(rng_state), _p(seen), _p(seen_rows), _p(scratch), _p(out_tokens), _p(error_flag),
                            _stream()), "sample", 2)
    return out_tokens


def mark_seen(tokens: torch.Tensor, rows: torch.Tensor, seen: torch.Tensor):
    _req(tokens, "tokens", torch.int32, 1)
    _req(rows, "rows", torch.int32, 1)
    _req(seen, "seen", torch.uint8, 2)
    L = _lib.load()
    _lib.check(L.qnn_mark_seen(_p(tokens), _p(rows), _p(seen), seen.shape[1], tokens.numel(), _stream()),
               "mark_seen")

"""Tensor-level wrappers of the CUDA launchers.

Each function checks devices, dtypes, shapes and contiguity on the host, then
calls the C entry point on the current CUDA stream.  Outputs are allocated by the
caller or here with ``torch.empty`` (the caching allocator, so that a step can be
captured in a CUDA graph).  Matrix products run on this library's own kernels:
float32 on FFMA kernels, bfloat16 on the mma.sync small-M kernel (up to 64 rows), the
cluster split-K tcgen05 kernel (9 to 128 rows) and the tcgen05/TMA GEMMs (whole
prompts; sizes they refuse go through the small-M kernel 64 rows at a time).  A library
product (cuBLAS through ``torch.matmul``) is used only when ``QNN_GEMM=cublas`` asks
for it, for comparisons.
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


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current device's current stream as a handle for the launchers.  Asked for at every launch, so by the
    two plain C calls where this torch has them (``torch.cuda.current_stream()`` walks a dozen Python frames, a
    third of the host time of a short step)."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
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


def embed_rmsnorm(tokens: torch.Tensor, table: torch.Tensor, scale: float, weight: torch.Tensor, eps: float,
                  unit_offset: bool, out_dtype: torch.dtype):
    """``embed`` and the first norm of what it gives in one kernel: (rows [T, H] float32, rmsnorm(rows))."""
    _req(tokens, "tokens", torch.int32, 1)
    _req(table, "table", None, 2)
    _req(weight, "weight", None, 1)
    T, (V, H) = tokens.numel(), table.shape
    if weight.numel() != H:
        raise ValueError(f"norm weight has {weight.numel()} elements for width {H}")
    out = torch.empty((T, H), dtype=torch.float32, device=tokens.device)
    normed = torch.empty((T, H), dtype=out_dtype, device=tokens.device)
    _lib.check(_lib.load().qnn_embed_rmsnorm(_p(tokens), _p(table), dt_code(table), float(scale), _p(out), _p(weight),
                                             dt_code(weight), float(eps), int(unit_offset), _p(normed), dt_code(normed),
                                             T, H, V, _stream()), "embed_rmsnorm")
    return out, normed


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


def check_finite(x: torch.Tensor, flag: Optional[torch.Tensor] = None):
    """Set ``flag`` (default: this device's non-finite word, read by ``raise_on_status``) if
    ``x`` holds NaN or Inf."""
    _req(x, "x", torch.float32)
    if flag is None:
        flag = finite_flag(x.device)
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


_no_freq = {}


def cache_append(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, tok_pos: torch.Tensor,
                 tok_slot: torch.Tensor, line) -> None:
    """Append the keys and values of the packed q|k|v rows to a cache line as they are (no rotation).
    ``line`` is a cache line view (k, v, page_table, page_size, ring, slot_len)."""
    f = _no_freq.get(qkv.device)
    if f is None:
        f = _no_freq[qkv.device] = torch.zeros(0, dtype=torch.float32, device=qkv.device)
    rope_cache_write(qkv, n_heads, n_kv, head_dim, 0, f, tok_pos, tok_slot, line.k, line.v, line.page_table,
                     line.page_size, line.ring, line.slot_len, True)


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


_status = {}


def status_words(device) -> torch.Tensor:
    """Two int32 words per device that kernels set and the host reads together: [0] the status of
    the tcgen05 kernels' bounded waits (1 loads, 2 tensor-core issue, 4 epilogue), [1] the
    non-finite flag of ``check_finite``."""
    device = torch.device(device)
    t = _status.get(device)
    if t is None:
        t = torch.zeros(2, dtype=torch.int32, device=device)
        _status[device] = t
    return t


def _status_word(device) -> torch.Tensor:
    return status_words(device)[0:1]


def finite_flag(device) -> torch.Tensor:
    return status_words(device)[1:2]


def wait_status_message(v: int) -> str:
    return (f"a tcgen05 kernel gave up waiting (status {v}: 1 loads, 2 tensor-core issue, 4 epilogue); "
            f"its result is not valid")


def raise_on_status(device) -> None:
    """Read both words (one 8-byte copy; it synchronises, so call it where the host waits anyway)
    and raise if a bounded wait ran out or a checked tensor held NaN or Inf since the last call."""
    t = _status.get(torch.device(device))
    if t is None:
        return
    wait, bad = t.tolist()
    if wait or bad:
        t.zero_()
    if wait:
        raise _lib.KernelError(wait_status_message(wait))
    if bad:
        raise _lib.NonFiniteLogits("the model produced non-finite logits")


check_gemm_status = raise_on_status


GEMM_2CTA = os.environ.get("QNN_GEMM_2CTA", "1") != "0"


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, *, epilogue: int = EPI_NONE, activation: str = "gelu_tanh",
                 pair: Optional[bool] = None, out: Optional[torch.Tensor] = None):
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
    if out is None:
        out = torch.empty((M, n_out), dtype=torch.bfloat16, device=x.device)
    else:
        _req(out, "out", torch.bfloat16, 2)
        if tuple(out.shape) != (M, n_out):
            raise ValueError(f"gemm_tcgen05: out is {tuple(out.shape)}, the product [{M}, {n_out}]")
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
                        activation: str = "gelu_tanh", out: Optional[torch.Tensor] = None):
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
    out_dtype = torch.float32 if epilogue == EPI_SOFTCAP else torch.bfloat16
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
    else:
        _req(out, "out", out_dtype, 2)
        if tuple(out.shape) != (M, n_out):
            raise ValueError(f"gemm_skinny_tcgen05: out is {tuple(out.shape)}, the product [{M}, {n_out}]")
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


_SM_COUNT: dict = {}


def _rows_for_the_small_kernel(M: int, n_out: int, K: int, epilogue: int, device) -> int:
    """How many of the last rows of a whole-prompt product go to the kernel for few rows instead (0: none).

    The prompt kernel works in 256 x 256 tiles (256 x 128 outputs when gated), a pair of SMs per tile, so its time
    goes up by a round of tiles when the tile count passes a multiple of the pairs.  Measured for the down product
    (2304 x 9216): 2048 rows (72 tiles on 74 pairs) 58 us, 2049 rows 92 us, 4096 / 4097 rows 114 / 140 us, 6144 /
    6145 rows 175 / 212 us: a round that only a few tiles open costs about 0.6 of a tile's time.  The kernel for few
    rows takes the weights' bytes once more plus 5 us up to 32 rows and 9 us up to 64 (2049 rows: 66 us together, 4097:
    123, 6145: 179); with more rows it costs what the round does (2200 rows in two launches: 90 against 92 us), and
    for the matrices with a short inner size the round is cheap, so only up to 64 rows are cut off, and only where
    the round costs well more than they do."""
    if not GEMM_2CTA or M <= 256:
        return 0
    tail = M % 256
    if tail == 0 or tail > 64:
        return 0
    key = str(device)
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(device).multi_processor_count if device.type == "cuda" else 148
    pairs = max(1, _SM_COUNT[key] // 2)
    per_row_tile = -(-n_out // (128 if epilogue == EPI_GATED else 256))
    rounds = lambda m_tiles: -(-m_tiles * per_row_tile // pairs)          # noqa: E731
    if rounds(-(-M // 256)) == rounds(M // 256):
        return 0
    weights = n_out * (2 if epilogue == EPI_GATED else 1) * K
    round_us = 0.6 * 2.0 * 256 * 256 * K / 22.0e6                # a tile at a pair's share of 1.6 PFLOP/s
    small_us = 2.0 * weights / 6.5e6 + (5.0 if tail <= 32 else 9.0)
    return tail if round_us > 1.5 * small_us else 0


def linear(x: torch.Tensor, w: torch.Tensor, *, epilogue: int = EPI_NONE, cap: Optional[float] = None,
           activation: str = "gelu_tanh", out_dtype: Optional[torch.dtype] = None):
    """y = x w^T with an optional epilogue.  x: [M, K]; w: [N, K] (gated: [2*N_out, K]).

    float32: FFMA kernels only.  bfloat16: the tensor-core small-M kernel up to 64 rows (the cluster
    split-K tcgen05 kernel from 9 rows on against big matrices), the tcgen05/TMA kernel above that; an inner
    size that is no multiple of 8 (rows that do not start on 16 bytes) goes to a plain kernel; a library
    product (cuBLAS) only when QNN_GEMM=cublas is set."""
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
    if K % 8:                                  # rows that do not start on 16 bytes: the plain kernel for any inner size
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        _lib.check(L.qnn_linear_bf16_any(_p(x), _p(w), _p(out), dt_code(out), M, N, K, epilogue, capv, act, _stream()),
                   "linear_bf16_any")
        return out
    if _takes_skinny_tcgen05(M, N, K) and out_dtype == (torch.float32 if epilogue == EPI_SOFTCAP else torch.bfloat16):
        y = gemm_skinny_tcgen05(x, w, epilogue=epilogue, cap=cap, activation=activation)
        if y is not None:
            return y
    def small(xr: torch.Tensor, out: torch.Tensor) -> None:
        _lib.check(L.qnn_skinny_bf16(_p(xr), _p(w), _p(out), dt_code(out), xr.shape[0], N, K, epilogue, capv, act,
                                     _stream()), "skinny_bf16")

    if M <= SKINNY_MAX_ROWS:
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        small(x, out)
        return out
    if USE_TCGEN05:
        if epilogue in (EPI_NONE, EPI_GATED) and out_dtype == torch.bfloat16:
            tail = _rows_for_the_small_kernel(M, n_out, K, epilogue, x.device)
            if tail:
                # the last rows would open one more round of 256 x 256 tiles: they go to the kernel for few rows
                head = M - tail
                out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
                ok = (gemm_tcgen05(x[:head], w, epilogue=epilogue, activation=activation, out=out[:head]) is not None
                      and gemm_skinny_tcgen05(x[head:], w, epilogue=epilogue, activation=activation,
                                              out=out[head:]) is not None)
                if ok:
                    return out
            y = gemm_tcgen05(x, w, epilogue=epilogue, activation=activation)
            if y is not None:
                return y
        elif epilogue == EPI_SOFTCAP:          # logits wanted at many places: the product, then the cap in float32
            y = gemm_tcgen05(x, w)
            if y is not None:
                return softcap(y, cap)
        # sizes that the tcgen05 kernels refuse: the small-M kernel, 64 rows at a time
        out = torch.empty((M, n_out), dtype=out_dtype, device=x.device)
        for r0 in range(0, M, SKINNY_MAX_ROWS):
            small(x[r0:r0 + SKINNY_MAX_ROWS], out[r0:r0 + SKINNY_MAX_ROWS])
        return out
    y = torch.matmul(x, w.t())                 # QNN_GEMM=cublas: the library product, for comparisons
    if epilogue == EPI_GATED:
        return gated_act(y, activation)
    if epilogue == EPI_SOFTCAP:
        return softcap(y, cap)
    return y if out_dtype == y.dtype else cast(y, out_dtype)


ATTN_TCGEN05 = os.environ.get("QNN_ATTN", "tcgen05") != "mma"
# A step that continues sequences takes the tensor-core prompt kernel from this many rows of a sequence on.  Measured
# at 8 heads of 256, one sequence, launched eagerly: 8 new rows on 4000 cached tokens 108 us against 3776 us of the
# generic kernel (a warp per row and kv head that walks the keys one after the other), 512 rows on 7000: 152 us against
# 8477; so always, where the sizes allow.
EXTEND_TENSOR_CORE_FROM = int(os.environ.get("QNN_EXTEND_TC_FROM", "1"))


def attention_refusal(dtype: torch.dtype, n_heads: int, n_kv: int, head_dim: int) -> Optional[str]:
    """None if the attention kernels take these head counts and this head size in ``dtype``, else the
    reason in words.  Asked when a model is loaded."""
    code = _lib.load().qnn_attn_supports(BF16 if dtype == torch.bfloat16 else F32, n_heads, n_kv, head_dim)
    if code == 0:
        return None
    vec = 8 if dtype == torch.bfloat16 else 4
    if code == _lib.ERR_ARGUMENT:
        return f"{n_kv} key/value heads do not divide {n_heads} query heads"
    return (f"head size {head_dim} in {dtype}: the attention kernels take multiples of {vec} up to {128 * vec} "
            f"(less when four or more query heads share a key/value head)")


def linear_refusal(dtype: torch.dtype, inner: int) -> Optional[str]:
    """None if the matrix products take this inner size in ``dtype``, else the reason.  Every size is taken:
    bfloat16 rows of whole 16-byte pieces (a multiple of 8) by the tensor-core kernels, others by a plain one."""
    if inner <= 0:
        return f"an inner size of {inner}"
    return None


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
                _p(qkv), T, _p(out), out.shape[1], _p(seq_row0), _p(seq_len), None, seq_row0.numel(), int(max_len),
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


def attn_extend(qkv: torch.Tensor, n_heads: int, n_kv: int, head_dim: int, k_pool: torch.Tensor, v_pool: torch.Tensor,
                page_table: torch.Tensor, page_size: int, ring: int, tok_pos: torch.Tensor, tok_row0: torch.Tensor,
                tok_slot: torch.Tensor, scale: float, cap: Optional[float], window: Optional[int], whole=None):
    """Attention of a step that continues sequences by several tokens: each row sees the cached
    positions before its sequence's first row of this step (from the cache, as earlier steps left it)
    and this step's own rows from there to itself (from ``qkv``, already rotated).  The caller appends
    this step's keys and values to the cache afterwards.

    ``whole`` (a ``WholeSequences``, optional) describes the step's sequences laid out with their cached
    tokens in front; with it, bfloat16 rows of head size 64, 128 or 256 go through the tensor-core prompt
    kernel: the cached keys and values are copied out of the pages into that layout, the kernel leaves out
    the query tiles that lie before each sequence's new rows, and the new rows' outputs are picked out.
    The generic kernel walks the keys once per row and kv head: it serves float32 and the other head sizes."""
    _req(qkv, "qkv", None, 2)
    _req(k_pool, "k_pool", qkv.dtype, 4)
    _req(v_pool, "v_pool", qkv.dtype, 4)
    for n, t in (("tok_pos", tok_pos), ("tok_row0", tok_row0), ("tok_slot", tok_slot)):
        _req(t, n, torch.int32, 1)
    T = qkv.shape[0]
    if (whole is not None and ATTN_TCGEN05 and qkv.dtype == torch.bfloat16 and head_dim in (64, 128, 256)
            and whole.most_new >= EXTEND_TENSOR_CORE_FROM):
        L = _lib.load()
        B = whole.row0.numel()
        rows = torch.empty((whole.total, qkv.shape[1]), dtype=qkv.dtype, device=qkv.device)
        _lib.check(L.qnn_attn_extend_gather(
            _p(qkv), _p(k_pool), _p(v_pool), _p(page_table), page_table.shape[1], page_size, ring, _p(whole.slots),
            _p(whole.start), _p(whole.new_row0), _p(whole.new_len), _p(whole.row0), _p(rows), B, whole.longest,
            n_heads, n_kv, head_dim, _stream()), "attn_extend_gather")
        out_rows = torch.empty((whole.total, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
        code = L.qnn_attn_prefill_tcgen05(
            _p(rows), whole.total, _p(out_rows), out_rows.shape[1], _p(whole.row0), _p(whole.length), _p(whole.start), B,
            whole.longest, n_heads, n_kv, head_dim, float(scale), float(cap or 0.0), int(window or 0),
            _p(_status_word(qkv.device)), _stream())
        if code != _lib.ERR_UNSUPPORTED:
            _lib.check(code, "attn_prefill_tcgen05")
            return gather_rows(out_rows, whole.tok_row, qkv.dtype)
    out = torch.empty((T, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    es = qkv.element_size()
    q_ptr = qkv.data_ptr()
    k_ptr = q_ptr + n_heads * head_dim * es
    v_ptr = k_ptr + n_kv * head_dim * es
    L = _lib.load()
    _lib.check(L.qnn_attn_extend(
        ctypes.c_void_p(q_ptr), ctypes.c_void_p(k_ptr), ctypes.c_void_p(v_ptr), qkv.shape[1], dt_code(qkv),
        _p(k_pool), _p(v_pool), _p(page_table), page_table.shape[1], page_size, ring, _p(out), out.shape[1],
        _p(tok_pos), _p(tok_row0), _p(tok_slot), T, n_heads, n_kv, head_dim, float(scale), float(cap or 0.0),
        int(window or 0), _stream()), "attn_extend")
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
           scratch: torch.Tensor, out_tokens: torch.Tensor, error_flag: Optional[torch.Tensor],
           status: Optional[torch.Tensor] = None):
    """``status`` (one int32 on the device) is OR-ed into ``error_flag`` as bit 1 plus its value
    from bit 8 up: what the step's kernels reported reaches the host with the ids."""
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
                            _p(status), _stream()), "sample", 4 if (temperature > 0 and top_k > 1 and V > 1) else 2)
    return out_tokens


def head_argmax_fusable(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``head_argmax`` takes this product: bfloat16 on both sides, an inner size in whole 16-byte
    vectors, and at most 128 rows."""
    M, K = x.shape
    return x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and 1 <= M <= 128


def head_candidates(vocab: int) -> int:
    """The most candidates per row that ``head_argmax`` writes (one per 16 output columns)."""
    return (vocab + 15) // 16


def head_argmax(x: torch.Tensor, w: torch.Tensor, cap: Optional[float], cand: torch.Tensor,
                error_flag: Optional[torch.Tensor]) -> Optional[int]:
    """softcap(x w^T) reduced in the product's epilogue to the best (value, id) of every group of output
    columns: ``cand`` (float32, at least rows * head_candidates(vocab) * 2) is filled, the logits are not
    written.  The product is the one that ``linear`` would run for these sizes: the mma.sync small-M kernel
    (a candidate per 16 columns) or, from 9 rows on against a big matrix, the tcgen05 kernel (a candidate
    per 128 columns).  Returns the number of candidates per row, or None when the sizes are refused (the
    caller then forms the logits).  NaN or Inf sets bit 0 of ``error_flag``."""
    _req(x, "x", torch.bfloat16, 2)
    _req(w, "w", torch.bfloat16, 2)
    _req(cand, "cand", torch.float32)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise ValueError(f"head_argmax: x is [*, {K}] but w is [*, {w.shape[1]}]")
    if cand.numel() < M * head_candidates(N) * 2:
        raise ValueError("head_argmax: the candidate buffer is too small")
    L = _lib.load()
    if _takes_skinny_tcgen05(M, N, K):
        code = L.qnn_gemm_skinny_tcgen05_argmax(_p(x), _p(w), _p(cand), M, N, K, float(cap or 0.0), _p(error_flag),
                                                _p(_status_word(x.device)), _stream())
        if code != _lib.ERR_UNSUPPORTED:
            _lib.check(code, "gemm_skinny_tcgen05_argmax")
            return (N + 127) // 128
    if M > SKINNY_MAX_ROWS:
        return None
    _lib.check(L.qnn_skinny_argmax(_p(x), _p(w), _p(cand), M, N, K, float(cap or 0.0), _p(error_flag), _stream()),
               "skinny_argmax")
    return (N + 15) // 16


def sample_candidates(cand: torch.Tensor, rows: int, ncand: int, vocab: int, top_k: int, temperature: float,
                      top_p: float, rng_state: torch.Tensor, seen: Optional[torch.Tensor],
                      seen_rows: Optional[torch.Tensor], out_tokens: torch.Tensor,
                      error_flag: Optional[torch.Tensor], status: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The merge-and-draw half of ``sample`` on candidates [rows, ncand] of (value, id) pairs."""
    _req(cand, "cand", torch.float32)
    _req(out_tokens, "out_tokens", torch.int32, 1)
    _req(rng_state, "rng_state", torch.int32, 1)
    if cand.numel() < rows * ncand * 2 or out_tokens.numel() < rows or rng_state.numel() < rows:
        raise ValueError("sample_candidates: a buffer is shorter than the batch")
    L = _lib.load()
    _lib.check(L.qnn_sample_candidates(_p(cand), rows, ncand, vocab, int(top_k), float(temperature), float(top_p),
                                       _p(rng_state), _p(seen), _p(seen_rows), _p(out_tokens), _p(error_flag),
                                       _p(status), _stream()), "sample_candidates")
    return out_tokens


def mark_seen(tokens: torch.Tensor, rows: torch.Tensor, seen: torch.Tensor):
    _req(tokens, "tokens", torch.int32, 1)
    _req(rows, "rows", torch.int32, 1)
    _req(seen, "seen", torch.uint8, 2)
    L = _lib.load()
    _lib.check(L.qnn_mark_seen(_p(tokens), _p(rows), _p(seen), seen.shape[1], tokens.numel(), _stream()),
               "mark_seen")

"""The entry point for callers that cannot allocate device memory, qnn_attn_decode_static,
called the way such a caller reaches it: through its exported C symbol, with raw pointers.

Its scratch is an array inside the library, shared by all calls, so the check runs two calls in a
row (different sizes, the second one reading what the first left behind) and compares each with
qnn_attn_decode given scratch of its own.  This file sorts last on purpose: if it fails, a run that
stops at the first failure has already run everything else.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, B, nq, nkv, hd, lens, dtype):
    rng = np.random.default_rng(seed)
    pages_per = max(-(-n // 64) for n in lens)
    n_pages = 1 + B * pages_per
    k_pool = torch.from_numpy(rng.normal(size=(n_pages, nkv, 64, hd)).astype(np.float32)).to(DEV).to(dtype)
    v_pool = torch.from_numpy(rng.normal(size=(n_pages, nkv, 64, hd)).astype(np.float32)).to(DEV).to(dtype)
    table = np.zeros((B, pages_per), dtype=np.int32)
    order = rng.permutation(np.arange(1, n_pages))
    for b in range(B):
        table[b] = order[b * pages_per:(b + 1) * pages_per]
    qkv = torch.from_numpy(rng.normal(size=(B, (nq + 2 * nkv) * hd)).astype(np.float32)).to(DEV).to(dtype)
    i32 = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)  # noqa: E731
    return qkv, k_pool, v_pool, i32(table), i32(np.arange(B)), i32(lens)


def test_static_scratch_entry_point_matches_the_allocating_one():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from quicknn_b200.kernels import lib, ops
    L = lib.load()
    fn = L.qnn_attn_decode_static                      # the exported C symbol
    vp, ll, ci, cf = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp, ll, ci, vp, vp, vp, ci, ci, ci, vp, vp, ci, ci, ci, ci, cf, cf, ci, ci, vp, ll, vp]
    fn.restype = ci
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731

    cases = [dict(seed=1, B=3, nq=8, nkv=4, hd=64, lens=[200, 65, 1], dtype=torch.bfloat16, splits=5, window=0, cap=50.0),
             dict(seed=2, B=2, nq=6, nkv=1, hd=24, lens=[130, 300], dtype=torch.float32, splits=3, window=100, cap=0.0)]
    for c in cases:                                    # two calls in a row on the one shared array
        qkv, k_pool, v_pool, table, slots, lens = _case(c["seed"], c["B"], c["nq"], c["nkv"], c["hd"], c["lens"], c["dtype"])
        B, nq, nkv, hd, S = c["B"], c["nq"], c["nkv"], c["hd"], c["splits"]
        scale = 1.0 / math.sqrt(hd)
        part_o = torch.empty(B * nq * S * hd, device=DEV)
        part_ml = torch.empty(B * nq * S * 2, device=DEV)
        want = ops.attn_decode(qkv, nq, nkv, hd, k_pool, v_pool, table, 64, 0, slots, lens, scale, c["cap"] or None,
                               c["window"] or None, S, part_o, part_ml)
        got = torch.full_like(want, float("nan"))
        code = fn(p(qkv), qkv.shape[1], ops.dt_code(qkv), p(k_pool), p(v_pool), p(table), table.shape[1], 64, 0,
                  p(slots), p(lens), B, nq, nkv, hd, scale, c["cap"], c["window"], S, p(got), got.shape[1], stream)
        assert code == 0, f"qnn_attn_decode_static returned {code}"
        torch.cuda.synchronize()
        w, g = want.float().cpu().numpy(), got.float().cpu().numpy()
        tol = (2e-6 if c["dtype"] == torch.float32 else 1.0 / 128) * max(1e-30, float(np.abs(w).max()))
        assert np.isfinite(g).all() and float(np.abs(g - w).max()) <= tol

    # beyond the stated maximum: refused with its own code, nothing launched
    qkv, k_pool, v_pool, table, slots, lens = _case(3, 2, 8, 4, 256, [10, 10], torch.bfloat16)
    out = torch.zeros((2, 8 * 256), dtype=torch.bfloat16, device=DEV)
    big = 1 + (4 << 20) // (2 * 8 * (256 + 2) * 4)
    code = fn(p(qkv), qkv.shape[1], 1, p(k_pool), p(v_pool), p(table), table.shape[1], 64, 0, p(slots), p(lens),
              2, 8, 4, 256, 0.0625, 0.0, 0, big, p(out), out.shape[1], stream)
    assert code == 10003
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0

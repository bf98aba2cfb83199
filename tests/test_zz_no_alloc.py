"""The entry point for callers that cannot allocate device memory, qnn_attn_decode_static,
called the way such a caller reaches it: through its exported C symbol, with raw pointers.

Its scratch is an array inside the library, shared by all calls, so the check runs several calls in
a row (different sizes and precisions, each reading what the one before left behind, one of them right
at the array's limit) and compares each with qnn_attn_decode given scratch of its own.  This file sorts last on purpose: if it fails, a run that
stops at the first failure has already run everything else.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, B, nq, nkv, hd, lens, dtype, ring=0, left_out=()):
    """Random queries, a paged cache with shuffled pages and the per-sequence arrays.  With ``ring`` a
    sequence holds ring/64 pages and position p lives at p mod ring; rows in ``left_out`` get slot -1
    (a row of the batch that belongs to no sequence: it must come out as zeros)."""
    rng = np.random.default_rng(seed)
    pages_per = ring // 64 if ring else max(-(-n // 64) for n in lens)
    n_pages = 1 + B * pages_per
    k_pool = torch.from_numpy(rng.normal(size=(n_pages, nkv, 64, hd)).astype(np.float32)).to(DEV).to(dtype)
    v_pool = torch.from_numpy(rng.normal(size=(n_pages, nkv, 64, hd)).astype(np.float32)).to(DEV).to(dtype)
    table = np.zeros((B, pages_per), dtype=np.int32)
    order = rng.permutation(np.arange(1, n_pages))
    for b in range(B):
        table[b] = order[b * pages_per:(b + 1) * pages_per]
    qkv = torch.from_numpy(rng.normal(size=(B, (nq + 2 * nkv) * hd)).astype(np.float32)).to(DEV).to(dtype)
    i32 = lambda a: torch.from_numpy(np.asarray(a, dtype=np.int32)).to(DEV)  # noqa: E731
    slots = np.arange(B)
    slots[list(left_out)] = -1
    return qkv, k_pool, v_pool, i32(table), i32(slots), i32(lens)


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

    # Calls in a row on the one shared array, each reading what the one before left behind: more key ranges
    # than a cluster merges (so the scratch and the combine pass are really used) in bfloat16 and in float32,
    # then a smaller bfloat16 call with a ring as long as its window and a row that belongs to no sequence,
    # whose partial results must all be written afresh (the reference's own scratch starts as NaN: whatever
    # the combine pass reads has been written by this call).
    cases = [dict(seed=1, B=3, nq=8, nkv=4, hd=64, lens=[200, 65, 1], dtype=torch.bfloat16, splits=5, window=0, cap=50.0),
             dict(seed=2, B=2, nq=6, nkv=1, hd=24, lens=[130, 300], dtype=torch.float32, splits=3, window=100, cap=0.0),
             dict(seed=4, B=3, nq=4, nkv=2, hd=128, lens=[300, 129, 40], dtype=torch.bfloat16, splits=6, window=128,
                  cap=30.0, ring=128, left_out=[1])]
    for c in cases:
        ring = c.get("ring", 0)
        qkv, k_pool, v_pool, table, slots, lens = _case(c["seed"], c["B"], c["nq"], c["nkv"], c["hd"], c["lens"], c["dtype"],
                                                       ring, c.get("left_out", ()))
        B, nq, nkv, hd, S = c["B"], c["nq"], c["nkv"], c["hd"], c["splits"]
        scale = 1.0 / math.sqrt(hd)
        part_o = torch.full((B * nq * S * hd,), float("nan"), device=DEV)
        part_ml = torch.full((B * nq * S * 2,), float("nan"), device=DEV)
        want = ops.attn_decode(qkv, nq, nkv, hd, k_pool, v_pool, table, 64, ring, slots, lens, scale, c["cap"] or None,
                               c["window"] or None, S, part_o, part_ml)
        got = torch.full_like(want, float("nan"))
        code = fn(p(qkv), qkv.shape[1], ops.dt_code(qkv), p(k_pool), p(v_pool), p(table), table.shape[1], 64, ring,
                  p(slots), p(lens), B, nq, nkv, hd, scale, c["cap"], c["window"], S, p(got), got.shape[1], stream)
        assert code == 0, f"qnn_attn_decode_static returned {code}"
        torch.cuda.synchronize()
        w, g = want.float().cpu().numpy(), got.float().cpu().numpy()
        tol = (2e-6 if c["dtype"] == torch.float32 else 1.0 / 128) * max(1e-30, float(np.abs(w).max()))
        assert np.isfinite(w).all() and np.isfinite(g).all() and float(np.abs(g - w).max()) <= tol
        for r in c.get("left_out", ()):
            assert float(np.abs(g[r]).max()) == 0.0

    # At the limit: 5 x 8 x 397 partial rows of 64 + 2 floats are 4,192,320 bytes, the most that these head
    # counts fit into the 4 MiB; it runs and agrees.  One more key range (4,202,880 bytes) is refused.
    qkv, k_pool, v_pool, table, slots, lens = _case(5, 5, 8, 4, 64, [900, 64, 397, 1000, 500], torch.bfloat16)
    assert 5 * 8 * 397 * 66 * 4 <= (4 << 20) < 5 * 8 * 398 * 66 * 4
    part_o = torch.empty(5 * 8 * 397 * 64, device=DEV)
    part_ml = torch.empty(5 * 8 * 397 * 2, device=DEV)
    want = ops.attn_decode(qkv, 8, 4, 64, k_pool, v_pool, table, 64, 0, slots, lens, 0.125, None, None, 397, part_o, part_ml)
    got = torch.full_like(want, float("nan"))
    args = [p(qkv), qkv.shape[1], 1, p(k_pool), p(v_pool), p(table), table.shape[1], 64, 0, p(slots), p(lens), 5, 8, 4, 64,
            0.125, 0.0, 0]
    assert fn(*args, 397, p(got), got.shape[1], stream) == 0
    torch.cuda.synchronize()
    w, g = want.float().cpu().numpy(), got.float().cpu().numpy()
    assert np.isfinite(g).all() and float(np.abs(g - w).max()) <= float(np.abs(w).max()) / 128
    untouched = torch.zeros_like(want)
    assert fn(*args, 398, p(untouched), untouched.shape[1], stream) == 10003
    torch.cuda.synchronize()
    assert float(untouched.float().abs().sum()) == 0.0

    # beyond the stated maximum: refused with its own code, nothing launched
    qkv, k_pool, v_pool, table, slots, lens = _case(3, 2, 8, 4, 256, [10, 10], torch.bfloat16)
    out = torch.zeros((2, 8 * 256), dtype=torch.bfloat16, device=DEV)
    big = 1 + (4 << 20) // (2 * 8 * (256 + 2) * 4)
    code = fn(p(qkv), qkv.shape[1], 1, p(k_pool), p(v_pool), p(table), table.shape[1], 64, 0, p(slots), p(lens),
              2, 8, 4, 256, 0.0625, 0.0, 0, big, p(out), out.shape[1], stream)
    assert code == 10003
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0

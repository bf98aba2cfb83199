"""Each CUDA kernel alone against its plain reference, at sizes other than the engine's:
widths and vocabularies that are no power of two, head sizes in steps of 8 and 16, any
number of heads and groups, float32 and bfloat16."""
import math

import numpy as np
import pytest
import torch

from plain import gemma2_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from quicknn_b200.kernels import ops as o
    return o


def T(a, dtype):
    return torch.from_numpy(np.asarray(a)).to(DEV).to(dtype).contiguous()


def N(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def bf16_round(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)


TOL = {torch.float32: 2e-6, torch.bfloat16: 1.0 / 128}


def assert_close(got, ref, dtype, what="", mult=1.0):
    ref = np.asarray(ref, dtype=np.float64)
    scale = max(1e-30, float(np.abs(ref).max()))
    g = N(got) if isinstance(got, torch.Tensor) else np.asarray(got, dtype=np.float64)
    err = float(np.abs(g - ref).max())
    assert err <= TOL[dtype] * mult * scale, f"{what}: error {err:.3g} > {TOL[dtype] * mult * scale:.3g}"


# ---- embedding, norms, elementwise --------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(ops, dtype):
    rng = np.random.default_rng(0)
    table = bf16_round(rng.normal(size=(37, 100)))
    ids = np.array([0, 36, 5, 37, -1, 12], dtype=np.int32)
    out = ops.embed(T(ids, torch.int32), T(table, dtype), math.sqrt(100))
    ref = P.embed(table, ids.tolist(), 100, np.float64)
    assert out.dtype == torch.float32
    assert_close(out, ref, torch.float32, "embed")
    assert float(out[3].abs().sum()) == 0.0 and float(out[4].abs().sum()) == 0.0   # ids outside the table
    # the same rows with their first norm from the same kernel
    w = bf16_round(rng.normal(size=100) * 0.2)
    for act in (torch.float32, torch.bfloat16):
        rows, normed = ops.embed_rmsnorm(T(ids, torch.int32), T(table, dtype), math.sqrt(100), T(w, dtype), 1e-6, True, act)
        assert torch.equal(rows, out) and normed.dtype == act
        assert_close(normed, P.rmsnorm(N(out), w, 1e-6), act, "embed + norm")


@pytest.mark.parametrize("H", [8, 100, 2304])
@pytest.mark.parametrize("act,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32)])
def test_rmsnorm_and_fused_residual(ops, H, act, wdt):
    rng = np.random.default_rng(H)
    x = rng.normal(size=(5, H)) * 3
    y = bf16_round(rng.normal(size=(5, H)))
    w1, w2 = bf16_round(rng.normal(size=H) * 0.2), bf16_round(rng.normal(size=H) * 0.2)
    out = ops.rmsnorm(T(x, torch.float32), T(w1, wdt), 1e-5, True, act)
    assert_close(out, P.rmsnorm(x.astype(np.float32).astype(np.float64), w1, 1e-5), act, "rmsnorm(1+w)")
    out = ops.rmsnorm(T(y, act), T(w1, wdt), 1e-6, False, act)
    assert_close(out, P.rmsnorm(y, w1 - 1.0, 1e-6), act, "rmsnorm(w)")
    resid = T(x, torch.float32)
    x32 = N(resid)
    nxt = ops.add_rmsnorm(resid, T(y, act), T(w1, wdt), 1e-5, True, T(w2, wdt), 1e-6, True, act)
    r_ref = x32 + P.rmsnorm(y, w1, 1e-5)
    assert_close(resid, r_ref, torch.float32, "residual", mult=4)
    assert_close(nxt, P.rmsnorm(r_ref, w2, 1e-6), act, "next norm")
    resid2 = T(x, torch.float32)
    assert ops.add_rmsnorm(resid2, T(y, act), T(w1, wdt), 1e-5, True) is None
    assert_close(resid2, r_ref, torch.float32, "residual only", mult=4)
    ops.add_(resid2, T(y, act))
    assert_close(resid2, r_ref + y, torch.float32, "add", mult=4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_activation_softcap_gather_cast(ops, dtype):
    rng = np.random.default_rng(3)
    gu = bf16_round(rng.normal(size=(7, 2 * 50)) * 2)
    out = ops.gated_act(T(gu, dtype), "gelu_tanh")
    assert_close(out, P.gelu_tanh(gu[:, :50]) * gu[:, 50:], dtype, "geglu")
    out = ops.gated_act(T(gu, dtype), "silu")
    g = gu[:, :50]
    assert_close(out, g / (1 + np.exp(-g)) * gu[:, 50:], dtype, "swiglu")
    x = bf16_round(rng.normal(size=(3, 33)) * 40)
    assert_close(ops.softcap(T(x, dtype), 15.0), P.softcap(x, 15.0), torch.float32, "softcap")
    assert_close(ops.softcap(T(x, dtype), None), x, torch.float32, "softcap off")
    bad = torch.tensor([float("nan"), float("inf"), -float("inf"), 1.0], dtype=dtype, device=DEV)
    capped = ops.softcap(bad, 15.0).cpu().numpy()          # NaN must stay visible to the finite check; Inf saturates
    assert np.isnan(capped[0]) and np.allclose(capped[1:3], [15.0, -15.0]) and np.isfinite(capped[3])
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.check_finite(ops.softcap(bad[3:], 15.0), flag)
    assert flag.item() == 0
    ops.check_finite(ops.softcap(bad, 15.0), flag)
    assert flag.item() != 0
    rows = T(np.array([2, 0, 2], dtype=np.int32), torch.int32)
    assert_close(ops.gather_rows(T(x, dtype), rows, torch.float32), x[[2, 0, 2]], torch.float32, "gather")
    assert ops.cast(T(x, torch.float32), torch.bfloat16).dtype == torch.bfloat16
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.check_finite(T(x, torch.float32), flag)
    assert int(flag) == 0
    x[1, 5] = np.inf
    ops.check_finite(T(x, torch.float32), flag)
    assert int(flag) == 1


# ---- matrix products ------------------------------------------------------------------

@pytest.mark.parametrize("M", [1, 5, 8, 17, 33, 64])
@pytest.mark.parametrize("N_,K", [(50, 96), (1000, 200), (2304, 2304), (24, 8)])
def test_skinny_bf16(ops, M, N_, K):
    rng = np.random.default_rng(M * 1000 + N_)
    x, w = bf16_round(rng.normal(size=(M, K))), bf16_round(rng.normal(size=(N_, K)) / math.sqrt(K))
    ref = x @ w.T
    y = ops.linear(T(x, torch.bfloat16), T(w, torch.bfloat16))
    assert y.dtype == torch.bfloat16 and tuple(y.shape) == (M, N_)
    assert_close(y, ref, torch.bfloat16, "skinny")
    y = ops.linear(T(x, torch.bfloat16), T(w, torch.bfloat16), epilogue=ops.EPI_SOFTCAP, cap=2.0)
    assert y.dtype == torch.float32
    assert_close(y, P.softcap(ref, 2.0), torch.float32, "skinny softcap", mult=50)
    y = ops.linear(T(x, torch.bfloat16), T(w, torch.bfloat16), epilogue=ops.EPI_GATED, activation="gelu_tanh")
    h = N_ // 2
    assert tuple(y.shape) == (M, h)
    assert_close(y, P.gelu_tanh(ref[:, :h]) * ref[:, h:], torch.bfloat16, "skinny geglu")


@pytest.mark.parametrize("M", [1, 7, 9, 70])
@pytest.mark.parametrize("N_,K", [(50, 100), (130, 50), (36, 7), (1001, 36)])
def test_bf16_products_of_inner_sizes_that_are_no_multiple_of_8(ops, M, N_, K):
    """Rows that do not start on 16 bytes go to the plain kernel: same roundings (bfloat16 in, float32 sums)."""
    rng = np.random.default_rng(M * 1000 + N_)
    x, w = bf16_round(rng.normal(size=(M, K))), bf16_round(rng.normal(size=(N_ & ~1, K)) / math.sqrt(K))
    ref = x @ w.T
    y = ops.linear(T(x, torch.bfloat16), T(w, torch.bfloat16))
    assert y.dtype == torch.bfloat16 and tuple(y.shape) == (M, N_ & ~1)
    assert_close(y, ref, torch.bfloat16, "any inner size")
    y = ops.linear(T(x, torch.bfloat16), T(w, torch.bfloat16), epilogue=ops.EPI_SOFTCAP, cap=2.0)
    assert y.dtype == torch.float32
    assert_close(y, P.softcap(ref, 2.0), torch.float32, "any inner size, softcap", mult=50)
    y = ops.linear(T(x, torch.bfloat16), T(w, torch.bfloat16), epilogue=ops.EPI_GATED, activation="gelu_tanh")
    h = (N_ & ~1) // 2
    assert tuple(y.shape) == (M, h)
    assert_close(y, P.gelu_tanh(ref[:, :h]) * ref[:, h:], torch.bfloat16, "any inner size, geglu")


def test_products_refuse_mixed_precisions(ops):
    with pytest.raises(TypeError):
        ops.linear(torch.zeros(2, 16, dtype=torch.bfloat16, device=DEV), torch.zeros(4, 16, device=DEV))


@pytest.mark.parametrize("M", [65, 200])
def test_bf16_large_m_library_product_with_epilogues(ops, M):
    rng = np.random.default_rng(M)
    x, w = bf16_round(rng.normal(size=(M, 96))), bf16_round(rng.normal(size=(40, 96)) / 10)
    ref = x @ w.T
    assert_close(ops.linear(T(x, torch.bfloat16), T(w, torch.bfloat16)), ref, torch.bfloat16, "gemm")
    y = ops.linear(T(x, torch.bfloat16), T(w, torch.bfloat16), epilogue=ops.EPI_GATED)
    assert_close(y, P.gelu_tanh(bf16_round(ref[:, :20])) * bf16_round(ref[:, 20:]), torch.bfloat16, "gemm geglu", mult=2)
    y = ops.linear(T(x, torch.bfloat16), T(w, torch.bfloat16), epilogue=ops.EPI_SOFTCAP, cap=3.0)
    assert y.dtype == torch.float32
    assert_close(y, P.softcap(bf16_round(ref), 3.0), torch.float32, "gemm softcap", mult=4000)


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("M,N_,K", [(65, 24, 8), (128, 256, 64), (200, 300, 96), (130, 1000, 200), (300, 2304, 2304),
                                     (2048, 512, 4160), (1, 40, 72), (700, 5000, 520)])
def test_tcgen05_product(ops, M, N_, K, pair):
    """The TMA + tcgen05 kernels alone (one CTA per 128 x 256 tile, and a pair of CTAs per 256 x 256
    tile): tiles that are cut by every edge (M, N, K not multiples of 128 or 256, 256, 64; an odd
    number of 128-row tiles), one slab and many, more tiles than CTAs, plain and gated epilogue."""
    import functools
    ops = type("O", (), {k: getattr(ops, k) for k in dir(ops) if not k.startswith("__")})
    ops.gemm_tcgen05 = staticmethod(functools.partial(ops.gemm_tcgen05, pair=pair))
    rng = np.random.default_rng(M + N_ + K)
    x, w = bf16_round(rng.normal(size=(M, K))), bf16_round(rng.normal(size=(N_, K)) / math.sqrt(K))
    ref = x @ w.T
    y = ops.gemm_tcgen05(T(x, torch.bfloat16), T(w, torch.bfloat16))
    torch.cuda.synchronize()
    ops.check_gemm_status(DEV)
    assert y is not None and y.dtype == torch.bfloat16 and tuple(y.shape) == (M, N_)
    assert_close(y, ref, torch.bfloat16, "tcgen05 product")
    y = ops.gemm_tcgen05(T(x, torch.bfloat16), T(w, torch.bfloat16), epilogue=ops.EPI_GATED, activation="gelu_tanh")
    torch.cuda.synchronize()
    ops.check_gemm_status(DEV)
    h = N_ // 2
    assert tuple(y.shape) == (M, h)
    assert_close(y, P.gelu_tanh(ref[:, :h]) * ref[:, h:], torch.bfloat16, "tcgen05 gated product", mult=1.5)
    y = ops.gemm_tcgen05(T(x, torch.bfloat16), T(w, torch.bfloat16), epilogue=ops.EPI_GATED, activation="silu")
    g = ref[:, :h]
    assert_close(y, g / (1 + np.exp(-g)) * ref[:, h:], torch.bfloat16, "tcgen05 silu-gated product", mult=1.5)
    assert ops.gemm_tcgen05(torch.zeros(70, 12, dtype=torch.bfloat16, device=DEV),
                            torch.zeros(8, 12, dtype=torch.bfloat16, device=DEV)) is None      # refused, not wrong


@pytest.mark.parametrize("M", [2049, 2110])
def test_rows_that_would_open_another_round_of_tiles_go_to_the_small_kernel(ops, M):
    """A product of 2049 or 2110 rows against [2304, 9216] is 81 tiles of 256 x 256 on 74 pairs of SMs: the rows
    beyond 2048 are computed by the kernel for few rows, into the same output."""
    N_, K = 2304, 9216
    assert ops._rows_for_the_small_kernel(M, N_, K, ops.EPI_NONE, torch.device(DEV)) == M - 2048
    assert ops._rows_for_the_small_kernel(2048, N_, K, ops.EPI_NONE, torch.device(DEV)) == 0
    assert ops._rows_for_the_small_kernel(2200, N_, K, ops.EPI_NONE, torch.device(DEV)) == 0      # too many rows to gain
    assert ops._rows_for_the_small_kernel(M, 4096, 2304, ops.EPI_NONE, torch.device(DEV)) == 0    # a cheap round stays
    g = torch.Generator(device=DEV).manual_seed(M)
    x = torch.randn(M, K, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(N_, K, generator=g, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    y = ops.linear(x, w)
    torch.cuda.synchronize()
    ops.check_gemm_status(DEV)
    rows = [0, 1000, 2047, 2048, M - 1]
    ref = N(x[rows].float()) @ N(w.float()).T
    assert_close(y[rows], ref, torch.bfloat16, "rows on either side of the cut")
    whole = ops.gemm_tcgen05(x, w)                               # the same product by the prompt kernel alone
    assert float((y.float() - whole.float()).abs().max()) <= 0.02 * float(whole.float().abs().max())
    assert torch.equal(y[:2048], whole[:2048])


@pytest.mark.parametrize("M,N_,K", [(1, 128, 64), (17, 300, 96), (64, 256, 512), (128, 1000, 200), (33, 2304, 2048),
                                     (64, 130, 4160), (9, 24, 8)])
def test_cluster_split_k_tcgen05_product(ops, M, N_, K):
    """The small-M tcgen05 kernel alone: K split over 1..8 CTAs of a cluster (chosen from the sizes)
    and summed through distributed shared memory; all three epilogues; edges in M, N and K."""
    rng = np.random.default_rng(M * 7 + N_ + K)
    x, w = bf16_round(rng.normal(size=(M, K))), bf16_round(rng.normal(size=(N_, K)) / math.sqrt(K))
    ref = x @ w.T
    y = ops.gemm_skinny_tcgen05(T(x, torch.bfloat16), T(w, torch.bfloat16))
    torch.cuda.synchronize()
    ops.check_gemm_status(DEV)
    assert y is not None and y.dtype == torch.bfloat16 and tuple(y.shape) == (M, N_)
    assert_close(y, ref, torch.bfloat16, "cluster product")
    y = ops.gemm_skinny_tcgen05(T(x, torch.bfloat16), T(w, torch.bfloat16), epilogue=ops.EPI_SOFTCAP, cap=2.0)
    assert y.dtype == torch.float32
    assert_close(y, P.softcap(ref, 2.0), torch.float32, "cluster product with softcap", mult=50)
    y = ops.gemm_skinny_tcgen05(T(x, torch.bfloat16), T(w, torch.bfloat16), epilogue=ops.EPI_GATED)
    h = N_ // 2
    assert_close(y, P.gelu_tanh(ref[:, :h]) * ref[:, h:], torch.bfloat16, "cluster gated product", mult=1.5)
    torch.cuda.synchronize()
    ops.check_gemm_status(DEV)
    assert ops.gemm_skinny_tcgen05(torch.zeros(129, 16, dtype=torch.bfloat16, device=DEV),
                                   torch.zeros(8, 16, dtype=torch.bfloat16, device=DEV)) is None


@pytest.mark.parametrize("M", [1, 3, 8, 9, 70, 130])
@pytest.mark.parametrize("N_,K", [(50, 96), (130, 50), (1000, 200), (7, 3)])
def test_fp32_products_are_true_fp32(ops, M, N_, K):
    rng = np.random.default_rng(M + N_)
    # values with 24 significant bits: a tf32 or bf16 product would be off by 1e-3
    x = rng.normal(size=(M, K)).astype(np.float32)
    w = (rng.normal(size=(N_, K)) / math.sqrt(K)).astype(np.float32)
    ref = x.astype(np.float64) @ w.astype(np.float64).T
    y = ops.linear(T(x, torch.float32), T(w, torch.float32))
    assert_close(y, ref, torch.float32, "fp32 product", mult=2)
    y = ops.linear(T(x, torch.float32), T(w, torch.float32), epilogue=ops.EPI_SOFTCAP, cap=1.5)
    assert_close(y, P.softcap(ref, 1.5), torch.float32, "fp32 softcap", mult=2)
    if N_ % 2 == 0:
        y = ops.linear(T(x, torch.float32), T(w, torch.float32), epilogue=ops.EPI_GATED)
        h = N_ // 2
        assert_close(y, P.gelu_tanh(ref[:, :h]) * ref[:, h:], torch.float32, "fp32 geglu", mult=4)


# ---- rotation and the cache write -----------------------------------------------------

def _pools(pages, nkv, hd, dtype):
    k = torch.zeros((pages, nkv, 64, hd), dtype=dtype, device=DEV)
    return k, torch.zeros_like(k)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd,rot,theta", [(4, 2, 16, 16, 1e4), (6, 1, 24, 24, 1e6), (3, 3, 32, 8, 100.0),
                                                 (2, 2, 16, 0, 1e4)])
def test_rope_and_cache_write(ops, dtype, nq, nkv, hd, rot, theta):
    rng = np.random.default_rng(hd + rot)
    lens = [70, 3]                                # sequence 0 crosses a page boundary
    slots = [2, 0]
    Tn = sum(lens)
    qkv = bf16_round(rng.normal(size=(Tn, (nq + 2 * nkv) * hd)))
    pos = np.concatenate([np.arange(n) for n in lens]).astype(np.int32)
    slot = np.concatenate([np.full(n, s) for n, s in zip(lens, slots)]).astype(np.int32)
    table = np.zeros((3, 4), dtype=np.int32)
    table[2, :2] = [5, 3]
    table[0, :1] = [1]
    slot_len = np.array([3, 0, 70], dtype=np.int32)
    k_pool, v_pool = _pools(7, nkv, hd, dtype)
    inv = torch.exp(-math.log(theta) * 2.0 * torch.arange(rot // 2, dtype=torch.float64) / max(rot, 1)).float().to(DEV)
    t = T(qkv, dtype)
    ops.rope_cache_write(t, nq, nkv, hd, rot, inv, T(pos, torch.int32), T(slot, torch.int32), k_pool, v_pool,
                         T(table, torch.int32), 64, 0, T(slot_len, torch.int32), True)
    q = qkv[:, :nq * hd].reshape(Tn, nq, hd)
    k = qkv[:, nq * hd:(nq + nkv) * hd].reshape(Tn, nkv, hd)
    v = qkv[:, (nq + nkv) * hd:].reshape(Tn, nkv, hd)

    def rot_ref(x):
        if rot == 0:
            return x
        return np.concatenate([P.rope(x[..., :rot], pos, theta), x[..., rot:]], axis=-1)
    got = N(t)
    assert_close(got[:, :nq * hd], rot_ref(q).reshape(Tn, -1), dtype, "q", mult=2)
    assert_close(got[:, nq * hd:(nq + nkv) * hd], rot_ref(k).reshape(Tn, -1), dtype, "k", mult=2)
    assert np.array_equal(got[:, (nq + nkv) * hd:], v.reshape(Tn, -1))
    kr = rot_ref(k)
    kp, vp = N(k_pool), N(v_pool)
    for r in range(Tn):
        page = table[slot[r], pos[r] // 64]
        assert_close(kp[page, :, pos[r] % 64, :], kr[r], dtype, "cached k", mult=2)
        assert np.array_equal(vp[page, :, pos[r] % 64, :], v[r])
    assert float(np.abs(kp[0]).sum()) == 0.0 and float(np.abs(kp[2]).sum()) == 0.0   # nobody's pages untouched
    assert float(np.abs(kp[5, :, 6:, :]).sum()) != 0.0 and float(np.abs(kp[3, :, 6:, :]).sum()) == 0.0


@pytest.mark.parametrize("M,K,nq,nkv,hd,ring", [(5, 200, 3, 1, 48, 0), (8, 264, 4, 2, 16, 128), (19, 136, 2, 2, 80, 0),
                                                (1, 2056, 2, 1, 32, 64)])
def test_qkv_product_with_rotate_and_append_epilogue(ops, M, K, nq, nkv, hd, ring):
    """The fused product against the product, rotation and append as separate kernels (same
    sums, so at most an ulp apart) and against the plain rotation of the plain product."""
    rng = np.random.default_rng(M * K + hd)
    Nw = (nq + 2 * nkv) * hd
    x = bf16_round(rng.normal(size=(M, K)))
    w = bf16_round(rng.normal(size=(Nw, K)) / math.sqrt(K))
    theta = 1e4
    pos = (rng.integers(0, 190, size=M)).astype(np.int32)
    slot = rng.permutation(M + 2)[:M].astype(np.int32)
    if M > 2:
        slot[1] = -1                                                      # a padding row writes nothing
    pages = 3
    table = np.zeros((M + 2, pages), dtype=np.int32)
    table[:, :] = 1 + rng.permutation((M + 2) * pages).reshape(M + 2, pages)
    slot_len = np.zeros(M + 2, dtype=np.int32)
    for r in range(M):
        if slot[r] >= 0:
            slot_len[slot[r]] = pos[r] + 1
    inv = torch.exp(-math.log(theta) * 2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd).float().to(DEV)
    args = (T(pos, torch.int32), T(slot, torch.int32))
    tab, sl = T(table, torch.int32), T(slot_len, torch.int32)
    k1, v1 = _pools((M + 2) * pages + 1, nkv, hd, torch.bfloat16)
    k2, v2 = _pools((M + 2) * pages + 1, nkv, hd, torch.bfloat16)
    xt, wt = T(x, torch.bfloat16), T(w, torch.bfloat16)
    fused = ops.qkv_rope_cache(xt, wt, nq, nkv, hd, inv, *args, k1, v1, tab, 64, ring, sl, True)
    sep = ops.linear(xt, wt)
    plain_qkv = N(sep).copy()
    ops.rope_cache_write(sep, nq, nkv, hd, hd, inv, *args, k2, v2, tab, 64, ring, sl, True)
    ulp = 2.0 ** -7
    for name, a, b in (("qkv", fused, sep), ("k pool", k1, k2), ("v pool", v1, v2)):
        a, b = N(a), N(b)
        assert np.all(np.abs(a - b) <= ulp * np.maximum(np.abs(b), 2.0 ** -20)), name
    assert np.array_equal(N(v1), N(v2))
    q = plain_qkv[:, :nq * hd].reshape(M, nq, hd)
    k = plain_qkv[:, nq * hd:(nq + nkv) * hd].reshape(M, nkv, hd)
    got = N(fused)
    assert_close(got[:, :nq * hd], P.rope(q, pos, theta).reshape(M, -1), torch.bfloat16, "q", mult=2)
    kr = P.rope(k, pos, theta)
    kp = N(k1)
    for r in range(M):
        if slot[r] < 0:
            continue
        c = pos[r] % ring if ring else pos[r]
        assert_close(kp[table[slot[r], c // 64], :, c % 64, :], kr[r], torch.bfloat16, "cached k", mult=2)
    assert float(np.abs(kp[0]).sum()) == 0.0
    written = sum(1 for r in range(M) if slot[r] >= 0)
    assert int((np.abs(N(v1)).sum(axis=(1, 3)) != 0).sum()) == written     # one cell per live row, no more
    # without the append nothing is written
    k3, v3 = _pools(4, nkv, hd, torch.bfloat16)
    again = ops.qkv_rope_cache(xt, wt, nq, nkv, hd, inv, *args, None, None, None, 64, ring, None, False)
    assert np.array_equal(N(again), N(fused))


def test_cache_write_ring_and_padding(ops):
    """A prompt longer than the ring leaves its last `ring` positions, each in its place; a
    row with a negative slot writes nothing."""
    nq, nkv, hd = 2, 1, 16
    n = 150
    qkv = np.zeros((n + 1, (nq + 2 * nkv) * hd), dtype=np.float32)
    qkv[:, (nq + nkv) * hd] = np.arange(n + 1) + 1.0                     # v[.., 0] = position + 1
    pos = np.concatenate([np.arange(n), [7]]).astype(np.int32)
    slot = np.concatenate([np.full(n, 1), [-1]]).astype(np.int32)
    table = np.array([[0, 0], [4, 2]], dtype=np.int32)
    k_pool, v_pool = _pools(6, nkv, hd, torch.float32)
    inv = torch.zeros(0, device=DEV)
    ops.rope_cache_write(T(qkv, torch.float32), nq, nkv, hd, 0, inv, T(pos, torch.int32), T(slot, torch.int32),
                         k_pool, v_pool, T(table, torch.int32), 64, 128, T(np.array([0, n], np.int32), torch.int32), True)
    vp = N(v_pool)[:, 0, :, 0]
    for p in range(n - 128, n):
        r = p % 128
        assert vp[table[1, r // 64], r % 64] == p + 1
    assert float(np.abs(vp[0]).sum()) == 0.0                               # the padding row wrote nothing


# ---- attention --------------------------------------------------------------------------

GEOMS = [(4, 2, 16), (6, 1, 24), (8, 4, 64), (3, 3, 40), (8, 4, 256), (8, 1, 128), (5, 5, 8)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd", GEOMS)
@pytest.mark.parametrize("window,cap", [(None, 50.0), (5, None), (64, 30.0)])
def test_attention_prefill(ops, dtype, nq, nkv, hd, window, cap):
    rng = np.random.default_rng(nq * hd + (window or 0))
    lens = [1, 37, 70]
    Tn = sum(lens)
    qkv = bf16_round(rng.normal(size=(Tn, (nq + 2 * nkv) * hd)))
    pos = np.concatenate([np.arange(n) for n in lens]).astype(np.int32)
    row0 = np.concatenate([np.full(n, s) for n, s in zip(lens, np.cumsum([0] + lens[:-1]))]).astype(np.int32)
    scale = 1.0 / math.sqrt(hd + 3)
    out = ops.attn_prefill(T(qkv, dtype), nq, nkv, hd, T(pos, torch.int32), T(row0, torch.int32), scale, cap, window)
    ref = np.zeros((Tn, nq * hd))
    r = 0
    for n in lens:
        blk = qkv[r:r + n]
        q = blk[:, :nq * hd].reshape(n, nq, hd)
        k = blk[:, nq * hd:(nq + nkv) * hd].reshape(n, nkv, hd)
        v = blk[:, (nq + nkv) * hd:].reshape(n, nkv, hd)
        ref[r:r + n] = P.attention(q, k, v, scale, cap, window).reshape(n, -1)
        r += n
    assert_close(out, ref, dtype, "prefill attention", mult=4)
    # with the per-sequence arrays, bfloat16 at head sizes 64/128/256 takes the tensor-core kernel
    starts = np.cumsum([0] + lens[:-1]).astype(np.int32)
    out2 = ops.attn_prefill(T(qkv, dtype), nq, nkv, hd, T(pos, torch.int32), T(row0, torch.int32), scale, cap, window,
                            T(starts, torch.int32), T(np.array(lens, np.int32), torch.int32), max(lens))
    assert_close(out2, ref, dtype, "prefill attention with sequence arrays", mult=4)


@pytest.mark.parametrize("nq,nkv,hd", [(8, 4, 256), (4, 1, 128), (6, 2, 64)])
@pytest.mark.parametrize("window,cap", [(None, 50.0), (100, None), (64, 30.0)])
@pytest.mark.parametrize("kernel", ["tcgen05", "mma"])
def test_attention_prefill_tensor_core_kernel_long_unequal(ops, monkeypatch, kernel, nq, nkv, hd, window, cap):
    """Sequences that span several 64-row tiles, of unequal lengths, against the plain attention; both
    tensor-core kernels (tcgen05, and the mma.sync one that stands behind it)."""
    monkeypatch.setattr(ops, "ATTN_TCGEN05", kernel == "tcgen05")
    rng = np.random.default_rng(hd + (window or 0))
    lens = [200, 1, 65, 130, 64]
    Tn = sum(lens)
    qkv = bf16_round(rng.normal(size=(Tn, (nq + 2 * nkv) * hd)))
    pos = np.concatenate([np.arange(n) for n in lens]).astype(np.int32)
    starts = np.cumsum([0] + lens[:-1]).astype(np.int32)
    row0 = np.concatenate([np.full(n, s) for n, s in zip(lens, starts)]).astype(np.int32)
    scale = 1.0 / math.sqrt(hd)
    out = ops.attn_prefill(T(qkv, torch.bfloat16), nq, nkv, hd, T(pos, torch.int32), T(row0, torch.int32), scale, cap,
                           window, T(starts, torch.int32), T(np.array(lens, np.int32), torch.int32), max(lens))
    r = 0
    for n in lens:
        blk = qkv[r:r + n]
        q = blk[:, :nq * hd].reshape(n, nq, hd)
        k = blk[:, nq * hd:(nq + nkv) * hd].reshape(n, nkv, hd)
        v = blk[:, (nq + nkv) * hd:].reshape(n, nkv, hd)
        ref = P.attention(q, k, v, scale, cap, window).reshape(n, -1)
        assert_close(out[r:r + n], ref, torch.bfloat16, f"sequence of {n}", mult=4)
        r += n


@pytest.mark.parametrize("hd", [64, 128, 256])
def test_attention_prefill_tcgen05_with_more_ctas_than_sms(ops, hd):
    """Enough heads, sequences and query tiles that the kernel runs one CTA per query tile (no pairs),
    several key tiles each, with a window that begins inside a tile."""
    nq, nkv, window, cap = 20, 4, 150, 40.0
    rng = np.random.default_rng(hd)
    lens = [300, 150, 260, 129]
    Tn = sum(lens)
    qkv = bf16_round(rng.normal(size=(Tn, (nq + 2 * nkv) * hd)))
    pos = np.concatenate([np.arange(n) for n in lens]).astype(np.int32)
    starts = np.cumsum([0] + lens[:-1]).astype(np.int32)
    row0 = np.concatenate([np.full(n, s) for n, s in zip(lens, starts)]).astype(np.int32)
    scale = 1.0 / math.sqrt(hd)
    out = ops.attn_prefill(T(qkv, torch.bfloat16), nq, nkv, hd, T(pos, torch.int32), T(row0, torch.int32), scale, cap,
                           window, T(starts, torch.int32), T(np.array(lens, np.int32), torch.int32), max(lens))
    r = 0
    for n in lens:
        blk = qkv[r:r + n]
        q = blk[:, :nq * hd].reshape(n, nq, hd)
        k = blk[:, nq * hd:(nq + nkv) * hd].reshape(n, nkv, hd)
        v = blk[:, (nq + nkv) * hd:].reshape(n, nkv, hd)
        ref = P.attention(q, k, v, scale, cap, window).reshape(n, -1)
        assert_close(out[r:r + n], ref, torch.bfloat16, f"sequence of {n}", mult=4)
        r += n


@pytest.mark.parametrize("hd", [64, 128, 256])
@pytest.mark.parametrize("window,cap", [(None, 50.0), (700, None)])
def test_attention_prefill_tcgen05_pairs_share_long_key_walks(ops, hd, window, cap):
    """Few heads and a sequence of 13 key tiles: the kernel runs pairs of CTAs that take alternate key
    tiles of a query tile and merge their halves; beside it a short sequence whose second CTA has nothing."""
    nq, nkv = 2, 1
    rng = np.random.default_rng(hd + 1)
    lens = [800, 130]
    Tn = sum(lens)
    qkv = bf16_round(rng.normal(size=(Tn, (nq + 2 * nkv) * hd)))
    pos = np.concatenate([np.arange(n) for n in lens]).astype(np.int32)
    starts = np.cumsum([0] + lens[:-1]).astype(np.int32)
    row0 = np.concatenate([np.full(n, s) for n, s in zip(lens, starts)]).astype(np.int32)
    scale = 1.0 / math.sqrt(hd)
    out = ops.attn_prefill(T(qkv, torch.bfloat16), nq, nkv, hd, T(pos, torch.int32), T(row0, torch.int32), scale, cap,
                           window, T(starts, torch.int32), T(np.array(lens, np.int32), torch.int32), max(lens))
    r = 0
    for n in lens:
        blk = qkv[r:r + n]
        q = blk[:, :nq * hd].reshape(n, nq, hd)
        k = blk[:, nq * hd:(nq + nkv) * hd].reshape(n, nkv, hd)
        v = blk[:, (nq + nkv) * hd:].reshape(n, nkv, hd)
        ref = P.attention(q, k, v, scale, cap, window).reshape(n, -1)
        assert_close(out[r:r + n], ref, torch.bfloat16, f"sequence of {n}", mult=4)
        r += n


def test_window_edge_in_the_tensor_core_prefill_kernel(ops):
    nq, nkv, hd, n, W = 2, 1, 64, 300, 100
    k = np.zeros((n, nkv, hd))
    v = np.zeros((n, nkv, hd))
    v[:, 0, 0] = np.arange(n) // 16
    v[:, 0, 1] = np.arange(n) % 16
    k[n - W, 0, 0] = 6.0
    k[n - W - 1, 0, 0] = 12.0
    q = np.zeros((n, nq, hd))
    q[:, :, 0] = 6.0
    qkv = np.concatenate([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], axis=1)
    i32 = lambda a: T(np.asarray(a, np.int32), torch.int32)  # noqa: E731
    out = ops.attn_prefill(T(qkv, torch.bfloat16), nq, nkv, hd, i32(np.arange(n)), i32(np.zeros(n)), 1.0, None, W,
                           i32([0]), i32([n]), n)
    o = N(out).reshape(n, nq, hd)
    found = np.rint(o[:, :, 0]) * 16 + np.rint(o[:, :, 1])
    assert np.all(found[-1] == n - W), found[-1]               # the key just inside the window
    assert np.all(found[-2] == n - W - 1), found[-2]           # one row earlier the outside key is still inside


def _fill_cache(k, v, tables, dtype, pages, ring=0):
    """k, v: per sequence [n, nkv, hd]; returns pools with every sequence in its pages."""
    nkv, hd = k[0].shape[1:]
    k_pool, v_pool = _pools(pages, nkv, hd, dtype)
    for s, (ks, vs) in enumerate(zip(k, v)):
        n = ks.shape[0]
        for p in range(max(0, n - ring) if ring else 0, n):
            r = p % ring if ring else p
            page = tables[s][r // 64]
            k_pool[page, :, r % 64, :] = T(ks[p], dtype)
            v_pool[page, :, r % 64, :] = T(vs[p], dtype)
    return k_pool, v_pool


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,hd", GEOMS)
@pytest.mark.parametrize("window,cap,splits", [(None, 50.0, 1), (None, None, 5), (40, 30.0, 3), (128, None, 4),
                                               (None, 30.0, 8), (128, 50.0, 9), (None, None, 20)])
def test_attention_decode(ops, dtype, nq, nkv, hd, window, cap, splits):
    rng = np.random.default_rng(nq + hd + splits)
    lens = [200, 1, 65, 130]
    tables = [[7, 2, 9, 11], [4, 0, 0, 0], [1, 6, 0, 0], [3, 8, 10, 0]]      # scattered, out of order
    slots = [3, 0, 2, 1]                                                       # rows are not in slot order
    ring = 128 if window == 128 else 0
    if ring:
        tables = [t[:2] + [0, 0] for t in tables]
    k = [bf16_round(rng.normal(size=(n, nkv, hd))) for n in lens]
    v = [bf16_round(rng.normal(size=(n, nkv, hd))) for n in lens]
    q = bf16_round(rng.normal(size=(len(lens) + 1, nq, hd)))
    k_pool, v_pool = _fill_cache(k, v, tables, dtype, 12, ring)
    table = np.zeros((4, 4), dtype=np.int32)
    slot_len = np.zeros(4, dtype=np.int32)
    for s, tb, n in zip(slots, tables, lens):
        table[s] = tb
        slot_len[s] = n
    qkv = np.zeros((len(lens) + 1, (nq + 2 * nkv) * hd))
    qkv[:, :nq * hd] = q.reshape(len(lens) + 1, -1)
    scale = 1.0 / math.sqrt(hd)
    B = len(lens) + 1
    part_o = torch.empty(B * nq * splits * hd, device=DEV)
    part_ml = torch.empty(B * nq * splits * 2, device=DEV)
    out = ops.attn_decode(T(qkv, dtype), nq, nkv, hd, k_pool, v_pool, T(table, torch.int32), 64, ring,
                          T(np.array(slots + [-1], np.int32), torch.int32), T(slot_len, torch.int32), scale, cap,
                          window, splits, part_o, part_ml)
    for b, n in enumerate(lens):
        qq = np.zeros((n, nq, hd))
        qq[-1] = q[b]
        ref = P.attention(qq, k[b], v[b], scale, cap, window)[-1].reshape(-1)
        assert_close(out[b], ref, dtype, f"decode attention row {b}", mult=4)
    assert float(out[-1].abs().sum()) == 0.0                                  # the padding row attends to nothing


@pytest.mark.parametrize("splits", [2, 3, 4])
def test_attention_decode_with_more_clusters_than_the_device_holds(ops, splits):
    """30 sequences x 4 kv heads at head size 256: 120 clusters of 3 CTAs do not fit the device at once, so the
    key ranges go through the scratch and the merge kernel; with 2 and 4 ranges they merge inside the clusters.
    The same numbers either way."""
    rng = np.random.default_rng(splits)
    nq, nkv, hd, B = 8, 4, 256, 30
    lens = [int(n) for n in rng.integers(1, 190, B)]
    k = [bf16_round(rng.normal(size=(n, nkv, hd))) for n in lens]
    v = [bf16_round(rng.normal(size=(n, nkv, hd))) for n in lens]
    q = bf16_round(rng.normal(size=(B, nq, hd)))
    tables = [[3 * b + 2, 3 * b, 3 * b + 1] for b in range(B)]
    k_pool, v_pool = _fill_cache(k, v, tables, torch.bfloat16, 3 * B, 0)
    qkv = np.zeros((B, (nq + 2 * nkv) * hd))
    qkv[:, :nq * hd] = q.reshape(B, -1)
    part_o = torch.empty(B * nq * splits * hd, device=DEV)
    part_ml = torch.empty(B * nq * splits * 2, device=DEV)
    out = ops.attn_decode(T(qkv, torch.bfloat16), nq, nkv, hd, k_pool, v_pool, T(np.array(tables, np.int32), torch.int32),
                          64, 0, T(np.arange(B, dtype=np.int32), torch.int32), T(np.array(lens, np.int32), torch.int32),
                          1.0 / 16, 50.0, None, splits, part_o, part_ml)
    for b, n in enumerate(lens):
        qq = np.zeros((n, nq, hd))
        qq[-1] = q[b]
        ref = P.attention(qq, k[b], v[b], 1.0 / 16, 50.0, None)[-1].reshape(-1)
        assert_close(out[b], ref, torch.bfloat16, f"decode attention row {b}", mult=4)


@pytest.mark.parametrize("dtype,nq,nkv,hd,tensor_cores", [
    (torch.float32, 4, 2, 16, False), (torch.bfloat16, 6, 1, 24, False), (torch.bfloat16, 8, 4, 64, True),
    (torch.bfloat16, 4, 2, 128, True), (torch.bfloat16, 8, 4, 256, True), (torch.bfloat16, 8, 4, 256, False)])
@pytest.mark.parametrize("window,cap", [(None, 50.0), (128, None), (100, 30.0)])
def test_attention_of_steps_that_continue_sequences(ops, dtype, nq, nkv, hd, tensor_cores, window, cap):
    """attn_extend: cached keys from the pages (a ring of 128 positions under a window, wrapped for the long
    sequence), the step's own rows from the packed projections; one sequence starts in this step, one brings a
    single row.  With the whole-sequence layout the bfloat16 rows of head size 64 / 128 / 256 go through the
    tensor-core prompt kernel, which leaves out the query tiles before the new rows."""
    from quicknn_b200.engine.batch import WholeSequences
    rng = np.random.default_rng(nq + hd + (window or 0))
    seqs = [(300, 40), (0, 70), (130, 1), (1000, 200)]                      # (cached, new)
    ring = 128 if window else 0
    per = 2 if ring else 19
    tables = (1 + rng.permutation(len(seqs) * per)).reshape(len(seqs), per).tolist()
    k = [bf16_round(rng.normal(size=(c + n, nkv, hd))) for c, n in seqs]
    v = [bf16_round(rng.normal(size=(c + n, nkv, hd))) for c, n in seqs]
    q = [bf16_round(rng.normal(size=(c + n, nq, hd))) for c, n in seqs]
    k_pool, v_pool = _fill_cache([kk[:c] for kk, (c, n) in zip(k, seqs)], [vv[:c] for vv, (c, n) in zip(v, seqs)],
                                 tables, dtype, 1 + len(seqs) * per, ring)
    packed = np.concatenate([np.concatenate([qq[c:].reshape(n, -1), kk[c:].reshape(n, -1), vv[c:].reshape(n, -1)], axis=1)
                             for qq, kk, vv, (c, n) in zip(q, k, v, seqs)])
    new = np.array([n for c, n in seqs], np.int32)
    start = np.array([c for c, n in seqs], np.int32)
    new_row0 = (np.cumsum(new) - new).astype(np.int32)
    tok_pos = np.concatenate([np.arange(c, c + n) for c, n in seqs]).astype(np.int32)
    tok_row0 = np.repeat(new_row0, new)
    slots = np.arange(len(seqs), dtype=np.int32)[::-1].copy()               # rows are not in slot order
    table = np.zeros((len(seqs), per), np.int32)
    for s_, tb in zip(slots, tables):
        table[s_] = tb
    tok_slot = np.repeat(slots, new)
    i32 = lambda a: T(np.asarray(a, np.int32), torch.int32)  # noqa: E731
    whole = None
    if tensor_cores:
        length = start + new
        row0 = (np.cumsum(length) - length).astype(np.int32)
        tok_row = (np.repeat(row0, new) + tok_pos).astype(np.int32)
        whole = WholeSequences(i32(slots), i32(start), i32(new_row0), i32(new), i32(row0), i32(length), i32(tok_row),
                               total=int(length.sum()), longest=int(length.max()), most_new=int(new.max()))
    scale = 1.0 / math.sqrt(hd)
    out = ops.attn_extend(T(packed, dtype), nq, nkv, hd, k_pool, v_pool, i32(table), 64, ring, i32(tok_pos), i32(tok_row0),
                          i32(tok_slot), scale, cap, window, whole=whole)
    ops.raise_on_status(DEV)
    assert tuple(out.shape) == (int(new.sum()), nq * hd)
    for b, (c, n) in enumerate(seqs):
        ref = P.attention(q[b], k[b], v[b], scale, cap, window)[c:].reshape(n, -1)
        assert_close(out[new_row0[b]:new_row0[b] + n], ref, dtype, f"sequence {b}", mult=4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decode_attention_finds_one_far_key_among_hundreds(ops, dtype):
    """Random keys would hide a skipped key: here one key per test scores far above the rest and
    carries a value of its own, at every position of a 700-key sequence in turn for the places
    where faults live (first key, page and split edges, last key)."""
    nq, nkv, hd, n, splits = 4, 2, 32, 700, 6
    rng = np.random.default_rng(0)
    base_k = bf16_round(rng.normal(size=(n, nkv, hd)) * 0.05)
    v = np.zeros((n, nkv, hd))
    v[:, :, 0] = (np.arange(n) // 16)[:, None]          # the position in two digits that bfloat16 holds exactly
    v[:, :, 1] = (np.arange(n) % 16)[:, None]
    q = np.zeros((1, nq, hd))
    q[0, :, 3] = 8.0
    tables = [[5, 1, 9, 2, 11, 3, 7, 4, 10, 6, 8]]
    table = np.array(tables, dtype=np.int32)
    part_o = torch.empty(nq * splits * hd, device=DEV)
    part_ml = torch.empty(nq * splits * 2, device=DEV)
    qkv = np.zeros((1, (nq + 2 * nkv) * hd))
    qkv[:, :nq * hd] = q.reshape(1, -1)
    per = -(-n // splits)
    places = sorted({0, 1, 63, 64, 65, 127, 128, per - 1, per, per + 1, 2 * per, 5 * per - 1, 5 * per, n - 2, n - 1})
    for far in places:
        k = base_k.copy()
        k[far, :, 3] = 8.0                                    # score 64 * scale against ~0 elsewhere
        k_pool, v_pool = _fill_cache([k], [v], tables, dtype, 12)
        out = ops.attn_decode(T(qkv, dtype), nq, nkv, hd, k_pool, v_pool, T(table, torch.int32), 64, 0,
                              T(np.array([0], np.int32), torch.int32), T(np.array([n], np.int32), torch.int32),
                              1.0, None, None, splits, part_o, part_ml)
        got = N(out).reshape(nq, hd)
        got = np.rint(got[:, 0]) * 16 + np.rint(got[:, 1])
        assert np.all(got == far), f"key {far} was not found: {got}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_window_edge_in_both_attention_kernels(ops, dtype):
    """The key just inside the window must be seen, the one just outside must not, although the
    outside one scores highest."""
    nq, nkv, hd, n, W = 2, 1, 16, 300, 100
    k = np.zeros((n, nkv, hd))
    v = np.zeros((n, nkv, hd))
    v[:, 0, 0] = np.arange(n)
    k[n - W, 0, 0] = 6.0          # first key inside the window of the last query
    k[n - W - 1, 0, 0] = 12.0     # just outside: would win if it were seen
    q = np.zeros((n, nq, hd))
    q[:, :, 0] = 6.0
    qkv = np.concatenate([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], axis=1)
    pos = np.arange(n, dtype=np.int32)
    out = ops.attn_prefill(T(qkv, dtype), nq, nkv, hd, T(pos, torch.int32), T(np.zeros(n, np.int32), torch.int32),
                           1.0, None, W)
    last = N(out)[-1].reshape(nq, hd)[:, 0]
    assert np.all(np.abs(last - (n - W)) < 0.5), last
    before = N(out)[-2].reshape(nq, hd)[:, 0]                 # the query before still sees the outside key
    assert np.all(np.abs(before - (n - W - 1)) < 0.5), before
    for ring in (0, 128):
        tables = [[3, 1, 4, 2, 5]] if not ring else [[3, 1, 0, 0, 0]]
        k_pool, v_pool = _fill_cache([k], [v], tables, dtype, 6, ring)
        part_o = torch.empty(nq * 4 * hd, device=DEV)
        part_ml = torch.empty(nq * 4 * 2, device=DEV)
        o = ops.attn_decode(T(qkv[-1:], dtype), nq, nkv, hd, k_pool, v_pool, T(np.array(tables, np.int32), torch.int32),
                            64, ring, T(np.array([0], np.int32), torch.int32), T(np.array([n], np.int32), torch.int32),
                            1.0, None, W, 4, part_o, part_ml)
        got = N(o).reshape(nq, hd)[:, 0]
        assert np.all(np.abs(got - (n - W)) < 0.5), (ring, got)


def test_attention_refuses_sizes_it_cannot_take(ops):
    from quicknn_b200.kernels.lib import KernelError
    qkv = torch.zeros((2, (2 + 2) * 12), dtype=torch.bfloat16, device=DEV)     # 12 * 2 bytes is no 16-byte vector
    z = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError):
        ops.attn_prefill(qkv, 2, 1, 12, z, z, 1.0, None, None)


# ---- sampling ---------------------------------------------------------------------------

@pytest.mark.parametrize("V", [100, 1000, 5000, 256000])
def test_sampling_follows_the_plain_sampler(ops, V):
    rng = np.random.default_rng(V)
    R = 6
    logits = rng.normal(size=(R, V)).astype(np.float32) * 3
    logits[0, 17] = logits[0, 5] = logits[0].max() + 1.0            # a tie: the lowest id wins
    seen = (rng.random(size=(R, V)) < 0.3).astype(np.uint8)
    lg = T(logits, torch.float32)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    for temp, k, p, pen in [(0.0, 20, 0.95, 1.0), (0.8, 20, 0.95, 1.0), (1.5, 64, 0.5, 1.3), (0.7, 3, 1.0, 0.8),
                            (1.0, 1, 1.0, 1.0)]:
        states = np.array([P.seed_state(42 + i) for i in range(R)], dtype=np.uint32)
        rng_state = T(states.view(np.int32), torch.int32)
        seen_t = T(seen, torch.uint8)
        scratch = torch.empty(ops.sample_scratch_bytes(R, V, k), dtype=torch.uint8, device=DEV)
        out = torch.zeros(R, dtype=torch.int32, device=DEV)
        seen_rows = torch.arange(R, dtype=torch.int32, device=DEV)
        st = states.copy()
        for draw in range(4):
            ops.sample(lg, k, temp, p, pen, rng_state, seen_t, seen_rows, scratch, out, flag)
            got = out.cpu().numpy()
            for r in range(R):
                u = 0.0
                if temp > 0 and min(k, V) > 1:
                    s, u = P.xorshift32(int(st[r]))
                    st[r] = s
                ref = P.sample(logits[r], temp, k, p, pen, seen[r] if pen != 1.0 else None, u)
                assert got[r] == ref, (temp, k, p, pen, draw, r, got[r], ref)
            if pen != 1.0:
                assert all(int(seen_t[r, got[r]]) == 1 for r in range(R))    # the chosen id is marked seen
                seen[np.arange(R), got] = 1
        if temp == 0.0:
            assert got[0] == 5
    assert int(flag) == 0


@pytest.mark.parametrize("V", [3000, 40000, 256000])
def test_sampling_when_many_values_crowd_the_top(ops, V):
    """The k best are looked for among the values at or above the k-th largest tile maximum, kept in a list of 4096;
    rows that overflow it take k rounds over everything instead: a row of equal logits (the lowest ids win), a row
    whose best thirty tiles are all outliers, a row of two values in halves; beside an ordinary row and one with
    fewer finite values than k."""
    rng = np.random.default_rng(V)
    R = 5
    logits = rng.normal(size=(R, V)).astype(np.float32)
    logits[0, :] = 1.25
    width = min(V, 31000)
    logits[1, V - width:] = 50.0 + rng.normal(size=width).astype(np.float32)
    logits[2, :] = np.where(np.arange(V) % 2 == 0, 3.0, -3.0)
    logits[4, :] = -np.inf
    logits[4, [7, V - 1, V // 2]] = [0.5, 0.25, 0.5]
    lg = T(logits, torch.float32)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    for temp, k, p in [(0.9, 20, 0.95), (1.3, 64, 1.0), (0.5, 2, 0.9)]:
        states = np.array([P.seed_state(7 + i) for i in range(R)], dtype=np.uint32)
        rng_state = T(states.view(np.int32), torch.int32)
        scratch = torch.empty(ops.sample_scratch_bytes(R, V, k), dtype=torch.uint8, device=DEV)
        out = torch.zeros(R, dtype=torch.int32, device=DEV)
        st = states.copy()
        for draw in range(6):
            ops.sample(lg, k, temp, p, 1.0, rng_state, None, None, scratch, out, flag)
            got = out.cpu().numpy()
            for r in range(R):
                s_, u = P.xorshift32(int(st[r]))
                st[r] = s_
                row = np.where(np.isfinite(logits[r]), logits[r], -3.0e38)        # non-finite values lose
                ref = P.sample(row, temp, min(k, 3) if r == 4 else k, p, 1.0, None, u)
                assert got[r] == ref, (temp, k, p, draw, r, got[r], ref)
    assert int(flag) == 1                                       # the infinities were seen


@pytest.mark.parametrize("M,V,K", [(1, 256000, 2304), (8, 256000, 2304), (5, 1000, 96), (20, 1000, 200), (30, 3001, 64),
                                   (12, 256000, 2304), (40, 3001, 64), (100, 30000, 256), (64, 20000, 128)])
def test_head_with_the_arg_max_in_its_epilogue(ops, M, V, K):
    """The greedy head: only the best (value, id) of every group of columns leaves the product (16 columns in
    the mma.sync kernel, 128 in the tcgen05 kernel that takes 9 rows and more against a big matrix).  The chosen
    ids are those of the largest logit as the ordinary head product writes it, the lowest id on ties; a
    vocabulary that is no multiple of the group; more than 64 rows (two rounds); NaN sets the error word."""
    g = torch.Generator(device=DEV)
    g.manual_seed(M * 1000 + K)
    x = torch.randn((M, K), generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn((V, K), generator=g, device=DEV) * 0.05).to(torch.bfloat16)
    big = (x[0].float() / x[0].float().norm()).to(torch.bfloat16)
    w[7] = big                                        # two columns with the same logit in every row,
    w[V - 3] = big                                    # row 0's largest: id 7 must win
    logits = ops.linear(x, w, epilogue=ops.EPI_SOFTCAP, cap=30.0).cpu().numpy()
    want = [P.argmax_lowest(r) for r in logits]
    assert want[0] == 7
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    cand = torch.full((M * ops.head_candidates(V) * 2,), float("nan"), device=DEV)
    assert ops.head_argmax_fusable(x, w)
    ncand = ops.head_argmax(x, w, 30.0, cand, flag)
    if ncand is None:                                 # more than 64 rows with the tcgen05 decode product switched off:
        assert M > 64 and not ops._takes_skinny_tcgen05(M, V, K)     # the caller forms the logits, as documented
        return
    group = {(V + 15) // 16: 16, (V + 127) // 128: 128}[ncand]
    c = cand[:M * ncand * 2].cpu().numpy().reshape(M, ncand, 2)
    ids = c[:, :, 1].copy().view(np.uint32)
    for m in range(M):                                # every candidate is the best of its group of columns
        for blk in (0, ncand // 2, ncand - 1):
            cols = logits[m, blk * group:(blk + 1) * group]
            assert c[m, blk, 0] == cols.max() and ids[m, blk] == blk * group + int(np.argmax(cols)), (m, blk)
    out = torch.zeros(M, dtype=torch.int32, device=DEV)
    rng_state = torch.ones(M, dtype=torch.int32, device=DEV)
    ops.sample_candidates(cand, M, ncand, V, 1, 0.0, 1.0, rng_state, None, None, out, flag)
    assert out.cpu().tolist() == want and int(flag) == 0
    x[M - 1, 3] = float("nan")
    ops.head_argmax(x, w, 30.0, cand, flag)
    assert int(flag) == 1
    ops.raise_on_status(DEV)


def test_sampling_flags_non_finite_logits_and_marks_prompts(ops):
    V = 300
    lg = torch.zeros((2, V), device=DEV)
    lg[1, 7] = float("nan")
    lg[0, 9] = 1.0
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.zeros(2, dtype=torch.int32, device=DEV)
    scratch = torch.empty(ops.sample_scratch_bytes(2, V, 1), dtype=torch.uint8, device=DEV)
    ops.sample(lg, 1, 0.0, 1.0, 1.0, torch.ones(2, dtype=torch.int32, device=DEV), None, None, scratch, out, flag)
    assert int(flag) == 1 and int(out[0]) == 9
    seen = torch.zeros((3, V), dtype=torch.uint8, device=DEV)
    ops.mark_seen(T(np.array([5, 6, 299, 5], np.int32), torch.int32), T(np.array([0, 0, 2, -1], np.int32), torch.int32), seen)
    assert seen.sum().item() == 3 and seen[0, 5] == 1 and seen[2, 299] == 1 and seen[1].sum() == 0

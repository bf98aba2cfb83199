// Matrix products of a few rows (decode batches of 17..128 sequences) against a big weight matrix:
//     C[M, N] = X[M, K] * W[N, K]^T,  M <= 128,  bfloat16 in, float32 accumulation
// These are bound by reading W once from HBM.  The product is taken transposed so that the WEIGHTS fill
// the 128-row side of tcgen05.mma and the few activation rows are its N (a multiple of 16):
//     D[128 weight rows x NM] += W_tile[128 x 64] * X_slab[NM x 64]^T
// A stage of the TMA ring is then 16 KB of weights and only NM x 128 bytes of activations, so 5 to 9
// stages fit and an SM keeps 80 to 144 KB of weights in flight (with the activations on the 128-row side a
// stage was half activations, four stages fit, and the products ran at a third of the memory bandwidth).
// A matrix with few rows (N = hidden size) gives too few tiles for 148 SMs, so a thread-block cluster of
// KS CTAs shares one 128-row tile of W and splits K:
//   * each CTA streams its part of K and accumulates in tensor memory (lane = weight row, column =
//     activation row);
//   * every rank finishes a slice of the tile's weight rows: the epilogue warps of each CTA move the float32
//     accumulator to shared memory (over the ring, which is idle by then) and one thread sends each rank its
//     slice with a bulk shared-to-shared copy (cp.async.bulk.shared::cluster into a receive buffer beside
//     the ring, counted in bytes on the receiver's mbarrier).  Measured: loads from another CTA's shared
//     memory cost a few hundred cycles each, and st.shared::cluster with one row per lane took 2.5 us for
//     64 activation rows; the bulk copies take a few hundred nanoseconds;
//   * when its mbarrier has counted all slices, every CTA sums them, from its own shared memory, always in
//     rank order, applies the epilogue (none, softcap -> float32, or gated activation) and stores.
// For the gated epilogue a tile is 64 gate rows and the 64 matching up rows.
// Reference: the matvec shaders of src/backends/vulkan/shaders/tensor.comp:87-120 (one row).
// Every mbarrier wait is bounded in time; on expiry a status word is set (1 loads, 2 tensor-core issue,
// 4 accumulator, 8 hand-over), and the CTA still sends its (then zero) rows, takes part in the cluster
// barriers, frees its tensor memory and returns.
#include "common.cuh"
#include "tcgen05.cuh"

using namespace qnn;

#define EPI_NONE 0
#define EPI_SOFTCAP 1
#define EPI_GATED 2
#define EPI_ARGMAX 3      // softcap, then only the best (value, column) of the CTA's 128 columns per row: cand[row][tile]

namespace {

using namespace qnn::tc;
// this file's short names for the single-CTA forms
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, uint64_t adesc, uint64_t bdesc, unsigned idesc, unsigned accumulate) {
    umma_bf16_cta1(tmem_d, adesc, bdesc, idesc, accumulate);
}
__device__ __forceinline__ void umma_commit(unsigned bar) { umma_commit_cta1(bar); }
__device__ __forceinline__ void tmem_ld32(unsigned taddr, uint32_t (&r)[32]) { tmem_ld32_sync(taddr, r); }
inline int make_map(CUtensorMap* map, const void* base, long long rows, long long width, int box_rows) {
    return make_map_bf16(map, base, rows, width, box_rows, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}

constexpr int BW = 128, BK = 64, MAX_STAGES = 10, UMMA_K = 16;     // BW: weight rows of a tile
constexpr int W_BYTES = BW * BK * 2;
constexpr int THREADS = 192;
constexpr int RECV_COLS = 64;              // activation rows that pass through the receive buffer in one round


struct __align__(8) Barriers {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t acc_ready;
    uint64_t recv_full;          // counts the bytes that the ranks send this CTA, one phase per round
    uint32_t tmem_base;
    uint32_t failed;
};

// grid.x = output tiles x KS, cluster (KS, 1, 1): the CTAs of a cluster share a tile, rank = K part.
// NM: activation rows rounded up to 16; stages: depth of the ring; tmem_cols: power of two >= max(32, NM).
template <int EPI>
__global__ void __launch_bounds__(THREADS)
gemm_skinny_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                           void* __restrict__ C, int M, int N, int K, int KS, int NM, int stages, int tmem_cols,
                           float cap, int act, int* __restrict__ status, int* __restrict__ err) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int x_bytes = NM * BK * 2, stage_bytes = W_BYTES + x_bytes;
    const int PL = min(NM, RECV_COLS) + 4;                   // row pitch of the partial tile in floats
    const int RPB = BW / KS;                                 // weight rows of the tile that one rank finishes
    float* part = reinterpret_cast<float*>(smem);            // [BW][PL]: this CTA's partial tile, over its idle ring
    // [source rank][row of my slice][PL]: what the ranks send me; beside the ring, which is still in use then
    // (a CTA that is alone on its tile finishes its own partial tile where it lies)
    float* recv = KS > 1 ? reinterpret_cast<float*>(smem + (size_t)stages * stage_bytes) : part;
    Barriers* bars = reinterpret_cast<Barriers*>(smem + (size_t)stages * stage_bytes + (KS > 1 ? (size_t)BW * PL * 4 : 0));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();
    const int tile = blockIdx.x / KS;
    const int Nout = (EPI == EPI_GATED) ? N / 2 : N;
    constexpr int OUT_ROWS = (EPI == EPI_GATED) ? BW / 2 : BW;   // output columns (weight rows) of a tile
    const int n0 = tile * OUT_ROWS;
    const int nk = (K + BK - 1) / BK;
    const int per = (nk + KS - 1) / KS;
    const int kb0 = min((int)rank * per, nk), kb1 = min(kb0 + per, nk);        // this CTA's slabs

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        mbar_init(smem_u32(&bars->acc_ready), 1);
        mbar_init(smem_u32(&bars->recv_full), 1);
        bars->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (threadIdx.x == 0) mbar_expect_tx(smem_u32(&bars->recv_full), (unsigned)(BW * PL * 4));   // the first round
    // The cluster barrier is used in two halves.  Every thread arrives here and waits before anything is sent to
    // a peer, by when the peers have long arrived: that makes sure that they run and that their barriers are
    // set up.  It is used again before a CTA leaves (arrive when everything this CTA is sent has come, wait at
    // the end): a CTA's shared memory is the source of copies until every receiver has them.
    cluster_arrive();
    const unsigned tmem = bars->tmem_base;
    // Barriers and tensor memory are set up.  The weights do not depend on the kernel before this one: the
    // producer asks for the weight tiles of the first ring of stages, and only then waits for that kernel,
    // whose output the activation loads read; every other thread waits before it touches global memory.
    const int n_it = kb1 - kb0;
    const int ahead = (warp == 0 && lane == 0) ? min(stages, n_it) : 0;
    auto load_weights = [&](int it) {
        const int s = it % stages, kb = kb0 + it;
        const unsigned full = smem_u32(&bars->full[s]);
        const unsigned w_dst = smem_u32(smem + (size_t)s * stage_bytes);
        mbar_expect_tx(full, (unsigned)stage_bytes);
        if (EPI == EPI_GATED) {
            tma_load_2d(w_dst, &map_w, full, kb * BK, n0);                        // 64 gate rows
            tma_load_2d(w_dst + W_BYTES / 2, &map_w, full, kb * BK, Nout + n0);   // the 64 up rows
        } else {
            tma_load_2d(w_dst, &map_w, full, kb * BK, n0);
        }
    };
    for (int it = 0; it < ahead; ++it) load_weights(it);
    pdl_wait();
    bool have_acc = false;     // epilogue warps: the accumulator is complete (else this CTA contributes zeros)

    if (warp == 0) {
        if (lane == 0) {
            for (int it = 0; it < n_it; ++it) {
                const int s = it % stages;
                if (it >= ahead) {
                    if (it >= stages && !mbar_wait(smem_u32(&bars->empty[s]), ((it / stages) - 1) & 1)) {
                        atomicOr(status, 1);
                        bars->failed = 1;
                        break;
                    }
                    load_weights(it);
                }
                const unsigned x_dst = smem_u32(smem + (size_t)s * stage_bytes) + W_BYTES;
                tma_load_2d(x_dst, &map_x, smem_u32(&bars->full[s]), (kb0 + it) * BK, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // D float32, A (weights) and B (activations) bfloat16, both K-major, N = NM, M = 128
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(NM >> 3) << 17) | ((unsigned)(BW >> 4) << 24);
            for (int kb = kb0, it = 0; kb < kb1; ++kb, ++it) {
                const int s = it % stages;
                if (!mbar_wait(smem_u32(&bars->full[s]), (it / stages) & 1)) {
                    atomicOr(status, 2);
                    bars->failed = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned w_addr = smem_u32(smem + (size_t)s * stage_bytes), x_addr = w_addr + W_BYTES;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    umma_bf16(tmem, umma_desc(w_addr + k * UMMA_K * 2), umma_desc(x_addr + k * UMMA_K * 2), idesc,
                              (it > 0 || k > 0) ? 1u : 0u);
                umma_commit(smem_u32(&bars->empty[s]));
            }
            umma_commit(smem_u32(&bars->acc_ready));
        }
    } else {
        // the accumulator is complete (a CTA without slabs contributes zeros)
        bool ok = true;
        if (kb1 > kb0) {
            ok = mbar_wait(smem_u32(&bars->acc_ready), 0);
            if (!ok) {
                atomicOr(status, 4);
                bars->failed = 1;
            }
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        have_acc = kb1 > kb0 && ok;
    }
    __syncwarp();
    cluster_wait();            // the peers run and their barriers are set up: they may be sent to

    // Activation rows pass 64 at a time (one round for up to 64 rows).  In a round the epilogue warps move their
    // accumulator rows to this CTA's partial tile [weight row][activation row], one thread sends every rank its
    // rows of it, and when all ranks' rows have arrived rank r finishes weight rows [r * rpr, (r + 1) * rpr) of
    // the tile, four activation rows at a time: sum over the ranks in ascending order, epilogue, store.
    // Consecutive threads take consecutive weight rows, i.e. consecutive elements of a row of C.  A gated tile is
    // 64 gate rows and their 64 up rows; a rank's slice is RPB / 2 of each.
    const int rpr = OUT_ROWS / KS;
    const int r_lo = (int)rank * rpr;
    const unsigned recv_bar = smem_u32(&bars->recv_full);
    bool arrived = true;
    int round = 0;
    for (int h = 0; h < NM; h += RECV_COLS, ++round) {
        const int hcols = min(NM - h, RECV_COLS);
        if (warp >= 2) {
            const int quarter = warp & 3;
            const int wrow = quarter * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < hcols; c0 += 32) {
                uint32_t v[32];
                if (have_acc) {
                    tmem_ld32(tmem + ((unsigned)(quarter * 32) << 16) + h + c0, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0u;
                }
                float4* dst = reinterpret_cast<float4*>(part + (size_t)wrow * PL + c0);
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    if (c0 + j < hcols)
                        dst[j / 4] = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                                 __uint_as_float(v[j + 3]));
            }
            if (KS > 1) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // visible to the copy engine
            asm volatile("bar.sync 1, 128;" ::: "memory");                   // the four epilogue warps
            if (KS > 1 && warp == 2 && lane == 0) {
                const unsigned part_addr = smem_u32(part), recv_addr = smem_u32(recv);
                for (int q = 0; q < KS; ++q) {
                    // rank q finishes rows [q * RPB, (q + 1) * RPB) of a plain tile; of a gated tile RPB / 2 gate rows
                    // and the RPB / 2 up rows 64 further on
                    if (EPI == EPI_GATED) {
                        const unsigned half = (unsigned)(RPB / 2) * PL * 4u;
                        bulk_copy_to_rank(recv_addr + (unsigned)rank * RPB * PL * 4u, part_addr + (unsigned)q * half, half, recv_bar, q);
                        bulk_copy_to_rank(recv_addr + (unsigned)rank * RPB * PL * 4u + half,
                                          part_addr + (unsigned)(BW / 2) * PL * 4u + (unsigned)q * half, half, recv_bar, q);
                    } else {
                        const unsigned bytes = (unsigned)RPB * PL * 4u;
                        bulk_copy_to_rank(recv_addr + (unsigned)rank * bytes, part_addr + (unsigned)q * bytes, bytes, recv_bar, q);
                    }
                }
            }
        }
        if (KS == 1) {
            __syncthreads();                                     // the partial tile is complete
        } else if (arrived && !mbar_wait(recv_bar, round & 1)) {  // every rank's rows have come
            atomicOr(status, 8);
            arrived = false;
        }
        if (EPI == EPI_ARGMAX) {
            // The head of a greedy step for 9 to 128 rows (always a tile of its own: KS = 1): a thread per activation
            // row walks the tile's 128 weight rows in ascending order (the lowest column wins a tie), the cap is
            // monotonic and is applied to the winner only; NaN and Inf set the error word and lose.  The logits are
            // not written: one (value, column) per row and tile.
            const int m = h + (int)threadIdx.x;
            if ((int)threadIdx.x < hcols && m < M) {
                float best = -3.402823466e38f;
                int best_n = -1;
                bool bad = false;
                const int rows = min(OUT_ROWS, Nout - n0);
                for (int rr = 0; rr < rows; ++rr) {
                    const float v = recv[(size_t)rr * PL + threadIdx.x];
                    if (!(fabsf(v) <= 3.402823466e38f)) { bad = true; continue; }
                    if (v > best) { best = v; best_n = n0 + rr; }
                }
                if (bad && err != nullptr) atomicOr(err, 1);
                reinterpret_cast<float2*>(C)[(size_t)m * gridDim.x + tile] =
                    make_float2(best_n >= 0 ? softcap(best, cap) : -3.402823466e38f, __uint_as_float(best_n >= 0 ? (unsigned)best_n : 0xffffffffu));
            }
        }
        const int mgroups = EPI == EPI_ARGMAX ? 0 : (min(M - h, hcols) + 3) / 4;
        for (int idx = threadIdx.x; idx < rpr * mgroups && arrived; idx += THREADS) {
            const int rr = idx % rpr, m4 = (idx / rpr) * 4;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f), up = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int q = 0; q < KS; ++q) {
                const float4 v = *reinterpret_cast<const float4*>(recv + ((size_t)q * RPB + rr) * PL + m4);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                if (EPI == EPI_GATED) {
                    const float4 w = *reinterpret_cast<const float4*>(recv + ((size_t)q * RPB + rpr + rr) * PL + m4);
                    up.x += w.x; up.y += w.y; up.z += w.z; up.w += w.w;
                }
            }
            const int n = n0 + r_lo + rr;
            if (n >= Nout) continue;
            const float a4[4] = {acc.x, acc.y, acc.z, acc.w}, u4[4] = {up.x, up.y, up.z, up.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int m = h + m4 + j;
                if (m >= M) continue;
                if (EPI == EPI_GATED) {
                    reinterpret_cast<bf16*>(C)[(size_t)m * Nout + n] = __float2bfloat16_rn(activate_fast(a4[j], act) * u4[j]);
                } else if (EPI == EPI_SOFTCAP) {
                    reinterpret_cast<float*>(C)[(size_t)m * Nout + n] = softcap(a4[j], cap);
                } else {
                    reinterpret_cast<bf16*>(C)[(size_t)m * Nout + n] = __float2bfloat16_rn(a4[j]);
                }
            }
        }
        if (h + RECV_COLS < NM) {
            // Before the partial tiles and the receive buffers are written again, every CTA must have what it was
            // sent (then the copies out of every partial tile are done) and must have read it.
            __syncthreads();
            if (KS > 1) {
                if (threadIdx.x == 0) mbar_expect_tx(recv_bar, (unsigned)(BW * PL * 4));
                cluster_arrive();
                cluster_wait();
            }
        }
    }
    // A CTA's partial tile is the source of copies until every receiver has them; each CTA arrives when it has
    // everything it is sent (it waited for that above), so after this barrier nothing is in flight anywhere.
    cluster_arrive();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
    }
    cluster_wait();
}



template <int EPI>
int launch(const CUtensorMap& map_x, const CUtensorMap& map_w, void* C, int M, int N, int K, int KS, int NM, int stages,
           float cap, int act, int* status, unsigned tiles, cudaStream_t st, int* err = nullptr) {
    auto kern = gemm_skinny_tcgen05_kernel<EPI>;
    const size_t smem = (size_t)stages * (W_BYTES + NM * BK * 2) + (KS > 1 ? (size_t)BW * ((NM < RECV_COLS ? NM : RECV_COLS) + 4) * 4 : 0) + sizeof(Barriers) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    int tmem_cols = 32;
    while (tmem_cols < NM) tmem_cols *= 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles * KS);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = KS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (qnn::pdl_enabled() && (long long)tiles * KS <= qnn::pdl_max_grid()) ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_x, map_w, C, M, N, K, KS, NM, stages, tmem_cols, cap, act, status, err);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // namespace

// C = X W^T for M <= 128 rows.  epi 0: bfloat16 out; 1: softcap, float32 out; 2: gated (W = [gate; up],
// C is [M, N/2], bfloat16).  `status` as in qnn_gemm_tcgen05.  Returns QNN_ERR_UNSUPPORTED for sizes it
// does not take.
static int skinny_tcgen05(const void* A, const void* B, void* C, int M, int N, int K, int epi, float cap, int act,
                         int* status, int* err, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 128 || K <= 0 || (K & 7) || ((((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) != 0)) return QNN_ERR_UNSUPPORTED;
    if (epi == EPI_GATED && (N & 1)) return QNN_ERR_ARGUMENT;
    const int NM = (M + 15) / 16 * 16;
    CUtensorMap map_x, map_w;
    int rc = make_map(&map_x, A, M, K, NM);
    if (rc) return rc;
    rc = make_map(&map_w, B, N, K, epi == EPI_GATED ? BW / 2 : BW);
    if (rc) return rc;
    const int Nout = epi == EPI_GATED ? N / 2 : N;
    const int rows = epi == EPI_GATED ? BW / 2 : BW;
    const long long tiles = (Nout + rows - 1) / rows;
    if (tiles > 0x3fffffffLL) return QNN_ERR_UNSUPPORTED;
    // split K over a cluster when the tiles alone do not fill the GPU; every CTA keeps >= 2 slabs
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0)
            sm_count = 148;
    }
    const int nk = (K + 63) / 64;
    int KS = 1;
    while (KS < 8 && tiles * KS * 2 <= sm_count && nk / (KS * 2) >= 2) KS *= 2;      // the doubled grid still fits one round
    // Depth of the ring: what fits beside the receive buffer (128 x (min(NM, 64) + 4) floats) and the barriers, if the device
    // then holds all clusters at once (clusters of 8 CTAs with 217 KB each do not: 15 of them fit); else, and
    // with more CTAs than SMs anyway, half of that, so that two CTAs share an SM (and one's set-up and
    // epilogue hide behind the other's main loop).  The gate|up product of the 9B sizes is 224 tiles: with an SM
    // to each CTA they ran in two rounds, 49.6 us in a step of 10 rows where the weights' traffic needs 31.6.
    const int stage_bytes = W_BYTES + NM * BK * 2;
    const int part_bytes = BW * ((NM < RECV_COLS ? NM : RECV_COLS) + 4) * 4;
    const int recv_bytes = KS > 1 ? part_bytes : 0;
    const int per = (nk + KS - 1) / KS;
    auto depth = [&](int kib) {
        int st = (int)(((long long)kib * 1024 - 1024 - recv_bytes - (long long)sizeof(Barriers)) / stage_bytes);
        if (st > MAX_STAGES) st = MAX_STAGES;
        if (st > per) st = per < 2 ? 2 : per;
        if (st < 2) st = 2;
        while ((long long)st * stage_bytes < part_bytes) ++st;      // the partial tile lies over the ring
        return st;
    };
    static int force_kib = -1;
    if (force_kib < 0) {
        const char* e = getenv("QNN_SKINNY_KIB");
        force_kib = e ? atoi(e) : 0;
    }
    int stages = depth(227);
    if (force_kib > 0) {
        stages = depth(force_kib);
    } else if (tiles * KS > (long long)sm_count || NM <= 32) {
        // also for up to 32 rows: consecutive products of a layer then share an SM, and the second one's first weights
        // are on their way while the first still runs (steps of 10 to 32 rows 1 to 2 % faster at the 2B sizes, nothing
        // lost at the 9B and 27B sizes; at 64 rows, where a stage is a third larger, the deep ring is 1 % better)
        stages = depth(113);
    } else if (KS > 1) {
        static int fits[4][MAX_STAGES + 1];                // clusters of 2^i CTAs that the device holds, by depth (0: not asked)
        int ki = KS == 2 ? 1 : (KS == 4 ? 2 : 3);
        if (fits[ki][stages] == 0) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(KS * 64);
            cfg.blockDim = dim3(THREADS);
            cfg.dynamicSmemBytes = (size_t)stages * stage_bytes + recv_bytes + sizeof(Barriers) + 1024;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = KS;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            (void)cudaFuncSetAttribute(gemm_skinny_tcgen05_kernel<EPI_NONE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (cudaOccupancyMaxActiveClusters(&n, gemm_skinny_tcgen05_kernel<EPI_NONE>, &cfg) != cudaSuccess || n <= 0) {
                (void)cudaGetLastError();
                n = -1;
            }
            fits[ki][stages] = n;
        }
        if (fits[ki][stages] < tiles) stages = depth(113);
    }
    if (stages > MAX_STAGES || (long long)stages * stage_bytes + recv_bytes + (long long)sizeof(Barriers) + 1024 > 227 * 1024)
        return QNN_ERR_UNSUPPORTED;
    if (epi == EPI_ARGMAX) {
        if (KS != 1) return QNN_ERR_UNSUPPORTED;        // so few columns that tiles share K: the caller writes logits
        return launch<EPI_ARGMAX>(map_x, map_w, C, M, N, K, KS, NM, stages, cap, act, status, (unsigned)tiles, st, err);
    }
    switch (epi) {
        case EPI_NONE: return launch<EPI_NONE>(map_x, map_w, C, M, N, K, KS, NM, stages, cap, act, status, (unsigned)tiles, st);
        case EPI_SOFTCAP: return launch<EPI_SOFTCAP>(map_x, map_w, C, M, N, K, KS, NM, stages, cap, act, status, (unsigned)tiles, st);
        case EPI_GATED: return launch<EPI_GATED>(map_x, map_w, C, M, N, K, KS, NM, stages, cap, act, status, (unsigned)tiles, st);
    }
    return QNN_ERR_ARGUMENT;
}

QNN_API int qnn_gemm_skinny_tcgen05(const void* A, const void* B, void* C, int M, int N, int K, int epi, float cap,
                                    int act, int* status, cudaStream_t st) {
    if (epi != EPI_NONE && epi != EPI_SOFTCAP && epi != EPI_GATED) return QNN_ERR_ARGUMENT;
    return skinny_tcgen05(A, B, C, M, N, K, epi, cap, act, status, nullptr, st);
}

// The head of a greedy step for up to 128 rows: cand[m][t] = the best (softcapped value, column) among the 128
// columns of W that tile t covers; ceil(N / 128) candidates per row, merged by qnn_sample_candidates.  err (may be
// null) gets bit 0 set if a logit is NaN or Inf.  QNN_ERR_UNSUPPORTED for a matrix of so few rows that its tiles
// would share K.
QNN_API int qnn_gemm_skinny_tcgen05_argmax(const void* A, const void* B, void* cand, int M, int N, int K, float cap,
                                           int* err, int* status, cudaStream_t st) {
    if ((uintptr_t)cand & 7) return QNN_ERR_ARGUMENT;
    return skinny_tcgen05(A, B, cand, M, N, K, EPI_ARGMAX, cap, 0, status, err, st);
}

// Whole-prompt matrix products on the 5th-generation tensor cores, two SMs per tile:
//     C[M, N] = A[M, K] * B[N, K]^T      bfloat16 in, float32 accumulation in tensor memory
// The same product and epilogues as gemm_tcgen05.cu; what differs is that a pair of CTAs (a
// thread-block cluster of two, on the two SMs of a TPC) computes a 256 x 256 tile with
// tcgen05.mma.cta_group::2.  Each CTA brings its own 128 rows of A and HALF of the B slab (128 of
// the 256 weight rows), so a CTA reads 32 KB from L2 per 64-deep slab instead of 48 KB for the same
// arithmetic; the single-CTA kernel is bound by exactly that traffic (its tensor pipe idles a quarter
// of the main loop), and the 32 KB stages leave room for 6 of them instead of 4.
//
//   * rank 0 of the pair is the leader: its lane issues every tcgen05.mma (M 256, N 256, K 16), reading
//     A and B from the shared memory of both CTAs and writing 128 accumulator rows into the tensor
//     memory of each;
//   * both CTAs run a TMA producer (cp.async.bulk.tensor with .cta_group::2, no multicast): the bytes of
//     both land on the LEADER's "full" barrier of the stage;
//   * tcgen05.commit.cta_group::2 with a CTA mask hands a stage back to both producers and, after the
//     last slab, an accumulator to the epilogue warps of both CTAs, each of which drains its own 128
//     rows; they return the accumulator with remote arrivals on the leader's barrier;
//   * the epilogue goes through shared memory (128 rows x 128 columns at a time) so that global memory
//     is written in whole 256-byte row pieces;
//   * tensor memory is allocated and freed with the .cta_group::2 forms by the same warp of both CTAs,
//     with cluster barriers after set-up and before the release.
// For the gated epilogue rank 0 loads the 128 gate rows and rank 1 the 128 matching up rows, so every
// accumulator row holds gate | up side by side, as in the single-CTA kernel.
//
// Every wait on an mbarrier is bounded (see gemm_tcgen05.cu); the two cluster barriers are reached by
// every thread of both CTAs on every path, in bounded time.
#include "common.cuh"
#include "tcgen05.cuh"

using namespace qnn;

#define EPI_NONE 0
#define EPI_GATED 2

namespace {

using namespace qnn::tc;
__device__ __forceinline__ void tmem_ld32(unsigned taddr, uint32_t (&r)[32]) { tmem_ld32_sync(taddr, r); }
inline int make_map(CUtensorMap* map, const void* base, long long rows, long long width, int box_rows) {
    return make_map_bf16(map, base, rows, width, box_rows, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
}

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 6, UMMA_K = 16;       // BM: rows per CTA; the pair does 256
constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;   // per CTA
constexpr int TMEM_COLS = 256;
constexpr int STAGING_BYTES = BM * 128 * 2;          // the epilogue's 128 rows x 128 columns of bfloat16
constexpr int GEMM_THREADS = 192;


// `bar` is a shared::cluster address: the leader's barrier, whichever CTA of the pair loads
__device__ __forceinline__ void tma_load_2d_pair(unsigned dst, const CUtensorMap* map, unsigned bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, uint64_t adesc, uint64_t bdesc, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once everything issued so far is done, on the barrier at this offset in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}


struct __align__(8) Barriers {
    uint64_t full[STAGES];      // leader only: the slabs of both CTAs have landed (TMA bytes)
    uint64_t empty[STAGES];     // in each CTA: the MMAs that read the stage are done
    uint64_t acc_ready[2];      // in each CTA: an accumulator is complete
    uint64_t acc_free[2];       // leader only: the epilogues of both CTAs have read an accumulator
    uint32_t tmem_base;
    uint32_t failed;
};

__device__ __forceinline__ bool has_failed(Barriers* b) { return *reinterpret_cast<volatile uint32_t*>(&b->failed) != 0; }

// Persistent: a pair of CTAs per TPC walks over 256-row tiles t = pair, pair + pairs, ... (row tiles
// fastest, so the pairs that run together share their B slabs in L2).
template <int EPI>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         bf16* __restrict__ C, int M, int N, int K, int act, int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* staging = smem + STAGES * STAGE_BYTES;
    Barriers* bars = reinterpret_cast<Barriers*>(staging + STAGING_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_rank();                 // 0: leader
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int Nout = (EPI == EPI_GATED) ? N / 2 : N;
    constexpr int OUT_COLS = (EPI == EPI_GATED) ? BN / 2 : BN;          // output columns of a tile
    const int m_tiles = (M + 2 * BM - 1) / (2 * BM), n_tiles = (Nout + OUT_COLS - 1) / OUT_COLS;
    const int ntiles = m_tiles * n_tiles;
    const int nk = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bars->acc_ready[a]), 1);
            mbar_init(smem_u32(&bars->acc_free[a]), 8);     // one arrival per epilogue warp of both CTAs
        }
        bars->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // the same warp of both CTAs allocates the pair's tensor memory, and frees it at the end
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"(2 * TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_barrier();           // the peer's barriers exist before anything is sent to them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = bars->tmem_base;
    // Barriers and tensor memory are set up; only now wait for the kernels before this one (whose output
    // the loads below read), so that the set-up overlaps their tail.
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer (both CTAs) ---------------------------------------------------------
            int it = 0;                                    // slabs issued so far, over all tiles
            for (int tile = pair; tile < ntiles && !has_failed(bars); tile += pairs) {
                const int m0 = (tile % m_tiles) * (2 * BM) + (int)rank * BM;
                const int n0 = (tile / m_tiles) * OUT_COLS;
                // this CTA's half of the B slab: for the gated product the gate rows (rank 0) or the up rows (rank 1)
                const int brow = (EPI == EPI_GATED) ? (rank == 0 ? n0 : Nout + n0) : n0 + (int)rank * (BN / 2);
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(smem_u32(&bars->empty[s]), ((it / STAGES) - 1) & 1)) {
                        atomicOr(status, 1);
                        bars->failed = 1;
                        break;
                    }
                    const unsigned full_local = smem_u32(&bars->full[s]);
                    const unsigned full_leader = map_to_rank(full_local, 0);
                    const unsigned a_dst = smem_u32(smem + s * STAGE_BYTES), b_dst = a_dst + A_BYTES;
                    if (rank == 0) mbar_expect_tx(full_local, 2 * STAGE_BYTES);
                    tma_load_2d_pair(a_dst, &map_a, full_leader, kb * BK, m0);
                    tma_load_2d_pair(b_dst, &map_b, full_leader, kb * BK, brow);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // ---- tensor-core issue (leader) ----------------------------------------------------
            // instruction descriptor: D float32, A and B bfloat16, both K-major, N >> 3, M >> 4 (M = 256 over the pair)
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)((2 * BM) >> 4) << 24);
            int it = 0, i = 0;                             // slabs consumed; tiles done by this pair
            for (int tile = pair; tile < ntiles && !has_failed(bars); tile += pairs, ++i) {
                const int a = i & 1;
                if (i >= 2 && !mbar_wait(smem_u32(&bars->acc_free[a]), ((i >> 1) - 1) & 1)) {
                    atomicOr(status, 8);
                    bars->failed = 1;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned acc = tmem + a * TMEM_COLS;
                bool ok = true;
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(smem_u32(&bars->full[s]), (it / STAGES) & 1)) {
                        atomicOr(status, 2);
                        bars->failed = 1;
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned a_addr = smem_u32(smem + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 elements further along K = 32 bytes inside the 128-byte swizzled row
                        umma_bf16(acc, umma_desc(a_addr + k * UMMA_K * 2), umma_desc(b_addr + k * UMMA_K * 2), idesc,
                                  (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(smem_u32(&bars->empty[s]));     // the stage is free in both CTAs once these MMAs have read it
                }
                umma_commit_pair(smem_u32(&bars->acc_ready[a]));     // arrives in both CTAs when everything issued so far is done
                if (!ok) break;
            }
        }
    } else {
        // ---- epilogue (both CTAs): warps 2..5, each owns the 32 accumulator lanes (rows) of its quarter ----
        const int quarter = warp & 3;
        int i = 0;
        for (int tile = pair; tile < ntiles; tile += pairs, ++i) {
            const int a = i & 1;
            const int m0 = (tile % m_tiles) * (2 * BM) + (int)rank * BM, n0 = (tile / m_tiles) * OUT_COLS;
            if (!mbar_wait(smem_u32(&bars->acc_ready[a]), (i >> 1) & 1)) {
                atomicOr(status, 4);
                bars->failed = 1;
                break;
            }
            if (has_failed(bars)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int m = m0 + quarter * 32 + lane;
            const unsigned lane_addr = tmem + a * TMEM_COLS + ((unsigned)(quarter * 32) << 16);
            if ((Nout & 7) == 0) {
                // Through shared memory, 128 columns at a time: each thread leaves its row as bfloat16
                // (16-byte chunks XOR-ed with the row number, so that neither side has bank conflicts), then
                // the warp writes its 32 rows to global memory two rows (2 x 256 bytes) per instruction.
                // A thread-per-row store straight from registers touches 32 lines per instruction and made
                // the epilogue 4.4 us of a 19 us product.
                unsigned char* mine = staging + quarter * (32 * 256);
#pragma unroll 1
                for (int h0 = 0; h0 < OUT_COLS; h0 += 128) {
#pragma unroll 1
                    for (int c0 = h0; c0 < h0 + 128; c0 += 32) {
                        uint32_t v[32];
                        tmem_ld32(lane_addr + c0, v);
                        float f[32];
                        if (EPI == EPI_GATED) {
                            uint32_t u[32];
                            tmem_ld32(lane_addr + BN / 2 + c0, u);
#pragma unroll
                            for (int j = 0; j < 32; ++j) f[j] = activate_fast(__uint_as_float(v[j]), act) * __uint_as_float(u[j]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
                        }
                        if (c0 + 32 >= OUT_COLS) {
                            // the last columns are in registers: hand the accumulator back to the leader
                            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                            __syncwarp();
                            if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&bars->acc_free[a]), 0));
                        }
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int ch = (c0 - h0) / 8 + j;
                            uint4 pk;
                            pk.x = pack_bf16(f[j * 8 + 0], f[j * 8 + 1]);
                            pk.y = pack_bf16(f[j * 8 + 2], f[j * 8 + 3]);
                            pk.z = pack_bf16(f[j * 8 + 4], f[j * 8 + 5]);
                            pk.w = pack_bf16(f[j * 8 + 6], f[j * 8 + 7]);
                            *reinterpret_cast<uint4*>(mine + lane * 256 + ((ch ^ (lane & 15)) << 4)) = pk;
                        }
                    }
                    __syncwarp();
#pragma unroll 4
                    for (int rr = 0; rr < 32; rr += 2) {
                        const int r = rr + (lane >> 4), pos = lane & 15;
                        const int row = m0 + quarter * 32 + r;
                        const int col = n0 + h0 + ((pos ^ (r & 15)) << 3);
                        const uint4 pk = *reinterpret_cast<const uint4*>(mine + r * 256 + (pos << 4));
                        if (row < M && col < Nout) *reinterpret_cast<uint4*>(C + (size_t)row * Nout + col) = pk;
                    }
                    __syncwarp();
                }
                continue;
            }
#pragma unroll 1
            for (int c0 = 0; c0 < OUT_COLS; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(lane_addr + c0, v);
                float f[32];
                if (EPI == EPI_GATED) {
                    uint32_t u[32];
                    tmem_ld32(lane_addr + BN / 2 + c0, u);
#pragma unroll
                    for (int j = 0; j < 32; ++j) f[j] = activate_fast(__uint_as_float(v[j]), act) * __uint_as_float(u[j]);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
                }
                if (c0 + 32 >= OUT_COLS) {
                    // the last columns are in registers: hand the accumulator back to the leader before storing them
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_rank(smem_u32(&bars->acc_free[a]), 0));
                }
                if (m < M) {
                    bf16* dst = C + (size_t)m * Nout + n0 + c0;
                    if (n0 + c0 + 32 <= Nout && ((Nout & 7) == 0)) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) Vec16<bf16>::store(dst + j, f + j);
                    } else {
                        for (int j = 0; j < 32; ++j)
                            if (n0 + c0 + j < Nout) dst[j] = __float2bfloat16_rn(f[j]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_barrier();           // neither CTA frees tensor memory, or leaves, while the other still uses the pair's
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * TMEM_COLS) : "memory");
    }
}



}  // namespace

// The product of qnn_gemm_tcgen05 (same arguments, same meaning of `status`) computed by pairs of CTAs.
// Returns QNN_ERR_UNSUPPORTED when the device cannot hold a pair (the caller then uses the single-CTA
// kernel).
QNN_API int qnn_gemm_tcgen05_2cta(const void* A, const void* B, void* C, int M, int N, int K, int epi, int act,
                                  int* status, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7) || ((((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) != 0)) return QNN_ERR_UNSUPPORTED;
    if (epi != EPI_NONE && epi != EPI_GATED) return QNN_ERR_ARGUMENT;
    if (epi == EPI_GATED && (N & 1)) return QNN_ERR_ARGUMENT;
    CUtensorMap map_a, map_b;
    int rc = make_map(&map_a, A, M, K, BM);
    if (rc) return rc;
    rc = make_map(&map_b, B, N, K, BN / 2);
    if (rc) return rc;
    const int Nout = epi == EPI_GATED ? N / 2 : N;
    const int cols = epi == EPI_GATED ? BN / 2 : BN;
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0)
            sm_count = 148;
    }
    const long long ntiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((Nout + cols - 1) / cols);
    if (ntiles > 0x3fffffffLL) return QNN_ERR_UNSUPPORTED;
    const size_t smem = (size_t)STAGES * STAGE_BYTES + STAGING_BYTES + sizeof(Barriers) + 1024;
    void (*kern)(CUtensorMap, CUtensorMap, bf16*, int, int, int, int, int*) =
        epi == EPI_GATED ? gemm_tcgen05_2cta_kernel<EPI_GATED> : gemm_tcgen05_2cta_kernel<EPI_NONE>;
    static bool configured[2] = {false, false};
    static int max_pairs = 0;
    const int which = epi == EPI_GATED ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    if (!configured[which]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured[which] = true;
    }
    if (max_pairs == 0) {        // pairs of this kernel that the device holds at once (asked once)
        cfg.gridDim = dim3(2 * (sm_count / 2));
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            max_pairs = -1;
        } else {
            max_pairs = n < sm_count / 2 ? n : sm_count / 2;
        }
    }
    if (max_pairs < 0) return QNN_ERR_UNSUPPORTED;
    const int pairs = ntiles < max_pairs ? (int)ntiles : max_pairs;
    cfg.gridDim = dim3(2 * pairs);
    cfg.numAttrs = (qnn::pdl_enabled() && 2ll * pairs <= qnn::pdl_max_grid()) ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_a, map_b, (bf16*)C, M, N, K, act, status);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Whole-prompt matrix products on the 5th-generation tensor cores:
//     C[M, N] = A[M, K] * B[N, K]^T      bfloat16 in, float32 accumulation in tensor memory
// with the epilogues that follow the products in the model (none, or the gated activation
// act(gate) * up for a weight matrix that stacks [gate; up]).
//
// Reference: the 64x64 fp32-FMA tile of src/backends/vulkan/shaders/gemm.comp:4-6 and the separate
// GO_GEGLU dispatch (src/models/QuickNN.Models.Gemma2.pas:184-186).  Here:
//   * a persistent CTA per SM computes 128 x 256 tiles; K is walked in slabs of 64 (128-byte rows,
//     128-byte swizzle); two accumulators in tensor memory let the epilogue of one tile overlap
//     the products of the next;
//   * warp 0 (one lane) is the producer: TMA (cp.async.bulk.tensor) loads of the A and B slabs into a
//     4-stage ring in shared memory, completion counted in bytes on an mbarrier per stage;
//   * warp 1 (one lane) issues tcgen05.mma (M 128, N 256, K 16; four per slab) from shared-memory
//     descriptors into a 256-column accumulator in tensor memory, and tcgen05.commit hands each stage
//     back to the producer and, after the last slab, the accumulator to the epilogue;
//   * warps 2..5 are the epilogue: tcgen05.ld (32 lanes x 32 columns at a time), activation, convert,
//     16-byte stores.  For the gated epilogue the B slab holds 128 gate rows and the 128 matching up
//     rows, so one accumulator holds both halves.
// Rows and columns beyond M, N, K are zero-filled by TMA and never stored.
//
// Every wait on an mbarrier is bounded: when it runs out, the thread sets a word in global memory
// (`status`), stops waiting, and the CTA still frees its tensor memory and returns; the host reads
// the word and raises.  No wait here can hang the GPU.
#include "common.cuh"
#include "tcgen05.cuh"

using namespace qnn;

#define EPI_NONE 0
#define EPI_GATED 2

namespace {

using namespace qnn::tc;
// this file's short names for the single-CTA forms
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, uint64_t adesc, uint64_t bdesc, unsigned idesc, unsigned accumulate) {
    umma_bf16_cta1(tmem_d, adesc, bdesc, idesc, accumulate);
}
__device__ __forceinline__ void umma_commit(unsigned bar) { umma_commit_cta1(bar); }
__device__ __forceinline__ void tmem_ld32(unsigned taddr, uint32_t (&r)[32]) { tmem_ld32_sync(taddr, r); }
inline int make_map(CUtensorMap* map, const void* base, long long rows, long long width, int box_rows) {
    return make_map_bf16(map, base, rows, width, box_rows, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
}

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 256;
constexpr int GEMM_THREADS = 192;



struct __align__(8) Barriers {
    uint64_t full[STAGES];      // a slab has landed (TMA bytes)
    uint64_t empty[STAGES];     // the MMAs that read a slab are done
    uint64_t acc_ready[2];      // an accumulator is complete
    uint64_t acc_free[2];       // the epilogue has read an accumulator out of tensor memory
    uint32_t tmem_base;
    uint32_t failed;
};

__device__ __forceinline__ bool has_failed(Barriers* b) { return *reinterpret_cast<volatile uint32_t*>(&b->failed) != 0; }

// Persistent: a CTA per SM walks over tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... (row tiles
// fastest, so the CTAs that run together share their B slabs in L2).  Tensor memory holds two
// accumulators of 256 columns; while the epilogue warps drain one, the MMAs of the next tile fill
// the other, and the TMA ring runs on across tile borders.
template <int EPI>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    bf16* __restrict__ C, int M, int N, int K, int act, int* __restrict__ status) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the operand ring wants 1024-byte alignment (8 swizzled rows); the barriers follow it
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Barriers* bars = reinterpret_cast<Barriers*>(smem + STAGES * STAGE_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int Nout = (EPI == EPI_GATED) ? N / 2 : N;
    constexpr int OUT_COLS = (EPI == EPI_GATED) ? BN / 2 : BN;          // output columns of a tile
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (Nout + OUT_COLS - 1) / OUT_COLS;
    const int ntiles = m_tiles * n_tiles;
    const int nk = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bars->acc_ready[a]), 1);
            mbar_init(smem_u32(&bars->acc_free[a]), 4);     // one arrival per epilogue warp
        }
        bars->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // this warp owns the tensor memory: allocates it here, frees it at the end
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"(2 * TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = bars->tmem_base;
    // Barriers and tensor memory are set up; only now wait for the kernels before this one (whose output
    // the loads below read), so that the set-up overlaps their tail.
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer -------------------------------------------------------------------
            int it = 0;                                    // slabs issued so far, over all tiles
            for (int tile = blockIdx.x; tile < ntiles && !has_failed(bars); tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * OUT_COLS;
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(smem_u32(&bars->empty[s]), ((it / STAGES) - 1) & 1)) {
                        atomicOr(status, 1);
                        bars->failed = 1;
                        break;
                    }
                    const unsigned full = smem_u32(&bars->full[s]);
                    const unsigned a_dst = smem_u32(smem + s * STAGE_BYTES), b_dst = a_dst + A_BYTES;
                    mbar_expect_tx(full, STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, full, kb * BK, m0);
                    if (EPI == EPI_GATED) {
                        tma_load_2d(b_dst, &map_b, full, kb * BK, n0);                        // 128 gate rows
                        tma_load_2d(b_dst + B_BYTES / 2, &map_b, full, kb * BK, Nout + n0);   // the 128 up rows
                    } else {
                        tma_load_2d(b_dst, &map_b, full, kb * BK, n0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- tensor-core issue ------------------------------------------------------------
            // instruction descriptor: D float32, A and B bfloat16, both K-major, N >> 3, M >> 4
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
            int it = 0, i = 0;                             // slabs consumed; tiles done by this CTA
            for (int tile = blockIdx.x; tile < ntiles && !has_failed(bars); tile += gridDim.x, ++i) {
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
                    umma_commit(smem_u32(&bars->empty[s]));     // the stage is free once these MMAs have read it
                }
                umma_commit(smem_u32(&bars->acc_ready[a]));     // arrives when everything issued so far is done
                if (!ok) break;
            }
        }
    } else {
        // ---- epilogue: warps 2..5, each owns the 32 accumulator lanes (rows) of its quarter ----------
        const int quarter = warp & 3;
        int i = 0;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++i) {
            const int a = i & 1;
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * OUT_COLS;
            if (!mbar_wait(smem_u32(&bars->acc_ready[a]), (i >> 1) & 1)) {
                atomicOr(status, 4);
                bars->failed = 1;
                break;
            }
            if (has_failed(bars)) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int m = m0 + quarter * 32 + lane;
            const unsigned lane_addr = tmem + a * TMEM_COLS + ((unsigned)(quarter * 32) << 16);
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
                    // the last columns are in registers: hand the accumulator back before storing them
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bars->acc_free[a])) : "memory");
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
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * TMEM_COLS) : "memory");
    }
}



}  // namespace

// C = A B^T (epi 0) or act(A Bgate^T) * (A Bup^T) with B = [gate; up] (epi 2; C is [M, N/2]).
// `status` is one int in device memory that the caller zeroed: a non-zero value after the kernel
// means a bounded wait ran out (bit 0 producer, bits 1 and 3 tensor-core issue, bit 2 epilogue) and C is
// not valid.  K must be a multiple of 8 (16-byte row pitch) and the bases 16-byte aligned.
QNN_API int qnn_gemm_tcgen05(const void* A, const void* B, void* C, int M, int N, int K, int epi, int act,
                             int* status, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7) || ((((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) != 0)) return QNN_ERR_UNSUPPORTED;
    if (epi != EPI_NONE && epi != EPI_GATED) return QNN_ERR_ARGUMENT;
    if (epi == EPI_GATED && (N & 1)) return QNN_ERR_ARGUMENT;
    CUtensorMap map_a, map_b;
    int rc = make_map(&map_a, A, M, K, BM);
    if (rc) return rc;
    rc = make_map(&map_b, B, N, K, epi == EPI_GATED ? BN / 2 : BN);
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
    const long long ntiles = (long long)((M + BM - 1) / BM) * ((Nout + cols - 1) / cols);
    if (ntiles > 0x7fffffffLL) return QNN_ERR_UNSUPPORTED;
    dim3 grid((unsigned)(ntiles < sm_count ? ntiles : sm_count));
    const size_t smem = (size_t)STAGES * STAGE_BYTES + sizeof(Barriers) + 1024;
    if (epi == EPI_GATED) {
        auto kern = gemm_tcgen05_kernel<EPI_GATED>;
        static bool configured = false;
        if (!configured) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
            configured = true;
        }
        cudaError_t e = qnn::launch_pdl(kern, grid, dim3(GEMM_THREADS), smem, st, map_a, map_b, (bf16*)C, M, N, K, act, status);
        return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
    }
    auto kern = gemm_tcgen05_kernel<EPI_NONE>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cudaError_t e = qnn::launch_pdl(kern, grid, dim3(GEMM_THREADS), smem, st, map_a, map_b, (bf16*)C, M, N, K, act, status);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// Prefill attention on the 5th-generation tensor cores, bfloat16, head sizes 64, 128 and 256: whole prompts
// packed one after another, causal, optional sliding window, optional tanh softcap, grouped
// query heads.  Formulas: attention.cu (reference: src/backends/vulkan/shaders/attention.comp:18-38).
//
// A CTA owns 128 query rows of one sequence and one query head and walks over its keys in tiles of 64, two tiles
// (a pair) at a time.  Twelve warps:
//   warp 0  (one lane)  TMA producer of Q (once, into the second stage of the K ring) and of K: a pair of key
//                       tiles is one operand of 128 rows (hd/64 boxes of 128 x 64), free again once S is formed.
//   warp 10 (one lane)  TMA producer of V, tiles of 64 keys, free only after O += P V.  128-byte swizzle throughout.
//   warp 1  (one lane)  issues S[128 x 128] = Q K^T for a pair of tiles: hd/16 tcgen05.mma of N = 128 whose A operand,
//                       Q, is read from tensor memory.  Issuing one tcgen05.mma occupies its thread for about 100
//                       cycles whatever its size (N = 32, 64, 128 alike; 138 at N = 256 with A from tensor memory,
//                       171 with A from shared memory), so products of N = 64 cost their issue, not their work.
//   warp 11 (one lane)  issues O[128 x hd] += P_j V_j (4 tcgen05.mma of N = hd, V as MN-major operand) for every tile.
//   warps 2..5          softmax, one thread per query row (tensor-memory lane = row, so row maxima and sums need no
//                       shuffles): first they copy Q from shared to tensor memory; then per tile tcgen05.ld of S
//                       (the S columns are handed back as soon as the scores are in registers), scale, softcap,
//                       mask, exp; P_j goes to shared memory as bfloat16 in the swizzled K-major layout the next
//                       product reads.  Without a softcap: a running maximum, and O is rescaled in tensor memory only
//                       when a row maximum has grown by more than 8 since the value the row's exponentials are taken
//                       against (the stale maximum cancels in the final division; P stays below e^8).
//   warps 6..9          a second softmax group, with a softcap only (FIXED).  A capped score lies in [-cap, cap], so
//                       exp(score) can neither overflow nor vanish in float32 and needs no running maximum:
//                       p = exp(cap tanh(s / cap)) against the fixed reference 0, the same softmax (it is invariant
//                       under the shift) with nothing carried from tile to tile but a row's sum.  The tiles are then
//                       independent: warps 2..5 take the lower tile of each pair, warps 6..9 the upper one, two tiles
//                       are in the softmax at any time, no maximum is tracked and O is never rescaled.
// What set the pace, in the order in which it was found (clock64 around the waits of each role): the softmax chain of
// one warp per scheduler (2350 cycles per tile); the issue of 16 + 4 products per tile by one thread (1850); shared
// memory bandwidth (Q, K, V, P and the TMA writes: 224 KB per tile, 160 with Q in tensor memory).  One prompt of 8192
// tokens, 8 heads of 256: 316 us with the running maximum and S of N = 64, 297 us with the fixed reference, two softmax
// groups and Q in tensor memory, 242 us (1.13 PFLOP/s) with S of N = 128 and P V issued by a thread of its own.
// With few CTAs the grid may be launched as clusters of two (the policy is in launch_attn): the CTAs of a pair take
// alternate pairs of key tiles of the same query tile; when both are done, rank 1 pushes its (reference maximum, sum,
// O) into rank 0's shared memory through the cluster's distributed shared memory and rank 0 merges and writes.
// Tensor memory: S 128 columns, O one column per head element, Q hd / 2 columns.  All softmax arithmetic is float32.
// Keys of other sequences that a tile drags in are masked; rows beyond the sequence are never stored.
// Every mbarrier wait is bounded in time; on expiry a status word is set and the CTA winds down.
#include "common.cuh"
#include "tcgen05.cuh"
#include <math_constants.h>

using namespace qnn;

namespace {

using namespace qnn::tc;
// this file's short names for the single-CTA forms
__device__ __forceinline__ void umma_bf16(unsigned tmem_d, uint64_t adesc, uint64_t bdesc, unsigned idesc, unsigned accumulate) {
    umma_bf16_cta1(tmem_d, adesc, bdesc, idesc, accumulate);
}
__device__ __forceinline__ void umma_commit(unsigned bar) { umma_commit_cta1(bar); }
__device__ __forceinline__ void tmem_ld32(unsigned taddr, uint32_t (&r)[32]) { tmem_ld32_nowait(taddr, r); }
inline int make_map(CUtensorMap* map, const void* base, long long rows, long long width, int box_rows) {
    return make_map_bf16(map, base, rows, width, box_rows, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
}

constexpr int BM = 128, BN = 64, MAX_KV_STAGES = 6, UMMA_K = 16;
// Depth of the rings: K in pairs of key tiles (128 keys), V in tiles of 64 keys; what fits beside P in 227 KB.
__host__ __device__ constexpr int k_stages(int hd) { return hd >= 256 ? 2 : (hd >= 128 ? 3 : 4); }
__host__ __device__ constexpr int v_stages(int hd) { return hd >= 256 ? 2 : (hd >= 128 ? 4 : 6); }
constexpr int P_BYTES = BM * BN * 2;                 // 16 KB
constexpr int THREADS = 384;       // K producer, S issue, two groups of four softmax warps, V producer, P V issue
constexpr int S_COL = 0, O_COL = 128;             // tensor-memory columns of S (two buffers of 64) and of O; Q follows O
// D[tmem] (+)= A[tmem] B[smem]: the A operand (here Q: lane = row, two bfloat16 per column) read from tensor memory
__device__ __forceinline__ void umma_bf16_a_tmem(unsigned tmem_d, unsigned tmem_a, uint64_t bdesc, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
constexpr float RESCALE_STEP = 8.f;
constexpr int MERGE_ML_BYTES = BM * 8;               // (reference maximum, sum) per row that rank 1 of a pair hands to rank 0

__device__ __forceinline__ float tanh_fast(float x) {
    float r;
    asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float exp2_fast(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
// 2^x on the FMA and integer pipes, for |x| < 126: x = n + f with n the nearest integer (the sum with 1.5 * 2^23
// leaves n in the low mantissa bits), 2^f by a cubic on [-0.5, 0.5] (relative error 7.5e-5, a thirtieth of
// bfloat16's rounding), n added to the exponent field.  The special-function unit does 16 operations a clock per
// SM and a capped score needs two (tanh, 2^x): taking some of the exponentials here relieves it.  Measured with
// 0, 2, 4, 6, 8 of every 8 columns done this way, 8 heads of 256, one prompt: 2048 tokens 36.8 / 36.1 / 35.1 / 35.2 /
// 38.4 us, 8192 tokens 243 / 241 / 238 / 239 / 253 us; 32 heads of 128 at 8192: 831 / 815 / 796 / 800 / 869 us.
constexpr int POLY = 4;            // of every 8 columns of a row
__device__ __forceinline__ float exp2_poly(float x) {
    const float magic = 12582912.f;
    const float xf = x + magic;
    const float f = x - (xf - magic);
    float p = fmaf(f, 0.055171407759189606f, 0.24261075258255005f);
    p = fmaf(p, f, 0.6932609677314758f);
    p = fmaf(p, f, 0.9999281167984009f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(xf) << 23));
}


struct __align__(8) Barriers {
    uint64_t q_full;
    uint64_t q_tmem;          // the softmax warps have copied Q from shared to tensor memory
    uint64_t k_full[MAX_KV_STAGES];
    uint64_t k_empty[MAX_KV_STAGES];   // S_j has read K_j
    uint64_t v_full[MAX_KV_STAGES];
    uint64_t v_empty[MAX_KV_STAGES];   // O += P_j V_j has read V_j
    uint64_t s_ready;         // S of a pair of key tiles is complete in tensor memory
    uint64_t s_free;          // the softmax warps have read it (8 arrivals: 4 warps for each tile of the pair)
    uint64_t p_ready[2];      // P_j is in shared memory and O has been corrected
    uint64_t pv_done[2];      // O += P_j V_j has completed
    uint64_t merge_full;      // rank 0 of a pair: rank 1's partial result has arrived (bytes)
    uint32_t tmem_base;
    uint32_t failed;
};

__device__ __forceinline__ bool has_failed(Barriers* b) { return *reinterpret_cast<volatile uint32_t*>(&b->failed) != 0; }

// HD: head size, 64, 128 or 256 (the operands are walked in blocks of 64 head elements = 128 bytes)
// FIXED: softcap with a fixed reference, both softmax groups at work (see the head of this file); else the running
// maximum, warps 2..5 only.
template <int HD, bool FIXED>
__global__ void __launch_bounds__(THREADS)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            bf16* __restrict__ out, size_t out_stride, const int* __restrict__ seq_row0,
                            const int* __restrict__ seq_len, const int* __restrict__ seq_q0, int nq, int nkv,
                            float scale, float cap, int window, int* __restrict__ status, int split_levels) {
    constexpr int KS = k_stages(HD), VS = v_stages(HD);
    constexpr int Q_BYTES = BM * HD * 2;                             // HD / 64 blocks of [128 x 64]
    constexpr int KP_BYTES = 2 * BN * HD * 2;                        // a pair of key tiles: HD / 64 blocks of [128 x 64]
    constexpr int V_BYTES = BN * HD * 2;                             // HD / 64 blocks of [64 x 64]
    constexpr int MERGE_O_BYTES = BM * HD * 4;                       // O of rank 1 of a pair, float32
    constexpr int Q_COL = O_COL + HD;                                // Q: HD / 2 columns (two bfloat16 each)
    constexpr int TMEM_COLS = HD > 64 ? 512 : 256;                   // 128 for S, HD for O, HD / 2 for Q; a power of two
    constexpr int CPR = HD / 8;                                      // 16-byte chunks of a bfloat16 output row
    static_assert(HD == 64 || HD == 128 || HD == 256, "head sizes 64, 128, 256");
    static_assert(KS >= 2 && Q_BYTES == KP_BYTES, "Q is staged in the second stage of the K ring");
    static_assert(MERGE_O_BYTES <= KS * KP_BYTES && MERGE_ML_BYTES <= 2 * P_BYTES, "the pair's hand-over fits");
    static_assert(BM * HD * 2 <= VS * V_BYTES, "the output is staged in the V ring");
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sK = smem;                                       // [KS] pairs of key tiles
    unsigned char* sV = sK + KS * KP_BYTES;                         // [VS] value tiles
    unsigned char* sP = sV + VS * V_BYTES;                          // [2][P]
    unsigned char* sQ = sK + KP_BYTES;                              // Q on its way to tensor memory: K stage 1, before its first use
    unsigned char* sOut = sV;                                       // the output rows, once every product is done
    Barriers* bars = reinterpret_cast<Barriers*>(sP + 2 * P_BYTES);

    // grid (heads [x 2 ranks], sequences, query tiles): the query tile is the slowest index, so that CTAs are
    // handed out from the heaviest tiles of all heads down to the lightest
    const int b = blockIdx.y, h = split_levels ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int len = seq_len[b];
    const int ntiles_q = (len + BM - 1) / BM;
    const int qx = (int)blockIdx.z;
    if (qx >= ntiles_q) return;                                      // before any barrier or tensor memory
    // split_levels > 0: the grid is clusters of two, blockIdx.x = 2 * head + rank.  The heaviest query tiles of a
    // sequence (the split_levels last ones) are shared by the pair; of every other tile rank 0 walks all keys and
    // rank 1 leaves at once (both CTAs of a pair agree on this, and an unshared tile uses nothing of the cluster).
    const bool split = qx < split_levels;
    if (split_levels && !split && (blockIdx.x & 1)) return;
    const int rank = split ? (int)(blockIdx.x & 1) : 0, stride = split ? 2 : 1;
    const int qt = ntiles_q - 1 - qx;                                // the longest rows first
    // seq_q0: the first rows of a sequence may be there for their keys and values only (a sequence that goes on from
    // cached tokens); query tiles that end before row seq_q0[b] are left out (both CTAs of a pair agree on this)
    if (seq_q0 != nullptr && (qt + 1) * BM <= seq_q0[b]) return;
    const int r0 = qt * BM, row0 = seq_row0[b];
    const int kh = h / (nq / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int last_row = min(r0 + BM, len) - 1;
    const int kv_lo = (window > 0 && r0 - window + 1 > 0) ? r0 - window + 1 : 0;
    // Keys are walked in pairs of 64-key tiles (S of a pair is one product of N = 128): pairs kv_lo / 128 ..
    // last_row / 128 of the query tile, of which this CTA takes jp0, jp0 + stride, ...  Local tile j is half j & 1 of
    // local pair j >> 1; a half outside the row range (the first pair's lower half under a window) is masked out
    // like any other key that a row does not see.
    const int jp1 = last_row / (2 * BN);
    const int jp0 = kv_lo / (2 * BN) + rank;
    const int np = jp1 >= jp0 ? (jp1 - jp0) / stride + 1 : 0;        // (none for rank 1 when there is a single pair)
    const int nt = 2 * np;

    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars->q_full), 1);
        mbar_init(smem_u32(&bars->q_tmem), 4);                       // one arrival per warp of the first softmax group
        for (int s = 0; s < KS; ++s) {
            mbar_init(smem_u32(&bars->k_full[s]), 1);
            mbar_init(smem_u32(&bars->k_empty[s]), 1);
        }
        for (int s = 0; s < VS; ++s) {
            mbar_init(smem_u32(&bars->v_full[s]), 1);
            mbar_init(smem_u32(&bars->v_empty[s]), 1);
        }
        mbar_init(smem_u32(&bars->s_ready), 1);
        mbar_init(smem_u32(&bars->s_free), 8);                       // one arrival per softmax warp and tile of the pair
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&bars->p_ready[i]), 4);               // one arrival per softmax warp
            mbar_init(smem_u32(&bars->pv_done[i]), 1);
        }
        mbar_init(smem_u32(&bars->merge_full), 1);
        if (split && rank == 0) mbar_expect_tx(smem_u32(&bars->merge_full), MERGE_O_BYTES + MERGE_ML_BYTES);
        bars->failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = bars->tmem_base;
    // Barriers and tensor memory are set up; only now wait for the kernel before this one, whose output the
    // loads below read (seq_row0 and seq_len, read above, come from the host before the step).
    pdl_wait();

    // The softmax warps' view of their row (warps 2..9; thread = query row), kept past the role branches
    // for the merge of a pair and the output.
    const int quarter = warp & 3;
    const int group = (warp >= 6 && warp < 10) ? 1 : 0;   // softmax group (warps 2..5 / 6..9)
    const bool grp0 = warp >= 2 && warp < 6;              // the group that also merges a pair and writes the output
    const int rloc = quarter * 32 + lane;                 // row within the tile = tensor-memory lane
    const int row = r0 + rloc;                            // position in the sequence
    const unsigned lane_base = tmem + ((unsigned)(quarter * 32) << 16);
    const float LOG2E = 1.4426950408889634f;
    const float k1 = cap > 0.f ? scale / cap : scale;
    const float k2 = (cap > 0.f ? cap : 1.f) * LOG2E;
    const float step = RESCALE_STEP / (cap > 0.f ? cap : 1.f);   // a growth of the maximum by 8 in the exponent
    float m_used = 0.f, l_sum = 0.f;                      // reference maximum of the exponentials, their sum
    bool alive = true;
    const int kx = (nq + kh) * HD, vx = (nq + nkv + kh) * HD;     // columns of K and V in the qkv rows

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer of Q and K --------------------------------------------------------------------
            // K of a pair of tiles is one operand of 128 rows; its stage is free again as soon as S of the pair has
            // been formed.  (The boxes of 128 rows x 64 columns are those of Q: the same tensor map.)
            const unsigned qf = smem_u32(&bars->q_full);
            mbar_expect_tx(qf, Q_BYTES);
            for (int d = 0; d < HD / 64; ++d)
                tma_load_2d(smem_u32(sQ + d * (BM * 128)), &map_q, qf, h * HD + d * 64, row0 + r0);
            for (int J = 0; J < np; ++J) {
                const int s = J % KS;
                if (J >= KS && !mbar_wait(smem_u32(&bars->k_empty[s]), ((J / KS) - 1) & 1)) {
                    atomicOr(status, 16);
                    bars->failed = 1;
                    break;
                }
                if (J == 1 && !mbar_wait(smem_u32(&bars->q_tmem), 0)) {      // stage 1 held Q until now
                    atomicOr(status, 32);
                    bars->failed = 1;
                    break;
                }
                const unsigned kfull = smem_u32(&bars->k_full[s]);
                unsigned char* kdst = sK + s * KP_BYTES;
                mbar_expect_tx(kfull, KP_BYTES);
                for (int d = 0; d < HD / 64; ++d)
                    tma_load_2d(smem_u32(kdst + d * (2 * BN * 128)), &map_q, kfull, kx + d * 64, row0 + (jp0 + J * stride) * 2 * BN);
            }
        }
    } else if (warp == 10) {
        if (lane == 0) {
            // ---- producer of V: a stage is free only after O += P_j V_j ------------------------------------
            for (int j = 0; j < nt; ++j) {
                const int s = j % VS;
                if (j >= VS && !mbar_wait(smem_u32(&bars->v_empty[s]), ((j / VS) - 1) & 1)) {
                    atomicOr(status, 16);
                    bars->failed = 1;
                    break;
                }
                const unsigned vfull = smem_u32(&bars->v_full[s]);
                unsigned char* vdst = sV + s * V_BYTES;
                mbar_expect_tx(vfull, V_BYTES);
                const int y = row0 + ((jp0 + (j >> 1) * stride) * 2 + (j & 1)) * BN;
                for (int d = 0; d < HD / 64; ++d)
                    tma_load_2d(smem_u32(vdst + d * (BN * 128)), &map_kv, vfull, vx + d * 64, y);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- tensor-core issue of S ----------------------------------------------------------------
            // Issuing one tcgen05.mma occupies its thread for about 100 cycles whatever its size (measured: N = 32,
            // 64 and 128 alike, 138 at N = 256), so S is formed for two key tiles at once, 16 products of N = 128 with
            // Q from tensor memory (M 128, B = K of the pair, K-major), and P V is issued by a thread of its own.
            // Operand descriptors differ only in their address field (bits 0..13, the address in 16-byte units; every
            // operand lies below 256 KB, so adding an offset never carries out of the field): one descriptor is
            // formed once and each product adds its offset.
            const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)((2 * BN) >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
            const uint64_t k_desc0 = umma_desc(smem_u32(sK), 16, 1024);
            bool ok = np > 0;
            if (ok && !mbar_wait(smem_u32(&bars->q_tmem), 0)) { atomicOr(status, 32); bars->failed = 1; ok = false; }
            for (int J = 0; J < np && ok; ++J) {
                ok = mbar_wait(smem_u32(&bars->k_full[J % KS]), (J / KS) & 1);
                if (!ok) { atomicOr(status, 2); bars->failed = 1; break; }
                // the S columns are free once the softmax warps have taken the pair before into their registers
                if (J >= 1 && !mbar_wait(smem_u32(&bars->s_free), (J - 1) & 1)) { atomicOr(status, 8); bars->failed = 1; break; }
                if (has_failed(bars)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t k_desc = k_desc0 + (uint64_t)(((J % KS) * KP_BYTES) >> 4);
#pragma unroll
                for (int d = 0; d < HD / 64; ++d)
#pragma unroll
                    for (int k = 0; k < 64 / UMMA_K; ++k)
                        umma_bf16_a_tmem(tmem + S_COL, tmem + Q_COL + d * 32 + k * (UMMA_K / 2),
                                         k_desc + (uint64_t)((d * (2 * BN * 128) + k * 32) >> 4), idesc_s, (d > 0 || k > 0) ? 1u : 0u);
                umma_commit(smem_u32(&bars->k_empty[J % KS]));
                umma_commit(smem_u32(&bars->s_ready));
            }
        }
    } else if (warp == 11) {
        if (lane == 0) {
            // ---- tensor-core issue of O += P_j V_j: M 128, N hd, A (P) K-major, B (V) MN-major -----------------
            const unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(HD >> 3) << 17) | ((unsigned)(BM >> 4) << 24);
            const uint64_t v_desc0 = umma_desc(smem_u32(sV), BN * 128, 1024);
            const uint64_t p_desc0 = umma_desc(smem_u32(sP), 16, 1024);
            bool ok = true;
            for (int j = 0; j < nt && ok; ++j) {
                ok = mbar_wait(smem_u32(&bars->p_ready[j & 1]), (j >> 1) & 1);
                if (!ok) { atomicOr(status, 8); bars->failed = 1; break; }
                if (has_failed(bars)) break;
                ok = mbar_wait(smem_u32(&bars->v_full[j % VS]), (j / VS) & 1);
                if (!ok) { atomicOr(status, 2); bars->failed = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t v_desc = v_desc0 + (uint64_t)(((j % VS) * V_BYTES) >> 4);
                const uint64_t p_desc = p_desc0 + (uint64_t)(((j & 1) * P_BYTES) >> 4);
#pragma unroll
                for (int k = 0; k < BN / UMMA_K; ++k)
                    // P: 16 keys further = 32 bytes in the swizzled row.  V (keys x dims, dims contiguous):
                    // 16 keys further = 16 rows of 128 bytes; the 64-dim blocks are BN*128 bytes apart.
                    umma_bf16(tmem + O_COL, p_desc + (uint64_t)((k * 32) >> 4), v_desc + (uint64_t)((k * UMMA_K * 128) >> 4),
                              idesc_o, (j > 0 || k > 0) ? 1u : 0u);
                umma_commit(smem_u32(&bars->v_empty[j % VS]));
                umma_commit(smem_u32(&bars->pv_done[j & 1]));
            }
        }
    } else {
        // ---- softmax: thread = query row ---------------------------------------------------------------
        // First, Q moves from shared to tensor memory, where S = Q K^T reads it as its A operand: 16 products per key
        // tile no longer read 64 KB of Q from shared memory, whose bandwidth (with K, V, P and the TMA writes about
        // 224 KB per tile) and not the tensor cores set the pace.  Thread = row; a row's 16-byte chunks are swizzled
        // within each 64-column block, and eight of them fill 32 columns.
        if (group == 0) {
            if (!mbar_wait_warp(smem_u32(&bars->q_full), 0)) {
                atomicOr(status, 32);
                bars->failed = 1;
                alive = false;
            }
#pragma unroll 1
            for (int d = 0; d < HD / 64; ++d) {
                uint32_t v[32];
                const unsigned char* qrow = sQ + d * (BM * 128) + rloc * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 w = *reinterpret_cast<const uint4*>(qrow + ((c ^ (rloc & 7)) << 4));
                    v[c * 4 + 0] = w.x; v[c * 4 + 1] = w.y; v[c * 4 + 2] = w.z; v[c * 4 + 3] = w.w;
                }
                tmem_st32(lane_base + Q_COL + d * 32, v);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->q_tmem));
        }
        float m_run = -CUDART_INF_F;
        // the keys this row sees: key_lo .. key_hi (none when the row lies beyond the sequence)
        const int key_hi = min(row, len - 1);
        const int key_lo = (window > 0 && row - window + 1 > 0) ? row - window + 1 : 0;
        const unsigned key_span = key_hi >= key_lo ? (unsigned)(key_hi - key_lo) : 0u;
        // FIXED: this group's tiles are group, group + 2, ...; else group 0 takes them all and group 1 none
        for (int j = FIXED ? group : (group == 0 ? 0 : nt); j < nt && alive; j += FIXED ? 2 : 1) {
            const int bsel = j & 1;                      // half of the pair = S columns = P buffer
            if (!mbar_wait_warp(smem_u32(&bars->s_ready), (j >> 1) & 1)) {
                atomicOr(status, 4);
                bars->failed = 1;
                alive = false;
                break;
            }
            if (__any_sync(0xffffffffu, has_failed(bars))) { alive = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float s[BN];
            {
                uint32_t v0[32], v1[32];
                tmem_ld32(lane_base + S_COL + bsel * BN, v0);
                tmem_ld32(lane_base + S_COL + bsel * BN + 32, v1);
                tmem_ld_wait();
                // the scores are in registers: the S columns may take the next pair
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars->s_free));
#pragma unroll
                for (int c = 0; c < 32; ++c) s[c] = __uint_as_float(v0[c]);
#pragma unroll
                for (int c = 0; c < 32; ++c) s[32 + c] = __uint_as_float(v1[c]);
            }
            // Scores in the unit the maximum is tracked in: tanh(score / cap) with a softcap (the clamp of
            // its argument to +-20 changes nothing: tanh.approx saturates), the scaled score without;
            // either times k2 is the exponent to base 2.  Tiles wholly inside every row's range of keys
            // skip the mask.
            const int col0 = ((jp0 + (j >> 1) * stride) * 2 + bsel) * BN;
            const bool interior = col0 + BN - 1 <= r0 && col0 + BN - 1 < len && (window <= 0 || col0 > r0 + BM - 1 - window);
            float corr = 1.f;
            bool rescale = false;
            if (FIXED) {
                // exp(capped score) against the reference 0: k2 = cap log2(e), the exponent stays within +-k2
                float rs4[4] = {0.f, 0.f, 0.f, 0.f};
                if (interior) {
#pragma unroll
                    for (int c = 0; c < BN; ++c) {
                        const float e = tanh_fast(s[c] * k1) * k2;
                        const float pv = (c & 7) < POLY ? exp2_poly(e) : exp2_fast(e);
                        s[c] = pv;
                        rs4[c & 3] += pv;
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < BN; ++c) {
                        const bool seen = (unsigned)(col0 + c - key_lo) <= key_span;      // key_lo <= column <= key_hi
                        const float e = tanh_fast(s[c] * k1) * k2;
                        const float pv = seen ? ((c & 7) < POLY ? exp2_poly(e) : exp2_fast(e)) : 0.f;
                        s[c] = pv;
                        rs4[c & 3] += pv;
                    }
                }
                l_sum += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
            } else {
            float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
            if (interior) {
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    const float x = cap > 0.f ? tanh_fast(s[c] * k1) : s[c] * k1;
                    s[c] = x;
                    mx4[c & 3] = fmaxf(mx4[c & 3], x);
                }
            } else {
#pragma unroll
                for (int c = 0; c < BN; ++c) {
                    float x = cap > 0.f ? tanh_fast(s[c] * k1) : s[c] * k1;
                    const bool seen = (unsigned)(col0 + c - key_lo) <= key_span;      // key_lo <= column <= key_hi
                    x = seen ? x : -CUDART_INF_F;
                    s[c] = x;
                    mx4[c & 3] = fmaxf(mx4[c & 3], x);
                }
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            m_run = fmaxf(m_run, mx);
            if (m_run != -CUDART_INF_F && (j == 0 || m_run > m_used + step || l_sum == 0.f)) {
                // take the exponentials against the new maximum from here on
                corr = (l_sum == 0.f) ? 0.f : exp2_fast((m_used - m_run) * k2);
                rescale = (j > 0);
                m_used = m_run;
            }
            const float moff = m_used * k2;
            float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < BN; ++c) {
                const float p = exp2_fast(fmaf(s[c], k2, -moff));         // exp(-inf) = 0 for masked keys
                s[c] = p;
                rs4[c & 3] += p;
            }
            const float rs = (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
            l_sum = l_sum * corr + rs;
            }
            // P_j overwrites the buffer that P_{j-2} V_{j-2} read: that product (issued by another thread than S, so
            // s_ready says nothing about it) has to be done.  Whoever writes P_j has seen every earlier phase of this
            // barrier, tile by tile.  (O may only be touched once P_{j-1} V_{j-1} is done: see the rescale below.)
            if (j >= 2 && !mbar_wait_warp(smem_u32(&bars->pv_done[bsel]), ((j - 2) >> 1) & 1)) {
                atomicOr(status, 64);
                bars->failed = 1;
                alive = false;
                break;
            }
            {
                unsigned char* prow = sP + bsel * P_BYTES + rloc * 128;
#pragma unroll
                for (int ch = 0; ch < BN / 8; ++ch) {
                    uint4 pk;
                    pk.x = pack_bf16(s[ch * 8 + 0], s[ch * 8 + 1]);
                    pk.y = pack_bf16(s[ch * 8 + 2], s[ch * 8 + 3]);
                    pk.z = pack_bf16(s[ch * 8 + 4], s[ch * 8 + 5]);
                    pk.w = pack_bf16(s[ch * 8 + 6], s[ch * 8 + 7]);
                    *reinterpret_cast<uint4*>(prow + ((ch ^ (rloc & 7)) << 4)) = pk;
                }
            }
            if (!FIXED && __any_sync(0xffffffffu, rescale)) {
                if (j >= 1 && !mbar_wait_warp(smem_u32(&bars->pv_done[(j - 1) & 1]), ((j - 1) >> 1) & 1)) {
                    atomicOr(status, 64);
                    bars->failed = 1;
                    alive = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const float f = rescale ? corr : 1.f;
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t v[32];
                    tmem_ld32(lane_base + O_COL + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * f);
                    tmem_st32(lane_base + O_COL + c0, v);
                }
            }
            // make P (generic-proxy writes) visible to the tensor core's reads, then hand over
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars->p_ready[bsel]));
        }
        // the last product, then O / l -> bfloat16 -> global
        // A waiter may only ask for a barrier's phase when it knows the phase before it to be over (a parity says
        // nothing about a phase that has not begun).  A group knows that of the barrier of its own tiles: S_j was
        // committed behind P_{j-2} V_{j-2}.  So each group waits for its own last product first; the products are
        // done in order, so after that the one before the very last is over too, and the very last may be asked for.
        if (alive && nt > 0) {
            const int jl = nt - 1;
            const int jmine = (FIXED && (jl & 1) != group) ? jl - 1 : jl;
            if (jmine >= 0 && jmine != jl && !mbar_wait_warp(smem_u32(&bars->pv_done[jmine & 1]), (jmine >> 1) & 1)) {
                atomicOr(status, 64);
                bars->failed = 1;
                alive = false;
            }
            if (alive && !mbar_wait_warp(smem_u32(&bars->pv_done[jl & 1]), (jl >> 1) & 1)) {
                atomicOr(status, 64);
                bars->failed = 1;
                alive = false;
            }
        }
        if (FIXED) {
            // a row's sum is the sum of its two groups' sums (both against the reference 0); the second group
            // leaves its own at the end of the P buffers, which no product reads any more
            float* l_second = reinterpret_cast<float*>(sP + 2 * P_BYTES - BM * 4);
            if (group == 1) l_second[rloc] = alive ? l_sum : 0.f;
            asm volatile("bar.sync 2, 256;" ::: "memory");       // the eight softmax warps
            if (group == 0) l_sum += l_second[rloc];
            if (__any_sync(0xffffffffu, has_failed(bars))) alive = false;
        }
    }

    // ---- a pair's second half hands its result to the first ---------------------------------------------
    // Rank 1 lays its O (float32, row by row, the 16-byte chunks XOR-ed with the row number) over its own
    // K/V stages and (reference maximum, sum) over its P buffer, and the copy engine moves both to the same
    // places in rank 0, whose operands no product reads any more (first cluster barrier).  Rank 0 waits for
    // the bytes on an mbarrier; the second cluster barrier keeps rank 1 alive until they have been read out
    // of its memory.
    float m_other = 0.f, l_other = 0.f;
    if (split) {
        if (grp0 && rank == 1) {
            const bool have = alive && nt > 0 && !has_failed(bars);
            if (have) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned char* orow = sK + rloc * (HD * 4);
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t v[32];
                if (have) {
                    tmem_ld32(lane_base + O_COL + c0, v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] = 0u;
                }
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4)
                    *reinterpret_cast<uint4*>(orow + ((((c0 >> 2) + c4) ^ (rloc & 7)) << 4)) =
                        make_uint4(v[c4 * 4], v[c4 * 4 + 1], v[c4 * 4 + 2], v[c4 * 4 + 3]);
            }
            *reinterpret_cast<float2*>(sP + rloc * 8) = make_float2(m_used, have ? l_sum : 0.f);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // visible to the copy engine
        }
        __syncthreads();
        cluster_barrier();                  // both CTAs are past their last product; rank 1's part is laid out
        if (rank == 1 && threadIdx.x == 64) {
            bulk_copy_to_rank(smem_u32(sK), smem_u32(sK), MERGE_O_BYTES, smem_u32(&bars->merge_full), 0);    // to the same place in rank 0
            bulk_copy_to_rank(smem_u32(sP), smem_u32(sP), MERGE_ML_BYTES, smem_u32(&bars->merge_full), 0);
        }
        if (grp0 && rank == 0) {
            if (!mbar_wait_warp(smem_u32(&bars->merge_full), 0)) {
                atomicOr(status, 128);
                bars->failed = 1;
                alive = false;
            } else {
                const float2 ml = *reinterpret_cast<const float2*>(sP + rloc * 8);
                m_other = ml.x;
                l_other = ml.y;
            }
        }
        __syncthreads();
        cluster_barrier();                  // the bytes have left rank 1's memory: it may go
    }

    if (grp0 && rank == 0) {
        // Every product is done, so the Q tile's shared memory is free: each thread leaves its row there as
        // bfloat16 (16-byte chunks XOR-ed with the row number, so that neither side conflicts), and the
        // warps then write whole rows of the head to global memory.
        const bool good = alive && !__any_sync(0xffffffffu, has_failed(bars));
        if (good) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // weights of the two halves against the larger reference maximum (a half without keys has sum 0)
            const bool have0 = l_sum > 0.f, have1 = l_other > 0.f;
            const float mm = fmaxf(have0 ? m_used : -CUDART_INF_F, have1 ? m_other : -CUDART_INF_F);
            const float w0 = have0 ? exp2_fast((m_used - mm) * k2) : 0.f;
            const float w1 = have1 ? exp2_fast((m_other - mm) * k2) : 0.f;
            const float l_row = l_sum * w0 + l_other * w1;
            const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
            const float f0 = w0 * inv, f1 = w1 * inv;
            unsigned char* orow = sOut + rloc * (HD * 2);
            const unsigned char* prow = sK + rloc * (HD * 4);
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 64) {
                uint32_t v0[32], v1[32];
                tmem_ld32(lane_base + O_COL + c0, v0);
                tmem_ld32(lane_base + O_COL + c0 + 32, v1);
                tmem_ld_wait();
                float o0[32], o1[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    o0[c] = __uint_as_float(v0[c]) * f0;
                    o1[c] = __uint_as_float(v1[c]) * f0;
                }
                if (have1) {
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const float4 a = *reinterpret_cast<const float4*>(prow + ((((c0 >> 2) + c4) ^ (rloc & 7)) << 4));
                        const float4 b = *reinterpret_cast<const float4*>(prow + ((((c0 >> 2) + 8 + c4) ^ (rloc & 7)) << 4));
                        o0[c4 * 4 + 0] += a.x * f1; o0[c4 * 4 + 1] += a.y * f1; o0[c4 * 4 + 2] += a.z * f1; o0[c4 * 4 + 3] += a.w * f1;
                        o1[c4 * 4 + 0] += b.x * f1; o1[c4 * 4 + 1] += b.y * f1; o1[c4 * 4 + 2] += b.z * f1; o1[c4 * 4 + 3] += b.w * f1;
                    }
                }
#pragma unroll
                for (int c8 = 0; c8 < 4; ++c8) {
                    uint4 pk;
                    pk.x = pack_bf16(o0[c8 * 8 + 0], o0[c8 * 8 + 1]);
                    pk.y = pack_bf16(o0[c8 * 8 + 2], o0[c8 * 8 + 3]);
                    pk.z = pack_bf16(o0[c8 * 8 + 4], o0[c8 * 8 + 5]);
                    pk.w = pack_bf16(o0[c8 * 8 + 6], o0[c8 * 8 + 7]);
                    *reinterpret_cast<uint4*>(orow + (((c0 / 8 + c8) ^ (rloc & (CPR - 1))) << 4)) = pk;
                    pk.x = pack_bf16(o1[c8 * 8 + 0], o1[c8 * 8 + 1]);
                    pk.y = pack_bf16(o1[c8 * 8 + 2], o1[c8 * 8 + 3]);
                    pk.z = pack_bf16(o1[c8 * 8 + 4], o1[c8 * 8 + 5]);
                    pk.w = pack_bf16(o1[c8 * 8 + 6], o1[c8 * 8 + 7]);
                    *reinterpret_cast<uint4*>(orow + (((c0 / 8 + 4 + c8) ^ (rloc & (CPR - 1))) << 4)) = pk;
                }
            }
        }
        __syncwarp();      // a warp stores the 32 rows that its own lanes wrote
        if (good) {
            constexpr int RPI = 32 / CPR;                        // rows that one warp-wide store covers
            for (int rr = 0; rr < 32; rr += RPI) {
                const int rl = quarter * 32 + rr + lane / CPR, pos = lane % CPR;
                if (r0 + rl >= len) continue;
                const uint4 pk = *reinterpret_cast<const uint4*>(sOut + rl * (HD * 2) + (pos << 4));
                bf16* dst = out + (size_t)(row0 + r0 + rl) * out_stride + (size_t)h * HD + ((pos ^ (rl & (CPR - 1))) << 3);
                *reinterpret_cast<uint4*>(dst) = pk;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}



template <int HD, bool FIXED>
int launch_attn(const void* qkv, long long total_rows, void* out, long long out_stride, const int* seq_row0,
                const int* seq_len, const int* seq_q0, int B, int max_len, int nq, int nkv, float scale, float cap,
                int window, int* status, cudaStream_t st) {
    const long long width = (long long)(nq + 2 * nkv) * HD;
    CUtensorMap map_q, map_kv;
    int rc = make_map(&map_q, qkv, total_rows, width, BM);
    if (rc) return rc;
    rc = make_map(&map_kv, qkv, total_rows, width, BN);
    if (rc) return rc;
    const size_t smem = (size_t)k_stages(HD) * 2 * BN * HD * 2 + (size_t)v_stages(HD) * BN * HD * 2 + 2 * P_BYTES + sizeof(Barriers) + 1024;
    auto kern = attn_prefill_tcgen05_kernel<HD, FIXED>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int ntq = (max_len + BM - 1) / BM;
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count <= 0)
            sm_count = 148;
    }
    // Few CTAs with long key walks: pairs of CTAs share a query tile's keys (see the head of this file).  A pair
    // pays for the cluster launch and the hand-over; the policy and its measurements are below.
    static int split_ok = -1;                      // the device holds a pair of these CTAs (asked once)
    const long long singles = (long long)ntq * B * nq;
    const int reach = window > 0 ? (max_len < window + BM - 1 ? max_len : window + BM - 1) : max_len;
    const int key_tiles = (reach + BN - 1) / BN;   // of the heaviest query tile
    static int no_split = -1;                       // QNN_ATTN_NO_SPLIT, read once
    if (no_split < 0) no_split = getenv("QNN_ATTN_NO_SPLIT") ? 1 : 0;
    // How many of the heaviest query tiles (counted from a sequence's last) are shared by pairs: all of them, when
    // both CTAs of every pair fit the device at once and the heaviest tile walks at least 12 key tiles; else none.
    // Measured inside a CUDA graph, head size 256, one prompt, pairs against single CTAs: 4 heads, 2048 tokens 28.6 /
    // 36.0 us; 2 heads, 2048 tokens 27.6 / 36.0; 4 heads, 1024 tokens 20.3 / 21.4.  With 8 heads and 2048 tokens (128
    // tiles on 148 SMs) pairs for every tile need a second round of CTAs (41.0 us), pairs for the two heaviest levels
    // only, so that everything still starts together, took 41.7 us, single CTAs 37.7 us: the cluster launch and the
    // hand-over cost more than the shorter key walk saves, so such a grid runs single CTAs.
    int levels = 0;
    if (ntq >= 2 && !no_split && 2 * singles <= sm_count && key_tiles >= 12) levels = ntq;
    const bool want_split = levels > 0;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    if (want_split && split_ok < 0) {
        cfg.gridDim = dim3(2, 1, 1);
        cfg.attrs = attr + 1;
        cfg.numAttrs = 1;
        int n = 0;
        split_ok = (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) ? 1 : 0;
        if (!split_ok) (void)cudaGetLastError();
        cfg.attrs = attr;
    }
    const int split = (want_split && split_ok == 1) ? levels : 0;
    cfg.gridDim = dim3((unsigned)(split ? 2 * nq : nq), B, ntq);
    const long long ctas = (long long)cfg.gridDim.x * B * ntq;
    const bool pdl = qnn::pdl_enabled() && ctas <= qnn::pdl_max_grid();
    if (split) {
        if (!pdl) cfg.attrs = attr + 1;
        cfg.numAttrs = pdl ? 2 : 1;
    } else {
        cfg.numAttrs = pdl ? 1 : 0;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, map_q, map_kv, (bf16*)out, (size_t)out_stride, seq_row0, seq_len, seq_q0, nq,
                                       nkv, scale, cap, window, status, split);
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

}  // namespace

// qkv: this step's projections, [T rows, (nq + 2 nkv) * hd] bfloat16, rotated; sequence b occupies rows
// seq_row0[b] .. + seq_len[b] - 1.  seq_q0 (may be null): row seq_q0[b] of sequence b is the first whose output is
// wanted; the rows before it bring keys and values only (qnn_attn_extend_gather lays cached tokens out that way) and
// their output rows hold nothing of use.  Head sizes 64, 128 and 256; QNN_ERR_UNSUPPORTED for others.  `status` as in
// qnn_gemm_tcgen05 (bits: 2 K/V wait, 4 S wait, 8 P wait, 16 ring wait, 32 Q wait, 64 product wait, 128 wait for
// the other half of a pair).  seq_row0 and seq_len are read before the kernel waits for the kernel launched
// in front of it on the stream: that kernel must not be the one that writes them (copies from the host and
// kernels further back are complete by then).
QNN_API int qnn_attn_prefill_tcgen05(const void* qkv, long long total_rows, void* out, long long out_stride,
                                     const int* seq_row0, const int* seq_len, const int* seq_q0, int B, int max_len,
                                     int nq, int nkv, int hd, float scale, float cap, int window, int* status,
                                     cudaStream_t st) {
    if (B <= 0 || max_len <= 0) return 0;
    if (hd != 64 && hd != 128 && hd != 256) return QNN_ERR_UNSUPPORTED;
    if (nkv <= 0 || nq % nkv) return QNN_ERR_ARGUMENT;
    if (B > 65535 || nq > 32767 || (max_len + BM - 1) / BM > 65535) return QNN_ERR_UNSUPPORTED;
    if (((uintptr_t)qkv & 15) || ((uintptr_t)out & 15) || (out_stride * 2) % 16) return QNN_ERR_UNSUPPORTED;
#define QNN_ATTN_ARGS qkv, total_rows, out, out_stride, seq_row0, seq_len, seq_q0, B, max_len, nq, nkv, scale, cap, window, status, st
    // With a softcap up to 70 the exponent cap * log2(e) stays below 101, so that neither exp(score) nor a row's
    // sum over a million keys leaves float32: the fixed-reference softmax with both groups of warps.  QNN_ATTN_FIXED=0
    // keeps the running maximum (for comparisons).
    static int fixed_ok = -1;
    if (fixed_ok < 0) {
        const char* e = getenv("QNN_ATTN_FIXED");
        fixed_ok = (e && e[0] == '0') ? 0 : 1;
    }
    const bool fixed = fixed_ok && cap > 0.f && cap <= 70.f;
    switch (hd) {
        case 64: return fixed ? launch_attn<64, true>(QNN_ATTN_ARGS) : launch_attn<64, false>(QNN_ATTN_ARGS);
        case 128: return fixed ? launch_attn<128, true>(QNN_ATTN_ARGS) : launch_attn<128, false>(QNN_ATTN_ARGS);
        default: return fixed ? launch_attn<256, true>(QNN_ATTN_ARGS) : launch_attn<256, false>(QNN_ATTN_ARGS);
    }
#undef QNN_ATTN_ARGS
}

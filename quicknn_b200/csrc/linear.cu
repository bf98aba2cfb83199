// Matrix products y[M,N] = x[M,K] * W[N,K]^T (weights stored [out, in], no bias), with
// the epilogues that follow them in the model.
//
// Reference: `Project` picks a matvec shader for one row and a tiled GEMM otherwise
// (src/models/QuickNN.Models.Gemma2.pas:142-148); matvec = 8 rows x 32 lanes x 4-wide
// bf16 loads with a shared-memory tree (shaders/tensor.comp:87-107), GEMM = 64x64 tile of
// fp32 FMA (shaders/gemm.comp:4-6).  GeGLU and the final softcap are separate dispatches
// there (Gemma2.pas:186,195); here they are epilogues.
//
//   qnn_skinny_bf16 : M <= 64 rows of bf16 activations against bf16 weights on the tensor
//                     cores (mma.sync m16n8k16, fp32 accumulate): a CTA owns 16 weight rows,
//                     its 8 to 32 warps split K, weights are read once with 16-byte loads.
//   qnn_gemv_f32    : true fp32, one warp per output column, up to 8 rows at a time.
//   qnn_sgemm_f32   : true fp32 tiled GEMM (FFMA only) for whole prompts.
//
// Epilogues: 0 none; 1 softcap (float32 out); 2 gated: W = [gate; up] stacked, the CTA
// computes rows n and N/2+n and stores act(gate)*up; 3 rotate and append: W = [q; k; v]
// stacked, the CTA computes 8 columns of a head with their partners half a head away, rotates
// the pairs by the token's position and writes K and V to the paged cache as well (what
// rope_cache.cu does as a kernel of its own; reference: Gemma2.pas:167-175 runs three
// projections, two rotations and a cache write as six dispatches); 4 arg-max: softcap, then only the
// best (value, id) of the CTA's 16 output columns is stored for each row, out[row][CTA] as float2
// (the head of a greedy decode step: the logits themselves are never written; the reference takes
// the top-k of 512-wide tiles straight from the logits tensor, shaders/tensor.comp:121-155).
#include "common.cuh"
#include <float.h>

using namespace qnn;

#define EPI_NONE 0
#define EPI_SOFTCAP 1
#define EPI_GATED 2
#define EPI_ROPE 3
#define EPI_ARGMAX 4

// What the rotate-and-append epilogue needs; the meaning of each field is that of the argument
// of the same name of qnn_rope_cache_write.
struct RopeEpi {
    int nq, nkv, hd;
    const float* inv_freq;
    const int* tok_pos;
    const int* tok_slot;
    bf16* k_pool;
    bf16* v_pool;
    const int* page_table;
    int max_pages, page_size, ring;
    const int* slot_len;
    int write_cache;
};

__device__ __forceinline__ void store_out(void* out, int out_dt, size_t i, float v) { store_from_f(out, out_dt, i, v); }

// ---------------------------------------------------------------------------------
// bf16, M <= 64, tensor cores.
//
// mma.m16n8k16 computes D[16x8] += A[16x16] * B[16x8]; A = 16 weight rows, B = 8
// activation rows (transposed).  The k index inside one mma is only a summation label, so
// each thread takes its fragment from one 16-byte load of 8 consecutive k of its weight
// row (and the same 8 k of its activation row) and feeds them to two mmas: the labels of A
// and B agree, which is all the instruction needs.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg16(const bf16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
// The same load as a volatile statement: it keeps its place relative to the dependency wait.
__device__ __forceinline__ uint4 ldg16_early(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Blocks per SM that the compiler has to leave room for.  The 16-warp kernels for 9 to 16 rows took 70 to 79
// registers, so one block of 512 threads filled an SM and the 256 blocks of a q|k|v product ran in two rounds (its
// share of a decode step of 10 rows: 10.4 us, with two blocks per SM 6.3); the kernels for 17 rows and more measured
// 2 us a layer faster when told that one block per SM is enough; the others are fastest left to the compiler (an
// explicit 1 cost the 8-row step 9 %).
template <int NT, int NW>
constexpr int skinny_min_blocks() { return (NW == 16 && NT >= 2) ? 2 : (NT >= 4 ? 1 : 0); }

template <int NT, int EPI, int NW>
__global__ void __launch_bounds__(NW * 32, skinny_min_blocks<NT, NW>()) skinny_bf16_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W,
                                                          void* __restrict__ out, int out_dt, int M, int N, int K,
                                                          float cap, int act, const RopeEpi rp, int* __restrict__ err) {
    constexpr int COLS = NT * 8;
    constexpr int THREADS = NW * 32;
    __shared__ float red[NW][16][COLS + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int Nout = (EPI == EPI_GATED) ? N / 2 : N;
    const int n0 = blockIdx.x * 16;
    int r0 = min(n0 + g, Nout - 1), r1 = min(n0 + g + 8, Nout - 1);
    // rotate and append: fragment rows 0-7 are columns j0..j0+7 of a head, rows 8-15 their partners
    int rope_base0 = 0, rope_base1 = 0, rope_blocks = 0;
    if constexpr (EPI == EPI_ROPE) {
        const int per = rp.hd / 16;
        rope_blocks = (rp.nq + rp.nkv) * per;
        if ((int)blockIdx.x < rope_blocks) {
            rope_base0 = ((int)blockIdx.x / per) * rp.hd + ((int)blockIdx.x % per) * 8;
            rope_base1 = rope_base0 + rp.hd / 2;
        } else {
            rope_base0 = (rp.nq + rp.nkv) * rp.hd + ((int)blockIdx.x - rope_blocks) * 16;
            rope_base1 = rope_base0 + 8;
        }
        r0 = rope_base0 + g;
        r1 = rope_base1 + g;
    }
    const int nchunks = K / 8;
    const int nkb = (nchunks + 3) / 4;
    const uint4 zero4 = make_uint4(0, 0, 0, 0);

    float acc[NT][4];
    float accu[(EPI == EPI_GATED) ? NT : 1][4];
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    if (EPI == EPI_GATED) {
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) accu[i][j] = 0.f;
    }

    const bf16* w0 = W + (size_t)r0 * K;
    const bf16* w1 = W + (size_t)r1 * K;
    const bf16* u0 = W + (size_t)(Nout + r0) * K;
    const bf16* u1 = W + (size_t)(Nout + r1) * K;

    // The weights do not depend on the kernel before this one, the activations do.  So each thread
    // takes its first PRE blocks of weights into registers, and asks for the rest of a small
    // matrix to be brought to L2, before it waits for that kernel: launched while the (short,
    // bandwidth-idle) kernel before it still runs, this kernel has most of its weight traffic
    // behind it when its activations arrive.  For the big matrices the L2 requests would only fill
    // the load queue.  The loads are volatile asm so that they stay in front of the wait.
    constexpr int PRE = (EPI == EPI_GATED) ? 1 : 4;
    uint4 pa_lo[PRE], pa_hi[PRE], pg_lo[(EPI == EPI_GATED) ? PRE : 1], pg_hi[(EPI == EPI_GATED) ? PRE : 1];
#pragma unroll
    for (int i = 0; i < PRE; ++i) {
        const int c = (warp + i * NW) * 4 + t;
        const bool valid = c < nchunks;
        const size_t ko = (size_t)c * 8;
        pa_lo[i] = valid ? ldg16_early(w0 + ko) : zero4;
        pa_hi[i] = valid ? ldg16_early(w1 + ko) : zero4;
        if (EPI == EPI_GATED) {
            pg_lo[i] = valid ? ldg16_early(u0 + ko) : zero4;
            pg_hi[i] = valid ? ldg16_early(u1 + ko) : zero4;
        }
    }
    if (t == 0 && (size_t)N * K <= ((size_t)1 << 24)) {
        for (int kb = warp + PRE * NW; kb < nkb; kb += NW) {
            const size_t ko = (size_t)kb * 32;
            if (ko < (size_t)K) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(w0 + ko));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(w1 + ko));
                if (EPI == EPI_GATED) {
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(u0 + ko));
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(u1 + ko));
                }
            }
        }
    }
    pdl_wait();

#pragma unroll
    for (int i = 0; i < PRE; ++i) {
        const int c = (warp + i * NW) * 4 + t;
        const bool valid = c < nchunks;
        const size_t ko = (size_t)c * 8;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int m = nt * 8 + g;
            uint4 b = (valid && m < M) ? ldg16(x + (size_t)m * K + ko) : zero4;
            mma_bf16_16816(acc[nt], pa_lo[i].x, pa_hi[i].x, pa_lo[i].y, pa_hi[i].y, b.x, b.y);
            mma_bf16_16816(acc[nt], pa_lo[i].z, pa_hi[i].z, pa_lo[i].w, pa_hi[i].w, b.z, b.w);
            if (EPI == EPI_GATED) {
                mma_bf16_16816(accu[nt], pg_lo[i].x, pg_hi[i].x, pg_lo[i].y, pg_hi[i].y, b.x, b.y);
                mma_bf16_16816(accu[nt], pg_lo[i].z, pg_hi[i].z, pg_lo[i].w, pg_hi[i].w, b.z, b.w);
            }
        }
    }
#pragma unroll 4
    for (int kb = warp + PRE * NW; kb < nkb; kb += NW) {
        const int c = kb * 4 + t;
        const bool valid = c < nchunks;
        const size_t ko = (size_t)c * 8;
        uint4 a_lo = valid ? ldg16(w0 + ko) : zero4;
        uint4 a_hi = valid ? ldg16(w1 + ko) : zero4;
        uint4 g_lo = zero4, g_hi = zero4;
        if (EPI == EPI_GATED) {
            g_lo = valid ? ldg16(u0 + ko) : zero4;
            g_hi = valid ? ldg16(u1 + ko) : zero4;
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int m = nt * 8 + g;
            uint4 b = (valid && m < M) ? ldg16(x + (size_t)m * K + ko) : zero4;
            mma_bf16_16816(acc[nt], a_lo.x, a_hi.x, a_lo.y, a_hi.y, b.x, b.y);
            mma_bf16_16816(acc[nt], a_lo.z, a_hi.z, a_lo.w, a_hi.w, b.z, b.w);
            if (EPI == EPI_GATED) {
                mma_bf16_16816(accu[nt], g_lo.x, g_hi.x, g_lo.y, g_hi.y, b.x, b.y);
                mma_bf16_16816(accu[nt], g_lo.z, g_hi.z, g_lo.w, g_hi.w, b.z, b.w);
            }
        }
    }

    // Sum the 8 warps' partial tiles in warp order; each thread then owns up to SLOTS
    // (row, col) pairs.  Consecutive threads take consecutive weight rows, so a row of `out`
    // is written in runs of 16 and the shared-memory reads (row stride COLS+1, odd) do not
    // conflict.
    constexpr int SLOTS = (16 * COLS + THREADS - 1) / THREADS;
    float gate_sum[SLOTS];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        red[warp][g][nt * 8 + 2 * t] = acc[nt][0];
        red[warp][g][nt * 8 + 2 * t + 1] = acc[nt][1];
        red[warp][g + 8][nt * 8 + 2 * t] = acc[nt][2];
        red[warp][g + 8][nt * 8 + 2 * t + 1] = acc[nt][3];
    }
    __syncthreads();
    if constexpr (EPI == EPI_ROPE) {
        // one thread per (pair, token): the two sums are rounded to bfloat16 first, as the product
        // without this epilogue would store them, then rotated in float32
        bf16* o = reinterpret_cast<bf16*>(out);
        const int hd = rp.hd, half = hd / 2;
        const size_t head_stride = (size_t)rp.page_size * hd;
        for (int e = threadIdx.x; e < 8 * COLS; e += THREADS) {
            const int j = e % 8, m = e / 8;
            if (m >= M) continue;
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) { s0 += red[w][j][m]; s1 += red[w][j + 8][m]; }
            const bf16 a = __float2bfloat16(s0), b = __float2bfloat16(s1);
            const int pos = rp.tok_pos[m], slot = rp.tok_slot[m];
            bool wr = rp.write_cache && slot >= 0;
            if (wr && rp.ring > 0 && pos + rp.ring < rp.slot_len[slot]) wr = false;
            size_t cache_base = 0;
            if (wr) {
                const int r = rp.ring > 0 ? pos % rp.ring : pos;
                const int page = rp.page_table[(size_t)slot * rp.max_pages + r / rp.page_size];
                cache_base = ((size_t)page * rp.nkv * rp.page_size + (r % rp.page_size)) * hd;
            }
            bf16* orow = o + (size_t)m * N;
            if ((int)blockIdx.x < rope_blocks) {
                const int h = rope_base0 / hd, d = rope_base0 % hd + j;
                float sn, cs;
                sincosf((float)pos * rp.inv_freq[d], &sn, &cs);
                const float fa = __bfloat162float(a), fb = __bfloat162float(b);
                const bf16 ra = __float2bfloat16(fa * cs - fb * sn), rb = __float2bfloat16(fa * sn + fb * cs);
                orow[h * hd + d] = ra;
                orow[h * hd + d + half] = rb;
                if (h >= rp.nq && wr) {
                    bf16* dst = rp.k_pool + cache_base + (size_t)(h - rp.nq) * head_stride;
                    dst[d] = ra;
                    dst[d + half] = rb;
                }
            } else {
                orow[rope_base0 + j] = a;
                orow[rope_base1 + j] = b;
                if (wr) {
                    const int c = rope_base0 - (rp.nq + rp.nkv) * hd + j;     // column of V; c + 8 is in the same head
                    bf16* dst = rp.v_pool + cache_base + (size_t)(c / hd) * head_stride + c % hd;
                    dst[0] = a;
                    dst[8] = b;
                }
            }
        }
    } else {
#pragma unroll
    for (int sl = 0; sl < SLOTS; ++sl) {
        const int e = threadIdx.x + sl * THREADS;
        float s = 0.f;
        if (e < 16 * COLS) {
            const int row = e % 16, col = e / 16;
#pragma unroll
            for (int w = 0; w < NW; ++w) s += red[w][row][col];
        }
        gate_sum[sl] = s;
    }
    if (EPI == EPI_GATED) {
        __syncthreads();
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            red[warp][g][nt * 8 + 2 * t] = accu[nt][0];
            red[warp][g][nt * 8 + 2 * t + 1] = accu[nt][1];
            red[warp][g + 8][nt * 8 + 2 * t] = accu[nt][2];
            red[warp][g + 8][nt * 8 + 2 * t + 1] = accu[nt][3];
        }
        __syncthreads();
    }
#pragma unroll
    for (int sl = 0; sl < SLOTS; ++sl) {
        const int e = threadIdx.x + sl * THREADS;
        if (e >= 16 * COLS) continue;
        const int row = e % 16, col = e / 16;
        const int n = n0 + row, m = col;
        float v = gate_sum[sl];
        if (EPI == EPI_GATED) {
            float u = 0.f;
#pragma unroll
            for (int w = 0; w < NW; ++w) u += red[w][row][col];
            v = activate_fast(v, act) * u;          // bfloat16 inputs and output: the fast activation
        } else if (EPI == EPI_SOFTCAP || EPI == EPI_ARGMAX) {
            v = softcap(v, cap);
        }
        if constexpr (EPI == EPI_ARGMAX) {
            // the 16 lanes of a half-warp hold the CTA's 16 columns of row m: the largest wins, the lowest
            // column on ties; NaN and Inf set the error word and lose (whole warps get here: 16 * COLS is a
            // multiple of 32)
            unsigned id = (n < Nout && m < M) ? (unsigned)n : 0xffffffffu;
            if (id != 0xffffffffu && (isnan(v) || isinf(v))) {
                if (err != nullptr) atomicOr(err, 1);
                v = -FLT_MAX;
            }
            if (id == 0xffffffffu) v = -FLT_MAX;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, v, o, 16);
                const unsigned oi = __shfl_xor_sync(0xffffffffu, id, o, 16);
                if (ov > v || (ov == v && oi < id)) { v = ov; id = oi; }
            }
            if (row == 0 && m < M)
                reinterpret_cast<float2*>(out)[(size_t)m * gridDim.x + blockIdx.x] = make_float2(v, __uint_as_float(id));
        } else {
            if (n < Nout && m < M) store_out(out, out_dt, (size_t)m * Nout + n, v);
        }
    }
    }
}

// The K range of a 16-row tile is split over the NW warps of its CTA.  Matrices with few rows
// (N/16 CTAs do not fill the GPU) get more warps per CTA, as far as K gives every warp at
// least two 32-wide blocks and the partial tiles fit in shared memory.
template <int EPI>
static int launch_skinny(const bf16* x, const bf16* W, void* out, int out_dt, int M, int N, int K, float cap, int act,
                         cudaStream_t st, const RopeEpi rp = RopeEpi(), int* err = nullptr) {
    const int Nout = (EPI == EPI_GATED) ? N / 2 : N;
    const unsigned blocks = (unsigned)((Nout + 15) / 16);
    const int nt = (M + 7) / 8;
    const int kblocks = (K + 31) / 32;
    int nw = 8;
    if (nt <= 2 && blocks * 8u < 3000u && kblocks >= 32) nw = 16;
    if (nt == 1 && blocks * 16u < 3000u && kblocks >= 64) nw = 32;
#define QNN_SK(NTV)                                                                                            \
    if (nw == 32 && NTV == 1)                                                                                  \
        qnn::launch_pdl(skinny_bf16_kernel<1, EPI, 32>, dim3(blocks), dim3(1024), 0, st, x, W, out, out_dt, M, N, K, cap, act, rp, err);         \
    else if (nw >= 16 && NTV <= 2)                                                                             \
        qnn::launch_pdl(skinny_bf16_kernel<(NTV <= 2 ? NTV : 1), EPI, 16>, dim3(blocks), dim3(512), 0, st, x, W, out, out_dt, M, N, K, cap, act, rp, err); \
    else                                                                                                       \
        qnn::launch_pdl(skinny_bf16_kernel<NTV, EPI, 8>, dim3(blocks), dim3(256), 0, st, x, W, out, out_dt, M, N, K, cap, act, rp, err);         \
    break;
    switch (nt) {
        case 1: QNN_SK(1)
        case 2: QNN_SK(2)
        case 3:
        case 4: QNN_SK(4)
        default: QNN_SK(8)
    }
#undef QNN_SK
    return (int)cudaGetLastError();
}

QNN_API int qnn_skinny_bf16(const void* x, const void* W, void* out, int out_dt, int M, int N, int K, int epi,
                            float cap, int act, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K % 8 != 0 || K <= 0) return QNN_ERR_UNSUPPORTED;
    if (epi == EPI_GATED && (N % 2)) return QNN_ERR_ARGUMENT;
    if (((uintptr_t)x | (uintptr_t)W) & 15) return QNN_ERR_ARGUMENT;
    switch (epi) {
        case EPI_NONE: return launch_skinny<EPI_NONE>((const bf16*)x, (const bf16*)W, out, out_dt, M, N, K, cap, act, st);
        case EPI_SOFTCAP: return launch_skinny<EPI_SOFTCAP>((const bf16*)x, (const bf16*)W, out, out_dt, M, N, K, cap, act, st);
        case EPI_GATED: return launch_skinny<EPI_GATED>((const bf16*)x, (const bf16*)W, out, out_dt, M, N, K, cap, act, st);
    }
    return QNN_ERR_ARGUMENT;
}

// The head of a greedy step: cand[m][c] = the best (softcapped value, column) among the 16 columns
// of W that CTA c owns, for each of the M rows; ceil(N / 16) candidates per row, merged by
// qnn_sample_candidates.  err (may be null) gets bit 0 set if a logit is NaN or Inf.
QNN_API int qnn_skinny_argmax(const void* x, const void* W, void* cand, int M, int N, int K, float cap, int* err,
                              cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K % 8 != 0 || K <= 0) return QNN_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)W) & 15 || ((uintptr_t)cand & 7)) return QNN_ERR_ARGUMENT;
    return launch_skinny<EPI_ARGMAX>((const bf16*)x, (const bf16*)W, cand, QNN_DT_F32, M, N, K, cap, 0, st, RopeEpi(), err);
}

// qkv[M, (nq+2nkv)*hd] = x[M,K] W^T with Q and K rotated by each row's position and K, V appended to
// the paged cache: qnn_skinny_bf16 followed by qnn_rope_cache_write (full-width rotation) in one
// kernel.  Head sizes in steps of 16; M <= 64.
QNN_API int qnn_skinny_qkv_rope(const void* x, const void* W, void* qkv, int M, int K, int nq, int nkv, int hd,
                                const float* inv_freq, const int* tok_pos, const int* tok_slot, void* k_pool,
                                void* v_pool, const int* page_table, int max_pages, int page_size, int ring,
                                const int* slot_len, int write_cache, cudaStream_t st) {
    if (M <= 0) return 0;
    if (M > 64 || K % 8 != 0 || K <= 0 || nq < 1 || nkv < 1 || hd < 16 || hd % 16) return QNN_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)W) & 15) return QNN_ERR_ARGUMENT;
    if (write_cache && (!k_pool || !v_pool || !page_table || !slot_len || page_size < 1)) return QNN_ERR_ARGUMENT;
    RopeEpi rp;
    rp.nq = nq; rp.nkv = nkv; rp.hd = hd;
    rp.inv_freq = inv_freq; rp.tok_pos = tok_pos; rp.tok_slot = tok_slot;
    rp.k_pool = (bf16*)k_pool; rp.v_pool = (bf16*)v_pool;
    rp.page_table = page_table; rp.max_pages = max_pages; rp.page_size = page_size; rp.ring = ring;
    rp.slot_len = slot_len; rp.write_cache = write_cache;
    return launch_skinny<EPI_ROPE>((const bf16*)x, (const bf16*)W, qkv, QNN_DT_BF16, M, (nq + 2 * nkv) * hd, K, 0.f, 0,
                                   st, rp);
}

// ---------------------------------------------------------------------------------
// fp32 GEMV: one warp per output column, MT rows at a time, lanes stride K.
// The order of additions for an output depends on K only.
// ---------------------------------------------------------------------------------
template <int MT, int EPI>
__global__ void gemv_f32_kernel(const float* __restrict__ x, const float* __restrict__ W, float* __restrict__ out,
                                int M, int N, int K, int m0, float cap, int act) {
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int Nout = (EPI == EPI_GATED) ? N / 2 : N;
    const int n = blockIdx.x * (blockDim.x >> 5) + warp;
    if (n >= Nout) return;
    float acc[MT], accu[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = accu[m] = 0.f;
    const float* w = W + (size_t)n * K;
    const float* u = W + (size_t)(Nout + n) * K;
    if ((K & 3) == 0) {
        for (int k = lane * 4; k < K; k += 128) {
            const float4 wv = __ldg(reinterpret_cast<const float4*>(w + k));
            float4 uv = make_float4(0, 0, 0, 0);
            if (EPI == EPI_GATED) uv = __ldg(reinterpret_cast<const float4*>(u + k));
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m0 + m < M) {
                    const float4 xv = *reinterpret_cast<const float4*>(x + (size_t)(m0 + m) * K + k);
                    acc[m] += xv.x * wv.x + xv.y * wv.y + xv.z * wv.z + xv.w * wv.w;
                    if (EPI == EPI_GATED) accu[m] += xv.x * uv.x + xv.y * uv.y + xv.z * uv.z + xv.w * uv.w;
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float wv = w[k];
            const float uv = (EPI == EPI_GATED) ? u[k] : 0.f;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m0 + m < M) {
                    const float xv = x[(size_t)(m0 + m) * K + k];
                    acc[m] += xv * wv;
                    if (EPI == EPI_GATED) accu[m] += xv * uv;
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        float v = warp_sum(acc[m]);
        float uu = (EPI == EPI_GATED) ? warp_sum(accu[m]) : 0.f;
        if (lane == 0 && m0 + m < M) {
            if (EPI == EPI_GATED) v = activate(v, act) * uu;
            else if (EPI == EPI_SOFTCAP) v = softcap(v, cap);
            out[(size_t)(m0 + m) * Nout + n] = v;
        }
    }
}

QNN_API int qnn_gemv_f32(const float* x, const float* W, float* out, int M, int N, int K, int epi, float cap, int act,
                         cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return QNN_ERR_ARGUMENT;
    if (epi == EPI_GATED && (N % 2)) return QNN_ERR_ARGUMENT;
    const int Nout = epi == EPI_GATED ? N / 2 : N;
    const int warps = 8;
    const unsigned blocks = (unsigned)((Nout + warps - 1) / warps);
    for (int m0 = 0; m0 < M; m0 += 4) {
        switch (epi) {
            case EPI_NONE: qnn::launch_pdl(gemv_f32_kernel<4, EPI_NONE>, dim3(blocks), dim3(warps * 32), 0, st, x, W, out, M, N, K, m0, cap, act); break;
            case EPI_SOFTCAP: qnn::launch_pdl(gemv_f32_kernel<4, EPI_SOFTCAP>, dim3(blocks), dim3(warps * 32), 0, st, x, W, out, M, N, K, m0, cap, act); break;
            case EPI_GATED: qnn::launch_pdl(gemv_f32_kernel<4, EPI_GATED>, dim3(blocks), dim3(warps * 32), 0, st, x, W, out, M, N, K, m0, cap, act); break;
            default: return QNN_ERR_ARGUMENT;
        }
    }
    QNN_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------
// fp32 tiled GEMM, FFMA only: 64x64 tile, 16-wide K slab, 256 threads x (4x4) outputs.
// Each output is summed over k in ascending order, whatever M and N are.
// ---------------------------------------------------------------------------------
template <int EPI>
__global__ void __launch_bounds__(256) sgemm_f32_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                        float* __restrict__ C, int M, int N, int K, float cap) {
    pdl_wait();
    __shared__ float As[16][64 + 4];
    __shared__ float Bs[16][64 + 4];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int lr = tid / 4, lk = (tid % 4) * 4;  // this thread loads row lr, k offset lk of each slab
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    const bool vec = (K & 3) == 0;
    for (int k0 = 0; k0 < K; k0 += 16) {
        float a[4] = {0, 0, 0, 0}, b[4] = {0, 0, 0, 0};
        const int am = m0 + lr, bn = n0 + lr, kk = k0 + lk;
        if (am < M) {
            if (vec && kk + 3 < K) {
                float4 v = *reinterpret_cast<const float4*>(A + (size_t)am * K + kk);
                a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (kk + i < K) a[i] = A[(size_t)am * K + kk + i];
            }
        }
        if (bn < N) {
            if (vec && kk + 3 < K) {
                float4 v = __ldg(reinterpret_cast<const float4*>(B + (size_t)bn * K + kk));
                b[0] = v.x; b[1] = v.y; b[2] = v.z; b[3] = v.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) if (kk + i < K) b[i] = B[(size_t)bn * K + kk + i];
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) { As[lk + i][lr] = a[i]; Bs[lk + i][lr] = b[i]; }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = As[k][ty * 4 + i]; bv[i] = Bs[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * N + n] = (EPI == EPI_SOFTCAP) ? softcap(acc[i][j], cap) : acc[i][j];
        }
    }
}

QNN_API int qnn_sgemm_f32(const float* A, const float* B, float* C, int M, int N, int K, int epi, float cap,
                          cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return QNN_ERR_ARGUMENT;
    dim3 grid((N + 63) / 64, (M + 63) / 64);
    if (grid.y > 65535) return QNN_ERR_UNSUPPORTED;
    if (epi == EPI_SOFTCAP) qnn::launch_pdl(sgemm_f32_kernel<EPI_SOFTCAP>, dim3(grid), dim3(256), 0, st, A, B, C, M, N, K, cap);
    else if (epi == EPI_NONE) qnn::launch_pdl(sgemm_f32_kernel<EPI_NONE>, dim3(grid), dim3(256), 0, st, A, B, C, M, N, K, cap);
    else return QNN_ERR_ARGUMENT;
    QNN_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------
// bfloat16 product for inner sizes that are no multiple of 8 (rows that do not start on 16 bytes, so
// neither the vector loads of the small-M kernel nor a TMA map can be used): one warp per output
// column, 8 rows at a time, lanes stride K with 2-byte loads, float32 sums.  Slow and only there so
// that such a width is served rather than refused; the order of additions depends on K only.
// ---------------------------------------------------------------------------------
template <int EPI>
__global__ void linear_bf16_any_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W, void* __restrict__ out,
                                       int out_f32, int M, int N, int K, float cap, int act) {
    pdl_wait();
    constexpr int MT = 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int Nout = (EPI == EPI_GATED) ? N / 2 : N;
    const int n = blockIdx.x * (blockDim.x >> 5) + warp;
    const int m0 = blockIdx.y * MT;
    if (n >= Nout) return;
    float acc[MT], accu[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = accu[m] = 0.f;
    const bf16* w = W + (size_t)n * K;
    const bf16* u = W + (size_t)(Nout + n) * K;
    for (int k = lane; k < K; k += 32) {
        const float wv = __bfloat162float(w[k]);
        const float uv = (EPI == EPI_GATED) ? __bfloat162float(u[k]) : 0.f;
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m0 + m < M) {
                const float xv = __bfloat162float(x[(size_t)(m0 + m) * K + k]);
                acc[m] += xv * wv;
                if (EPI == EPI_GATED) accu[m] += xv * uv;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        float v = warp_sum(acc[m]);
        const float uu = (EPI == EPI_GATED) ? warp_sum(accu[m]) : 0.f;
        if (lane == 0 && m0 + m < M) {
            if (EPI == EPI_GATED) v = activate(v, act) * uu;
            else if (EPI == EPI_SOFTCAP) v = softcap(v, cap);
            const size_t at = (size_t)(m0 + m) * Nout + n;
            if (out_f32) reinterpret_cast<float*>(out)[at] = v;
            else reinterpret_cast<bf16*>(out)[at] = __float2bfloat16_rn(v);
        }
    }
}

QNN_API int qnn_linear_bf16_any(const void* x, const void* W, void* out, int out_dt, int M, int N, int K, int epi,
                                float cap, int act, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return QNN_ERR_ARGUMENT;
    if (epi == EPI_GATED && (N % 2)) return QNN_ERR_ARGUMENT;
    if (out_dt != QNN_DT_BF16 && out_dt != QNN_DT_F32) return QNN_ERR_ARGUMENT;
    const int Nout = epi == EPI_GATED ? N / 2 : N;
    const int warps = 4;
    const dim3 grid((unsigned)((Nout + warps - 1) / warps), (unsigned)((M + 7) / 8));
    if (grid.y > 65535) return QNN_ERR_UNSUPPORTED;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)W;
    const int f32 = out_dt == QNN_DT_F32;
    switch (epi) {
        case EPI_NONE: qnn::launch_pdl(linear_bf16_any_kernel<EPI_NONE>, grid, dim3(warps * 32), 0, st, xp, wp, out, f32, M, N, K, cap, act); break;
        case EPI_SOFTCAP: qnn::launch_pdl(linear_bf16_any_kernel<EPI_SOFTCAP>, grid, dim3(warps * 32), 0, st, xp, wp, out, f32, M, N, K, cap, act); break;
        case EPI_GATED: qnn::launch_pdl(linear_bf16_any_kernel<EPI_GATED>, grid, dim3(warps * 32), 0, st, xp, wp, out, f32, M, N, K, cap, act); break;
        default: return QNN_ERR_ARGUMENT;
    }
    QNN_LAUNCH_CHECK();
}

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
// computes rows n and N/2+n and stores act(gate)*up.
#include "common.cuh"

using namespace qnn;

#define EPI_NONE 0
#define EPI_SOFTCAP 1
#define EPI_GATED 2

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

template <int NT, int EPI, int NW>
__global__ void __launch_bounds__(NW * 32) skinny_bf16_kernel(const bf16* __restrict__ x, const bf16* __restrict__ W,
                                                          void* __restrict__ out, int out_dt, int M, int N, int K,
                                                          float cap, int act) {
    constexpr int COLS = NT * 8;
    constexpr int THREADS = NW * 32;
    __shared__ float red[NW][16][COLS + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int Nout = (EPI == EPI_GATED) ? N / 2 : N;
    const int n0 = blockIdx.x * 16;
    const int r0 = min(n0 + g, Nout - 1), r1 = min(n0 + g + 8, Nout - 1);
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

    // The weights do not depend on the kernel before this one: pull this warp's share of them
    // towards L2 while that kernel is still running, then wait for the activations.  Only for the
    // smaller matrices, whose kernels are too short to reach full bandwidth on their own; for the
    // big ones the extra instructions only fill the load queue.
    if (t == 0 && (size_t)N * K <= ((size_t)1 << 24)) {
        for (int kb = warp; kb < nkb; kb += NW) {
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

#pragma unroll 4
    for (int kb = warp; kb < nkb; kb += NW) {
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
        } else if (EPI == EPI_SOFTCAP) {
            v = softcap(v, cap);
        }
        if (n < Nout && m < M) store_out(out, out_dt, (size_t)m * Nout + n, v);
    }
}

// The K range of a 16-row tile is split over the NW warps of its CTA.  Matrices with few rows
// (N/16 CTAs do not fill the GPU) get more warps per CTA, as far as K gives every warp at
// least two 32-wide blocks and the partial tiles fit in shared memory.
template <int EPI>
static int launch_skinny(const bf16* x, const bf16* W, void* out, int out_dt, int M, int N, int K, float cap, int act,
                         cudaStream_t st) {
    const int Nout = (EPI == EPI_GATED) ? N / 2 : N;
    const unsigned blocks = (unsigned)((Nout + 15) / 16);
    const int nt = (M + 7) / 8;
    const int kblocks = (K + 31) / 32;
    int nw = 8;
    if (nt <= 2 && blocks * 8u < 3000u && kblocks >= 32) nw = 16;
    if (nt == 1 && blocks * 16u < 3000u && kblocks >= 64) nw = 32;
#define QNN_SK(NTV)                                                                                            \
    if (nw == 32 && NTV == 1)                                                                                  \
        qnn::launch_pdl(skinny_bf16_kernel<1, EPI, 32>, dim3(blocks), dim3(1024), 0, st, x, W, out, out_dt, M, N, K, cap, act);         \
    else if (nw >= 16 && NTV <= 2)                                                                             \
        qnn::launch_pdl(skinny_bf16_kernel<(NTV <= 2 ? NTV : 1), EPI, 16>, dim3(blocks), dim3(512), 0, st, x, W, out, out_dt, M, N, K, cap, act); \
    else                                                                                                       \
        qnn::launch_pdl(skinny_bf16_kernel<NTV, EPI, 8>, dim3(blocks), dim3(256), 0, st, x, W, out, out_dt, M, N, K, cap, act);         \
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

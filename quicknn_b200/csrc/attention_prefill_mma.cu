// Prefill attention on the tensor cores, bfloat16, head sizes 64, 128 and 256: whole prompts
// packed one after another, causal, optional sliding window, optional tanh softcap, grouped
// query heads.
//
// Formulas: those of attention.cu (reference: src/backends/vulkan/shaders/attention.comp:18-38,
// which gives every (query row, head) a workgroup of its own).  Here a CTA of 4 warps owns 64
// query rows of one sequence and one query head and walks over the 64-key tiles that those rows
// can see (from the window's edge to the diagonal) in tiles of BN keys (64, or 32 at head size 256 so
// that two CTAs fit an SM), keys and values double-buffered in shared memory by cp.async:
//     S[16 x BN] = Q K^T      per warp, mma.m16n8k16, Q and K fragments by ldmatrix
//     scale, softcap, mask (key <= row, key > row - window, key < length), online softmax in float32
//     O[16 x hd] += P V       P taken from S's accumulators, V fragments by ldmatrix.trans
// K and V are read from this step's own projections (rows of the qkv buffer), so a prompt longer
// than the window does not depend on the ring in the cache.  Rows of shared memory are
// XOR-swizzled by 16-byte chunk against ldmatrix bank conflicts.
#include "common.cuh"
#include <math_constants.h>

using namespace qnn;

namespace {

constexpr int BM = 64, PF_WARPS = 4;

__device__ __forceinline__ void cp_async_16(unsigned smem_dst, const void* gmem_src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_dst), "l"(gmem_src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float tanh_fast(float x) {
    float r;
    asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int HD, int BN>
__global__ void __launch_bounds__(PF_WARPS * 32, (BM + 4 * BN) * HD * 2 <= 112 * 1024 ? 2 : 1)
attn_prefill_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k, const bf16* __restrict__ v,
                        size_t row_stride, bf16* __restrict__ out, size_t out_stride,
                        const int* __restrict__ seq_row0, const int* __restrict__ seq_len, int nq, int nkv, float scale,
                        float cap, int window) {
    pdl_wait();
    constexpr int KSTEPS = HD / 16, CH = HD / 8, ROWB = HD * 2, NDT = HD / 8;
    constexpr int TILEB = BN * ROWB;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // grid (heads, sequences, query tiles): the tile is the slowest index, so that CTAs are handed out from
    // the heaviest tiles of all heads down to the lightest
    const int b = blockIdx.y, h = blockIdx.x;
    const int len = seq_len[b];
    const int ntiles = (len + BM - 1) / BM;
    if ((int)blockIdx.z >= ntiles) return;
    const int tile = ntiles - 1 - blockIdx.z;          // the longest rows first
    const int r0 = tile * BM, row0 = seq_row0[b];
    const int kh = h / (nq / nkv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const unsigned sQ = (unsigned)__cvta_generic_to_shared(smem_raw);
    const unsigned sK = sQ + BM * ROWB, sV = sK + 2 * TILEB;

    // Q tile
    {
        const bf16* qb = q + (size_t)(row0 + r0) * row_stride + (size_t)h * HD;
        for (int idx = tid; idx < BM * CH; idx += PF_WARPS * 32) {
            const int row = idx / CH, chunk = idx % CH;
            cp_async_16(sQ + row * ROWB + ((chunk ^ (row & 7)) << 4), qb + (size_t)row * row_stride + chunk * 8,
                        r0 + row < len);
        }
    }
    const int last_row = min(r0 + BM, len) - 1;
    const int kv_lo = (window > 0 && r0 - window + 1 > 0) ? r0 - window + 1 : 0;
    const int jt_first = kv_lo / BN, jt_last = last_row / BN;
    const bf16* kb = k + (size_t)row0 * row_stride + (size_t)kh * HD;
    const bf16* vb = v + (size_t)row0 * row_stride + (size_t)kh * HD;
    auto load_kv = [&](int jt, int stage) {
        const unsigned dK = sK + stage * TILEB, dV = sV + stage * TILEB;
        for (int idx = tid; idx < BN * CH; idx += PF_WARPS * 32) {
            const int row = idx / CH, chunk = idx % CH;
            const int key = jt * BN + row;
            const bool valid = key < len;
            const size_t off = (size_t)(valid ? key : 0) * row_stride + chunk * 8;
            const unsigned dst = row * ROWB + ((chunk ^ (row & 7)) << 4);
            cp_async_16(dK + dst, kb + off, valid);
            cp_async_16(dV + dst, vb + off, valid);
        }
    };
    load_kv(jt_first, 0);
    cp_async_commit();

    float o[NDT][4];
#pragma unroll
    for (int i = 0; i < NDT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m_[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_[2] = {0.f, 0.f};
    const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
    const int qrow_lo = r0 + warp * 16 + g;            // this lane's rows: qrow_lo and qrow_lo + 8

    for (int jt = jt_first, n = 0; jt <= jt_last; ++jt, ++n) {
        const int stage = n & 1;
        if (jt < jt_last) {
            load_kv(jt + 1, stage ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const unsigned cK = sK + stage * TILEB, cV = sV + stage * TILEB;

        float s[BN / 8][4];
#pragma unroll
        for (int i = 0; i < BN / 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
            uint32_t a[4];
            {
                const int row = warp * 16 + (lane & 15), chunk = ks * 2 + (lane >> 4);
                ldmatrix_x4(a, sQ + row * ROWB + ((chunk ^ (row & 7)) << 4));
            }
#pragma unroll
            for (int np = 0; np < BN / 16; ++np) {
                uint32_t bf[4];
                const int row = np * 16 + (lane & 7) + ((lane >> 4) << 3), chunk = ks * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(bf, cK + row * ROWB + ((chunk ^ (row & 7)) << 4));
                mma_16816(s[np * 2], a, bf[0], bf[1]);
                mma_16816(s[np * 2 + 1], a, bf[2], bf[3]);
            }
        }
        // scale, softcap, mask; row maxima
        float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int col = jt * BN + nt * 8 + 2 * t + (j & 1);
                const int row = qrow_lo + ((j >> 1) << 3);
                float x = s[nt][j] * scale;
                if (cap > 0.f) x = cap * tanh_fast(fminf(fmaxf(x * inv_cap, -20.f), 20.f));
                const bool seen = col <= row && col < len && (window <= 0 || col > row - window);
                x = seen ? x : -CUDART_INF_F;
                s[nt][j] = x;
                mx[j >> 1] = fmaxf(mx[j >> 1], x);
            }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float mn = fmaxf(m_[r], mx[r]);
            corr[r] = (mn == -CUDART_INF_F) ? 1.f : __expf(m_[r] - mn);
            m_[r] = mn;
            mx[r] = (mn == -CUDART_INF_F) ? 0.f : mn;      // what is subtracted below; exp(-inf - 0) = 0
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float p = __expf(s[nt][j] - mx[j >> 1]);
                s[nt][j] = p;
                rs[j >> 1] += p;
            }
        l_[0] = l_[0] * corr[0] + rs[0];                   // per-lane partial sums; reduced at the end
        l_[1] = l_[1] * corr[1] + rs[1];
#pragma unroll
        for (int nd = 0; nd < NDT; ++nd) {
            o[nd][0] *= corr[0];
            o[nd][1] *= corr[0];
            o[nd][2] *= corr[1];
            o[nd][3] *= corr[1];
        }
        // O += P V
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
            a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
            a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
                uint32_t bf[4];
                const int row = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), chunk = dp * 2 + (lane >> 4);
                ldmatrix_x4_trans(bf, cV + row * ROWB + ((chunk ^ (row & 7)) << 4));
                mma_16816(o[dp * 2], a, bf[0], bf[1]);
                mma_16816(o[dp * 2 + 1], a, bf[2], bf[3]);
            }
        }
        __syncthreads();   // the other stage is refilled at the top of the next round
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_[r] += __shfl_xor_sync(0xffffffffu, l_[r], 1);
        l_[r] += __shfl_xor_sync(0xffffffffu, l_[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = qrow_lo + r * 8;
        if (row < len) {
            const float inv = l_[r] > 0.f ? 1.f / l_[r] : 0.f;
            uint32_t* dst = reinterpret_cast<uint32_t*>(out + (size_t)(row0 + row) * out_stride + (size_t)h * HD);
#pragma unroll
            for (int nd = 0; nd < NDT; ++nd) dst[nd * 4 + t] = pack_bf16(o[nd][2 * r] * inv, o[nd][2 * r + 1] * inv);
        }
    }
}

template <int HD, int BN>
int launch(const void* q, const void* k, const void* v, long long row_stride, void* out, long long out_stride,
           const int* seq_row0, const int* seq_len, int B, int max_len, int nq, int nkv, float scale, float cap,
           int window, cudaStream_t st) {
    auto kern = attn_prefill_mma_kernel<HD, BN>;
    const size_t smem = (size_t)(BM + 4 * BN) * HD * 2;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(nq, B, (max_len + BM - 1) / BM);
    qnn::launch_pdl(kern, dim3(grid), dim3(PF_WARPS * 32), smem, st, (const bf16*)q, (const bf16*)k, (const bf16*)v, (size_t)row_stride,
                                            (bf16*)out, (size_t)out_stride, seq_row0, seq_len, nq, nkv, scale, cap,
                                            window);
    return (int)cudaGetLastError();
}

}  // namespace

// q, k, v: this step's projections (row_stride elements between rows); sequence b occupies rows
// seq_row0[b] .. seq_row0[b] + seq_len[b] - 1, its positions start at 0.  max_len bounds the
// lengths.  Returns QNN_ERR_UNSUPPORTED for head sizes other than 64, 128, 256.
QNN_API int qnn_attn_prefill_mma(const void* q, const void* k, const void* v, long long row_stride, void* out,
                                 long long out_stride, const int* seq_row0, const int* seq_len, int B, int max_len,
                                 int nq, int nkv, int hd, float scale, float cap, int window, cudaStream_t st) {
    if (B <= 0 || max_len <= 0) return 0;
    if (nkv <= 0 || nq % nkv) return QNN_ERR_ARGUMENT;
    if (B > 65535 || (max_len + BM - 1) / BM > 65535) return QNN_ERR_UNSUPPORTED;
    if ((row_stride * 2) % 16 || (out_stride * 2) % 4 ||
        (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) || ((uintptr_t)out & 3))
        return QNN_ERR_ARGUMENT;
    switch (hd) {
        case 64: return launch<64, 64>(q, k, v, row_stride, out, out_stride, seq_row0, seq_len, B, max_len, nq, nkv, scale, cap, window, st);
        case 128: return launch<128, 64>(q, k, v, row_stride, out, out_stride, seq_row0, seq_len, B, max_len, nq, nkv, scale, cap, window, st);
        case 256: return launch<256, 32>(q, k, v,      // 32-key tiles: 96 KB of shared memory, two CTAs per SM
                                          row_stride, out, out_stride, seq_row0, seq_len, B, max_len, nq, nkv, scale, cap, window, st);
        default: return QNN_ERR_UNSUPPORTED;
    }
}

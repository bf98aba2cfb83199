// Attention over keys and values: the generic kernels, for float32 and bfloat16 and any
// head size that is a multiple of 16 bytes of elements.
//
// Reference: one workgroup per (query row, head) streaming the cache in 128-key blocks
// with an online softmax (src/backends/vulkan/shaders/attention.comp:18-38):
//   s_j = (q . k_j) * scale;  s_j = cap * tanh(clamp(s_j / cap, -20, 20)) if cap > 0   (:26-27)
//   keys j in [keyStart, keyEnd), keyEnd = p + 1, keyStart = keyEnd - window when
//   window > 0 and keyEnd > window, else 0                                            (:21-24)
//   running max / sum rescaling, O += w_j v_j, A = O / sum                           (:28-37)
//   query head h reads kv head h / (heads / kvHeads)                                  (:14)
//
// Here a warp is the unit: the lanes of a warp are split into groups of LPT lanes, each
// group dots one key with the query (16-byte loads, CPL chunks per lane), so a warp takes
// 32/LPT keys per step; every group carries its own (max, sum, O) and the groups are merged
// at the end.  A warp serves GT query heads of one kv head at once, so K and V are read
// once per group of query heads.  All softmax arithmetic is float32.
//
//   decode : grid (splits, kv heads x head tiles, sequences); the keys of a sequence are cut
//            into `splits` equal ranges (a fixed number, so results do not depend on the
//            batch); each CTA writes (max, sum, O) of its range to scratch and
//            qnn_attn_combine merges them in split order.  K and V come from the paged cache.
//   prefill: one warp per (token, kv head, head tile); K and V come from this step's own
//            packed projections (rows of the qkv buffer), which is what makes a prompt
//            longer than the window independent of the ring in the cache.
#include "common.cuh"
#include <math_constants.h>

using namespace qnn;

namespace {

// expf in the float32 path, the fast exponential where the data are bfloat16 anyway
template <typename T> __device__ __forceinline__ float fexp(float x);
template <> __device__ __forceinline__ float fexp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ float fexp<bf16>(float x) { return __expf(x); }

template <typename T>
struct PagedKV {
    const T* k_pool;
    const T* v_pool;
    const int* page_row;  // page table row of this sequence
    int page_size, nkv, hd, ring, kh;
    __device__ __forceinline__ size_t off(int p) const {
        const int r = ring > 0 ? p % ring : p;
        const int page = page_row[r / page_size];
        return (((size_t)page * nkv + kh) * page_size + (r % page_size)) * hd;
    }
    __device__ __forceinline__ const T* k(int p) const { return k_pool + off(p); }
    __device__ __forceinline__ const T* v(int p) const { return v_pool + off(p); }
};

template <typename T>
struct PackedKV {
    const T* kbase;  // already offset to this kv head
    const T* vbase;
    size_t row_stride;
    int row0;
    __device__ __forceinline__ const T* k(int p) const { return kbase + (size_t)(row0 + p) * row_stride; }
    __device__ __forceinline__ const T* v(int p) const { return vbase + (size_t)(row0 + p) * row_stride; }
};

// One warp over the keys [begin, end), taking keys begin + first + i*stride + group.
template <typename T, int CPL, int GT, typename KV>
__device__ __forceinline__ void attend_range(const float (&q)[GT][CPL][Vec16<T>::N], const KV& kv, int begin, int end,
                                             int first, int stride, int LPT, int chunks, float cap,
                                             float (&m)[GT], float (&l)[GT], float (&o)[GT][CPL][Vec16<T>::N]) {
    constexpr int VEC = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int sl = lane % LPT, ti = lane / LPT;
    for (int base = begin + first; base < end; base += stride) {
        const int p = base + ti;
        const bool valid = p < end;
        float s[GT];
#pragma unroll
        for (int g = 0; g < GT; ++g) s[g] = 0.f;
        float vv[CPL][VEC];
        if (valid) {
            const T* kp = kv.k(p);
            const T* vp = kv.v(p);
            Vec16<T> kvec[CPL], vvec[CPL];
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                const int c = sl + i * LPT;
                if (c < chunks) {
                    kvec[i].load(kp + c * VEC);
                    vvec[i].load(vp + c * VEC);
                }
            }
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                const int c = sl + i * LPT;
                if (c < chunks) {
                    float kk[VEC];
                    kvec[i].unpack(kk);
                    vvec[i].unpack(vv[i]);
#pragma unroll
                    for (int g = 0; g < GT; ++g)
#pragma unroll
                        for (int e = 0; e < VEC; ++e) s[g] = fmaf(q[g][i][e], kk[e], s[g]);
                } else {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) vv[i][e] = 0.f;
                }
            }
        }
#pragma unroll
        for (int g = 0; g < GT; ++g)
            for (int off = LPT >> 1; off > 0; off >>= 1) s[g] += __shfl_xor_sync(0xffffffffu, s[g], off);
        if (valid) {
#pragma unroll
            for (int g = 0; g < GT; ++g) {
                const float sc = softcap(s[g], cap);
                const float mn = fmaxf(m[g], sc);
                const float corr = fexp<T>(m[g] - mn);  // m = -inf on the first key gives 0
                const float w = fexp<T>(sc - mn);
                l[g] = l[g] * corr + w;
#pragma unroll
                for (int i = 0; i < CPL; ++i)
#pragma unroll
                    for (int e = 0; e < VEC; ++e) o[g][i][e] = o[g][i][e] * corr + w * vv[i][e];
                m[g] = mn;
            }
        }
    }
}

// Merge the states of the 32/LPT lane groups of a warp; afterwards every lane holds the
// merged state for its own chunks.
template <int CPL, int GT, int VEC>
__device__ __forceinline__ void merge_groups(int LPT, float (&m)[GT], float (&l)[GT], float (&o)[GT][CPL][VEC]) {
    for (int off = LPT; off < 32; off <<= 1) {
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[g], off);
            const float lo = __shfl_xor_sync(0xffffffffu, l[g], off);
            const float mn = fmaxf(m[g], mo);
            const float ca = (m[g] == -CUDART_INF_F) ? 0.f : expf(m[g] - mn);
            const float cb = (mo == -CUDART_INF_F) ? 0.f : expf(mo - mn);
            l[g] = l[g] * ca + lo * cb;
#pragma unroll
            for (int i = 0; i < CPL; ++i)
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    const float oo = __shfl_xor_sync(0xffffffffu, o[g][i][e], off);
                    o[g][i][e] = o[g][i][e] * ca + oo * cb;
                }
            m[g] = mn;
        }
    }
}

template <typename T, int CPL, int GT>
__device__ __forceinline__ void load_query(const T* qrow0, int hd, int G, int gt0, int LPT, int chunks, float scale,
                                           float (&q)[GT][CPL][Vec16<T>::N]) {
    constexpr int VEC = Vec16<T>::N;
    const int sl = (threadIdx.x & 31) % LPT;
#pragma unroll
    for (int g = 0; g < GT; ++g)
#pragma unroll
        for (int i = 0; i < CPL; ++i) {
            const int c = sl + i * LPT;
            if (gt0 + g < G && c < chunks) {
                Vec16<T> v;
                v.load(qrow0 + (size_t)(gt0 + g) * hd + c * VEC);
                v.unpack(q[g][i]);
#pragma unroll
                for (int e = 0; e < VEC; ++e) q[g][i][e] *= scale;
            } else {
#pragma unroll
                for (int e = 0; e < VEC; ++e) q[g][i][e] = 0.f;
            }
        }
}

constexpr int DEC_WARPS = 4;

template <typename T, int CPL, int GT>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_kernel(const T* __restrict__ q, size_t q_stride, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                   const int* __restrict__ page_table, int max_pages, int page_size, int ring,
                   const int* __restrict__ slots, const int* __restrict__ slot_len, int nq, int nkv, int hd, int LPT,
                   float scale, float cap, int window, float* __restrict__ part_o, float* __restrict__ part_ml,
                   int n_splits) {
    constexpr int VEC = Vec16<T>::N;
    extern __shared__ float smem[];  // [DEC_WARPS][GT][hd + 2]
    const int split = blockIdx.x, b = blockIdx.z;
    const int G = nq / nkv, gtiles = (G + GT - 1) / GT;
    const int kh = blockIdx.y / gtiles, gt0 = (blockIdx.y % gtiles) * GT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = hd / VEC;
    const int sl = lane % LPT, ti = lane / LPT, TPW = 32 / LPT;
    const int slot = slots[b];

    float m[GT], l[GT], o[GT][CPL][VEC];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        m[g] = -CUDART_INF_F;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < CPL; ++i)
#pragma unroll
            for (int e = 0; e < VEC; ++e) o[g][i][e] = 0.f;
    }
    if (slot >= 0) {
        const int n = slot_len[slot];
        const int kbeg = (window > 0 && n > window) ? n - window : 0;
        const int count = n - kbeg;
        const int per = (count + n_splits - 1) / n_splits;
        const int begin = kbeg + split * per;
        const int end = min(begin + per, n);
        if (begin < end) {
            float qr[GT][CPL][VEC];
            load_query<T, CPL, GT>(q + (size_t)b * q_stride + (size_t)kh * G * hd, hd, G, gt0, LPT, chunks, scale, qr);
            PagedKV<T> kv{k_pool, v_pool, page_table + (size_t)slot * max_pages, page_size, nkv, hd, ring, kh};
            attend_range<T, CPL, GT>(qr, kv, begin, end, warp * TPW, DEC_WARPS * TPW, LPT, chunks, cap, m, l, o);
        }
    }
    merge_groups<CPL, GT, VEC>(LPT, m, l, o);
    // warps -> shared memory -> merged in warp order by the threads that own a dimension
    const int row = hd + 2;
    if (ti == 0) {
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            float* dst = smem + ((size_t)warp * GT + g) * row;
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                const int c = sl + i * LPT;
                if (c < chunks)
#pragma unroll
                    for (int e = 0; e < VEC; ++e) dst[c * VEC + e] = o[g][i][e];
            }
            if (sl == 0) {
                dst[hd] = m[g];
                dst[hd + 1] = l[g];
            }
        }
    }
    __syncthreads();
    for (int g = 0; g < GT; ++g) {
        if (gt0 + g >= G) break;
        const int h = kh * G + gt0 + g;
        float mm = -CUDART_INF_F;
        for (int w = 0; w < DEC_WARPS; ++w) mm = fmaxf(mm, smem[((size_t)w * GT + g) * row + hd]);
        float coef[DEC_WARPS], ll = 0.f;
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float mw = smem[((size_t)w * GT + g) * row + hd];
            coef[w] = (mw == -CUDART_INF_F) ? 0.f : expf(mw - mm);
            ll += coef[w] * smem[((size_t)w * GT + g) * row + hd + 1];
        }
        const size_t pbase = ((size_t)b * nq + h) * n_splits + split;
        for (int d = threadIdx.x; d < hd; d += blockDim.x) {
            float acc = 0.f;
            for (int w = 0; w < DEC_WARPS; ++w) acc += coef[w] * smem[((size_t)w * GT + g) * row + d];
            part_o[pbase * hd + d] = acc;
        }
        if (threadIdx.x == 0) {
            part_ml[pbase * 2] = mm;
            part_ml[pbase * 2 + 1] = ll;
        }
    }
}

// out[b, h, :] = sum_s e^{m_s - M} O_s / sum_s e^{m_s - M} l_s, splits in ascending order.
template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    T* __restrict__ out, size_t out_stride, int nq, int hd, int n_splits) {
    const int b = blockIdx.x / nq, h = blockIdx.x % nq;
    const size_t pbase = ((size_t)b * nq + h) * n_splits;
    float mm = -CUDART_INF_F;
    for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, part_ml[(pbase + s) * 2]);
    float ll = 0.f;
    for (int s = 0; s < n_splits; ++s) {
        const float ms = part_ml[(pbase + s) * 2];
        if (ms != -CUDART_INF_F) ll += expf(ms - mm) * part_ml[(pbase + s) * 2 + 1];
    }
    const float inv = ll > 0.f ? 1.f / ll : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float ms = part_ml[(pbase + s) * 2];
            if (ms != -CUDART_INF_F) acc += expf(ms - mm) * part_o[(pbase + s) * hd + d];
        }
        out[(size_t)b * out_stride + (size_t)h * hd + d] = from_f<T>(acc * inv);
    }
}

constexpr int PRE_WARPS = 4;

// One warp per (token, kv head, head tile).  PAGED = false: keys are rows of this step's
// packed projections (k, v, row_stride, tok_row0).  PAGED = true: keys come from the paged
// cache of the token's sequence (k = K pool, v = V pool, tok_row0 = slot per token); used
// by a layer that reads a cache line which another layer wrote.
template <typename T, int CPL, int GT, bool PAGED>
__global__ void __launch_bounds__(PRE_WARPS * 32)
attn_prefill_generic_kernel(const T* __restrict__ q, size_t q_stride, const T* __restrict__ k, const T* __restrict__ v,
                            size_t row_stride, T* __restrict__ out, size_t out_stride, const int* __restrict__ tok_pos,
                            const int* __restrict__ tok_row0, int n_tokens, int nq, int nkv, int hd, int LPT,
                            float scale, float cap, int window, const int* __restrict__ page_table, int max_pages,
                            int page_size, int ring) {
    constexpr int VEC = Vec16<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * PRE_WARPS + warp;
    if (t >= n_tokens) return;
    const int G = nq / nkv, gtiles = (G + GT - 1) / GT;
    const int kh = blockIdx.y / gtiles, gt0 = (blockIdx.y % gtiles) * GT;
    const int chunks = hd / VEC;
    const int sl = lane % LPT, ti = lane / LPT, TPW = 32 / LPT;
    const int row0 = tok_row0[t];

    float m[GT], l[GT], o[GT][CPL][VEC];
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        m[g] = -CUDART_INF_F;
        l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < CPL; ++i)
#pragma unroll
            for (int e = 0; e < VEC; ++e) o[g][i][e] = 0.f;
    }
    if (row0 >= 0) {
        const int p = tok_pos[t];
        const int end = p + 1;
        const int begin = (window > 0 && end > window) ? end - window : 0;
        float qr[GT][CPL][VEC];
        load_query<T, CPL, GT>(q + (size_t)t * q_stride + (size_t)kh * G * hd, hd, G, gt0, LPT, chunks, scale, qr);
        if (PAGED) {
            PagedKV<T> kv{k, v, page_table + (size_t)row0 * max_pages, page_size, nkv, hd, ring, kh};
            attend_range<T, CPL, GT>(qr, kv, begin, end, 0, TPW, LPT, chunks, cap, m, l, o);
        } else {
            PackedKV<T> kv{k + (size_t)kh * hd, v + (size_t)kh * hd, row_stride, row0};
            attend_range<T, CPL, GT>(qr, kv, begin, end, 0, TPW, LPT, chunks, cap, m, l, o);
        }
    }
    merge_groups<CPL, GT, VEC>(LPT, m, l, o);
    if (ti == 0) {
#pragma unroll
        for (int g = 0; g < GT; ++g) {
            if (gt0 + g >= G) continue;
            const float inv = l[g] > 0.f ? 1.f / l[g] : 0.f;
            T* dst = out + (size_t)t * out_stride + (size_t)(kh * G + gt0 + g) * hd;
#pragma unroll
            for (int i = 0; i < CPL; ++i) {
                const int c = sl + i * LPT;
                if (c < chunks) {
                    float r[VEC];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) r[e] = o[g][i][e] * inv;
                    Vec16<T>::store(dst + c * VEC, r);
                }
            }
        }
    }
}

struct Geometry {
    int cpl, lpt, gt;
    bool ok;
};

template <typename T>
Geometry geometry(int hd, int G) {
    constexpr int VEC = 16 / sizeof(T);
    Geometry g{0, 0, 0, false};
    if (hd <= 0 || hd % VEC) return g;
    const int chunks = hd / VEC;
    int cpl = (chunks + 31) / 32;
    cpl = cpl <= 1 ? 1 : (cpl <= 2 ? 2 : 4);
    if (chunks > 32 * 4) return g;
    const int per = (chunks + cpl - 1) / cpl;
    int lpt = 1;
    while (lpt < per) lpt <<= 1;
    g.cpl = cpl;
    g.lpt = lpt;
    g.gt = G <= 1 ? 1 : (G <= 2 ? 2 : 4);
    g.ok = true;
    return g;
}

}  // namespace

#define QNN_DISPATCH_CPL_GT(CPLV, GTV, ...)                                   \
    if (geo.cpl == CPLV && geo.gt == GTV) {                                    \
        constexpr int CPL = CPLV;                                              \
        constexpr int GT = GTV;                                                \
        __VA_ARGS__                                                            \
    }
#define QNN_DISPATCH_ALL(...)                                                                       \
    QNN_DISPATCH_CPL_GT(1, 1, __VA_ARGS__) QNN_DISPATCH_CPL_GT(1, 2, __VA_ARGS__)                    \
    QNN_DISPATCH_CPL_GT(1, 4, __VA_ARGS__) QNN_DISPATCH_CPL_GT(2, 1, __VA_ARGS__)                    \
    QNN_DISPATCH_CPL_GT(2, 2, __VA_ARGS__) QNN_DISPATCH_CPL_GT(2, 4, __VA_ARGS__)                    \
    QNN_DISPATCH_CPL_GT(4, 1, __VA_ARGS__) QNN_DISPATCH_CPL_GT(4, 2, __VA_ARGS__)                    \
    QNN_DISPATCH_CPL_GT(4, 4, __VA_ARGS__)

template <typename T>
static int decode_launch(const void* q, long long q_stride, const void* k_pool, const void* v_pool,
                         const int* page_table, int max_pages, int page_size, int ring, const int* slots,
                         const int* slot_len, int B, int nq, int nkv, int hd, float scale, float cap, int window,
                         float* part_o, float* part_ml, int n_splits, void* out, long long out_stride,
                         cudaStream_t st) {
    if (nkv <= 0 || nq % nkv) return QNN_ERR_ARGUMENT;
    const Geometry geo = geometry<T>(hd, nq / nkv);
    if (!geo.ok) return QNN_ERR_UNSUPPORTED;
    if ((q_stride * sizeof(T)) % 16 || ((uintptr_t)q & 15)) return QNN_ERR_ARGUMENT;
    const int gtiles = (nq / nkv + geo.gt - 1) / geo.gt;
    dim3 grid(n_splits, nkv * gtiles, B);
    const size_t smem = (size_t)DEC_WARPS * geo.gt * (hd + 2) * sizeof(float);
    if (smem > 48 * 1024) return QNN_ERR_UNSUPPORTED;
    QNN_DISPATCH_ALL({
        attn_decode_kernel<T, CPL, GT><<<grid, DEC_WARPS * 32, smem, st>>>(
            (const T*)q, (size_t)q_stride, (const T*)k_pool, (const T*)v_pool, page_table, max_pages, page_size, ring,
            slots, slot_len, nq, nkv, hd, geo.lpt, scale, cap, window, part_o, part_ml, n_splits);
    })
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    attn_combine_kernel<T><<<B * nq, 128, 0, st>>>(part_o, part_ml, (T*)out, (size_t)out_stride, nq, hd, n_splits);
    QNN_LAUNCH_CHECK();
}

// Scratch: part_o needs B*nq*n_splits*hd floats, part_ml B*nq*n_splits*2 floats.
QNN_API int qnn_attn_decode(const void* q, long long q_stride, int dtype, const void* k_pool, const void* v_pool,
                            const int* page_table, int max_pages, int page_size, int ring, const int* slots,
                            const int* slot_len, int B, int nq, int nkv, int hd, float scale, float cap, int window,
                            float* part_o, float* part_ml, int n_splits, void* out, long long out_stride,
                            cudaStream_t st) {
    if (B <= 0) return 0;
    if (n_splits < 1 || n_splits > 65535 || B > 65535) return QNN_ERR_ARGUMENT;
    if (dtype == QNN_DT_BF16)
        return decode_launch<bf16>(q, q_stride, k_pool, v_pool, page_table, max_pages, page_size, ring, slots, slot_len,
                                   B, nq, nkv, hd, scale, cap, window, part_o, part_ml, n_splits, out, out_stride, st);
    return decode_launch<float>(q, q_stride, k_pool, v_pool, page_table, max_pages, page_size, ring, slots, slot_len, B,
                                nq, nkv, hd, scale, cap, window, part_o, part_ml, n_splits, out, out_stride, st);
}

template <typename T>
static int prefill_launch(const void* q, long long q_stride, const void* k, const void* v, long long row_stride,
                          void* out, long long out_stride, const int* tok_pos, const int* tok_row0, int n_tokens,
                          int nq, int nkv, int hd, float scale, float cap, int window, const int* page_table,
                          int max_pages, int page_size, int ring, bool paged, cudaStream_t st) {
    if (nkv <= 0 || nq % nkv) return QNN_ERR_ARGUMENT;
    const Geometry geo = geometry<T>(hd, nq / nkv);
    if (!geo.ok) return QNN_ERR_UNSUPPORTED;
    if ((q_stride * sizeof(T)) % 16 || (row_stride * sizeof(T)) % 16 || (out_stride * sizeof(T)) % 16 ||
        (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15))
        return QNN_ERR_ARGUMENT;
    const int gtiles = (nq / nkv + geo.gt - 1) / geo.gt;
    dim3 grid((n_tokens + PRE_WARPS - 1) / PRE_WARPS, nkv * gtiles);
    QNN_DISPATCH_ALL({
        if (paged)
            attn_prefill_generic_kernel<T, CPL, GT, true><<<grid, PRE_WARPS * 32, 0, st>>>(
                (const T*)q, (size_t)q_stride, (const T*)k, (const T*)v, (size_t)row_stride, (T*)out,
                (size_t)out_stride, tok_pos, tok_row0, n_tokens, nq, nkv, hd, geo.lpt, scale, cap, window, page_table,
                max_pages, page_size, ring);
        else
            attn_prefill_generic_kernel<T, CPL, GT, false><<<grid, PRE_WARPS * 32, 0, st>>>(
                (const T*)q, (size_t)q_stride, (const T*)k, (const T*)v, (size_t)row_stride, (T*)out,
                (size_t)out_stride, tok_pos, tok_row0, n_tokens, nq, nkv, hd, geo.lpt, scale, cap, window, page_table,
                max_pages, page_size, ring);
    })
    QNN_LAUNCH_CHECK();
}

// q, k, v: rows of this step's projections (row_stride elements apart); key p of the
// sequence of token t is row tok_row0[t] + p.  tok_row0[t] < 0 marks padding (zeros out).
QNN_API int qnn_attn_prefill_generic(const void* q, const void* k, const void* v, long long row_stride, int dtype,
                                     void* out, long long out_stride, const int* tok_pos, const int* tok_row0,
                                     int n_tokens, int nq, int nkv, int hd, float scale, float cap, int window,
                                     cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (dtype == QNN_DT_BF16)
        return prefill_launch<bf16>(q, row_stride, k, v, row_stride, out, out_stride, tok_pos, tok_row0, n_tokens, nq,
                                    nkv, hd, scale, cap, window, nullptr, 0, 1, 0, false, st);
    return prefill_launch<float>(q, row_stride, k, v, row_stride, out, out_stride, tok_pos, tok_row0, n_tokens, nq, nkv,
                                 hd, scale, cap, window, nullptr, 0, 1, 0, false, st);
}

// Several query rows per sequence against the paged cache: token t of the sequence in slot
// tok_slot[t] at position tok_pos[t] sees the cached positions up to its own.  With a ring
// the caller must make sure that no needed position has been overwritten.
QNN_API int qnn_attn_prefill_paged(const void* q, long long q_stride, int dtype, const void* k_pool, const void* v_pool,
                                   const int* page_table, int max_pages, int page_size, int ring, void* out,
                                   long long out_stride, const int* tok_pos, const int* tok_slot, int n_tokens, int nq,
                                   int nkv, int hd, float scale, float cap, int window, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (dtype == QNN_DT_BF16)
        return prefill_launch<bf16>(q, q_stride, k_pool, v_pool, 0, out, out_stride, tok_pos, tok_slot, n_tokens, nq,
                                    nkv, hd, scale, cap, window, page_table, max_pages, page_size, ring, true, st);
    return prefill_launch<float>(q, q_stride, k_pool, v_pool, 0, out, out_stride, tok_pos, tok_slot, n_tokens, nq, nkv,
                                 hd, scale, cap, window, page_table, max_pages, page_size, ring, true, st);
}

// What the generic attention kernels share: the lane-group walk over keys with its online softmax, the
// merge of a warp's lane groups, the geometry that a head size gets, and the dispatch over it.
// Included by attention.cu (decode: one query row per sequence against the paged cache) and by
// attention_rows.cu (whole prompts and continued sequences: many rows a step).  See the head of
// attention.cu for the scheme and the reference.
#pragma once
#include "common.cuh"
#include <math_constants.h>

using namespace qnn;

namespace {

// expf in the float32 path, the fast exponential where the data are bfloat16 anyway
template <typename T> __device__ __forceinline__ float fexp(float x);
template <> __device__ __forceinline__ float fexp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ float fexp<bf16>(float x) { return __expf(x); }

// softcap with the exact tanhf in the float32 path and the hardware tanh where the data are
// bfloat16 (its error, about 2^-11, is below bfloat16's own rounding)
template <typename T> __device__ __forceinline__ float softcap_t(float x, float cap);
template <> __device__ __forceinline__ float softcap_t<float>(float x, float cap) { return softcap(x, cap); }
template <> __device__ __forceinline__ float softcap_t<bf16>(float x, float cap) {
    if (cap > 0.f) {
        float t = fminf(fmaxf(__fdividef(x, cap), -20.f), 20.f), r;
        asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(t));
        return cap * r;
    }
    return x;
}

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

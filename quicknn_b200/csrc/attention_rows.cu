// Generic attention for steps of many rows: whole prompts from this step's own packed projections,
// prompts whose keys lie in the paged cache (layers that read another layer's cache line), and
// sequences continued by several tokens (cached keys before the step, the step's own rows from there on).
// One warp per (token, kv head, head tile); float32 and bfloat16, any head size that is a multiple of 16
// bytes of elements.  The scheme and the reference are described at the head of attention.cu.
#include "attention_generic.cuh"

namespace {

constexpr int PRE_WARPS = 4;

// After the lane groups of a warp have been merged: group 0 normalises and stores the rows of
// the head tile.
template <typename T, int CPL, int GT>
__device__ __forceinline__ void store_rows(T* __restrict__ out_row, int kh, int G, int gt0, int hd, int LPT, int chunks,
                                           const float (&l)[GT], const float (&o)[GT][CPL][Vec16<T>::N]) {
    constexpr int VEC = Vec16<T>::N;
    const int lane = threadIdx.x & 31, sl = lane % LPT, ti = lane / LPT;
    if (ti != 0) return;
#pragma unroll
    for (int g = 0; g < GT; ++g) {
        if (gt0 + g >= G) continue;
        const float inv = l[g] > 0.f ? 1.f / l[g] : 0.f;
        T* dst = out_row + (size_t)(kh * G + gt0 + g) * hd;
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
    pdl_wait();
    constexpr int VEC = Vec16<T>::N;
    const int warp = threadIdx.x >> 5;
    const int t = blockIdx.x * PRE_WARPS + warp;
    if (t >= n_tokens) return;
    const int G = nq / nkv, gtiles = (G + GT - 1) / GT;
    const int kh = blockIdx.y / gtiles, gt0 = (blockIdx.y % gtiles) * GT;
    const int chunks = hd / VEC;
    const int TPW = 32 / LPT;
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
    store_rows<T, CPL, GT>(out + (size_t)t * out_stride, kh, G, gt0, hd, LPT, chunks, l, o);
}

// A step that continues sequences by several tokens (or starts some and continues others): token t
// of the sequence in slot tok_slot[t] at position tok_pos[t] sees the cached positions before its
// sequence's first token of this step from the paged cache (k_pool, v_pool: what earlier steps wrote;
// this step's keys are appended only after this kernel, so that a ring may be as short as the window)
// and the positions from there up to its own from this step's packed projections (k, v).  The first
// packed row of the token's sequence is tok_row0[t]; that row's position is the sequence's length
// before the step.
template <typename T, int CPL, int GT>
__global__ void __launch_bounds__(PRE_WARPS * 32)
attn_extend_generic_kernel(const T* __restrict__ q, size_t q_stride, const T* __restrict__ k, const T* __restrict__ v,
                           size_t row_stride, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                           T* __restrict__ out, size_t out_stride, const int* __restrict__ tok_pos,
                           const int* __restrict__ tok_row0, const int* __restrict__ tok_slot, int n_tokens, int nq,
                           int nkv, int hd, int LPT, float scale, float cap, int window,
                           const int* __restrict__ page_table, int max_pages, int page_size, int ring) {
    pdl_wait();
    constexpr int VEC = Vec16<T>::N;
    const int warp = threadIdx.x >> 5;
    const int t = blockIdx.x * PRE_WARPS + warp;
    if (t >= n_tokens) return;
    const int G = nq / nkv, gtiles = (G + GT - 1) / GT;
    const int kh = blockIdx.y / gtiles, gt0 = (blockIdx.y % gtiles) * GT;
    const int chunks = hd / VEC;
    const int TPW = 32 / LPT;
    const int slot = tok_slot[t];

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
        const int p = tok_pos[t], row0 = tok_row0[t];
        const int first = p - (t - row0);                 // position of the sequence's first token of this step
        const int end = p + 1;
        const int begin = (window > 0 && end > window) ? end - window : 0;
        float qr[GT][CPL][VEC];
        load_query<T, CPL, GT>(q + (size_t)t * q_stride + (size_t)kh * G * hd, hd, G, gt0, LPT, chunks, scale, qr);
        if (begin < first) {
            PagedKV<T> kv{k_pool, v_pool, page_table + (size_t)slot * max_pages, page_size, nkv, hd, ring, kh};
            attend_range<T, CPL, GT>(qr, kv, begin, first, 0, TPW, LPT, chunks, cap, m, l, o);
        }
        PackedKV<T> kv{k + (size_t)kh * hd, v + (size_t)kh * hd, row_stride, row0 - first};
        attend_range<T, CPL, GT>(qr, kv, begin > first ? begin : first, end, 0, TPW, LPT, chunks, cap, m, l, o);
    }
    merge_groups<CPL, GT, VEC>(LPT, m, l, o);
    store_rows<T, CPL, GT>(out + (size_t)t * out_stride, kh, G, gt0, hd, LPT, chunks, l, o);
}

}  // namespace

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
            qnn::launch_pdl(attn_prefill_generic_kernel<T, CPL, GT, true>, dim3(grid), dim3(PRE_WARPS * 32), 0, st, 
                (const T*)q, (size_t)q_stride, (const T*)k, (const T*)v, (size_t)row_stride, (T*)out,
                (size_t)out_stride, tok_pos, tok_row0, n_tokens, nq, nkv, hd, geo.lpt, scale, cap, window, page_table,
                max_pages, page_size, ring);
        else
            qnn::launch_pdl(attn_prefill_generic_kernel<T, CPL, GT, false>, dim3(grid), dim3(PRE_WARPS * 32), 0, st, 
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

// Cached keys before this step's tokens, this step's own rows from there on (see
// attn_extend_generic_kernel).  q, k, v: this step's packed, already rotated projections.
template <typename T>
static int extend_launch(const void* q, const void* k, const void* v, long long row_stride, const void* k_pool,
                         const void* v_pool, const int* page_table, int max_pages, int page_size, int ring, void* out,
                         long long out_stride, const int* tok_pos, const int* tok_row0, const int* tok_slot, int n_tokens,
                         int nq, int nkv, int hd, float scale, float cap, int window, cudaStream_t st) {
    if (nkv <= 0 || nq % nkv) return QNN_ERR_ARGUMENT;
    const Geometry geo = geometry<T>(hd, nq / nkv);
    if (!geo.ok) return QNN_ERR_UNSUPPORTED;
    if ((row_stride * sizeof(T)) % 16 || (out_stride * sizeof(T)) % 16 ||
        (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15))
        return QNN_ERR_ARGUMENT;
    const int gtiles = (nq / nkv + geo.gt - 1) / geo.gt;
    dim3 grid((n_tokens + PRE_WARPS - 1) / PRE_WARPS, nkv * gtiles);
    QNN_DISPATCH_ALL({
        qnn::launch_pdl(attn_extend_generic_kernel<T, CPL, GT>, dim3(grid), dim3(PRE_WARPS * 32), 0, st, (const T*)q,
                        (size_t)row_stride, (const T*)k, (const T*)v, (size_t)row_stride, (const T*)k_pool,
                        (const T*)v_pool, (T*)out, (size_t)out_stride, tok_pos, tok_row0, tok_slot, n_tokens, nq, nkv, hd,
                        geo.lpt, scale, cap, window, page_table, max_pages, page_size, ring);
    })
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_attn_extend(const void* q, const void* k, const void* v, long long row_stride, int dtype,
                            const void* k_pool, const void* v_pool, const int* page_table, int max_pages, int page_size,
                            int ring, void* out, long long out_stride, const int* tok_pos, const int* tok_row0,
                            const int* tok_slot, int n_tokens, int nq, int nkv, int hd, float scale, float cap,
                            int window, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (dtype == QNN_DT_BF16)
        return extend_launch<bf16>(q, k, v, row_stride, k_pool, v_pool, page_table, max_pages, page_size, ring, out,
                                   out_stride, tok_pos, tok_row0, tok_slot, n_tokens, nq, nkv, hd, scale, cap, window, st);
    return extend_launch<float>(q, k, v, row_stride, k_pool, v_pool, page_table, max_pages, page_size, ring, out,
                                out_stride, tok_pos, tok_row0, tok_slot, n_tokens, nq, nkv, hd, scale, cap, window, st);
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

// ---------------------------------------------------------------------------------
// Whole sequences laid out as rows, for the tensor-core prompt kernel: sequence b, whose first seq_start[b]
// tokens are cached and which brings seq_len[b] new rows in `qkv`, gets rows whole_row0[b] .. of `whole`
// ([rows, (nq + 2 nkv) * hd] bfloat16): a cached position carries its keys and values from the paged cache (zeros
// where a ring no longer holds it, and in the query columns), a new position the step's own projections.
// qnn_attn_prefill_tcgen05 with seq_q0 = seq_start then computes the new rows against everything before them.
// grid (longest whole sequence, sequences).
// ---------------------------------------------------------------------------------
__global__ void extend_gather_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ k_pool,
                                     const bf16* __restrict__ v_pool, const int* __restrict__ page_table, int max_pages,
                                     int page_size, int ring, const int* __restrict__ slots,
                                     const int* __restrict__ seq_start, const int* __restrict__ seq_row0,
                                     const int* __restrict__ seq_len, const int* __restrict__ whole_row0,
                                     bf16* __restrict__ whole, int nq, int nkv, int hd) {
    pdl_wait();
    const int p = blockIdx.x, b = blockIdx.y;
    const int start = seq_start[b], n = seq_len[b];
    if (p >= start + n) return;
    const int width = (nq + 2 * nkv) * hd, chunks = width / 8;
    uint4* dst = reinterpret_cast<uint4*>(whole + ((size_t)whole_row0[b] + p) * width);
    if (p >= start) {
        const uint4* src = reinterpret_cast<const uint4*>(qkv + ((size_t)seq_row0[b] + (p - start)) * width);
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) dst[c] = src[c];
        return;
    }
    const int slot = slots[b];
    const bool held = slot >= 0 && (ring <= 0 || p >= start - ring);
    const int r = ring > 0 ? p % ring : p;
    size_t base = 0;
    if (held) {
        const int page = page_table[(size_t)slot * max_pages + r / page_size];
        base = ((size_t)page * nkv * page_size + (r % page_size)) * hd;
    }
    const int qc = nq * hd / 8, hc = hd / 8, kvc = nkv * hc;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
        uint4 v = zero;
        if (held && c >= qc) {
            const int e = c - qc;
            const bf16* pool = e < kvc ? k_pool : v_pool;
            const int e2 = e < kvc ? e : e - kvc;
            const int kh = e2 / hc, d = (e2 % hc) * 8;
            v = *reinterpret_cast<const uint4*>(pool + base + (size_t)kh * page_size * hd + d);
        }
        dst[c] = v;
    }
}

QNN_API int qnn_attn_extend_gather(const void* qkv, const void* k_pool, const void* v_pool, const int* page_table,
                                   int max_pages, int page_size, int ring, const int* slots, const int* seq_start,
                                   const int* seq_row0, const int* seq_len, const int* whole_row0, void* whole, int B,
                                   int longest, int nq, int nkv, int hd, cudaStream_t st) {
    if (B <= 0 || longest <= 0) return 0;
    if (hd <= 0 || (hd & 7) || page_size <= 0 || B > 65535) return QNN_ERR_UNSUPPORTED;
    if ((((uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)whole) & 15)) return QNN_ERR_ARGUMENT;
    qnn::launch_pdl(extend_gather_kernel, dim3((unsigned)longest, (unsigned)B), dim3(128), 0, st, (const bf16*)qkv,
                    (const bf16*)k_pool, (const bf16*)v_pool, page_table, max_pages, page_size, ring, slots, seq_start,
                    seq_row0, seq_len, whole_row0, (bf16*)whole, nq, nkv, hd);
    QNN_LAUNCH_CHECK();
}

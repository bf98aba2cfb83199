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
#include "attention_generic.cuh"

namespace {

constexpr int DEC_WARPS = 4;

// The warps of a CTA hand their states to shared memory; the threads that own a dimension
// merge them in warp order and write the CTA's partial (max, sum, O) for its split.
template <int CPL, int GT, int VEC>
__device__ __forceinline__ void write_partials(float* smem, const float (&m)[GT], const float (&l)[GT],
                                               const float (&o)[GT][CPL][VEC], int hd, int LPT, int chunks, int G,
                                               int gt0, int kh, int nq, int b, int split, int n_splits,
                                               float* __restrict__ part_o, float* __restrict__ part_ml) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sl = lane % LPT, ti = lane / LPT;
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


template <typename T, int CPL, int GT>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_kernel(const T* __restrict__ q, size_t q_stride, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                   const int* __restrict__ page_table, int max_pages, int page_size, int ring,
                   const int* __restrict__ slots, const int* __restrict__ slot_len, int nq, int nkv, int hd, int LPT,
                   float scale, float cap, int window, float* __restrict__ part_o, float* __restrict__ part_ml,
                   int n_splits) {
    pdl_wait();
    constexpr int VEC = Vec16<T>::N;
    extern __shared__ float smem[];  // [DEC_WARPS][GT][hd + 2]
    const int split = blockIdx.x, b = blockIdx.z;
    const int G = nq / nkv, gtiles = (G + GT - 1) / GT;
    const int kh = blockIdx.y / gtiles, gt0 = (blockIdx.y % gtiles) * GT;
    const int warp = threadIdx.x >> 5;
    const int chunks = hd / VEC;
    const int TPW = 32 / LPT;
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
    write_partials<CPL, GT, VEC>(smem, m, l, o, hd, LPT, chunks, G, gt0, kh, nq, b, split, n_splits, part_o, part_ml);
}

// The tiled, pipelined decode kernel.  Same grid, same scratch and same results (up to
// rounding) as attn_decode_kernel, but
//   * a lane group takes TT keys per step instead of one, and the keys and values of the next
//     steps are already on their way: every warp owns DEC_STAGES buffers in shared memory that it
//     fills with cp.async (16 bytes per lane, zero-filled beyond the end of its range), so about
//     two tiles per warp are in flight while the third is being worked on;
//   * the GT*TT partial dot products of a lane are summed over the group by a transposed
//     reduction (each exchange halves what a lane still carries: GT*TT - 1 shuffles instead of
//     GT*TT*log2(LPT)), after which every score lives on one lane (replicated LPT/(GT*TT) times),
//     so softcap and exp are evaluated once per score, not once per lane;
//   * the running maximum is updated once per tile, so O is rescaled once per TT keys.
// Needs GT*TT <= LPT and a page size that is a power of two.
constexpr int DEC_STAGES = 3;

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src, bool valid) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(gmem_src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

template <typename T, int CPL, int GT, int TT>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_tiled_kernel(const T* __restrict__ q, size_t q_stride, const T* __restrict__ k_pool,
                         const T* __restrict__ v_pool, const int* __restrict__ page_table, int max_pages,
                         int page_size, int ring, const int* __restrict__ slots, const int* __restrict__ slot_len,
                         int nq, int nkv, int hd, int LPT, float scale, float cap, int window,
                         float* __restrict__ part_o, float* __restrict__ part_ml, int n_splits) {
    pdl_wait();
    constexpr int VEC = Vec16<T>::N;
    constexpr int NV = GT * TT;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int split = blockIdx.x, b = blockIdx.z;
    const int G = nq / nkv, gtiles = (G + GT - 1) / GT;
    const int kh = blockIdx.y / gtiles, gt0 = (blockIdx.y % gtiles) * GT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = hd / VEC;
    const int sl = lane % LPT, grp = lane / LPT, TPW = 32 / LPT;
    const int group_base = grp * LPT;
    const int R = LPT / NV;                    // lanes that hold the same score after the reduction
    const int my_idx = sl / R, my_g = my_idx / TT, my_tt = my_idx % TT;
    const int slot = slots[b];
    const int tile = TT * TPW;                 // keys per warp step
    const size_t tile_elems = (size_t)tile * hd;
    // this warp's buffers: [stage][K | V][key of the tile][hd]
    T* wbuf = reinterpret_cast<T*>(smem_raw) + (size_t)warp * DEC_STAGES * 2 * tile_elems;
    int* pages_s = reinterpret_cast<int*>(reinterpret_cast<T*>(smem_raw) + (size_t)DEC_WARPS * DEC_STAGES * 2 * tile_elems);

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
            // The page ids of this CTA's key range go to shared memory once, so that the fetches
            // below do not wait on a lookup in global memory.  Entry u is the page of the u-th
            // page-sized stretch counted from the range's first key (unwrapped over a ring).
            const int page_shift = 31 - __clz(page_size), page_mask = page_size - 1;
            const int* page_row = page_table + (size_t)slot * max_pages;
            const int rb0 = ring > 0 ? begin % ring : begin;
            const int first_pg = rb0 >> page_shift;
            const int npg = ((rb0 + (end - begin) - 1) >> page_shift) - first_pg + 1;
            const int ring_pages = ring > 0 ? ring >> page_shift : 0x7fffffff;
            for (int u = threadIdx.x; u < npg; u += blockDim.x) {
                int pi = first_pg + u;
                if (pi >= ring_pages) pi -= ring_pages;
                pages_s[u] = page_row[pi];
            }
            __syncthreads();
            const int first = begin + warp * tile, stride = DEC_WARPS * tile;
            const int my_tiles = first < end ? (end - first + stride - 1) / stride : 0;

            // fetch tile `it` of this warp into stage it % DEC_STAGES
            auto fetch = [&](int it) {
                if (it < my_tiles) {
                    const int base = first + it * stride;
                    T* kst = wbuf + (size_t)(it % DEC_STAGES) * 2 * tile_elems;
                    T* vst = kst + tile_elems;
                    const int rbase = rb0 + (base - begin);            // unwrapped place in the ring
#pragma unroll
                    for (int tt = 0; tt < TT; ++tt) {
                        const int j = tt * TPW + grp;
                        const bool valid = base + j < end;
                        const int r = rbase + j;
                        const int page = valid ? pages_s[(r >> page_shift) - first_pg] : 0;
                        const size_t off = ((size_t)(page * nkv + kh) * page_size + (r & page_mask)) * hd;
#pragma unroll
                        for (int i = 0; i < CPL; ++i) {
                            const int c = sl + i * LPT;
                            if (c < chunks) {
                                cp_async_16(kst + (size_t)j * hd + c * VEC, k_pool + off + c * VEC, valid);
                                cp_async_16(vst + (size_t)j * hd + c * VEC, v_pool + off + c * VEC, valid);
                            }
                        }
                    }
                }
                cp_async_commit();   // an empty group keeps the count of outstanding groups uniform
            };
#pragma unroll
            for (int it = 0; it < DEC_STAGES - 1; ++it) fetch(it);

            for (int it = 0; it < my_tiles; ++it) {
                fetch(it + DEC_STAGES - 1);
                cp_async_wait<DEC_STAGES - 1>();
                __syncwarp();
                const int base = first + it * stride;
                const T* kst = wbuf + (size_t)(it % DEC_STAGES) * 2 * tile_elems;
                const T* vst = kst + tile_elems;
                float s[NV];
#pragma unroll
                for (int j = 0; j < NV; ++j) s[j] = 0.f;
#pragma unroll
                for (int tt = 0; tt < TT; ++tt)
#pragma unroll
                    for (int i = 0; i < CPL; ++i) {
                        const int c = sl + i * LPT;
                        if (c < chunks) {
                            Vec16<T> kv_;
                            kv_.load(kst + (size_t)(tt * TPW + grp) * hd + c * VEC);
                            float kk[VEC];
                            kv_.unpack(kk);
#pragma unroll
                            for (int g = 0; g < GT; ++g)
#pragma unroll
                                for (int e = 0; e < VEC; ++e) s[g * TT + tt] = fmaf(qr[g][i][e], kk[e], s[g * TT + tt]);
                        }
                    }
                // transposed reduction over the LPT lanes of the group
                int d = LPT >> 1;
#pragma unroll
                for (int h = NV / 2; h >= 1; h >>= 1) {
                    const bool upper = (sl & d) != 0;
#pragma unroll
                    for (int j = 0; j < h; ++j) {
                        const float keep = upper ? s[j + h] : s[j];
                        const float send = upper ? s[j] : s[j + h];
                        s[j] = keep + __shfl_xor_sync(0xffffffffu, send, d);
                    }
                    d >>= 1;
                }
                float sc = s[0];
                for (; d >= 1; d >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, d);
                // this lane now owns the score of (head my_g, key my_tt of the tile)
                const bool mine = (base + my_tt * TPW + grp) < end;
                sc = mine ? softcap_t<T>(sc, cap) : -CUDART_INF_F;
                float tmax = sc;
                for (int off = R; off < R * TT; off <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
                float m_old = m[0];
#pragma unroll
                for (int g = 1; g < GT; ++g) m_old = (my_g == g) ? m[g] : m_old;
                const float m_new = fmaxf(m_old, tmax);
                float pw = (m_new == -CUDART_INF_F) ? 0.f : fexp<T>(sc - m_new);
                float tsum = pw;
                for (int off = R; off < R * TT; off <<= 1) tsum += __shfl_xor_sync(0xffffffffu, tsum, off);
#pragma unroll
                for (int g = 0; g < GT; ++g) {
                    const int src = group_base + (g * TT) * R;
                    const float mg = __shfl_sync(0xffffffffu, m_new, src);
                    const float ls = __shfl_sync(0xffffffffu, tsum, src);
                    const float corr = (mg == -CUDART_INF_F) ? 1.f : fexp<T>(m[g] - mg);
                    l[g] = l[g] * corr + ls;
                    m[g] = mg;
#pragma unroll
                    for (int i = 0; i < CPL; ++i)
#pragma unroll
                        for (int e = 0; e < VEC; ++e) o[g][i][e] *= corr;
                }
#pragma unroll
                for (int tt = 0; tt < TT; ++tt) {
                    float pg[GT];
#pragma unroll
                    for (int g = 0; g < GT; ++g) pg[g] = __shfl_sync(0xffffffffu, pw, group_base + (g * TT + tt) * R);
#pragma unroll
                    for (int i = 0; i < CPL; ++i) {
                        const int c = sl + i * LPT;
                        if (c < chunks) {
                            Vec16<T> vv_;
                            vv_.load(vst + (size_t)(tt * TPW + grp) * hd + c * VEC);
                            float vv[VEC];
                            vv_.unpack(vv);
#pragma unroll
                            for (int g = 0; g < GT; ++g)
#pragma unroll
                                for (int e = 0; e < VEC; ++e) o[g][i][e] = fmaf(pg[g], vv[e], o[g][i][e]);
                        }
                    }
                }
                __syncwarp();   // everybody is done with this stage before a later fetch refills it
            }
            cp_async_wait<0>();
        }
    }
    merge_groups<CPL, GT, VEC>(LPT, m, l, o);
    __syncthreads();            // the stage buffers are free now: reuse them for the merge of the warps
    write_partials<CPL, GT, VEC>(reinterpret_cast<float*>(smem_raw), m, l, o, hd, LPT, chunks, G, gt0, kh, nq, b, split,
                                 n_splits, part_o, part_ml);
}

// out[b, h, :] = sum_s e^{m_s - M} O_s / sum_s e^{m_s - M} l_s.  The block is cut into G groups of hd/4
// threads; group g adds up splits g, g + G, g + 2G, ... (four head elements per thread, 16-byte loads that
// do not wait for one another), and the G partial sums are added in ascending order of g: an order that
// depends on the number of splits and the head size only.
template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                    T* __restrict__ out, size_t out_stride, int nq, int hd, int n_splits) {
    pdl_wait();
    extern __shared__ __align__(16) float comb[];  // [G][hd] partial sums, then [n_splits] weights and 1/sum
    const int lpg = hd / 4, G = max(1, min((int)blockDim.x / lpg, n_splits));
    float* coef = comb + max((size_t)G * hd, (size_t)n_splits);
    const int b = blockIdx.x / nq, h = blockIdx.x % nq;
    const size_t pbase = ((size_t)b * nq + h) * n_splits;
    // A thread's first partial outputs do not depend on the ranges' weights: they are asked for first, and
    // the (maximum, sum) pairs right after, so that the kernel waits for global memory once.
    constexpr int AHEAD = 4;
    const int g = threadIdx.x / lpg, c = (threadIdx.x % lpg) * 4;
    float4 first[AHEAD];
#pragma unroll
    for (int i = 0; i < AHEAD; ++i) {
        const int s = g + i * G;
        first[i] = (g < G && s < n_splits) ? *reinterpret_cast<const float4*>(part_o + (pbase + s) * hd + c)
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (threadIdx.x < 32) {
        // every (maximum, sum) pair is loaded once (up to 128 ranges stay in registers between the two passes);
        // the weighted sums go through shared memory so that one thread can add them in ascending order
        // without waiting for global memory at every term
        float* wl = comb;                                   // [n_splits], before the partial sums take the space
        float2 ml[4];
        float mm = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int s = threadIdx.x + i * 32;
            ml[i] = s < n_splits ? *reinterpret_cast<const float2*>(part_ml + (pbase + s) * 2) : make_float2(-CUDART_INF_F, 0.f);
            mm = fmaxf(mm, ml[i].x);
        }
        for (int s = threadIdx.x + 128; s < n_splits; s += 32) mm = fmaxf(mm, part_ml[(pbase + s) * 2]);
        mm = warp_max(mm);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int s = threadIdx.x + i * 32;
            if (s < n_splits) {
                const float w = (ml[i].x == -CUDART_INF_F) ? 0.f : expf(ml[i].x - mm);
                coef[s] = w;
                wl[s] = w * ml[i].y;
            }
        }
        for (int s = threadIdx.x + 128; s < n_splits; s += 32) {
            const float2 v = *reinterpret_cast<const float2*>(part_ml + (pbase + s) * 2);
            const float w = (v.x == -CUDART_INF_F) ? 0.f : expf(v.x - mm);
            coef[s] = w;
            wl[s] = w * v.y;
        }
        __syncwarp();
        if (threadIdx.x == 0) {
            float ll = 0.f;
            for (int s = 0; s < n_splits; ++s) ll += wl[s];   // ascending order
            coef[n_splits] = ll > 0.f ? 1.f / ll : 0.f;
        }
    }
    __syncthreads();
    if (g < G) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int i = 0; i < AHEAD; ++i) {
            const int s = g + i * G;
            if (s < n_splits) {
                const float w = coef[s];
                acc.x += w * first[i].x;
                acc.y += w * first[i].y;
                acc.z += w * first[i].z;
                acc.w += w * first[i].w;
            }
        }
#pragma unroll 4
        for (int s = g + AHEAD * G; s < n_splits; s += G) {
            const float w = coef[s];
            const float4 v = *reinterpret_cast<const float4*>(part_o + (pbase + s) * hd + c);
            acc.x += w * v.x;
            acc.y += w * v.y;
            acc.z += w * v.z;
            acc.w += w * v.w;
        }
        *reinterpret_cast<float4*>(comb + (size_t)g * hd + c) = acc;
    }
    __syncthreads();
    const float inv = coef[n_splits];
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.f;
        for (int gg = 0; gg < G; ++gg) acc += comb[(size_t)gg * hd + d];
        out[(size_t)b * out_stride + (size_t)h * hd + d] = from_f<T>(acc * inv);
    }
}

}  // namespace

extern "C" int qnn_attn_decode_mma_split(const void* q, long long q_stride, const void* k_pool, const void* v_pool,
                                         const int* page_table, int max_pages, int page_size, int ring,
                                         const int* slots, const int* slot_len, int B, int nq, int nkv, int hd,
                                         float scale, float cap, int window, float* part_o, float* part_ml,
                                         int n_splits, void* out, long long out_stride, int* combined,
                                         cudaStream_t st);

// threads of the combine kernel's block: a group of hd/4 threads for every key range, up to 1024; and the
// groups that such a block has (see attn_combine_kernel)
static int combine_threads(int hd, int n_splits) {
    const int lpg = hd / 4 > 0 ? hd / 4 : 1;
    long long t = ((long long)lpg * n_splits + 31) / 32 * 32;
    if (t < 64) t = 64;
    const int most = lpg > 1024 ? lpg : 1024;      // at least one whole group
    return (int)(t > most ? most : t);
}
static int combine_groups(int hd, int n_splits) {
    const int lpg = hd / 4;
    int g = lpg > 0 ? combine_threads(hd, n_splits) / lpg : 1;
    if (g > n_splits) g = n_splits;
    return g < 1 ? 1 : g;
}

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
#define QNN_DEC_ARGS                                                                                              \
    (const T*)q, (size_t)q_stride, (const T*)k_pool, (const T*)v_pool, page_table, max_pages, page_size, ring, slots, \
        slot_len, nq, nkv, hd, geo.lpt, scale, cap, window, part_o, part_ml, n_splits
    int tt = (geo.cpl == 1 && geo.gt * 8 <= geo.lpt) ? 8 : ((geo.cpl <= 2 && geo.gt * 4 <= geo.lpt) ? 4 : 0);
    if (page_size <= 0 || (page_size & (page_size - 1)) || (ring > 0 && ring < 8 * 32)) tt = 0;   // the tiled kernel's address arithmetic
    bool launched = false;
    if (sizeof(T) == 2) {   // bfloat16: the tensor-core kernel where it takes the sizes
        int combined = 0;
        const int rc = qnn_attn_decode_mma_split(q, q_stride, k_pool, v_pool, page_table, max_pages, page_size, ring,
                                                 slots, slot_len, B, nq, nkv, hd, scale, cap, window, part_o, part_ml,
                                                 n_splits, out, out_stride, &combined, st);
        if (rc == 0 && combined) return 0;            // merged inside the kernel's clusters
        if (rc == 0) launched = true;
        else if (rc != QNN_ERR_UNSUPPORTED) return rc;
    }
    const size_t tile_bytes = (size_t)tt * (32 / geo.lpt) * hd * sizeof(T) * 2;
    size_t smem_tiled = (size_t)DEC_WARPS * DEC_STAGES * tile_bytes;
    if (smem_tiled < smem) smem_tiled = smem;      // the merge of the warps reuses the stage buffers
    smem_tiled += ((size_t)max_pages + 2) * sizeof(int);   // page ids of the CTA's key range
    if (smem_tiled > 100 * 1024) tt = 0;
#define QNN_TILED(CPLV, GTV, TTV)                                                                          \
    if (!launched && geo.cpl == CPLV && geo.gt == GTV && tt == TTV) {                                        \
        auto kern = attn_decode_tiled_kernel<T, CPLV, GTV, TTV>;                                            \
        static bool configured = false;                                                                     \
        if (!configured) {                                                                                  \
            cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
            if (ce != cudaSuccess) return (int)ce;                                                          \
            configured = true;                                                                              \
        }                                                                                                   \
        qnn::launch_pdl(kern, dim3(grid), dim3(DEC_WARPS * 32), smem_tiled, st, QNN_DEC_ARGS);                                       \
        launched = true;                                                                                    \
    }
    QNN_TILED(1, 1, 8) QNN_TILED(1, 2, 8) QNN_TILED(1, 4, 8)
    QNN_TILED(1, 1, 4) QNN_TILED(1, 2, 4) QNN_TILED(1, 4, 4)
    QNN_TILED(2, 1, 4) QNN_TILED(2, 2, 4) QNN_TILED(2, 4, 4)
#undef QNN_TILED
    if (!launched) {
        QNN_DISPATCH_ALL({ qnn::launch_pdl(attn_decode_kernel<T, CPL, GT>, dim3(grid), dim3(DEC_WARPS * 32), smem, st, QNN_DEC_ARGS); })
    }
#undef QNN_DEC_ARGS
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    size_t comb_floats = (size_t)combine_groups(hd, n_splits) * hd;
    if (comb_floats < (size_t)n_splits) comb_floats = (size_t)n_splits;      // the weighted sums pass through it first
    qnn::launch_pdl(attn_combine_kernel<T>, dim3(B * nq), dim3(combine_threads(hd, n_splits)), (comb_floats + n_splits + 1) * sizeof(float), st, part_o, part_ml, (T*)out, (size_t)out_stride, nq, hd, n_splits);
    QNN_LAUNCH_CHECK();
}

// Whether the attention kernels of this file take these sizes (the checks that the launchers make, without
// launching): 0, or QNN_ERR_UNSUPPORTED / QNN_ERR_ARGUMENT.  A model asks this when it is loaded, so that an
// unsupported head size is refused there and not at the first step.
template <typename T>
static int supports(int nq, int nkv, int hd) {
    if (nkv <= 0 || nq <= 0 || nq % nkv) return QNN_ERR_ARGUMENT;
    const Geometry geo = geometry<T>(hd, nq / nkv);
    if (!geo.ok) return QNN_ERR_UNSUPPORTED;
    if ((size_t)DEC_WARPS * geo.gt * (hd + 2) * sizeof(float) > 48 * 1024) return QNN_ERR_UNSUPPORTED;
    return 0;
}
QNN_API int qnn_attn_supports(int dtype, int nq, int nkv, int hd) {
    return dtype == QNN_DT_BF16 ? supports<bf16>(nq, nkv, hd) : supports<float>(nq, nkv, hd);
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

// Decode attention over the paged cache on the tensor cores, bfloat16, for head sizes 64, 128
// and 256 and up to 8 query heads per kv head (more heads take several CTAs).
//
// Formulas: those of attention.cu (reference: src/backends/vulkan/shaders/attention.comp:18-38).
// What differs is the mapping.  One query row per sequence leaves the matrix shapes lopsided, so
// the products are taken transposed and the keys, not the queries, fill the 16-row side of
// mma.m16n8k16:
//     S^T[16 keys x 8 heads]  = K[16 keys x hd]   * Q^T[hd x 8 heads]        (A = K,   B = Q^T)
//     O^T[hd x 8 heads]      += V^T[hd x 16 keys] * P^T[16 keys x 8 heads]   (A = V^T, B = P^T)
// K and V tiles of 16 keys travel global -> shared memory by cp.async in a 3-stage pipeline per
// warp (rows XOR-swizzled by 16-byte chunk so that ldmatrix does not conflict); K fragments come
// from ldmatrix, V^T fragments from ldmatrix.trans; Q^T stays in registers for the whole kernel;
// P^T is rearranged from the accumulator layout of S^T with eight shuffles.  Softmax state
// (max, sum) is float32, one pair of heads per lane; O^T accumulates in float32.
//
// Grid (splits, kv heads x head tiles, sequences), 2 warps per CTA; the warps of a CTA interleave
// the 16-key tiles of the CTA's key range and are merged through shared memory in warp order.
// With up to 4 splits the CTAs of one (sequence, kv head) form a thread-block cluster: each leaves
// (max, sum, O) of its range in its own shared memory, and after a cluster barrier every CTA
// merges a share of the output elements over all ranks, in rank order, reading the others through
// distributed shared memory, and writes bfloat16 output: no scratch, no second kernel.  With more
// splits the CTA writes (max, sum, O) to the scratch that the combine kernel of attention.cu reads.
#include "common.cuh"
#include <math_constants.h>
#include <stdlib.h>

using namespace qnn;

namespace {

constexpr int TILE = 16;   // keys per warp step

__device__ __forceinline__ void cp_async_16(unsigned smem_dst, const void* gmem_src, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the destination is zero-filled
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
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// float at `local_addr` (a shared-memory address of this CTA) in the CTA of rank `rank`
__device__ __forceinline__ float ld_cluster(unsigned local_addr, unsigned rank) {
    unsigned remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// out[h, d] = sum_r e^{m_r - M} O_r[d] / sum_r e^{m_r - M} l_r over the ranks of the cluster in
// ascending order: the sums that the combine kernel forms from the scratch.  `cs` is this CTA's
// [head][HD + 2] (O, max, sum) in shared memory, at the same address in every CTA of the cluster;
// every CTA merges a share of the (head, d) pairs.  Kept out of line so that the main loop of the
// kernel compiles as it does without it.
template <int HD>
__device__ __noinline__ void cluster_merge(const float* cs, int S, int heads, bf16* __restrict__ out) {
    constexpr int ROW = HD + 2;
    cluster_barrier();
    const unsigned rank = cluster_rank();
    const unsigned cs_addr = (unsigned)__cvta_generic_to_shared(cs);
    for (int i = rank * blockDim.x + threadIdx.x; i < heads * HD; i += S * blockDim.x) {
        const int hh = i / HD, d = i % HD;
        const unsigned row = cs_addr + (unsigned)(hh * ROW) * 4u;
        float mr[8], lr[8], orr[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const bool on = r < S;
            mr[r] = on ? ld_cluster(row + HD * 4u, r) : -CUDART_INF_F;
            lr[r] = on ? ld_cluster(row + (HD + 1) * 4u, r) : 0.f;
            orr[r] = on ? ld_cluster(row + (unsigned)d * 4u, r) : 0.f;
        }
        float mm = -CUDART_INF_F;
#pragma unroll
        for (int r = 0; r < 8; ++r) mm = fmaxf(mm, mr[r]);
        float ll = 0.f, acc = 0.f;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            const float c = (mr[r] == -CUDART_INF_F) ? 0.f : expf(mr[r] - mm);
            ll += c * lr[r];
            acc += c * orr[r];
        }
        const float inv = ll > 0.f ? 1.f / ll : 0.f;
        out[(size_t)hh * HD + d] = __float2bfloat16(acc * inv);
    }
    cluster_barrier();                            // nobody leaves while its memory is still read
}

template <int HD, int MMA_WARPS, int MMA_STAGES>
__global__ void __launch_bounds__(MMA_WARPS * 32)
attn_decode_mma_kernel(const bf16* __restrict__ q, size_t q_stride, const bf16* __restrict__ k_pool,
                       const bf16* __restrict__ v_pool, const int* __restrict__ page_table, int max_pages,
                       int page_size, int ring, const int* __restrict__ slots, const int* __restrict__ slot_len,
                       int nq, int nkv, float scale, float cap, int window, float* __restrict__ part_o,
                       float* __restrict__ part_ml, int n_splits, bf16* __restrict__ out, size_t out_stride) {
    const bool CLUSTER = out != nullptr;         // launched as clusters of n_splits CTAs that merge their ranges
    constexpr int KSTEPS = HD / 16;              // k16 steps of S^T, and 16-row tiles of O^T
    constexpr int CH = HD / 8;                   // 16-byte chunks per row
    constexpr int ROW_BYTES = HD * 2;
    constexpr int TILE_BYTES = TILE * ROW_BYTES; // one of K or V
    constexpr int PER_LANE = TILE * CH / 32;     // cp.async per lane for K (and as many for V)
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int split = blockIdx.x, b = blockIdx.z;
    const int G = nq / nkv, htiles = (G + 7) / 8;
    const int kh = blockIdx.y / htiles, h0 = (blockIdx.y % htiles) * 8;   // first query head of this CTA within the group
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int slot = slots[b];
    const unsigned wbase = (unsigned)__cvta_generic_to_shared(smem_raw) + warp * MMA_STAGES * 2 * TILE_BYTES;
    int* pages_s = reinterpret_cast<int*>(smem_raw + (size_t)MMA_WARPS * MMA_STAGES * 2 * TILE_BYTES);

    float o[KSTEPS][4];
#pragma unroll
    for (int i = 0; i < KSTEPS; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;   // heads h0 + 2t and h0 + 2t + 1

    int begin = 0, end = 0;
    if (slot >= 0) {
        const int n = slot_len[slot];
        const int kbeg = (window > 0 && n > window) ? n - window : 0;
        const int per = (n - kbeg + n_splits - 1) / n_splits;
        begin = kbeg + split * per;
        end = min(begin + per, n);
    }
    // The sequence's length and page ids come from the host before the step, not from the kernel in front:
    // this chain of dependent loads (slot -> length -> page row) runs before the wait for that kernel, whose
    // query row and newest key are read only after it.  (Asking for the first key tiles before the wait as
    // well, all but the one with the newest key, measured no further gain.)
    const int page_shift = 31 - __clz(page_size), page_mask = page_size - 1;
    const int rb0 = ring > 0 ? begin % ring : begin;
    const int first_pg = rb0 >> page_shift;
    if (begin < end) {
        const int* page_row = page_table + (size_t)slot * max_pages;
        const int npg = ((rb0 + (end - begin) - 1) >> page_shift) - first_pg + 1;
        const int ring_pages = ring > 0 ? ring >> page_shift : 0x7fffffff;
        for (int u = threadIdx.x; u < npg; u += blockDim.x) {
            int pi = first_pg + u;
            if (pi >= ring_pages) pi -= ring_pages;
            pages_s[u] = page_row[pi];
        }
    }
    pdl_wait();
    __syncthreads();
    if (begin < end) {
        // Q^T fragments: b0 = Q[head g][16 ks + 2t, +1], b1 = Q[head g][16 ks + 8 + 2t, +1]
        uint32_t qf[KSTEPS][2];
        {
            const bool have = h0 + g < G;
            const uint32_t* qrow = reinterpret_cast<const uint32_t*>(q + (size_t)b * q_stride + (size_t)(kh * G + h0 + g) * HD);
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ++ks) {
                qf[ks][0] = have ? qrow[ks * 8 + t] : 0u;
                qf[ks][1] = have ? qrow[ks * 8 + 4 + t] : 0u;
            }
        }
        const int first = begin + warp * TILE, stride = MMA_WARPS * TILE;
        const int my_tiles = first < end ? (end - first + stride - 1) / stride : 0;

        auto fetch = [&](int it) {
            if (it < my_tiles) {
                const int base = first + it * stride;
                const unsigned kst = wbase + (it % MMA_STAGES) * 2 * TILE_BYTES, vst = kst + TILE_BYTES;
                const int rbase = rb0 + (base - begin);
#pragma unroll
                for (int i = 0; i < PER_LANE; ++i) {
                    const int idx = i * 32 + lane;
                    const int row = idx / CH, chunk = idx % CH;
                    const bool valid = base + row < end;
                    const int r = rbase + row;
                    const int page = valid ? pages_s[(r >> page_shift) - first_pg] : 0;
                    const size_t off = ((size_t)(page * nkv + kh) * page_size + (r & page_mask)) * HD + chunk * 8;
                    const unsigned dst = row * ROW_BYTES + ((chunk ^ (row & 7)) << 4);
                    cp_async_16(kst + dst, k_pool + off, valid);
                    cp_async_16(vst + dst, v_pool + off, valid);
                }
            }
            cp_async_commit();
        };
#pragma unroll
        for (int it = 0; it < MMA_STAGES - 1; ++it) fetch(it);

        const float inv_cap = cap > 0.f ? 1.f / cap : 0.f;
        for (int it = 0; it < my_tiles; ++it) {
            fetch(it + MMA_STAGES - 1);
            cp_async_wait<MMA_STAGES - 1>();
            __syncwarp();
            const int base = first + it * stride;
            const unsigned kst = wbase + (it % MMA_STAGES) * 2 * TILE_BYTES, vst = kst + TILE_BYTES;

            // S^T = K Q^T
            float s[4] = {0.f, 0.f, 0.f, 0.f};
            {
                const int row = lane & 15, half = lane >> 4;
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ++ks) {
                    uint32_t a[4];
                    const int chunk = ks * 2 + half;
                    ldmatrix_x4(a, kst + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4));
                    mma_16816(s, a, qf[ks][0], qf[ks][1]);
                }
            }
            // s[0], s[1]: key base+g, heads 2t, 2t+1;  s[2], s[3]: key base+g+8
            const bool v_lo = base + g < end, v_hi = base + g + 8 < end;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float x = s[j] * scale;
                if (cap > 0.f) x = cap * tanh_fast(fminf(fmaxf(x * inv_cap, -20.f), 20.f));
                s[j] = ((j < 2) ? v_lo : v_hi) ? x : -CUDART_INF_F;
            }
            float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
            }
            const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);    // finite: every tile has a valid key
            const float c0 = __expf(m0 - mn0), c1 = __expf(m1 - mn1);
            float p[4];
            p[0] = __expf(s[0] - mn0);
            p[1] = __expf(s[1] - mn1);
            p[2] = __expf(s[2] - mn0);
            p[3] = __expf(s[3] - mn1);
            float ls0 = p[0] + p[2], ls1 = p[1] + p[3];
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                ls0 += __shfl_xor_sync(0xffffffffu, ls0, off);
                ls1 += __shfl_xor_sync(0xffffffffu, ls1, off);
            }
            l0 = l0 * c0 + ls0;
            l1 = l1 * c1 + ls1;
            m0 = mn0;
            m1 = mn1;
#pragma unroll
            for (int i = 0; i < KSTEPS; ++i) {
                o[i][0] *= c0;
                o[i][1] *= c1;
                o[i][2] *= c0;
                o[i][3] *= c1;
            }
            // P^T fragments for B: b0 = P[key 2t, 2t+1][head g], b1 = P[key 2t+8, 2t+9][head g];
            // P[key a][head g] sits on lane ((a & 7) << 2) | (g >> 1), in p[g & 1] (a < 8) or p[2 + (g & 1)]
            uint32_t pb0, pb1;
            {
                const int srcA = ((2 * t) << 2) | (g >> 1), srcB = ((2 * t + 1) << 2) | (g >> 1);
                const bool odd = g & 1;
                const float a0 = __shfl_sync(0xffffffffu, p[0], srcA), a1 = __shfl_sync(0xffffffffu, p[1], srcA);
                const float b0 = __shfl_sync(0xffffffffu, p[0], srcB), b1 = __shfl_sync(0xffffffffu, p[1], srcB);
                const float a2 = __shfl_sync(0xffffffffu, p[2], srcA), a3 = __shfl_sync(0xffffffffu, p[3], srcA);
                const float b2 = __shfl_sync(0xffffffffu, p[2], srcB), b3 = __shfl_sync(0xffffffffu, p[3], srcB);
                pb0 = pack_bf16(odd ? a1 : a0, odd ? b1 : b0);
                pb1 = pack_bf16(odd ? a3 : a2, odd ? b3 : b2);
            }
            // O^T += V^T P^T
            {
                const int row = (lane & 7) + ((lane >> 4) << 3), sub = (lane >> 3) & 1;
#pragma unroll
                for (int mt = 0; mt < KSTEPS; ++mt) {
                    uint32_t a[4];
                    const int chunk = mt * 2 + sub;
                    ldmatrix_x4_trans(a, vst + row * ROW_BYTES + ((chunk ^ (row & 7)) << 4));
                    mma_16816(o[mt], a, pb0, pb1);
                }
            }
            __syncwarp();   // the stage may be refilled by a later fetch
        }
        cp_async_wait<0>();
    }
    __syncthreads();
    // The warps' states go to shared memory as [warp][head][HD + 2]; then as in attention.cu.
    float* ms = reinterpret_cast<float*>(smem_raw);
    constexpr int ROW = HD + 2;
#pragma unroll
    for (int mt = 0; mt < KSTEPS; ++mt) {
        float* r0 = ms + ((size_t)warp * 8 + 2 * t) * ROW;
        float* r1 = r0 + ROW;
        r0[mt * 16 + g] = o[mt][0];
        r1[mt * 16 + g] = o[mt][1];
        r0[mt * 16 + g + 8] = o[mt][2];
        r1[mt * 16 + g + 8] = o[mt][3];
    }
    if (g == 0) {
        float* r0 = ms + ((size_t)warp * 8 + 2 * t) * ROW;
        r0[HD] = m0;
        r0[HD + 1] = l0;
        r0[ROW + HD] = m1;
        r0[ROW + HD + 1] = l1;
    }
    __syncthreads();
    float* cs = ms + (size_t)MMA_WARPS * 8 * ROW;      // cluster mode: this CTA's merged [head][HD + 2]
    for (int hh = 0; hh < 8; ++hh) {
        if (h0 + hh >= G) break;
        const int h = kh * G + h0 + hh;
        float mm = -CUDART_INF_F;
        for (int w = 0; w < MMA_WARPS; ++w) mm = fmaxf(mm, ms[((size_t)w * 8 + hh) * ROW + HD]);
        float coef[MMA_WARPS], ll = 0.f;
        for (int w = 0; w < MMA_WARPS; ++w) {
            const float mw = ms[((size_t)w * 8 + hh) * ROW + HD];
            coef[w] = (mw == -CUDART_INF_F) ? 0.f : expf(mw - mm);
            ll += coef[w] * ms[((size_t)w * 8 + hh) * ROW + HD + 1];
        }
        const size_t pbase = ((size_t)b * nq + h) * n_splits + split;
        for (int d = threadIdx.x; d < HD; d += blockDim.x) {
            float acc = 0.f;
            for (int w = 0; w < MMA_WARPS; ++w) acc += coef[w] * ms[((size_t)w * 8 + hh) * ROW + d];
            if (CLUSTER) cs[hh * ROW + d] = acc;
            else part_o[pbase * HD + d] = acc;
        }
        if (threadIdx.x == 0) {
            if (CLUSTER) {
                cs[hh * ROW + HD] = mm;
                cs[hh * ROW + HD + 1] = ll;
            } else {
                part_ml[pbase * 2] = mm;
                part_ml[pbase * 2 + 1] = ll;
            }
        }
    }
    if (CLUSTER)
        cluster_merge<HD>(cs, n_splits, min(8, G - h0), out + (size_t)b * out_stride + (size_t)(kh * G + h0) * HD);
}

// Largest cluster that merges in the kernel.  Clusters of 8 CTAs with 98 KB of shared memory each
// (head size 256) fit the device only just, and a step with them measured 28 % slower than the
// plain grid followed by the combine kernel; clusters of 2 and 4 measured equal or slightly faster.
constexpr int CLUSTER_MAX = 4;

template <int HD, bool CLUSTER>
constexpr int stages() { return 3; }   // of the cp.async pipeline

template <int HD, int MMA_WARPS, bool CLUSTER>
size_t smem_bytes(int max_pages) {
    constexpr int MMA_STAGES = stages<HD, CLUSTER>();
    size_t smem = (size_t)MMA_WARPS * MMA_STAGES * 2 * TILE * HD * 2;
    const size_t merge = (size_t)(MMA_WARPS + 1) * 8 * (HD + 2) * sizeof(float);
    if (smem < merge) smem = merge;
    return smem + ((size_t)max_pages + 2) * sizeof(int);
}

// How many clusters of `size` CTAs of this kernel the device holds at once (asked once per size; 0: none, or
// clusters are switched off).  Clusters are placed inside a GPC, so fewer CTAs may fit than as a plain grid.
template <int HD, int MMA_WARPS>
int clusters_at_once(size_t smem, int size) {
    constexpr int ST = stages<HD, true>();
    static int known[CLUSTER_MAX + 1] = {-1, -1, -1, -1, -1};
    if (size < 1 || size > CLUSTER_MAX) return 0;
    if (known[size] < 0) {
        const char* e = getenv("QNN_ATTN_CLUSTER");
        known[size] = 0;
        if (!(e && e[0] == '0')) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(size, 1, 1);
            cfg.blockDim = dim3(MMA_WARPS * 32);
            cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = size;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, attn_decode_mma_kernel<HD, MMA_WARPS, ST>, &cfg) == cudaSuccess && n > 0)
                known[size] = n;
            else
                (void)cudaGetLastError();
        }
    }
    return known[size];
}

// CTAs of this kernel that the device holds at once as a plain grid (asked once).
template <int HD, int MMA_WARPS>
int ctas_at_once(size_t smem) {
    constexpr int ST = stages<HD, false>();
    static int known = -1;
    if (known < 0) {
        int per_sm = 0, dev = 0, sms = 0;
        known = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_mma_kernel<HD, MMA_WARPS, ST>,
                                                          MMA_WARPS * 32, smem) == cudaSuccess &&
            cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess)
            known = per_sm * sms;
        else
            (void)cudaGetLastError();
    }
    return known;
}

// Whether a grid of `clusters` clusters of `size` CTAs merges its key ranges inside the clusters.  Yes if
// they all fit the device at once, or if the device holds nearly as many CTAs in clusters of this size as
// it holds plain ones (a grid of several rounds loses little then).  Measured at head size 256, 24
// sequences x 4 kv heads x 3 ranges at context 8192: 96 clusters of 3 do not fit at once where 288 plain
// CTAs do, and a step of 6 layers took 1.58 ms against 1.08 ms with the combine kernel.
template <int HD, int MMA_WARPS>
bool merge_in_clusters(size_t smem_plain, size_t smem_cluster, int size, long long clusters) {
    const int at_once = clusters_at_once<HD, MMA_WARPS>(smem_cluster, size);
    if (at_once <= 0) return false;
    if (clusters <= at_once) return true;
    return (long long)at_once * size * 100 >= (long long)ctas_at_once<HD, MMA_WARPS>(smem_plain) * 95;
}

template <int HD, int MMA_WARPS>
int launch(const void* q, long long q_stride, const void* k_pool, const void* v_pool, const int* page_table,
           int max_pages, int page_size, int ring, const int* slots, const int* slot_len, int B, int nq, int nkv,
           float scale, float cap, int window, float* part_o, float* part_ml, int n_splits, void* out,
           long long out_stride, int* combined, cudaStream_t st) {
    const size_t smem = smem_bytes<HD, MMA_WARPS, false>(max_pages);
    const size_t smem_c = smem_bytes<HD, MMA_WARPS, true>(max_pages);
    if (smem > 220 * 1024 || smem_c > 220 * 1024) return QNN_ERR_UNSUPPORTED;
    constexpr int ST = stages<HD, false>(), STC = stages<HD, true>();
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_mma_kernel<HD, MMA_WARPS, ST>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_decode_mma_kernel<HD, MMA_WARPS, STC>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int G = nq / nkv;
    dim3 grid(n_splits, nkv * ((G + 7) / 8), B);
    *combined = 0;
    if (out != nullptr && n_splits <= CLUSTER_MAX &&
        merge_in_clusters<HD, MMA_WARPS>(smem, smem_c, n_splits, (long long)grid.y * grid.z)) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(MMA_WARPS * 32);
        cfg.dynamicSmemBytes = smem_c;
        cfg.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = n_splits;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = (qnn::pdl_enabled() && (long long)grid.x * grid.y * grid.z <= qnn::pdl_max_grid()) ? 2 : 1;
        cudaError_t e = cudaLaunchKernelEx(&cfg, attn_decode_mma_kernel<HD, MMA_WARPS, STC>, (const bf16*)q,
                                           (size_t)q_stride, (const bf16*)k_pool, (const bf16*)v_pool, page_table,
                                           max_pages, page_size, ring, slots, slot_len, nq, nkv, scale, cap, window,
                                           part_o, part_ml, n_splits, (bf16*)out, (size_t)out_stride);
        if (e != cudaSuccess) return (int)e;
        *combined = 1;
        return (int)cudaGetLastError();
    }
    qnn::launch_pdl(attn_decode_mma_kernel<HD, MMA_WARPS, ST>, dim3(grid), dim3(MMA_WARPS * 32), smem, st, (const bf16*)q, (size_t)q_stride, (const bf16*)k_pool, (const bf16*)v_pool,
                                             page_table, max_pages, page_size, ring, slots, slot_len, nq, nkv, scale,
                                             cap, window, part_o, part_ml, n_splits, (bf16*)nullptr, (size_t)0);
    return (int)cudaGetLastError();
}

}  // namespace

// Decode attention for bfloat16 on the tensor cores.  Returns QNN_ERR_UNSUPPORTED for sizes it
// does not take (the caller then uses the generic kernel).  On success *combined says whether
// `out` ([B, out_stride] bfloat16, may be null) already holds the result (up to 4 splits, merged
// inside a cluster) or the caller still has to run the combine pass over part_o / part_ml.
// slots, slot_len and page_table are read before the kernel waits for the kernel launched in front of it
// on the stream (programmatic dependent launch): that kernel must not be the one that writes them.  Copies
// from the host and kernels further back are complete by then.
extern "C" int qnn_attn_decode_mma_split(const void* q, long long q_stride, const void* k_pool, const void* v_pool,
                                         const int* page_table, int max_pages, int page_size, int ring,
                                         const int* slots, const int* slot_len, int B, int nq, int nkv, int hd,
                                         float scale, float cap, int window, float* part_o, float* part_ml,
                                         int n_splits, void* out, long long out_stride, int* combined,
                                         cudaStream_t st) {
    if (nkv <= 0 || nq % nkv) return QNN_ERR_ARGUMENT;
    if (page_size < TILE || (page_size & (page_size - 1))) return QNN_ERR_UNSUPPORTED;
    if (ring > 0 && (ring % page_size)) return QNN_ERR_UNSUPPORTED;
    if ((q_stride * 2) % 4 || ((uintptr_t)q & 3)) return QNN_ERR_UNSUPPORTED;
#define QNN_MMA_ARGS q, q_stride, k_pool, v_pool, page_table, max_pages, page_size, ring, slots, slot_len, B, nq, nkv, \
                     scale, cap, window, part_o, part_ml, n_splits, out, out_stride, combined, st
    static int warps = 0;
    if (warps == 0) {
        const char* e = getenv("QNN_MMA_WARPS");
        warps = (e && atoi(e) == 4) ? 4 : 2;
    }
    if (warps == 4) {
        switch (hd) {
            case 64: return launch<64, 4>(QNN_MMA_ARGS);
            case 128: return launch<128, 4>(QNN_MMA_ARGS);
            case 256: return launch<256, 4>(QNN_MMA_ARGS);
            default: return QNN_ERR_UNSUPPORTED;
        }
    }
    switch (hd) {
        case 64: return launch<64, 2>(QNN_MMA_ARGS);
        case 128: return launch<128, 2>(QNN_MMA_ARGS);
        case 256: return launch<256, 2>(QNN_MMA_ARGS);
        default: return QNN_ERR_UNSUPPORTED;
    }
#undef QNN_MMA_ARGS
}

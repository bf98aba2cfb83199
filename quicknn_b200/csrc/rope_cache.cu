// Rotary position encoding of Q and K in place, fused with the append of K and V to
// the paged cache.
//
// Reference: two GO_LLM_ROPE dispatches and one GO_LLM_CACHE_WRITE per layer
// (src/models/QuickNN.Models.Gemma2.pas:170-175; shaders/tensor.comp:318-327 and :312-317).
// The rotation is the half-split one over the rotated width:
//   x' = x_j cos(a) - x_{j+r/2} sin(a),  y' = x_j sin(a) + x_{j+r/2} cos(a),
//   a = float(position) * inv_freq[j],  inv_freq[j] = theta^(-2j/r) rounded to float32 on the host.
// The reference computes inv_freq in the shader and reduces the angle by hand before
// native sin/cos; here sincosf() does the full-range reduction.
//
// Cache layout of one line: K and V pools [page][kv_head][slot_in_page][head_dim]; the
// page of position p of a sequence is page_table[slot][ (p mod ring) / page_size ] where
// ring = 0 means "no ring" (every position kept).
#include "common.cuh"

using namespace qnn;

template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, int nq, int nkv, int hd, int rot,
                                  const float* __restrict__ inv_freq, const int* __restrict__ tok_pos,
                                  const int* __restrict__ tok_slot, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                  const int* __restrict__ page_table, int max_pages, int page_size, int ring,
                                  const int* __restrict__ slot_len, int write_cache) {
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int slot = tok_slot[t];
    const int half = hd / 2, rh = rot / 2;
    const size_t row = (size_t)t * (nq + 2 * nkv) * hd;
    T* q = qkv + row;
    T* k = q + (size_t)nq * hd;
    T* v = k + (size_t)nkv * hd;

    size_t cache_base = 0;
    bool wr = write_cache && slot >= 0;
    // A prompt longer than the ring would write one cell from several positions in this
    // launch; only the last `ring` positions of the sequence (its length after this step
    // is slot_len[slot]) are kept.
    if (wr && ring > 0 && pos + ring < slot_len[slot]) wr = false;
    if (wr) {
        const int r = ring > 0 ? pos % ring : pos;
        const int page = page_table[(size_t)slot * max_pages + r / page_size];
        cache_base = ((size_t)page * nkv * page_size + (r % page_size)) * hd;  // + h * page_size * hd
    }
    const size_t head_stride = (size_t)page_size * hd;

    const int nwork = (nq + nkv) * half;
    for (int w = threadIdx.x; w < nwork; w += blockDim.x) {
        const int h = w / half, idx = w % half;
        const bool is_k = h >= nq;
        T* x = is_k ? k + (size_t)(h - nq) * hd : q + (size_t)h * hd;
        if (idx < rh) {
            float s, c;
            sincosf((float)pos * inv_freq[idx], &s, &c);
            const float a = to_f(x[idx]), b = to_f(x[idx + rh]);
            const T ra = from_f<T>(a * c - b * s), rb = from_f<T>(a * s + b * c);
            x[idx] = ra;
            x[idx + rh] = rb;
            if (is_k && wr) {
                T* dst = k_pool + cache_base + (size_t)(h - nq) * head_stride;
                dst[idx] = ra;
                dst[idx + rh] = rb;
            }
        } else if (is_k && wr) {
            const int d = rot + 2 * (idx - rh);
            T* dst = k_pool + cache_base + (size_t)(h - nq) * head_stride;
            dst[d] = x[d];
            dst[d + 1] = x[d + 1];
        }
    }
    if (wr) {
        for (int w = threadIdx.x; w < nkv * hd; w += blockDim.x) {
            const int h = w / hd, d = w % hd;
            v_pool[cache_base + (size_t)h * head_stride + d] = v[w];
        }
    }
}

// The same with 16-byte accesses: a work item rotates VEC pairs (x_j .. x_{j+VEC-1} with their
// partners half the rotated width away) or copies VEC values.  Needs rot/2, hd - rot and hd to be
// multiples of VEC.
template <typename T>
__global__ void rope_cache_vec_kernel(T* __restrict__ qkv, int nq, int nkv, int hd, int rot,
                                      const float* __restrict__ inv_freq, const int* __restrict__ tok_pos,
                                      const int* __restrict__ tok_slot, T* __restrict__ k_pool,
                                      T* __restrict__ v_pool, const int* __restrict__ page_table, int max_pages,
                                      int page_size, int ring, const int* __restrict__ slot_len, int write_cache) {
    pdl_wait();
    constexpr int VEC = Vec16<T>::N;
    const int t = blockIdx.x;
    const int pos = tok_pos[t];
    const int slot = tok_slot[t];
    const int rh = rot / 2;
    T* q = qkv + (size_t)t * (nq + 2 * nkv) * hd;
    T* k = q + (size_t)nq * hd;
    T* v = k + (size_t)nkv * hd;
    size_t cache_base = 0;
    bool wr = write_cache && slot >= 0;
    if (wr && ring > 0 && pos + ring < slot_len[slot]) wr = false;
    if (wr) {
        const int r = ring > 0 ? pos % ring : pos;
        const int page = page_table[(size_t)slot * max_pages + r / page_size];
        cache_base = ((size_t)page * nkv * page_size + (r % page_size)) * hd;
    }
    const size_t head_stride = (size_t)page_size * hd;
    // The angles depend on the position and the pair only, not on the head: the block forms each
    // (cos, sin) once (sincosf is the expensive part of this kernel) and every head reads it.
    extern __shared__ float2 angles[];             // [rh]
    for (int j = threadIdx.x; j < rh; j += blockDim.x) {
        float sn, cs;
        sincosf((float)pos * inv_freq[j], &sn, &cs);
        angles[j] = make_float2(cs, sn);
    }
    __syncthreads();
    const int rc = rh / VEC;                       // rotating items per head
    const int pc = (hd - rot) / VEC;               // pass-through items per kv head
    const int vc = hd / VEC;                       // value items per kv head
    const int n_rot = (nq + nkv) * rc, n_pass = wr ? nkv * pc : 0, n_val = wr ? nkv * vc : 0;
    for (int w = threadIdx.x; w < n_rot + n_pass + n_val; w += blockDim.x) {
        if (w < n_rot) {
            const int h = w / rc, j = (w % rc) * VEC;
            const bool is_k = h >= nq;
            T* x = is_k ? k + (size_t)(h - nq) * hd : q + (size_t)h * hd;
            Vec16<T> av, bv;
            av.load(x + j);
            bv.load(x + j + rh);
            float a[VEC], b[VEC], ra[VEC], rb[VEC];
            av.unpack(a);
            bv.unpack(b);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float cs = angles[j + e].x, sn = angles[j + e].y;
                ra[e] = a[e] * cs - b[e] * sn;
                rb[e] = a[e] * sn + b[e] * cs;
            }
            Vec16<T>::store(x + j, ra);
            Vec16<T>::store(x + j + rh, rb);
            if (is_k && wr) {
                T* dst = k_pool + cache_base + (size_t)(h - nq) * head_stride;
                Vec16<T>::store(dst + j, ra);
                Vec16<T>::store(dst + j + rh, rb);
            }
        } else if (w < n_rot + n_pass) {
            const int u = w - n_rot, h = u / pc, d = rot + (u % pc) * VEC;
            Vec16<T> xv;
            xv.load(k + (size_t)h * hd + d);
            *reinterpret_cast<decltype(xv.raw)*>(k_pool + cache_base + (size_t)h * head_stride + d) = xv.raw;
        } else {
            const int u = w - n_rot - n_pass, h = u / vc, d = (u % vc) * VEC;
            Vec16<T> xv;
            xv.load(v + (size_t)h * hd + d);
            *reinterpret_cast<decltype(xv.raw)*>(v_pool + cache_base + (size_t)h * head_stride + d) = xv.raw;
        }
    }
}

QNN_API int qnn_rope_cache_write(void* qkv, int dtype, int T, int nq, int nkv, int hd, int rot,
                                 const float* inv_freq, const int* tok_pos, const int* tok_slot, void* k_pool,
                                 void* v_pool, const int* page_table, int max_pages, int page_size, int ring,
                                 const int* slot_len, int write_cache, cudaStream_t st) {
    if (T <= 0) return 0;
    if (hd % 2 || rot % 2 || rot > hd || rot < 0) return QNN_ERR_UNSUPPORTED;
    const int vec = dtype == QNN_DT_BF16 ? 8 : 4;
    const bool aligned = ((((uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0);
    if (aligned && hd % vec == 0 && (rot / 2) % vec == 0 && (hd - rot) % vec == 0) {
        const int items = (nq + nkv) * (rot / 2) / vec + nkv * (hd - rot) / vec + nkv * hd / vec;
        // a token per block; few tokens: many threads each (the step waits for this kernel's latency); many tokens:
        // small blocks, more of them on an SM (measured at 12 heads of 256: 2048 tokens 9.4 us with 64 threads,
        // 10.8 with 256; 65536 tokens 212 against 321 us; 64 tokens 3.9 against 2.7)
        int threads = items >= 256 ? 256 : (items >= 128 ? 128 : 64);
        if (T > 1024) threads = 64;
        else if (T > 256 && threads > 128) threads = 128;
        if (dtype == QNN_DT_BF16)
            qnn::launch_pdl(rope_cache_vec_kernel<bf16>, dim3(T), dim3(threads), (size_t)(rot / 2) * sizeof(float2), st, (bf16*)qkv, nq, nkv, hd, rot,
                            inv_freq, tok_pos, tok_slot, (bf16*)k_pool, (bf16*)v_pool, page_table, max_pages, page_size,
                            ring, slot_len, write_cache);
        else
            qnn::launch_pdl(rope_cache_vec_kernel<float>, dim3(T), dim3(threads), (size_t)(rot / 2) * sizeof(float2), st, (float*)qkv, nq, nkv, hd, rot,
                            inv_freq, tok_pos, tok_slot, (float*)k_pool, (float*)v_pool, page_table, max_pages,
                            page_size, ring, slot_len, write_cache);
        QNN_LAUNCH_CHECK();
    }
    const int work = (nq + nkv) * hd / 2;
    const int threads = work >= 1024 ? 256 : (work >= 256 ? 128 : 64);
    if (dtype == QNN_DT_BF16)
        qnn::launch_pdl(rope_cache_kernel<bf16>, dim3(T), dim3(threads), 0, st, (bf16*)qkv, nq, nkv, hd, rot, inv_freq,
                        tok_pos, tok_slot, (bf16*)k_pool, (bf16*)v_pool, page_table, max_pages, page_size, ring,
                        slot_len, write_cache);
    else
        qnn::launch_pdl(rope_cache_kernel<float>, dim3(T), dim3(threads), 0, st, (float*)qkv, nq, nkv, hd, rot,
                        inv_freq, tok_pos, tok_slot, (float*)k_pool, (float*)v_pool, page_table, max_pages, page_size,
                        ring, slot_len, write_cache);
    QNN_LAUNCH_CHECK();
}

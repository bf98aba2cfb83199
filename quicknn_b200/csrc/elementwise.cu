// Embedding, norms, gated activation, softcap and small helpers.
//
// Reference formulas (HemulGM/QuickNN, src/backends/vulkan/shaders/tensor.comp):
//   embedding gather, id >= vocab -> 0 ........ :237-242 (op 15), scale :309 (op 43)
//   RMSNorm: inv = rsqrt(sum(x^2)/dim + eps) ... :63-72 (op 2), "+1" weight bit :70
//   residual add .............................. :221 (op 4)
//   gelu_tanh(gate) * up ...................... :23, :228 (op 75)
//   final softcap ............................. :308 (op 76)
//   finite check into an error word ........... :235 (op 13)
// The reference runs each as its own dispatch; here the post-sublayer norm, the
// residual add and the next pre-norm are one kernel, and sums are always float32.
#include "common.cuh"

using namespace qnn;

// ---------------------------------------------------------------------------------
// out[t, :] = table[token_t, :] * scale   (float32 residual stream)
// ---------------------------------------------------------------------------------
template <typename W>
__global__ void embed_kernel(const int* __restrict__ tokens, const W* __restrict__ table, float scale,
                             float* __restrict__ out, int H, int V) {
    pdl_wait();
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float* o = out + (size_t)t * H;
    if (tok < 0 || tok >= V) {
        for (int j = threadIdx.x; j < H; j += blockDim.x) o[j] = 0.f;
        return;
    }
    const W* row = table + (size_t)tok * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) o[j] = to_f(row[j]) * scale;
}

// The same with the first norm of the first layer in the same kernel: out[t] as above, and
// normed[t] = rmsnorm(out[t]; w) in `normed_dt` (one kernel less at the head of every step).
template <typename W>
__global__ void embed_rmsnorm_kernel(const int* __restrict__ tokens, const W* __restrict__ table, float scale,
                                     float* __restrict__ out, int H, int V, const void* __restrict__ w, int w_dt,
                                     float eps, float offset, void* __restrict__ normed, int normed_dt) {
    pdl_wait();
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int tok = tokens[t];
    const bool valid = tok >= 0 && tok < V;
    const W* row = table + (size_t)(valid ? tok : 0) * H;
    float* o = out + (size_t)t * H;
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const float v = valid ? to_f(row[j]) * scale : 0.f;
        o[j] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int j = threadIdx.x; j < H; j += blockDim.x) {       // each thread re-reads what it wrote itself
        const float g = load_as_f(w, w_dt, j) + offset;
        store_from_f(normed, normed_dt, (size_t)t * H + j, o[j] * inv * g);
    }
}

QNN_API int qnn_embed_rmsnorm(const int* tokens, const void* table, int table_dtype, float scale, float* out,
                              const void* w, int w_dt, float eps, int unit_offset, void* normed, int normed_dt,
                              int T, int H, int V, cudaStream_t st) {
    if (T <= 0) return 0;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    const float off = unit_offset ? 1.f : 0.f;
    if (table_dtype == QNN_DT_BF16)
        qnn::launch_pdl(embed_rmsnorm_kernel<bf16>, dim3(T), dim3(threads), 0, st, tokens, (const bf16*)table, scale, out, H,
                        V, w, w_dt, eps, off, normed, normed_dt);
    else
        qnn::launch_pdl(embed_rmsnorm_kernel<float>, dim3(T), dim3(threads), 0, st, tokens, (const float*)table, scale, out,
                        H, V, w, w_dt, eps, off, normed, normed_dt);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_embed(const int* tokens, const void* table, int table_dtype, float scale, float* out,
                      int T, int H, int V, cudaStream_t st) {
    if (T <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == QNN_DT_BF16)
        qnn::launch_pdl(embed_kernel<bf16>, dim3(T), dim3(threads), 0, st, tokens, (const bf16*)table, scale, out, H, V);
    else
        qnn::launch_pdl(embed_kernel<float>, dim3(T), dim3(threads), 0, st, tokens, (const float*)table, scale, out, H, V);
    QNN_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------
// RMSNorm of one row per block.
// ---------------------------------------------------------------------------------
__global__ void rmsnorm_kernel(const void* __restrict__ x, int x_dt, const void* __restrict__ w, int w_dt,
                               float eps, float offset, void* __restrict__ out, int out_dt, int H) {
    pdl_wait();
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * H;
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = load_as_f(x, x_dt, base + j);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = load_as_f(x, x_dt, base + j);
        float g = load_as_f(w, w_dt, j) + offset;
        store_from_f(out, out_dt, base + j, v * inv * g);
    }
}

static inline int norm_threads(int H) { return H >= 2048 ? 512 : (H >= 512 ? 256 : 128); }

QNN_API int qnn_rmsnorm(const void* x, int x_dt, const void* w, int w_dt, float eps, int unit_offset,
                        void* out, int out_dt, int T, int H, cudaStream_t st) {
    if (T <= 0) return 0;
    qnn::launch_pdl(rmsnorm_kernel, dim3(T), dim3(norm_threads(H)), 0, st, x, x_dt, w, w_dt, eps, unit_offset ? 1.f : 0.f, out, out_dt, H);
    QNN_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------
// resid += rmsnorm(y; w_post);  optionally  out_next = rmsnorm(resid; w_next).
// Three passes over a row by the same thread -> element mapping, so a thread re-reads
// only what it wrote itself.
// ---------------------------------------------------------------------------------
// PER = elements per thread held in registers (H <= PER * blockDim): every global load of the
// kernel is issued before the first reduction, so the row costs two block reductions and no
// dependent reloads.  PER = 0 is the looping form for rows that do not fit.
template <int PER>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const void* __restrict__ y, int y_dt,
                                   const void* __restrict__ w_post, int w_post_dt, float eps_post, float off_post,
                                   const void* __restrict__ w_next, int w_next_dt, float eps_next, float off_next,
                                   void* __restrict__ out_next, int out_dt, int H) {
    pdl_wait();
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * H;
    if (PER > 0) {
        float yv[PER > 0 ? PER : 1], rv[PER > 0 ? PER : 1], g1[PER > 0 ? PER : 1], g2[PER > 0 ? PER : 1];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int j = threadIdx.x + i * blockDim.x;
            const bool in = j < H;
            yv[i] = in ? load_as_f(y, y_dt, base + j) : 0.f;
            rv[i] = in ? resid[base + j] : 0.f;
            g1[i] = in ? load_as_f(w_post, w_post_dt, j) + off_post : 0.f;
            g2[i] = (in && w_next != nullptr) ? load_as_f(w_next, w_next_dt, j) + off_next : 0.f;
            ss += yv[i] * yv[i];
        }
        ss = block_sum(ss, red);
        const float inv = rsqrtf(ss / (float)H + eps_post);
        float ss2 = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int j = threadIdx.x + i * blockDim.x;
            rv[i] = rv[i] + yv[i] * inv * g1[i];
            if (j < H) resid[base + j] = rv[i];
            ss2 += rv[i] * rv[i];
        }
        if (w_next == nullptr) return;
        ss2 = block_sum(ss2, red);
        const float inv2 = rsqrtf(ss2 / (float)H + eps_next);
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int j = threadIdx.x + i * blockDim.x;
            if (j < H) store_from_f(out_next, out_dt, base + j, rv[i] * inv2 * g2[i]);
        }
        return;
    }
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = load_as_f(y, y_dt, base + j);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps_post);
    float ss2 = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = load_as_f(y, y_dt, base + j);
        float g = load_as_f(w_post, w_post_dt, j) + off_post;
        float r = resid[base + j] + v * inv * g;
        resid[base + j] = r;
        ss2 += r * r;
    }
    if (w_next == nullptr) return;
    ss2 = block_sum(ss2, red);
    const float inv2 = rsqrtf(ss2 / (float)H + eps_next);
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float r = resid[base + j];
        float g = load_as_f(w_next, w_next_dt, j) + off_next;
        store_from_f(out_next, out_dt, base + j, r * inv2 * g);
    }
}

// The same with 8 consecutive elements per access (H a multiple of 8, 16-byte aligned rows):
// CH chunks of 8 per thread.
template <int CH>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const void* __restrict__ y, int y_dt,
                                       const void* __restrict__ w_post, int w_post_dt, float eps_post, float off_post,
                                       const void* __restrict__ w_next, int w_next_dt, float eps_next, float off_next,
                                       void* __restrict__ out_next, int out_dt, int H) {
    __shared__ float red[32];
    const size_t base = (size_t)blockIdx.x * H;
    const int nchunks = H >> 3;
    float yv[CH][8], rv[CH][8], g1[CH][8];
    // The norm weights are written by no kernel of the step: they are fetched before the wait for the
    // kernel in front, so that their latency is hidden behind its tail (with one chunk per thread, the few
    // rows of a decode step, also those of the second norm, which otherwise sit behind two reductions).
    constexpr bool EARLY2 = CH == 1;
    float g2e[EARLY2 ? 8 : 1];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < nchunks) {
            load8_as_f(w_post, w_post_dt, (size_t)c * 8, g1[i]);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) g1[i][e] = 0.f;
        }
    }
    if constexpr (EARLY2) {
        if (w_next != nullptr && (int)threadIdx.x < nchunks) load8_as_f(w_next, w_next_dt, (size_t)threadIdx.x * 8, g2e);
        else {
#pragma unroll
            for (int e = 0; e < 8; ++e) g2e[e] = 0.f;
        }
    }
    pdl_wait();
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < nchunks) {
            load8_as_f(y, y_dt, base + c * 8, yv[i]);
            load8_as_f(resid, QNN_DT_F32, base + c * 8, rv[i]);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) yv[i][e] = rv[i][e] = 0.f;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += yv[i][e] * yv[i][e];
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps_post);
    float ss2 = 0.f;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            rv[i][e] = rv[i][e] + yv[i][e] * inv * (g1[i][e] + off_post);
            ss2 += (c < nchunks) ? rv[i][e] * rv[i][e] : 0.f;
        }
        if (c < nchunks) store8_from_f(resid, QNN_DT_F32, base + c * 8, rv[i]);
    }
    if (w_next == nullptr) return;
    ss2 = block_sum(ss2, red);
    const float inv2 = rsqrtf(ss2 / (float)H + eps_next);
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < nchunks) {
            float g2[8], o[8];
            if constexpr (EARLY2) {
#pragma unroll
                for (int e = 0; e < 8; ++e) g2[e] = g2e[e];
            } else {
                load8_as_f(w_next, w_next_dt, (size_t)c * 8, g2);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = rv[i][e] * inv2 * (g2[e] + off_next);
            store8_from_f(out_next, out_dt, base + c * 8, o);
        }
    }
}

QNN_API int qnn_add_rmsnorm(float* resid, const void* y, int y_dt, const void* w_post, int w_post_dt,
                            float eps_post, int unit_post, const void* w_next, int w_next_dt, float eps_next,
                            int unit_next, void* out_next, int out_dt, int T, int H, cudaStream_t st) {
    if (T <= 0) return 0;
    const float o1 = unit_post ? 1.f : 0.f, o2 = unit_next ? 1.f : 0.f;
    const bool aligned = ((((uintptr_t)resid | (uintptr_t)y | (uintptr_t)w_post | (uintptr_t)w_next | (uintptr_t)out_next) & 15) == 0);
    if ((H & 7) == 0 && aligned && H <= 8 * 4 * 1024) {
        // a thread per 8 elements as long as a block can hold the row (measured against two chunks per thread:
        // 2048 rows of 2304 the same, 16384 and 65536 rows 5.35 and 5.56 TB/s against 5.02 and 5.25)
        const int chunks = H >> 3;
        int ch = 1;
        while ((chunks + ch - 1) / ch > 1024) ch *= 2;
        const int threads = (((chunks + ch - 1) / ch) + 31) / 32 * 32;
#define QNN_ARV(CHV)                                                                                                 \
    qnn::launch_pdl(add_rmsnorm_vec_kernel<CHV>, dim3(T), dim3(threads), 0, st, resid, y, y_dt, w_post, w_post_dt,    \
                    eps_post, o1, w_next, w_next_dt, eps_next, o2, out_next, out_dt, H)
        if (ch == 1) QNN_ARV(1);
        else if (ch == 2) QNN_ARV(2);
        else QNN_ARV(4);
#undef QNN_ARV
        QNN_LAUNCH_CHECK();
    }
    const int threads = norm_threads(H);
#define QNN_ARN(PERV)                                                                                              \
    qnn::launch_pdl(add_rmsnorm_kernel<PERV>, dim3(T), dim3(threads), 0, st, resid, y, y_dt, w_post, w_post_dt,     \
                    eps_post, o1, w_next, w_next_dt, eps_next, o2, out_next, out_dt, H)
    const int per = (H + threads - 1) / threads;
    if (per <= 2) QNN_ARN(2);
    else if (per <= 5) QNN_ARN(5);
    else if (per <= 8) QNN_ARN(8);
    else QNN_ARN(0);
#undef QNN_ARN
    QNN_LAUNCH_CHECK();
}

// resid[i] += y[i]   (generic residual add for blocks that do not fuse)
__global__ void add_kernel(float* __restrict__ resid, const void* __restrict__ y, int y_dt, size_t n) {
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) resid[i] += load_as_f(y, y_dt, i);
}
QNN_API int qnn_add(float* resid, const void* y, int y_dt, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    qnn::launch_pdl(add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, resid, y, y_dt, (size_t)n);
    QNN_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------
// out[t, i] = act(gu[t, i]) * gu[t, I + i]
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void gated_act_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, int act, size_t n) {
    pdl_wait();
    size_t id = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (id >= n) return;
    size_t t = id / I;
    int i = (int)(id % I);
    float g = to_f(gu[t * 2 * I + i]), u = to_f(gu[t * 2 * I + I + i]);
    out[id] = from_f<T>(activate(g, act) * u);
}
// 8 consecutive columns per thread, one row per blockIdx.y (I a multiple of 8)
template <typename T>
__global__ void gated_act_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, int act) {
    pdl_wait();
    constexpr int VEC = Vec16<T>::N;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c * VEC >= I) return;
    const size_t row = blockIdx.y;
    Vec16<T> gv, uv;
    gv.load(gu + row * 2 * I + (size_t)c * VEC);
    uv.load(gu + row * 2 * I + I + (size_t)c * VEC);
    float g[VEC], u[VEC];
    gv.unpack(g);
    uv.unpack(u);
#pragma unroll
    for (int e = 0; e < VEC; ++e) g[e] = (sizeof(T) == 2 ? activate_fast(g[e], act) : activate(g[e], act)) * u[e];
    Vec16<T>::store(out + row * I + (size_t)c * VEC, g);
}

QNN_API int qnn_gated_act(const void* gu, void* out, int dtype, int T, int I, int act, cudaStream_t st) {
    size_t n = (size_t)T * I;
    if (n == 0) return 0;
    const int vec = dtype == QNN_DT_BF16 ? 8 : 4;
    if (I % vec == 0 && T <= 65535 && ((((uintptr_t)gu | (uintptr_t)out) & 15) == 0)) {
        dim3 grid((I / vec + 255) / 256, T);
        if (dtype == QNN_DT_BF16)
            qnn::launch_pdl(gated_act_vec_kernel<bf16>, grid, dim3(256), 0, st, (const bf16*)gu, (bf16*)out, I, act);
        else
            qnn::launch_pdl(gated_act_vec_kernel<float>, grid, dim3(256), 0, st, (const float*)gu, (float*)out, I, act);
        QNN_LAUNCH_CHECK();
    }
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == QNN_DT_BF16)
        qnn::launch_pdl(gated_act_kernel<bf16>, dim3(blocks), dim3(256), 0, st, (const bf16*)gu, (bf16*)out, I, act, n);
    else
        qnn::launch_pdl(gated_act_kernel<float>, dim3(blocks), dim3(256), 0, st, (const float*)gu, (float*)out, I, act, n);
    QNN_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------
// out[i] = softcap(x[i])  -> float32 (the logits)
// ---------------------------------------------------------------------------------
__global__ void softcap_kernel(const void* __restrict__ x, int x_dt, float* __restrict__ out, float cap, size_t n) {
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = softcap(load_as_f(x, x_dt, i), cap);
}
QNN_API int qnn_softcap(const void* x, int x_dt, float* out, float cap, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    qnn::launch_pdl(softcap_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, x, x_dt, out, cap, (size_t)n);
    QNN_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------
// dst[r, :] = src[rows[r], :]  with dtype conversion (gather the rows whose logits are wanted)
// ---------------------------------------------------------------------------------
__global__ void gather_rows_kernel(const void* __restrict__ src, int src_dt, const int* __restrict__ rows,
                                   void* __restrict__ dst, int dst_dt, int H) {
    pdl_wait();
    const size_t s = (size_t)rows[blockIdx.x] * H, d = (size_t)blockIdx.x * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) store_from_f(dst, dst_dt, d + j, load_as_f(src, src_dt, s + j));
}
QNN_API int qnn_gather_rows(const void* src, int src_dt, const int* rows, void* dst, int dst_dt, int R, int H,
                            cudaStream_t st) {
    if (R <= 0) return 0;
    qnn::launch_pdl(gather_rows_kernel, dim3(R), dim3(256), 0, st, src, src_dt, rows, dst, dst_dt, H);
    QNN_LAUNCH_CHECK();
}

// dst = convert(src)
__global__ void cast_kernel(const void* __restrict__ src, int src_dt, void* __restrict__ dst, int dst_dt, size_t n) {
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) store_from_f(dst, dst_dt, i, load_as_f(src, src_dt, i));
}
QNN_API int qnn_cast(const void* src, int src_dt, void* dst, int dst_dt, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    qnn::launch_pdl(cast_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, src, src_dt, dst, dst_dt, (size_t)n);
    QNN_LAUNCH_CHECK();
}

// flag |= 1 when any value is NaN or Inf
__global__ void finite_kernel(const float* __restrict__ x, size_t n, int* __restrict__ flag) {
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        float v = x[i];
        if (isnan(v) || isinf(v)) atomicOr(flag, 1);
    }
}
QNN_API int qnn_check_finite(const float* x, long long n, int* flag, cudaStream_t st) {
    if (n <= 0) return 0;
    qnn::launch_pdl(finite_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, x, (size_t)n, flag);
    QNN_LAUNCH_CHECK();
}

// Token selection on the device: greedy, and temperature sampling with top-k, nucleus cut
// and repetition penalty.  Only the chosen ids (and an error word) cross to the host.
//
// Reference (src/backends/vulkan/shaders/tensor.comp):
//   op 50 :121-155  exact top-k of each 512-token tile; k = 1 is an arg-max; repetition
//                   penalty s<0 ? s*pen : s/pen on seen ids; ties go to the lowest id
//   op 51/46 :156-199  merge to the global top-k (k <= 64), p_j = exp((s_j - s_0)/T), keep the
//                   shortest prefix with mass >= top_p * total, draw target = u * retained,
//                   first j whose running sum exceeds it, else the last kept
//   op 48 :328      mark ids in the "seen" table
//   op 13 :235      NaN/Inf -> error word
// Host side of the reference: xorshift32 per token, u = min(0.99999994, (x + 0.5) / 2^32)
// (src/models/QuickNN.Models.LLM.pas:625-628); temperature 0 forces k = 1
// (QuickNN.Vulkan.Context.Implementation.inc:1169-1170).  Here the generator state lives on
// the device, one per row, and tiles are 1024 wide.  For k > 1 the tiles only give their maxima, from which a
// threshold is taken that few values pass (see sample_tilemax_kernel and the three kernels after it).
#include "common.cuh"
#include <float.h>

using namespace qnn;

#define SAMPLE_TILE 1024
#define SAMPLE_THREADS 256
#define SAMPLE_MAX_K 64
#define NO_ID 0xffffffffu

__device__ __forceinline__ bool better(float a, unsigned ia, float b, unsigned ib) {
    return a > b || (a == b && ia < ib);
}

// Block-wide arg-max with lowest-id ties; every thread gets the winner.
__device__ __forceinline__ void block_argmax(float& v, unsigned& id, float* sv, unsigned* si) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const unsigned oi = __shfl_xor_sync(0xffffffffu, id, o);
        if (better(ov, oi, v, id)) { v = ov; id = oi; }
    }
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = id; }
    __syncthreads();
    float rv = lane < nwarp ? sv[lane] : -FLT_MAX;
    unsigned ri = lane < nwarp ? si[lane] : NO_ID;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, rv, o);
        const unsigned oi = __shfl_xor_sync(0xffffffffu, ri, o);
        if (better(ov, oi, rv, ri)) { rv = ov; ri = oi; }
    }
    v = rv;
    id = ri;
}

// cand[(r * tiles + tile) * k + j] = j-th best (value, id) of the tile
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_tile_kernel(const float* __restrict__ logits, int V, int k, float penalty, const unsigned char* __restrict__ seen,
                   const int* __restrict__ seen_rows, float2* __restrict__ cand, int* __restrict__ error_flag) {
    pdl_wait();
    __shared__ float sv[32];
    __shared__ unsigned si[32];
    const int tile = blockIdx.x, r = blockIdx.y, tiles = gridDim.x;
    const float* row = logits + (size_t)r * V;
    const unsigned char* srow = nullptr;
    if (seen != nullptr && seen_rows != nullptr && seen_rows[r] >= 0) srow = seen + (size_t)seen_rows[r] * V;
    constexpr int PER = SAMPLE_TILE / SAMPLE_THREADS;
    float val[PER];
    unsigned ids[PER];
    bool bad = false;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        const int tok = tile * SAMPLE_TILE + i * SAMPLE_THREADS + threadIdx.x;
        val[i] = -FLT_MAX;
        ids[i] = NO_ID;
        if (tok < V) {
            float s = row[tok];
            if (isnan(s) || isinf(s)) { bad = true; s = -FLT_MAX; }
            else if (srow != nullptr && srow[tok]) s = s < 0.f ? s * penalty : s / penalty;
            val[i] = s;
            ids[i] = (unsigned)tok;
        }
    }
    if (bad && error_flag != nullptr) atomicOr(error_flag, 1);
    for (int j = 0; j < k; ++j) {
        float bv = -FLT_MAX;
        unsigned bi = NO_ID;
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (better(val[i], ids[i], bv, bi)) { bv = val[i]; bi = ids[i]; }
        block_argmax(bv, bi, sv, si);
        if (threadIdx.x == 0) cand[((size_t)r * tiles + tile) * k + j] = make_float2(bv, __uint_as_float(bi));
#pragma unroll
        for (int i = 0; i < PER; ++i)
            if (ids[i] == bi && bi != NO_ID) { val[i] = -FLT_MAX; ids[i] = NO_ID; }
    }
}

// The draw among the k best of a row (values in descending order, NO_ID where a row has fewer): softmax at the
// temperature, the shortest prefix with at least top_p of the mass, one xorshift32 step of the row's generator.
__device__ void draw(float* top_v, const unsigned* top_i, int k, float temperature, float top_p,
                     unsigned* __restrict__ rng_state, int* __restrict__ out_tokens, unsigned char* __restrict__ seen,
                     const int* __restrict__ seen_rows, int V, int r) {
    unsigned selected = top_i[0];
    if (temperature > 0.f && k > 1) {
        unsigned x = rng_state[r];
        x ^= x << 13; x ^= x >> 17; x ^= x << 5;
        rng_state[r] = x;
        const float u = fminf(0.99999994f, (float)(((double)x + 0.5) / 4294967296.0));
        int kk = k;
        while (kk > 1 && top_i[kk - 1] == NO_ID) --kk;  // fewer valid ids than k
        float total = 0.f;
        const float mx = top_v[0];
        for (int j = 0; j < kk; ++j) { top_v[j] = expf((top_v[j] - mx) / temperature); total += top_v[j]; }
        float retained = 0.f;
        int count = 0;
        do { retained += top_v[count]; ++count; } while (count < kk && retained < top_p * total);
        const float target = u * retained;
        float acc = 0.f;
        selected = top_i[count - 1];
        for (int j = 0; j < count; ++j) { acc += top_v[j]; if (target < acc) { selected = top_i[j]; break; } }
    }
    out_tokens[r] = (selected == NO_ID) ? -1 : (int)selected;
    if (seen != nullptr && seen_rows != nullptr && seen_rows[r] >= 0 && selected != NO_ID)
        seen[(size_t)seen_rows[r] * V + selected] = 1;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_merge_kernel(float2* __restrict__ cand, int ncand, int k, float temperature, float top_p,
                    unsigned* __restrict__ rng_state, int* __restrict__ out_tokens, unsigned char* __restrict__ seen,
                    const int* __restrict__ seen_rows, int V, const int* __restrict__ status_in,
                    int* __restrict__ error_flag) {
    pdl_wait();
    // what the kernels of this step reported (a bounded wait that ran out) joins the error word
    // that the host reads with the chosen ids: bit 1 = "a kernel gave up", its status from bit 8 up
    if (blockIdx.x == 0 && threadIdx.x == 0 && status_in != nullptr && error_flag != nullptr) {
        const int s = *status_in;
        if (s != 0) atomicOr(error_flag, 2 | (s << 8));
    }
    __shared__ float sv[32];
    __shared__ unsigned si[32];
    __shared__ float top_v[SAMPLE_MAX_K];
    __shared__ unsigned top_i[SAMPLE_MAX_K];
    const int r = blockIdx.x;
    float2* c = cand + (size_t)r * ncand;
    for (int j = 0; j < k; ++j) {
        float bv = -FLT_MAX;
        unsigned bi = NO_ID;
        for (int i = threadIdx.x; i < ncand; i += blockDim.x) {
            const float2 e = c[i];
            const unsigned id = __float_as_uint(e.y);
            if (better(e.x, id, bv, bi)) { bv = e.x; bi = id; }
        }
        block_argmax(bv, bi, sv, si);
        if (threadIdx.x == 0) { top_v[j] = bv; top_i[j] = bi; }
        if (bi != NO_ID)
            for (int i = threadIdx.x; i < ncand; i += blockDim.x)
                if (__float_as_uint(c[i].y) == bi) c[i] = make_float2(-FLT_MAX, __uint_as_float(NO_ID));
        __syncthreads();
    }
    if (threadIdx.x == 0)
        draw(top_v, top_i, k, temperature, top_p, rng_state, out_tokens, seen, seen_rows, V, r);
}

// ---------------------------------------------------------------------------------
// The k best of a row without k rounds over everything.  If T is the k-th largest of the tiles' maxima, at least k
// values of the row are >= T, so the k best are all among the values >= T, and these are few (k of them and what
// else the best tiles hold above T).  Four short kernels: the maximum of every tile; T per row (the rank of every
// maximum by counting, no rounds); the values >= T appended to a short list per row (tiles whose maximum is below
// T leave at once); the k best of the list by rank counting, then the draw.  Ties are decided by the lowest id
// everywhere, so the result is that of the exact top-k (reference: tensor.comp:121-199).  A list that overflows
// (thousands of values above T: a tile of outliers) is not used: the last kernel then takes k rounds over the row.
// ---------------------------------------------------------------------------------
#define SAMPLE_LIST 4096

__device__ __forceinline__ float penalised(const float* row, const unsigned char* srow, float penalty, int tok, bool& bad) {
    float s = row[tok];
    if (isnan(s) || isinf(s)) { bad = true; return -FLT_MAX; }
    if (srow != nullptr && srow[tok]) s = s < 0.f ? s * penalty : s / penalty;
    return s;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_tilemax_kernel(const float* __restrict__ logits, int V, int tile, float penalty, const unsigned char* __restrict__ seen,
                      const int* __restrict__ seen_rows, float* __restrict__ tmax, int* __restrict__ error_flag) {
    pdl_wait();
    __shared__ float sv[32];
    const int t = blockIdx.x, r = blockIdx.y, tiles = gridDim.x;
    const float* row = logits + (size_t)r * V;
    const unsigned char* srow = nullptr;
    if (seen != nullptr && seen_rows != nullptr && seen_rows[r] >= 0) srow = seen + (size_t)seen_rows[r] * V;
    bool bad = false;
    float m = -FLT_MAX;
    for (int i = threadIdx.x; i < tile; i += blockDim.x) {
        const int tok = t * tile + i;
        if (tok < V) m = fmaxf(m, penalised(row, srow, penalty, tok, bad));
    }
    if (bad && error_flag != nullptr) atomicOr(error_flag, 1);
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) sv[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x < 32) {
        m = threadIdx.x < (blockDim.x >> 5) ? sv[threadIdx.x] : -FLT_MAX;
        m = warp_max(m);
        if (threadIdx.x == 0) tmax[(size_t)r * tiles + t] = m;
    }
}

// thr[r] = the k-th largest of the row's tile maxima (-FLT_MAX with fewer than k tiles); count[r] = 0
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_threshold_kernel(const float* __restrict__ tmax, int tiles, int k, float* __restrict__ thr, int* __restrict__ count) {
    pdl_wait();
    extern __shared__ float sm_max[];
    const int r = blockIdx.x;
    for (int i = threadIdx.x; i < tiles; i += blockDim.x) sm_max[i] = tmax[(size_t)r * tiles + i];
    if (threadIdx.x == 0) {
        count[r] = 0;
        if (tiles < k) thr[r] = -FLT_MAX;
    }
    __syncthreads();
    if (tiles < k) return;
    for (int i = threadIdx.x; i < tiles; i += blockDim.x) {
        const float v = sm_max[i];
        int rank = 0;
        for (int j = 0; j < tiles; ++j) rank += better(sm_max[j], (unsigned)j, v, (unsigned)i) ? 1 : 0;
        if (rank == k - 1) thr[r] = v;
    }
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_collect_kernel(const float* __restrict__ logits, int V, int tile, float penalty, const unsigned char* __restrict__ seen,
                      const int* __restrict__ seen_rows, const float* __restrict__ tmax, const float* __restrict__ thr,
                      int* __restrict__ count, float2* __restrict__ list) {
    pdl_wait();
    const int t = blockIdx.x, r = blockIdx.y, tiles = gridDim.x;
    const float T = thr[r];
    if (tmax[(size_t)r * tiles + t] < T) return;
    const float* row = logits + (size_t)r * V;
    const unsigned char* srow = nullptr;
    if (seen != nullptr && seen_rows != nullptr && seen_rows[r] >= 0) srow = seen + (size_t)seen_rows[r] * V;
    bool bad = false;
    for (int i = threadIdx.x; i < tile; i += blockDim.x) {
        const int tok = t * tile + i;
        if (tok >= V) continue;
        const float s = penalised(row, srow, penalty, tok, bad);
        if (s >= T && !bad) {
            const int pos = atomicAdd(&count[r], 1);
            if (pos < SAMPLE_LIST) list[(size_t)r * SAMPLE_LIST + pos] = make_float2(s, __uint_as_float((unsigned)tok));
        }
        bad = false;
    }
}

__global__ void __launch_bounds__(1024)
sample_pick_kernel(const float* __restrict__ logits, int V, float penalty, const float2* __restrict__ list,
                   const int* __restrict__ count, int k, float temperature, float top_p, unsigned* __restrict__ rng_state,
                   int* __restrict__ out_tokens, unsigned char* __restrict__ seen, const int* __restrict__ seen_rows,
                   const int* __restrict__ status_in, int* __restrict__ error_flag) {
    pdl_wait();
    if (blockIdx.x == 0 && threadIdx.x == 0 && status_in != nullptr && error_flag != nullptr) {
        const int s = *status_in;
        if (s != 0) atomicOr(error_flag, 2 | (s << 8));
    }
    __shared__ float2 sl[SAMPLE_LIST];
    __shared__ float sv[32];
    __shared__ unsigned si[32];
    __shared__ float top_v[SAMPLE_MAX_K];
    __shared__ unsigned top_i[SAMPLE_MAX_K];
    const int r = blockIdx.x;
    const int n = count[r];
    if (threadIdx.x < SAMPLE_MAX_K) { top_v[threadIdx.x] = -FLT_MAX; top_i[threadIdx.x] = NO_ID; }
    if (n <= SAMPLE_LIST) {
        for (int i = threadIdx.x; i < n; i += blockDim.x) sl[i] = list[(size_t)r * SAMPLE_LIST + i];
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float v = sl[i].x;
            const unsigned id = __float_as_uint(sl[i].y);
            int rank = 0;
            for (int j = 0; j < n; ++j) rank += better(sl[j].x, __float_as_uint(sl[j].y), v, id) ? 1 : 0;
            if (rank < k) { top_v[rank] = v; top_i[rank] = id; }
        }
    } else {
        // the list overflowed: k rounds over the whole row, each for the best value after the one before
        const float* row = logits + (size_t)r * V;
        const unsigned char* srow = nullptr;
        if (seen != nullptr && seen_rows != nullptr && seen_rows[r] >= 0 && penalty != 1.f) srow = seen + (size_t)seen_rows[r] * V;
        float pv = FLT_MAX;
        unsigned pi = 0;
        bool first = true;
        for (int j = 0; j < k; ++j) {
            float bv = -FLT_MAX;
            unsigned bi = NO_ID;
            for (int tok = threadIdx.x; tok < V; tok += blockDim.x) {
                bool bad = false;
                const float s = penalised(row, srow, penalty, tok, bad);
                if (bad) continue;
                if ((first || better(pv, pi, s, (unsigned)tok)) && better(s, (unsigned)tok, bv, bi)) { bv = s; bi = (unsigned)tok; }
            }
            block_argmax(bv, bi, sv, si);
            if (threadIdx.x == 0) { top_v[j] = bv; top_i[j] = bi; }
            if (bi == NO_ID) break;
            pv = bv;
            pi = bi;
            first = false;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0)
        draw(top_v, top_i, k, temperature, top_p, rng_state, out_tokens, seen, seen_rows, V, r);
}

static int sample_tile_for(int V) { return V >= 65536 ? 1024 : (V >= 16384 ? 256 : 64); }

// Scratch `cand`: R * ceil(V/1024) * k float2.
QNN_API int qnn_sample(const float* logits, int R, int V, int top_k, float temperature, float top_p, float penalty,
                       unsigned* rng_state, unsigned char* seen, const int* seen_rows, void* cand, int* out_tokens,
                       int* error_flag, const int* status_in, cudaStream_t st) {
    if (R <= 0) return 0;
    if (V <= 0 || top_k < 1 || !(temperature >= 0.f) || !(top_p > 0.f && top_p <= 1.f) || !(penalty > 0.f))
        return QNN_ERR_ARGUMENT;
    int k = top_k > SAMPLE_MAX_K ? SAMPLE_MAX_K : top_k;
    if (k > V) k = V;
    if (temperature <= 0.f) k = 1;
    if (R > 65535) return QNN_ERR_UNSUPPORTED;
    if (k > 1) {
        const int tile = sample_tile_for(V), nt = (V + tile - 1) / tile;
        if (nt <= 8192) {
            const unsigned char* sn = penalty != 1.f ? seen : nullptr;
            float* tmax = (float*)cand;
            float* thr = tmax + (size_t)R * nt;
            int* count = (int*)(thr + R);
            float2* list = (float2*)(((uintptr_t)(count + R) + 15) & ~(uintptr_t)15);
            const int threads = tile < SAMPLE_THREADS ? tile : SAMPLE_THREADS;
            qnn::launch_pdl(sample_tilemax_kernel, dim3(nt, R), dim3(threads), 0, st, logits, V, tile, penalty, sn, seen_rows,
                            tmax, error_flag);
            qnn::launch_pdl(sample_threshold_kernel, dim3(R), dim3(SAMPLE_THREADS), (size_t)nt * sizeof(float), st,
                            (const float*)tmax, nt, k, thr, count);
            qnn::launch_pdl(sample_collect_kernel, dim3(nt, R), dim3(threads), 0, st, logits, V, tile, penalty, sn, seen_rows,
                            (const float*)tmax, (const float*)thr, count, list);
            qnn::launch_pdl(sample_pick_kernel, dim3(R), dim3(1024), 0, st, logits, V, penalty, (const float2*)list,
                            (const int*)count, k, temperature, top_p, rng_state, out_tokens, seen, seen_rows, status_in,
                            error_flag);
            QNN_LAUNCH_CHECK();
        }
    }
    const int tiles = (V + SAMPLE_TILE - 1) / SAMPLE_TILE;
    qnn::launch_pdl(sample_tile_kernel, dim3(dim3(tiles, R)), dim3(SAMPLE_THREADS), 0, st, logits, V, k, penalty, penalty != 1.f ? seen : nullptr,
                                                                 seen_rows, (float2*)cand, error_flag);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
    qnn::launch_pdl(sample_merge_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, st, (float2*)cand, tiles * k, k, temperature, top_p, rng_state,
                                                      out_tokens, seen, seen_rows, V, status_in, error_flag);
    QNN_LAUNCH_CHECK();
}

// k = 1 over many candidates (the 16-column candidates of the head's arg-max epilogue: 16,000 per row at a
// vocabulary of 256,000): one block of 1024 threads per row, every thread's loads independent of one another,
// one block-wide arg-max.  Nothing is erased: the candidates stay as they were.
__global__ void __launch_bounds__(1024)
argmax_candidates_kernel(const float2* __restrict__ cand, int ncand, int* __restrict__ out_tokens,
                         const int* __restrict__ status_in, int* __restrict__ error_flag) {
    pdl_wait();
    if (blockIdx.x == 0 && threadIdx.x == 0 && status_in != nullptr && error_flag != nullptr) {
        const int s = *status_in;
        if (s != 0) atomicOr(error_flag, 2 | (s << 8));
    }
    __shared__ float sv[32];
    __shared__ unsigned si[32];
    const float2* c = cand + (size_t)blockIdx.x * ncand;
    float bv = -FLT_MAX;
    unsigned bi = NO_ID;
    int i = threadIdx.x;
    for (; i + 3 * 1024 < ncand; i += 4 * 1024) {
        float2 e[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) e[j] = __ldg(c + i + j * 1024);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const unsigned id = __float_as_uint(e[j].y);
            if (better(e[j].x, id, bv, bi)) { bv = e[j].x; bi = id; }
        }
    }
    for (; i < ncand; i += 1024) {
        const float2 e = __ldg(c + i);
        const unsigned id = __float_as_uint(e.y);
        if (better(e.x, id, bv, bi)) { bv = e.x; bi = id; }
    }
    block_argmax(bv, bi, sv, si);
    if (threadIdx.x == 0) out_tokens[blockIdx.x] = (bi == NO_ID) ? -1 : (int)bi;
}

// The second half of qnn_sample alone, on candidates that another kernel produced (the arg-max
// epilogue of the head product): cand[r][0..ncand) = (value, id), k best of them per row, then the
// draw.  The candidates are consumed (overwritten), except for a plain arg-max (k = 1, no table of seen ids).
QNN_API int qnn_sample_candidates(void* cand, int R, int ncand, int V, int top_k, float temperature, float top_p,
                                  unsigned* rng_state, unsigned char* seen, const int* seen_rows, int* out_tokens,
                                  int* error_flag, const int* status_in, cudaStream_t st) {
    if (R <= 0) return 0;
    if (ncand <= 0 || top_k < 1 || !(temperature >= 0.f) || !(top_p > 0.f && top_p <= 1.f)) return QNN_ERR_ARGUMENT;
    int k = top_k > SAMPLE_MAX_K ? SAMPLE_MAX_K : top_k;
    if (k > ncand) k = ncand;
    if (temperature <= 0.f) k = 1;
    if (k == 1 && seen == nullptr) {
        qnn::launch_pdl(argmax_candidates_kernel, dim3(R), dim3(1024), 0, st, (const float2*)cand, ncand, out_tokens,
                        status_in, error_flag);
        QNN_LAUNCH_CHECK();
    }
    qnn::launch_pdl(sample_merge_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, st, (float2*)cand, ncand, k, temperature, top_p,
                    rng_state, out_tokens, seen, seen_rows, V, status_in, error_flag);
    QNN_LAUNCH_CHECK();
}

QNN_API int qnn_sample_scratch_bytes(int R, int V, int top_k) {
    int k = top_k > SAMPLE_MAX_K ? SAMPLE_MAX_K : (top_k < 1 ? 1 : top_k);
    const long long tiles = (V + SAMPLE_TILE - 1) / SAMPLE_TILE;
    long long b = (long long)R * tiles * k * 8;
    // the threshold selection: tile maxima, threshold and count per row, the list
    const int tile = sample_tile_for(V);
    const long long nt = (V + tile - 1) / tile;
    const long long b2 = (long long)R * nt * 4 + (long long)R * 8 + 16 + (long long)R * SAMPLE_LIST * 8;
    if (b2 > b) b = b2;
    return b > 0x7fffffff ? -1 : (int)b;
}

// seen[rows[t]][tokens[t]] = 1   (prompt tokens; rows[t] < 0 is skipped)
__global__ void mark_seen_kernel(const int* __restrict__ tokens, const int* __restrict__ rows,
                                 unsigned char* __restrict__ seen, int V, int T) {
    pdl_wait();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const int tok = tokens[t], r = rows[t];
    if (r >= 0 && tok >= 0 && tok < V) seen[(size_t)r * V + tok] = 1;
}
QNN_API int qnn_mark_seen(const int* tokens, const int* rows, unsigned char* seen, int V, int T, cudaStream_t st) {
    if (T <= 0) return 0;
    qnn::launch_pdl(mark_seen_kernel, dim3((T + 255) / 256), dim3(256), 0, st, tokens, rows, seen, V, T);
    QNN_LAUNCH_CHECK();
}

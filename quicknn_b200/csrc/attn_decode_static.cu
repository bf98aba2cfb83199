// The no-allocation variant of decode attention; see qnn_no_alloc.h for who needs it and the
// rules of use.  The kernels are those of attention.cu, reached through qnn_attn_decode; only
// the scratch differs: it is the array below instead of buffers the caller allocated.
#include "common.cuh"
#include "qnn_no_alloc.h"
#include <stdio.h>
#include <mutex>

// Partial (max, sum, O) of every key range of every (sequence, head).  In host code this name
// is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_decode_scratch[QNN_NO_ALLOC_SCRATCH_BYTES];

extern "C" int qnn_attn_decode(const void* q, long long q_stride, int dtype, const void* k_pool, const void* v_pool,
                               const int* page_table, int max_pages, int page_size, int ring, const int* slots,
                               const int* slot_len, int B, int nq, int nkv, int hd, float scale, float cap,
                               int window, float* part_o, float* part_ml, int n_splits, void* out,
                               long long out_stride, cudaStream_t st);

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_setup_lock;
void* g_scratch_address[kMaxDevices];   // device address of g_decode_scratch, per device; null = not looked up yet

// Once per device, with that device current: ask the runtime where the array lives there.
int scratch_for_current_device(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return QNN_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> hold(g_setup_lock);
    if (g_scratch_address[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_decode_scratch);
        if (e != cudaSuccess) return (int)e;
        if (p == nullptr) return QNN_ERR_ARGUMENT;
        g_scratch_address[dev] = p;
    }
    *out = g_scratch_address[dev];
    return 0;
}
}  // namespace

QNN_API int qnn_attn_decode_static(const void* q, long long q_stride, int dtype, const void* k_pool,
                                   const void* v_pool, const int* page_table, int max_pages, int page_size, int ring,
                                   const int* slots, const int* slot_len, int B, int n_heads, int n_kv_heads,
                                   int head_dim, float scale, float cap, int window, int n_splits, void* out,
                                   long long out_stride, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (n_heads <= 0 || head_dim <= 0 || n_splits <= 0) return QNN_ERR_ARGUMENT;
    const unsigned long long rows = (unsigned long long)B * (unsigned long long)n_heads * (unsigned long long)n_splits;
    const unsigned long long o_bytes = rows * (unsigned long long)head_dim * sizeof(float);
    const unsigned long long need = o_bytes + rows * 2ull * sizeof(float);
    if (need > QNN_NO_ALLOC_SCRATCH_BYTES) {
        fprintf(stderr,
                "qnn_attn_decode_static: %llu bytes of scratch needed (B=%d heads=%d splits=%d head_dim=%d) but the "
                "built-in scratch holds %u; use fewer splits or a smaller batch, or call qnn_attn_decode with "
                "buffers of your own\n",
                need, B, n_heads, n_splits, head_dim, QNN_NO_ALLOC_SCRATCH_BYTES);
        return QNN_ERR_NO_ALLOC_TOO_LARGE;
    }
    void* base = nullptr;
    const int rc = scratch_for_current_device(&base);
    if (rc != 0) return rc;
    float* part_o = reinterpret_cast<float*>(base);
    float* part_ml = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(base) + o_bytes);
    return qnn_attn_decode(q, q_stride, dtype, k_pool, v_pool, page_table, max_pages, page_size, ring, slots, slot_len,
                           B, n_heads, n_kv_heads, head_dim, scale, cap, window, part_o, part_ml, n_splits, out,
                           out_stride, stream);
}

// qnn_attn_decode_static: decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in HemulGM/QuickNN; it exists for hosts that embed this
// library through its C symbols rather than through PyTorch.  Such a host often cannot call
// cudaMalloc once it is running: a serving process whose device memory was carved up at start
// by an arena of its own (a later driver allocation would either fail or steal from that
// budget), a latency-bound loop in which cudaMalloc's implicit device-wide synchronisation is
// not acceptable, or a sandboxed worker whose policy forbids driver allocations after set-up.
// qnn_attn_decode needs two scratch buffers for the partial results of its key ranges; here
// they live in a fixed array inside the library instead.
//
//   * The scratch is a file-scope `static __device__` array of QNN_NO_ALLOC_SCRATCH_BYTES
//     (4 MiB).  Every GPU on which the library's module gets loaded holds these 4 MiB until the
//     process exits, whether or not this entry point is ever called.
//   * A call needs  B * n_heads * n_splits * (head_dim + 2) * 4  bytes of it.  More than the
//     maximum is refused: the function prints one line to stderr naming the need and the limit
//     and returns QNN_ERR_NO_ALLOC_TOO_LARGE; nothing is launched.
//   * It calls no cudaMalloc, cudaFree or any allocating library routine.  The first call on
//     each device looks up the array's device address (cudaGetSymbolAddress) and remembers it;
//     make that first call outside any stream capture.  Later calls on that device only launch.
//     The address is the current device's: `stream` must be a stream of the device that is
//     current when the function is called (cudaSetDevice first, as for any launch).
//   * All calls share the one array, and it keeps the previous call's partial results.  Nothing
//     in it has to start at zero: a call writes every element that it later reads.  Two calls
//     that overlap on the GPU (different streams, or different host threads without ordering)
//     race on it; serialise them on one stream or with events.
//
// Arguments and result are those of qnn_attn_decode (attention.cu) without the two scratch
// pointers: inputs, outputs, page tables and lengths are still the caller's device memory.
#pragma once
#include <cuda_runtime.h>

#define QNN_NO_ALLOC_SCRATCH_BYTES (4u << 20)
#define QNN_ERR_NO_ALLOC_TOO_LARGE 10003

#ifdef __cplusplus
extern "C" {
#endif

int qnn_attn_decode_static(const void* q, long long q_stride, int dtype, const void* k_pool, const void* v_pool,
                           const int* page_table, int max_pages, int page_size, int ring, const int* slots,
                           const int* slot_len, int B, int n_heads, int n_kv_heads, int head_dim, float scale,
                           float cap, int window, int n_splits, void* out, long long out_stride,
                           cudaStream_t stream);

#ifdef __cplusplus
}
#endif

// Shared device helpers for the sm_100a kernels of quicknn_b200.
//
// Conventions of every launcher in this directory:
//   * plain C entry points, raw device pointers, an explicit cudaStream_t;
//   * dtype codes: 0 = float32, 1 = bfloat16;
//   * the return value is a cudaError_t cast to int (0 = launched);
//   * sizes that a kernel cannot take are refused on the host side of the launcher
//     with QNN_ERR_UNSUPPORTED, never computed wrongly.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdlib.h>

#define QNN_ERR_UNSUPPORTED 10001
#define QNN_ERR_ARGUMENT 10002

#define QNN_DT_F32 0
#define QNN_DT_BF16 1

#define QNN_API extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;

namespace qnn {

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

// A value of runtime dtype read as float.
__device__ __forceinline__ float load_as_f(const void* p, int dtype, size_t i) {
    return dtype == QNN_DT_BF16 ? __bfloat162float(((const bf16*)p)[i]) : ((const float*)p)[i];
}
__device__ __forceinline__ void store_from_f(void* p, int dtype, size_t i, float v) {
    if (dtype == QNN_DT_BF16) ((bf16*)p)[i] = __float2bfloat16_rn(v);
    else ((float*)p)[i] = v;
}

// 16-byte vectors: 4 floats or 8 bf16.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    float4 raw;
    __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
    __device__ __forceinline__ void zero() { raw = make_float4(0.f, 0.f, 0.f, 0.f); }
    __device__ __forceinline__ void unpack(float* o) const { o[0] = raw.x; o[1] = raw.y; o[2] = raw.z; o[3] = raw.w; }
    __device__ __forceinline__ static void store(float* p, const float* v) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec16<bf16> {
    static constexpr int N = 8;
    uint4 raw;
    __device__ __forceinline__ void load(const bf16* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void zero() { raw = make_uint4(0u, 0u, 0u, 0u); }
    __device__ __forceinline__ void unpack(float* o) const {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[2 * i] = __uint_as_float(w[i] << 16);
            o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ __forceinline__ static void store(bf16* p, const float* v) {
        uint4 r;
        uint32_t* w = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = r;
    }
};

// Eight consecutive values of runtime dtype, 16-byte aligned, as floats (and back).
__device__ __forceinline__ void load8_as_f(const void* p, int dtype, size_t i, float* o) {
    if (dtype == QNN_DT_BF16) {
        Vec16<bf16> v;
        v.load((const bf16*)p + i);
        v.unpack(o);
    } else {
        const float4 a = *reinterpret_cast<const float4*>((const float*)p + i);
        const float4 b = *reinterpret_cast<const float4*>((const float*)p + i + 4);
        o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
    }
}
__device__ __forceinline__ void store8_from_f(void* p, int dtype, size_t i, const float* v) {
    if (dtype == QNN_DT_BF16) {
        Vec16<bf16>::store((bf16*)p + i, v);
    } else {
        *reinterpret_cast<float4*>((float*)p + i) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>((float*)p + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of
// additions depends only on blockDim, so a row gives the same sum in any batch.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem32[warp] = v;
    __syncthreads();
    float r = (lane < nwarp) ? smem32[lane] : 0.f;
    r = warp_sum(r);
    return r;
}

// cap * tanh(clamp(x / cap, -20, 20)); cap <= 0 switches it off.  NaN stays NaN.
__device__ __forceinline__ float softcap(float x, float cap) {
    if (cap > 0.f) {
        float t = fminf(fmaxf(x / cap, -20.f), 20.f);
        return x == x ? cap * tanhf(t) : x;   // fminf/fmaxf drop a NaN; it has to reach the finite check

    }
    return x;
}

__device__ __forceinline__ float gelu_tanh(float x) {
    return 0.5f * x * (1.f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }

// activation codes of the gated feed-forward
#define QNN_ACT_GELU_TANH 0
#define QNN_ACT_SILU 1
__device__ __forceinline__ float activate(float x, int act) {
    return act == QNN_ACT_SILU ? silu(x) : gelu_tanh(x);
}
// The same for results that are rounded to bfloat16 anyway: the hardware tanh (error about
// 2^-11, below bfloat16's rounding) and the fast exponential.
__device__ __forceinline__ float tanh_approx(float x) {
    float r;
    asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float activate_fast(float x, int act) {
    if (act == QNN_ACT_SILU) return __fdividef(x, 1.f + __expf(-x));
    return 0.5f * x * (1.f + tanh_approx(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

}  // namespace qnn

// ---- programmatic dependent launch ---------------------------------------------------------
// Every kernel of this library calls pdl_wait() before it touches memory that another kernel
// writes.  It blocks until everything before this kernel in the stream has completed and its
// writes are visible, and then lets the kernel that follows in the stream be scheduled while
// this one still runs.  Ordering is what it would be without the feature; what is saved is the
// follower's launch latency, and whatever a kernel chooses to do before pdl_wait() (prefetching
// weights, which no kernel writes) overlaps its predecessor.
//
// Measured on decode steps (batch 8, context 8192): releasing the follower before the wait (so
// that several kernels of the chain are resident at once) gained 1 % at hidden size 2304 and lost
// 40 % at hidden size 4608; releasing it after the wait gained 2 % and lost 9 %; and launching
// only grids of at most 1184 blocks this way gained 2 % and lost under 1 %.  Hence the order in
// pdl_wait() and the limit in launch_pdl(); QNN_PDL=0 switches the feature off and
// QNN_PDL_MAX_GRID changes the limit.
namespace qnn {
__device__ __forceinline__ void pdl_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("QNN_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}
inline long long pdl_max_grid() {
    static long long v = -1;
    if (v < 0) {
        const char* e = getenv("QNN_PDL_MAX_GRID");
        v = e ? atoll(e) : 1184;
    }
    return v;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl_enabled() && (long long)grid.x * grid.y * grid.z <= pdl_max_grid()) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
}  // namespace qnn

#define QNN_LAUNCH_CHECK() return (int)cudaGetLastError()

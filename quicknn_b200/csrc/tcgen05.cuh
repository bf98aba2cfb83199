// What the tcgen05 / TMA kernels of this directory share: mbarriers with bounded waits, tensor-map
// loads, shared-memory operand descriptors, tensor-memory loads and stores, the cluster's barrier and
// distributed shared memory, and the host-side tensor-map encoder.  Everything is inline PTX for
// sm_100a; nothing here comes from a library.
//
// Waits are bounded: mbar_wait returns false after about a second of SM clock, the caller then sets a
// status word in global memory and winds down (frees its tensor memory, joins its cluster barriers),
// so that a fault in a pipeline shows as an error on the host and never as a hung GPU.
#pragma once
#include "common.cuh"
#include <cuda.h>

namespace qnn {
namespace tc {

constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;   // SM clock cycles before a wait gives up
constexpr unsigned WAIT_HINT_NS = 1000u;                // longest suspension inside one try_wait

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

// ---- mbarriers ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// arrive on a barrier of another CTA of the cluster (`cluster_addr` from map_to_rank)
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// true when the phase with this parity has completed; false when the time limit ran out
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    const long long start = clock64();
    for (;;) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(bar), "r"(parity), "r"(WAIT_HINT_NS) : "memory");
        if (done) return true;
        if (clock64() - start > WAIT_LIMIT_CYCLES) return false;
    }
}
// the same for a whole warp: either every lane goes on or none does (for the warp-wide tcgen05.ld / st
// and votes that follow)
__device__ __forceinline__ bool mbar_wait_warp(unsigned bar, unsigned parity) {
    return __all_sync(0xffffffffu, mbar_wait(bar, parity));
}

// ---- TMA -----------------------------------------------------------------------------------------
// one box of a 2-d tensor map into this CTA's shared memory; bytes are counted on `bar`.  The innermost
// coordinate x times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, unsigned bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}

// ---- tensor-core operands and issue ------------------------------------------------------------
// Shared-memory operand descriptor with the 128-byte swizzle; leading and stride byte offsets in bytes.
__device__ __forceinline__ uint64_t umma_desc(unsigned smem_addr, unsigned lbo, unsigned sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);        // start address
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;         // leading byte offset
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;         // stride byte offset
    d |= (uint64_t)1 << 46;                             // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                             // 128-byte swizzle
    return d;
}
// K-major operand: rows of 128 bytes, groups of 8 rows 1024 bytes apart (the leading offset is unused)
__device__ __forceinline__ uint64_t umma_desc(unsigned smem_addr) { return umma_desc(smem_addr, 16, 1024); }

// D[tmem] (+)= A[smem] B[smem], bfloat16 operands, float32 accumulation, issued by one thread of one CTA
__device__ __forceinline__ void umma_bf16_cta1(unsigned tmem_d, uint64_t adesc, uint64_t bdesc, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on `bar` once everything this thread has issued so far is done
__device__ __forceinline__ void umma_commit_cta1(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- tensor memory -----------------------------------------------------------------------------
// 32 consecutive columns of this thread's lane; the values are valid after tmem_ld_wait()
__device__ __forceinline__ void tmem_ld32_nowait(unsigned taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32_sync(unsigned taddr, uint32_t (&r)[32]) {
    tmem_ld32_nowait(taddr, r);
    tmem_ld_wait();
}
__device__ __forceinline__ void tmem_st32(unsigned taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// ---- thread-block clusters ---------------------------------------------------------------------
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_barrier() {
    cluster_arrive();
    cluster_wait();
}
// the shared::cluster address of `local_addr` in the CTA of rank `rank`
__device__ __forceinline__ unsigned map_to_rank(unsigned local_addr, unsigned rank) {
    unsigned remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}
// `bytes` (a multiple of 16) from `src_local` in this CTA's shared memory to `dst_local` in the CTA of rank
// `rank`; completion is counted in bytes on that CTA's mbarrier at `bar_local`.
__device__ __forceinline__ void bulk_copy_to_rank(unsigned dst_local, unsigned src_local, unsigned bytes, unsigned bar_local,
                                                  unsigned rank) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(map_to_rank(dst_local, rank)), "r"(src_local), "r"(bytes), "r"(map_to_rank(bar_local, rank)) : "memory");
}

// ---- host: tensor maps ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's entry-point query (the library does not link libcuda)
inline EncodeTiled tensor_map_encoder() {
    static EncodeTiled fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiled>(p);
    }
    return fn;
}

// rows x width bfloat16, row-major; box = 64 columns x box_rows rows, 128-byte swizzle, zero fill outside.
// Returns 0, QNN_ERR_UNSUPPORTED (no encoder) or QNN_ERR_ARGUMENT (the driver refused base or strides).
inline int make_map_bf16(CUtensorMap* map, const void* base, long long rows, long long width, int box_rows,
                         CUtensorMapL2promotion promotion = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
    EncodeTiled enc = tensor_map_encoder();
    if (enc == nullptr) return QNN_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)width * 2};
    const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promotion,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : QNN_ERR_ARGUMENT;
}

}  // namespace tc
}  // namespace qnn

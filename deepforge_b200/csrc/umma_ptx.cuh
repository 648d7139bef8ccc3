// PTX wrappers shared by the tcgen05 kernels (TMA, mbarrier, tensor memory, UMMA) and the
// host-side tensor-map helper. Every wait goes through mbar_wait(), which gives up after ~2 s of
// wall clock and records a code in g_device_status, so no kernel can spin forever.
#pragma once

#include <cuda.h>

#include "umma.cuh"

namespace dfgpu {

namespace {

// One status word per translation unit (device globals are not shared across units without
// relocatable device code); dfgpu_device_status() reads and clears all of them.
__device__ int g_device_status = 0;

inline int read_and_clear_device_status(int* status) {
    int zero = 0;
    cudaError_t error = cudaMemcpyFromSymbol(status, g_device_status, sizeof(int));
    if (error == cudaSuccess) error = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    if (error != cudaSuccess) return fail(kExecutionFailed, "device_status: %s", cudaGetErrorString(error));
    return kOk;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
// Non-blocking probe: a completed phase is the common case in the steady state of a pipeline, and the
// potentially-suspending try_wait form costs a few hundred cycles even then.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: false after ~2 s, with `code` left in g_device_status. The common case (the phase
// is already complete, or completes within the hardware's own suspend window) stays inline; only
// the long wait is a call, so the hot loops do not pay a call's register save/restore.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, int code) {
    const uint64_t start = global_timer_ns();
    for (;;) {
        for (int spin = 0; spin < 128; ++spin)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - start > 2000000000ull) {
            atomicCAS(&g_device_status, 0, code);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code) {
    if (mbar_test_wait(bar, parity)) return true;
#pragma unroll 1
    for (int spin = 0; spin < 64; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, code);
}

// Whole-warp forms for the loader and issuing warps. Their loops run on all 32 lanes with warp-uniform
// control flow, so addresses, descriptors and counters live in uniform registers (the operands the TMA
// and tcgen05 instructions take) and only the asynchronous instruction itself is predicated on one
// elected lane; a loop that runs inside `if (lane == 0)` pays a vector-to-uniform move per operand.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, int code) {
    if (__all_sync(0xffffffffu, mbar_test_wait(bar, parity))) return true;
#pragma unroll 1
    for (int spin = 0; spin < 64; ++spin)
        if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    return __all_sync(0xffffffffu, mbar_wait_slow(bar, parity, code)) != 0;
}
__device__ __forceinline__ bool elect_one() {
    uint32_t elected;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(elected));
    return elected != 0;
}
__device__ __forceinline__ int uniform_warp_index() { return __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
}

// Starts the fetch of a tensor map into the TMA unit's descriptor cache; the first copy that uses the map otherwise
// pays that global-memory round trip on the critical path of the kernel's prologue.
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void epilogue_barrier(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
// RELU_FWD with the same result as relu_forward() in fewer instructions: NaN in -> NaN out,
// x < lower takes the sloped branch, otherwise clip to [lower, upper].
__device__ __forceinline__ float relu_fast(float x, float lower, float upper, float slope) {
    float clipped = fminf(fmaxf(x, lower), upper);
    float result = x < lower ? fmaf(slope, x - lower, lower) : clipped;
    return x != x ? x : result;
}

__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, Blackwell version bit set.
// K-major operand: rows of 64 bf16 (128 B), 8-row groups 1024 B apart (SBO); LBO unused (1).
// MN-major operand: 64-element chunks along MN are `lbo_bytes` apart, 8-row K groups 1024 B apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t address, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((address & 0x3FFFFu) >> 4);
    desc |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    desc |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    desc |= 1ull << 46;
    desc |= 2ull << 61;
    return desc;
}

// The same descriptor as two 32-bit words. Issuing one product costs about as many cycles as the
// instructions around it (a lone lane has nothing to hide latency with): building the 64-bit value with
// shifts and ORs per product makes a 128 x 128 x 16 product issue in ~120 cycles, twice what the tensor pipe
// needs to run it. The high word never changes and the low word advances by (bytes >> 4), so a K step is
// one 32-bit add.
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t address, uint32_t lbo_bytes) {
    return ((address & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ constexpr uint32_t smem_desc_hi(uint32_t sbo_bytes) { return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29); }
__device__ __forceinline__ uint64_t desc_words(uint32_t lo, uint32_t hi) {
    uint64_t desc;
    asm("mov.b64 %0, {%1, %2};" : "=l"(desc) : "r"(lo), "r"(hi));
    return desc;
}

// ---- host: tensor maps ------------------------------------------------------------------------

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The encoder is a DRIVER entry point and needs a current context. A host thread that has made no runtime call yet
// (a worker thread of the caller's pool running its first launch) has none: bind the primary context of the thread's
// current device once per thread, the way the first runtime call would.
inline void bind_primary_context() {
    thread_local const bool bound = [] {
        int device = 0;
        return cudaGetDevice(&device) == cudaSuccess && cudaSetDevice(device) == cudaSuccess;  // (binds; allocates nothing)
    }();
    (void)bound;
}

inline EncodeTiled encode_tiled() {
    bind_primary_context();
    static EncodeTiled fn = [] {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            entry = nullptr;
        return reinterpret_cast<EncodeTiled>(entry);
    }();
    return fn;
}

// bf16 tensor map with a 64-element (128-byte) swizzled inner box.
inline int make_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
             const uint32_t* box, const char* what) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return fail(kExecutionFailed, "%s: cuTensorMapEncodeTiled is unavailable", what);
    cuuint32_t element_strides[5] = {1, 1, 1, 1, 1};
    CUresult result = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base),
                             reinterpret_cast<const cuuint64_t*>(dims), reinterpret_cast<const cuuint64_t*>(strides_bytes),
                             reinterpret_cast<const cuuint32_t*>(box), element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS) return fail(kExecutionFailed, "%s: tensor map encode failed (CUresult %d)", what, static_cast<int>(result));
    return kOk;
}


}  // namespace
}  // namespace dfgpu

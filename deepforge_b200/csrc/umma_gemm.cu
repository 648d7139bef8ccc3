// bf16 GEMM and implicit-GEMM convolution on the 5th-generation tensor cores.
//
// One CTA computes a 128 x BN tile of D = A * B^T with f32 accumulation in tensor
// memory. Roles (192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of 128x64 (A) and BNx64 (B)
//               bf16 tiles into a STAGES-deep shared-memory ring (128-byte swizzle),
//   warp 1      allocates TMEM, then one lane issues tcgen05.mma (M128 x BN x K16) and
//               releases ring slots with tcgen05.commit,
//   warps 2..5  epilogue: tcgen05.ld the accumulator (one row per thread), apply the
//               fused ADD / RELU steps, convert, store.
// A convolution is the same kernel with a different A producer: NHWC input is seen
// through a 4-D tensor map (C, W, H, N); a tile is `rows` whole output rows of one
// image, and for filter tap (r, s) the producer loads the box that starts at
// (c0, s - pad_w, h0 + r - pad_h, n). Out-of-range coordinates are zero-filled by the
// TMA unit, which is the convolution's padding. KRSC weights are already the K-major
// B operand with k = (r*S + s)*C + c.
//
// Every wait is bounded (wall-clock, ~2 s): on expiry the waiter records a code in
// g_device_status and all roles fall through to the common exit, so TMEM is always
// freed and the kernel always returns.
#include <cuda.h>

#include "umma.cuh"

namespace dfgpu {

__device__ int g_device_status = 0;

namespace {

// ---- PTX wrappers -------------------------------------------------------------------

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
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: false after ~2 s, with `code` left in g_device_status.
__device__ __noinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code) {
    if (mbar_try_wait(bar, parity)) return true;
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

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar) : "memory");
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

// ---- kernel ---------------------------------------------------------------------------

constexpr int kTileM = 128;
constexpr int kBlockK = 64;
constexpr int kThreads = 192;

enum { kEpiBias = 1, kEpiFull = 2, kEpiRelu = 3 };

struct GemmArgs {
    // problem
    int32_t k_blocks;          // total 64-wide K slices (taps * C/64 for a convolution)
    int32_t k_blocks_per_tap;  // C / 64
    int32_t is_conv;
    int32_t filter_s;          // S
    int32_t pad_h, pad_w;
    int32_t rows_per_tile;     // output rows of one image per tile (conv)
    int32_t tiles_per_image;   // ceil(P / rows_per_tile)
    int32_t out_p, out_q;      // P, Q
    int32_t b_mn_major;        // B given as [K, N] with N contiguous
    int64_t m_total;           // GEMM rows (non-conv)
    int64_t n_total;
    // output
    void* out;
    int64_t out_ld;            // elements between consecutive output rows
    int32_t out_dtype;         // DFGPU_BF16 or DFGPU_F32
    // epilogue
    int32_t epi_count;
    int32_t epi_kind[DFGPU_MAX_EPILOGUE];
    const void* epi_data[DFGPU_MAX_EPILOGUE];
    int32_t epi_dtype[DFGPU_MAX_EPILOGUE];
    int64_t epi_ld[DFGPU_MAX_EPILOGUE];
    float epi_lower[DFGPU_MAX_EPILOGUE], epi_upper[DFGPU_MAX_EPILOGUE], epi_slope[DFGPU_MAX_EPILOGUE];
};

template <int BN, int STAGES>
struct SmemLayout {
    static constexpr int kABytes = kTileM * kBlockK * 2;  // 16 KiB
    static constexpr int kBBytes = BN * kBlockK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarrierOffset = STAGES * kStageBytes;
    static constexpr int kTotal = kBarrierOffset + (2 * STAGES + 1) * 8 + 8;
    static constexpr int kDynamic = kTotal + 1024;  // slack for the 1024-byte alignment of the ring
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads)
umma_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmArgs args) {
    using L = SmemLayout<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + L::kBarrierOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    const uint32_t tmem_full_bar = bar_base + 8u * (2 * STAGES);
    const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 1);
    uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(generic_base + L::kBarrierOffset + 8 * (2 * STAGES + 1));

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tile = blockIdx.x, n_tile = blockIdx.y;
    const int n0 = n_tile * BN;

    // tile geometry
    int64_t out_row0;
    int valid_rows;
    int image = 0, h0 = 0;
    if (args.is_conv) {
        image = m_tile / args.tiles_per_image;
        h0 = (m_tile % args.tiles_per_image) * args.rows_per_tile;
        int rows = min(args.rows_per_tile, args.out_p - h0);
        valid_rows = rows * args.out_q;
        out_row0 = (static_cast<int64_t>(image) * args.out_p + h0) * args.out_q;
    } else {
        out_row0 = static_cast<int64_t>(m_tile) * kTileM;
        int64_t remaining = args.m_total - out_row0;
        valid_rows = remaining < kTileM ? static_cast<int>(remaining) : kTileM;
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(tmem_full_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, BN);
        tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        if (lane == 0) {
            const uint32_t a_bytes = args.is_conv ? static_cast<uint32_t>(args.rows_per_tile * args.out_q * kBlockK * 2) : L::kABytes;
            for (int kb = 0; kb < args.k_blocks; ++kb) {
                const int s = kb % STAGES;
                const uint32_t parity = ((kb / STAGES) & 1) ^ 1;
                if (!mbar_wait(empty_bar(s), parity, 101)) break;
                const uint32_t a_dst = smem_base + s * L::kStageBytes;
                const uint32_t b_dst = a_dst + L::kABytes;
                mbar_expect_tx(full_bar(s), a_bytes + L::kBBytes);
                const int tap = kb / args.k_blocks_per_tap;
                const int c0 = (kb - tap * args.k_blocks_per_tap) * kBlockK;
                if (args.is_conv) {
                    const int r = tap / args.filter_s, sx = tap - r * args.filter_s;
                    tma_load_4d(a_dst, &map_a, c0, sx - args.pad_w, h0 + r - args.pad_h, image, full_bar(s));
                } else {
                    tma_load_2d(a_dst, &map_a, kb * kBlockK, m_tile * kTileM, full_bar(s));
                }
                if (args.b_mn_major) {
#pragma unroll
                    for (int j = 0; j < BN / 64; ++j)
                        tma_load_2d(b_dst + j * (kBlockK * 128), &map_b, n0 + 64 * j, kb * kBlockK, full_bar(s));
                } else {
                    tma_load_2d(b_dst, &map_b, kb * kBlockK, n0, full_bar(s));
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D f32, A/B bf16, A K-major, B per flag, N = BN, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(args.b_mn_major) << 16) |
                                   (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < args.k_blocks && ok; ++kb) {
                const int s = kb % STAGES;
                const uint32_t parity = (kb / STAGES) & 1;
                ok = mbar_wait(full_bar(s), parity, 102);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_src = smem_base + s * L::kStageBytes;
                const uint32_t b_src = a_src + L::kABytes;
#pragma unroll
                for (int k = 0; k < kBlockK / 16; ++k) {
                    const uint64_t desc_a = smem_desc(a_src + k * 32, 16, 1024);
                    const uint64_t desc_b = args.b_mn_major ? smem_desc(b_src + k * 2048, kBlockK * 128, 1024)
                                                            : smem_desc(b_src + k * 32, 16, 1024);
                    umma_bf16(tmem_base, desc_a, desc_b, idesc, (kb | k) != 0 ? 1u : 0u);
                }
                umma_commit(empty_bar(s));
            }
            // always arrive, so the epilogue's wait ends even after a failed wait above
            umma_commit(tmem_full_bar);
        }
    } else {
        const int quadrant = warp & 3;  // TMEM lanes 32*quadrant .. +31 belong to this warp
        const int row = quadrant * 32 + lane;
        const bool ok = mbar_wait(tmem_full_bar, 0, 103);
        tc_fence_after();
        if (ok && g_device_status == 0) {
            const bool row_valid = row < valid_rows;
            const int64_t out_row = out_row0 + row;
#pragma unroll 1
            for (int chunk = 0; chunk < BN / 32; ++chunk) {
                uint32_t raw[32];
                tmem_load_32(tmem_base + (static_cast<uint32_t>(quadrant * 32) << 16) + chunk * 32, raw);
                tmem_load_wait();
                const int64_t col0 = n0 + chunk * 32;
                if (!row_valid || col0 >= args.n_total) continue;
                float v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
                for (int e = 0; e < args.epi_count; ++e) {
                    const int kind = args.epi_kind[e];
                    if (kind == kEpiRelu) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = relu_forward(v[i], args.epi_lower[e], args.epi_upper[e], args.epi_slope[e]);
                    } else {
                        const int64_t base = kind == kEpiBias ? col0 : out_row * args.epi_ld[e] + col0;
                        if (args.epi_dtype[e] == DFGPU_BF16) {
                            const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(args.epi_data[e]) + base);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint4 q = __ldg(p + j);
                                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                                for (int t = 0; t < 4; ++t) {
                                    v[8 * j + 2 * t] = __fadd_rn(v[8 * j + 2 * t], __uint_as_float(w[t] << 16));
                                    v[8 * j + 2 * t + 1] = __fadd_rn(v[8 * j + 2 * t + 1], __uint_as_float(w[t] & 0xffff0000u));
                                }
                            }
                        } else {
                            const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(args.epi_data[e]) + base);
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float4 q = __ldg(p + j);
                                v[4 * j] = __fadd_rn(v[4 * j], q.x);
                                v[4 * j + 1] = __fadd_rn(v[4 * j + 1], q.y);
                                v[4 * j + 2] = __fadd_rn(v[4 * j + 2], q.z);
                                v[4 * j + 3] = __fadd_rn(v[4 * j + 3], q.w);
                            }
                        }
                    }
                }
                if (args.out_dtype == DFGPU_BF16) {
                    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(args.out) + out_row * args.out_ld + col0);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t w[4];
#pragma unroll
                        for (int t = 0; t < 4; ++t)
                            w[t] = f32_to_bf16_bits(v[8 * j + 2 * t]) | (static_cast<uint32_t>(f32_to_bf16_bits(v[8 * j + 2 * t + 1])) << 16);
                        dst[j] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                } else {
                    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(args.out) + out_row * args.out_ld + col0);
#pragma unroll
                    for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, BN);
    }
}

// ---- host side ----------------------------------------------------------------------------

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
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
int make_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
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

template <int BN, int STAGES>
int launch(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmArgs& args, dim3 grid, cudaStream_t stream) {
    using L = SmemLayout<BN, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t error = cudaFuncSetAttribute(umma_gemm_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
        if (error != cudaSuccess) return fail(kExecutionFailed, "tcgen05 GEMM: cannot reserve %d bytes of shared memory: %s", L::kDynamic, cudaGetErrorString(error));
        configured = true;
    }
    umma_gemm_kernel<BN, STAGES><<<grid, kThreads, L::kDynamic, stream>>>(map_a, map_b, args);
    return check_launch("tcgen05 GEMM");
}

// Ring depth: shallow K loops (the 1x1 convolutions) get short rings so that several CTAs fit on
// one SM and overlap each other's load / MMA / epilogue phases; deep K loops (matmul) get 4 stages.
int dispatch(int bn, int k_blocks, const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmArgs& args, dim3 grid, cudaStream_t stream) {
    const int stages = k_blocks <= 1 ? 1 : (k_blocks <= 12 ? 2 : 4);
    if (bn == 64) {
        if (stages == 1) return launch<64, 1>(map_a, map_b, args, grid, stream);
        if (stages == 2) return launch<64, 2>(map_a, map_b, args, grid, stream);
        return launch<64, 4>(map_a, map_b, args, grid, stream);
    }
    if (bn == 128) {
        if (stages == 1) return launch<128, 1>(map_a, map_b, args, grid, stream);
        if (stages == 2) return launch<128, 2>(map_a, map_b, args, grid, stream);
        return launch<128, 4>(map_a, map_b, args, grid, stream);
    }
    if (stages <= 2) return launch<256, 2>(map_a, map_b, args, grid, stream);
    return launch<256, 4>(map_a, map_b, args, grid, stream);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool nhwc_packed(const dfgpu_tensor& t) {
    // logical [N, C, H, W] with strides [H*W*C, 1, W*C, C]
    return t.rank == 4 && t.stride[1] == 1 && t.stride[3] == t.dim[1] && t.stride[2] == t.dim[3] * t.dim[1] &&
           t.stride[0] == t.dim[2] * t.dim[3] * t.dim[1];
}

// Translate the generic epilogue into the kernel's three step kinds. Returns false when a
// step needs something the kernel does not do (then the CUDA-core kernel runs instead).
bool translate_epilogue(int count, const dfgpu_epilogue_step* steps, const dfgpu_tensor* extra, const dfgpu_tensor& out,
                        int channel_axis, bool out_rows_packed, int64_t out_ld, void* const* extra_pointers, GemmArgs* args) {
    if (count < 0 || count > DFGPU_MAX_EPILOGUE) return false;
    if (args) args->epi_count = count;
    for (int i = 0; i < count; ++i) {
        if (steps[i].op == DFGPU_EPI_RELU) {
            if (args) {
                args->epi_kind[i] = kEpiRelu;
                args->epi_lower[i] = steps[i].relu_lower;
                args->epi_upper[i] = steps[i].relu_upper;
                args->epi_slope[i] = steps[i].relu_slope;
            }
            continue;
        }
        if (steps[i].op != DFGPU_EPI_ADD || steps[i].operand < 0 || steps[i].operand > 1) return false;
        const dfgpu_tensor& t = extra[steps[i].operand];
        if (t.rank < 1 || t.rank > out.rank) return false;
        if (t.dtype != DFGPU_BF16 && t.dtype != DFGPU_F32) return false;
        const int shift = out.rank - t.rank;
        bool per_channel = true, full = t.rank == out.rank;
        for (int axis = 0; axis < t.rank; ++axis) {
            const int out_axis = axis + shift;
            if (out_axis == channel_axis) {
                if (t.dim[axis] != out.dim[out_axis] || t.stride[axis] != 1) per_channel = false;
            } else if (t.dim[axis] != 1) {
                per_channel = false;
            }
            if (t.dim[axis] != out.dim[out_axis] || t.stride[axis] != out.stride[out_axis]) full = false;
        }
        if (shift > channel_axis) per_channel = false;
        if (!per_channel && !(full && out_rows_packed)) return false;
        if (args) {
            args->epi_kind[i] = per_channel ? kEpiBias : kEpiFull;
            args->epi_data[i] = extra_pointers[steps[i].operand];
            args->epi_dtype[i] = t.dtype;
            args->epi_ld[i] = out_ld;
            if (!aligned16(args->epi_data[i])) return false;
        }
    }
    return true;
}

// Wide N tiles pay off when the K loop is long (matmul); with a short K loop a narrower tile keeps
// more CTAs resident per SM (less shared memory and TMEM each).
int pick_bn(int64_t n, int64_t k_blocks) {
    if (k_blocks > 12 && n % 256 == 0) return 256;
    return n % 128 == 0 ? 128 : 64;
}

}  // namespace

bool conv_umma_supported(const dfgpu_conv_params& p) {
    if (p.x.dtype != DFGPU_BF16 || p.w.dtype != DFGPU_BF16 || (p.y.dtype != DFGPU_BF16 && p.y.dtype != DFGPU_F32)) return false;
    if (!nhwc_packed(p.x) || !nhwc_packed(p.w) || !nhwc_packed(p.y)) return false;
    if (p.x.dim[1] != p.w.dim[1]) return false;  // groups == 1
    const int64_t C = p.x.dim[1], K = p.y.dim[1], Q = p.y.dim[3];
    if (C % 64 != 0 || K % 64 != 0 || Q > 128 || Q < 1) return false;
    if (p.stride[0] != 1 || p.stride[1] != 1 || p.dilation[0] != 1 || p.dilation[1] != 1 || p.reverse_filter) return false;
    if (p.w.dim[2] * p.w.dim[3] > 49 || p.x.dim[0] * p.y.dim[2] > (1 << 22)) return false;
    if (p.x.dim[2] > 65535 || p.x.dim[3] > 65535 || p.pre_pad[0] > 64 || p.pre_pad[1] > 64) return false;
    return translate_epilogue(p.epilogue_count, p.epilogue, p.extra, p.y, 1, true, K, nullptr, nullptr);
}

int launch_conv_umma(const dfgpu_conv_params& p, void* const* tensors, cudaStream_t stream) {
    const int64_t N = p.x.dim[0], C = p.x.dim[1], H = p.x.dim[2], W = p.x.dim[3];
    const int64_t K = p.y.dim[1], P = p.y.dim[2], Q = p.y.dim[3], R = p.w.dim[2], S = p.w.dim[3];
    if (!aligned16(tensors[0]) || !aligned16(tensors[1]) || !aligned16(tensors[2]))
        return fail(kInvalidArgument, "CONV_FPROP: the tcgen05 kernel needs 16-byte aligned X, W and Y");
    GemmArgs args{};
    const bool pointwise = R == 1 && S == 1 && p.pre_pad[0] == 0 && p.pre_pad[1] == 0 && p.post_pad[0] == 0 && p.post_pad[1] == 0;
    const int bn = pick_bn(K, R * S * (C / kBlockK));
    CUtensorMap map_a, map_b;
    int status;
    int64_t m_tiles;
    if (pointwise) {
        const int64_t M = N * H * W;
        uint64_t dims[2] = {static_cast<uint64_t>(C), static_cast<uint64_t>(M)};
        uint64_t strides[1] = {static_cast<uint64_t>(C) * 2};
        uint32_t box[2] = {kBlockK, kTileM};
        status = make_map(&map_a, tensors[0], 2, dims, strides, box, "CONV_FPROP X");
        if (status) return status;
        args.is_conv = 0;
        args.m_total = M;
        m_tiles = (M + kTileM - 1) / kTileM;
    } else {
        const int rows = static_cast<int>(kTileM / Q);
        uint64_t dims[4] = {static_cast<uint64_t>(C), static_cast<uint64_t>(W), static_cast<uint64_t>(H), static_cast<uint64_t>(N)};
        uint64_t strides[3] = {static_cast<uint64_t>(C) * 2, static_cast<uint64_t>(W * C) * 2, static_cast<uint64_t>(H * W * C) * 2};
        uint32_t box[4] = {kBlockK, static_cast<uint32_t>(Q), static_cast<uint32_t>(rows), 1};
        status = make_map(&map_a, tensors[0], 4, dims, strides, box, "CONV_FPROP X");
        if (status) return status;
        args.is_conv = 1;
        args.rows_per_tile = rows;
        args.tiles_per_image = static_cast<int>((P + rows - 1) / rows);
        m_tiles = N * args.tiles_per_image;
    }
    {
        uint64_t dims[2] = {static_cast<uint64_t>(R * S * C), static_cast<uint64_t>(K)};
        uint64_t strides[1] = {static_cast<uint64_t>(R * S * C) * 2};
        uint32_t box[2] = {kBlockK, static_cast<uint32_t>(bn)};
        status = make_map(&map_b, tensors[1], 2, dims, strides, box, "CONV_FPROP W");
        if (status) return status;
    }
    args.k_blocks_per_tap = static_cast<int>(C / kBlockK);
    args.k_blocks = static_cast<int>(R * S) * args.k_blocks_per_tap;
    args.filter_s = static_cast<int>(S);
    args.pad_h = static_cast<int>(p.pre_pad[0]);
    args.pad_w = static_cast<int>(p.pre_pad[1]);
    args.out_p = static_cast<int>(P);
    args.out_q = static_cast<int>(Q);
    args.b_mn_major = 0;
    args.n_total = K;
    args.out = tensors[2];
    args.out_ld = K;
    args.out_dtype = p.y.dtype;
    if (!translate_epilogue(p.epilogue_count, p.epilogue, p.extra, p.y, 1, true, K, tensors + 3, &args))
        return fail(kUnsupported, "CONV_FPROP: the fused epilogue is not one the tcgen05 kernel applies");
    dim3 grid(static_cast<unsigned>(m_tiles), static_cast<unsigned>(K / bn));
    return dispatch(bn, args.k_blocks, map_a, map_b, args, grid, stream);
}

bool matmul_umma_supported(const dfgpu_matmul_params& p, int kernel) {
    if (kernel != DFGPU_MATMUL_UMMA_BF16) return false;  // the MXFP8 variant is not built yet
    if (p.a_scale.rank || p.b_scale.rank) return false;
    if (p.a.dtype != DFGPU_BF16 || p.b.dtype != DFGPU_BF16 || (p.c.dtype != DFGPU_BF16 && p.c.dtype != DFGPU_F32)) return false;
    const int rank = p.c.rank;
    if (rank < 2) return false;
    for (int i = 0; i < rank - 2; ++i)
        if (p.c.dim[i] != 1 || p.a.dim[i] != 1 || p.b.dim[i] != 1) return false;
    const int64_t M = p.c.dim[rank - 2], N = p.c.dim[rank - 1], K = p.a.dim[rank - 1];
    if (K % 64 != 0 || N % 64 != 0 || M < 1 || M > (1ll << 30)) return false;
    if (p.a.stride[rank - 1] != 1 || p.a.stride[rank - 2] % 8 != 0 || p.a.stride[rank - 2] < K) return false;
    const bool b_k_major = p.b.stride[rank - 2] == 1 && p.b.stride[rank - 1] % 8 == 0 && p.b.stride[rank - 1] >= K;
    const bool b_n_major = p.b.stride[rank - 1] == 1 && p.b.stride[rank - 2] % 8 == 0 && p.b.stride[rank - 2] >= N;
    if (!b_k_major && !b_n_major) return false;
    if (p.c.stride[rank - 1] != 1 || p.c.stride[rank - 2] % 8 != 0 || p.c.stride[rank - 2] < N) return false;
    return translate_epilogue(p.epilogue_count, p.epilogue, p.extra, p.c, rank - 1, true, p.c.stride[rank - 2], nullptr, nullptr);
}

int launch_matmul_umma(const dfgpu_matmul_params& p, void* const* tensors, int kernel, cudaStream_t stream) {
    (void)kernel;
    const int rank = p.c.rank;
    const int64_t M = p.c.dim[rank - 2], N = p.c.dim[rank - 1], K = p.a.dim[rank - 1];
    if (!aligned16(tensors[0]) || !aligned16(tensors[1]) || !aligned16(tensors[2]))
        return fail(kInvalidArgument, "MATMUL: the tcgen05 kernel needs 16-byte aligned A, B and C");
    const int bn = pick_bn(N, K / kBlockK);
    const bool b_k_major = p.b.stride[rank - 2] == 1 && p.b.stride[rank - 1] % 8 == 0 && p.b.stride[rank - 1] >= K;
    const bool b_n_major = !b_k_major;
    GemmArgs args{};
    CUtensorMap map_a, map_b;
    {
        uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
        uint64_t strides[1] = {static_cast<uint64_t>(p.a.stride[rank - 2]) * 2};
        uint32_t box[2] = {kBlockK, kTileM};
        int status = make_map(&map_a, tensors[0], 2, dims, strides, box, "MATMUL A");
        if (status) return status;
    }
    if (b_n_major) {
        uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
        uint64_t strides[1] = {static_cast<uint64_t>(p.b.stride[rank - 2]) * 2};
        uint32_t box[2] = {64, kBlockK};
        int status = make_map(&map_b, tensors[1], 2, dims, strides, box, "MATMUL B");
        if (status) return status;
    } else {
        uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
        uint64_t strides[1] = {static_cast<uint64_t>(p.b.stride[rank - 1]) * 2};
        uint32_t box[2] = {kBlockK, static_cast<uint32_t>(bn)};
        int status = make_map(&map_b, tensors[1], 2, dims, strides, box, "MATMUL B");
        if (status) return status;
    }
    args.is_conv = 0;
    args.m_total = M;
    args.k_blocks_per_tap = static_cast<int>(K / kBlockK);
    args.k_blocks = args.k_blocks_per_tap;
    args.filter_s = 1;
    args.b_mn_major = b_n_major ? 1 : 0;
    args.n_total = N;
    args.out = tensors[2];
    args.out_ld = p.c.stride[rank - 2];
    args.out_dtype = p.c.dtype;
    if (!translate_epilogue(p.epilogue_count, p.epilogue, p.extra, p.c, rank - 1, true, args.out_ld, tensors + 5, &args))
        return fail(kUnsupported, "MATMUL: the fused epilogue is not one the tcgen05 kernel applies");
    dim3 grid(static_cast<unsigned>((M + kTileM - 1) / kTileM), static_cast<unsigned>(N / bn));
    return dispatch(bn, args.k_blocks, map_a, map_b, args, grid, stream);
}

bool sdpa_umma_supported(const dfgpu_sdpa_params&) { return false; }
int launch_sdpa_umma(const dfgpu_sdpa_params&, void* const*, void*, cudaStream_t) {
    return fail(kUnsupported, "SDPA: the tcgen05 kernel is not built");
}

}  // namespace dfgpu

// Reads and clears the device-side status word the bounded waits write (0 = none).
// Synchronises the device; meant for tests and for the runtime's post-mortem path.
extern "C" int dfgpu_device_status(int* status) {
    using namespace dfgpu;
    if (!status) return fail(kInvalidArgument, "device_status: null pointer");
    int zero = 0;
    cudaError_t error = cudaMemcpyFromSymbol(status, g_device_status, sizeof(int));
    if (error == cudaSuccess) error = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    if (error != cudaSuccess) return fail(kExecutionFailed, "device_status: %s", cudaGetErrorString(error));
    return kOk;
}

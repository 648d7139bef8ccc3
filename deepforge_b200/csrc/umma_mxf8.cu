// MATMUL on MXFP8 operands without a dequantize pass: C = (A_codes * 2^SFA) (B_codes * 2^SFB).
//
// The E4M3 codes and their E8M0 block scales (one per 32 elements along K) go straight into the
// block-scaled tensor-core instruction (tcgen05.mma.kind::mxf8f6f4.block_scale): the products of two
// E4M3 values are exact, the power-of-two scales are applied per 32-deep block, accumulation is f32 in
// tensor memory. That is the arithmetic of BLOCK_SCALE_DEQUANTIZE -> MATMUL in the reference
// (lib/Compiler/SpecializedGraph.cpp:752-795 feeding FoundationalGraph.cpp:3167-3295) up to the order
// of the f32 additions, and it reads 1 byte per element instead of writing and re-reading bf16 copies.
//
// Persistent kernel, one CTA per SM, 128 x BN output tile, K in steps of 128 elements (one 128-byte
// swizzled row):
//   warp 0      TMA: A tile (128 rows x 128 B) and B tile (BN x 128 B, K-major or N-major) into a 4-slot ring
//   warp 1      per slot: tcgen05.cp of the slot's scale factors into tensor memory, then 4 products of K = 32,
//               each selecting its scale byte through the instruction descriptor
//   warps 2-5   epilogue: tcgen05.ld -> fused steps -> bf16 / f32 -> global
//   warps 6-9   scale loaders, one ring slot each: gather the slot's 128 + BN scale words from the plain
//               [rows, K/32] / [K/32, cols] tensors and lay them out in shared memory the way the tensor core wants
//               them: 512-byte chunks of 128 rows x 4 K-blocks at (row % 32) * 16 + (row / 32) * 4 + block.
// Whole-warp uniform loops with one elected lane issuing, bounded waits, no spinning on other launches.
#include "umma.cuh"
#include "umma_ptx.cuh"

namespace dfgpu {
namespace {

constexpr int kTileM = 128;
constexpr int kBlockK = 128;   // fp8 elements = bytes per swizzled row
constexpr int kStages = 4;
constexpr int kABytes = kTileM * kBlockK;
constexpr int kSfaBytes = 512;
constexpr int kMxThreads = 320;
constexpr int kMaxSteps = DFGPU_MAX_EPILOGUE;

enum { kStepRelu = 1, kStepBias = 2, kStepFull = 3 };

struct MxArgs {
    const uint8_t* sfa;  // [M, K/32] plain
    const uint8_t* sfb;  // [K/32, N] plain
    int64_t sfa_ld, sfb_ld;
    void* out;
    int64_t out_ld;
    int32_t out_dtype;
    int32_t m_tiles, n_tiles, k_blocks;
    int32_t whole_items;   // work items that are whole 128 x BN tiles; the items after them are 128-column halves of the
    int32_t total_items;   // remaining tiles, so that the last round over the SMs takes half a tile's time instead of a whole one
    int32_t b_mn_major;
    int32_t a_format, b_format;  // operand formats of the instruction descriptor: 0 E4M3, 1 E5M2
    // MATMUL_FP8 form: sfa == nullptr (every block scale is 1), and after the fused steps value = acc * *descale_a * *descale_b,
    // *amax_bits = max over all elements of |value| (bits of the non-negative f32, NaN canonical), C = value * *scale_c
    const float* descale_a;
    const float* descale_b;
    const float* scale_c;
    unsigned int* amax_bits;
    int32_t step_count;
    int32_t step_kind[kMaxSteps];
    float relu_lower[kMaxSteps], relu_upper[kMaxSteps], relu_slope[kMaxSteps];
    const void* step_data[kMaxSteps];
    int32_t step_dtype[kMaxSteps];
    int64_t step_ld[kMaxSteps];
};

template <int BN>
struct MxSmem {
    static constexpr int kBBytes = BN * kBlockK;
    static constexpr int kSfbBytes = (BN / 128) * 512;
    static constexpr int kSfaOffset = kABytes + kBBytes;
    static constexpr int kSfbOffset = kSfaOffset + kSfaBytes;
    static constexpr int kStageBytes = kSfbOffset + 1024;  // keeps every slot 1024-byte aligned
    static constexpr int kBarriers = kStages * kStageBytes;
    // full[4], empty[4], acc_full, acc_empty
    static constexpr int kBarrierCount = 2 * kStages + 2;
    static constexpr int kTotal = kBarriers + kBarrierCount * 8 + 16;
    static constexpr int kDynamic = kTotal + 1024;
};

// 32 rows x 16 bytes of shared memory -> 4 columns of tensor memory, replicated to the four lane quarters.
__device__ __forceinline__ void tmem_copy_scales(uint32_t tmem_dst, uint64_t smem_descriptor) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(smem_descriptor) : "memory");
}
// Descriptor of an unswizzled K-major block for tcgen05.cp: 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t scale_desc(uint32_t address) {
    uint64_t desc = 0;
    desc |= static_cast<uint64_t>((address & 0x3FFFFu) >> 4);
    desc |= static_cast<uint64_t>(128u >> 4) << 32;
    desc |= 1ull << 46;
    return desc;
}
__device__ __forceinline__ void umma_mxf8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate,
                                          uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb) : "memory");
}

__device__ __forceinline__ float load_step_f32(const void* base, int dtype, int64_t index) {
    if (dtype == DFGPU_F32) return static_cast<const float*>(base)[index];
    return __uint_as_float(static_cast<uint32_t>(static_cast<const uint16_t*>(base)[index]) << 16);
}

// One thread's row of a finished tile: tensor memory -> fused steps -> bf16 / f32 -> global, 32 columns at a time.
struct MxScalars {
    bool on;
    float descale_a, descale_b, scale_c;
    float magnitude;  // running max |value| of this thread (NaN sticks)
};
__device__ __forceinline__ void mx_store_row(const MxArgs& args, uint32_t tmem_row_base, int64_t out_row, int64_t n0, int width, bool healthy, MxScalars& scalars) {
#pragma unroll 1
    for (int chunk = 0; chunk < width / 32; ++chunk) {
        uint32_t raw[32];
        tmem_load_32(tmem_row_base + chunk * 32, raw);
        tmem_load_wait();
        float v[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(raw[e]);
        const int64_t col0 = static_cast<int64_t>(n0) + chunk * 32;
        for (int s = 0; s < args.step_count; ++s) {
            const int kind = args.step_kind[s];
            if (kind == kStepRelu) {
                const float lower = args.relu_lower[s], upper = args.relu_upper[s], slope = args.relu_slope[s];
#pragma unroll
                for (int e = 0; e < 32; ++e) v[e] = relu_fast(v[e], lower, upper, slope);
            } else if (kind == kStepBias) {
#pragma unroll
                for (int e = 0; e < 32; ++e) v[e] = __fadd_rn(v[e], load_step_f32(args.step_data[s], args.step_dtype[s], col0 + e));
            } else {
#pragma unroll
                for (int e = 0; e < 32; ++e) v[e] = __fadd_rn(v[e], load_step_f32(args.step_data[s], args.step_dtype[s], out_row * args.step_ld[s] + col0 + e));
            }
        }
        if (scalars.on) {
            float top = scalars.magnitude;
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                // (+0.0 first: the reference's sum starts from +0.0 and so is never -0.0, the tensor core's can be)
                const float value = __fmul_rn(__fmul_rn(__fadd_rn(v[e], 0.0f), scalars.descale_a), scalars.descale_b);
                top = maximum_nan(top, fabsf(value));
                v[e] = __fmul_rn(value, scalars.scale_c);
            }
            scalars.magnitude = top;
        }
        if (healthy) {
            if (args.out_dtype == DFGPU_E4M3) {
                uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(args.out) + out_row * args.out_ld + col0);
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    uint32_t w[4];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        const float* f = v + 16 * q + 4 * t;
                        uint32_t lo = encode_e4m3_pair(f[0], f[1]), hi = encode_e4m3_pair(f[2], f[3]);
                        // NaN -> 0x7f whatever its sign (the hardware convert keeps the sign bit)
                        if (f[0] != f[0]) lo = (lo & 0xff00u) | 0x7fu;
                        if (f[1] != f[1]) lo = (lo & 0x00ffu) | 0x7f00u;
                        if (f[2] != f[2]) hi = (hi & 0xff00u) | 0x7fu;
                        if (f[3] != f[3]) hi = (hi & 0x00ffu) | 0x7f00u;
                        w[t] = lo | (hi << 16);
                    }
                    dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
                }
            } else if (args.out_dtype == DFGPU_BF16) {
                uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(args.out) + out_row * args.out_ld + col0);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t w[4];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        __nv_bfloat162 pair = __floats2bfloat162_rn(v[8 * q + 2 * t], v[8 * q + 2 * t + 1]);
                        w[t] = *reinterpret_cast<uint32_t*>(&pair);
                    }
                    dst[q] = make_uint4(w[0], w[1], w[2], w[3]);
                }
            } else {
                float4* dst = reinterpret_cast<float4*>(static_cast<float*>(args.out) + out_row * args.out_ld + col0);
#pragma unroll
                for (int q = 0; q < 8; ++q) dst[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            }
        }
    }
}

template <int BN>
__global__ void __launch_bounds__(kMxThreads, 1)
umma_mxf8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, MxArgs args) {
    using L = MxSmem<BN>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + L::kBarriers;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    const uint32_t acc_full_bar = bar_base + 8u * (2 * kStages);
    const uint32_t acc_empty_bar = bar_base + 8u * (2 * kStages + 1);
    const uint32_t tmem_slot = bar_base + 8u * L::kBarrierCount;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(generic_base + L::kBarriers + 8 * L::kBarrierCount);

    const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
    const bool leader = elect_one();
    const int total_tiles = args.total_items;
    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
    }
    // work item -> (row tile, first column, width in columns)
    auto decode_item = [&](int item, int& m_tile, int& n0, int& width) {
        int tile = item, half = -1;
        if (item >= args.whole_items) {
            const int h = item - args.whole_items;
            tile = args.whole_items + (h >> 1);
            half = h & 1;
        }
        m_tile = tile % args.m_tiles;
        n0 = (tile / args.m_tiles) * BN;
        width = BN;
        if (half >= 0) {
            width = BN / 2;
            n0 += half * (BN / 2);
        }
    };
    chain_release();

    if (warp == 0) {
        if (leader) {
            for (int s = 0; s < kStages; ++s) {
                mbar_init(full_bar(s), 2);   // the loader's expect_tx arrival + the scale warp of that slot
                mbar_init(empty_bar(s), 1);  // tcgen05.commit
            }
            mbar_init(acc_full_bar, 1);
            mbar_init(acc_empty_bar, 4);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    chain_wait();  // barriers and tensor memory are set up; from here on the previous kernel's output is read

    if (warp == 0) {
        // ---- TMA loader ----
        int stage = 0;
        uint32_t phase = 1;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            int m_tile, n0, width;
            decode_item(tile, m_tile, n0, width);
            for (int kb = 0; kb < args.k_blocks; ++kb) {
                ok = mbar_wait_warp(empty_bar(stage), phase, 401);
                if (!ok) break;
                const uint32_t a_dst = smem_base + stage * L::kStageBytes;
                const uint32_t b_dst = a_dst + kABytes;
                if (leader) {
                    mbar_expect_tx(full_bar(stage), kABytes + width * kBlockK);
                    tma_load_2d(a_dst, &map_a, kb * kBlockK, m_tile * kTileM, full_bar(stage));
                    // B arrives as boxes of 128 columns: 128 x 128 bytes each, consecutive in the slot in either layout
                    for (int j = 0; j < width / 128; ++j) {
                        if (args.b_mn_major) tma_load_2d(b_dst + j * (kBlockK * 128), &map_b, n0 + 128 * j, kb * kBlockK, full_bar(stage));
                        else tma_load_2d(b_dst + j * (128 * kBlockK), &map_b, kb * kBlockK, n0 + 128 * j, full_bar(stage));
                    }
                }
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---- issuing warp ----
        // instruction descriptor: E4M3 x E4M3, E8M0 scales, A K-major, B per flag, N = BN, M = 128; the two
        // scale-id fields (bits 4-5 for B, 29-30 for A) pick the K block's byte inside the scale columns
        const uint32_t idesc_fixed = (static_cast<uint32_t>(args.a_format) << 7) | (static_cast<uint32_t>(args.b_format) << 10) |
                                     (static_cast<uint32_t>(args.b_mn_major) << 16) | (1u << 23) | (static_cast<uint32_t>(kTileM >> 4) << 24);
        const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        int local = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
            int m_tile, n0, width;
            decode_item(tile, m_tile, n0, width);
            const uint32_t idesc_base = idesc_fixed | (static_cast<uint32_t>(width >> 3) << 17);
            if (ok) ok = mbar_wait_warp(acc_empty_bar, (local & 1) ^ 1, 402);
            tc_fence_after();
            for (int kb = 0; kb < args.k_blocks && ok; ++kb) {
                ok = mbar_wait_warp(full_bar(stage), phase, 403);
                if (!ok) break;  // (operands by TMA, scales by generic stores + fence.proxy.async: no tcgen05 fence needed)
                const uint32_t a_src = smem_base + stage * L::kStageBytes;
                const uint32_t b_src = a_src + kABytes;
                const uint32_t sf_tmem = tmem_u + 256 + (stage & 1) * 16;  // SFA at +0..3, SFB at +4..
                if (leader) {
                    tmem_copy_scales(sf_tmem, scale_desc(a_src + L::kSfaOffset));
                    for (int c = 0; c < width / 128; ++c) tmem_copy_scales(sf_tmem + 4 + 4 * c, scale_desc(a_src + L::kSfbOffset + 512 * c));
                }
                const uint32_t a_lo = smem_desc_lo(a_src, 16);
                const uint32_t b_lo = args.b_mn_major ? smem_desc_lo(b_src, kBlockK * 128) : smem_desc_lo(b_src, 16);
                const uint32_t b_step = args.b_mn_major ? (4096u >> 4) : (32u >> 4);
                if (leader) {
#pragma unroll
                    for (int j = 0; j < kBlockK / 32; ++j) {
                        const uint32_t idesc = idesc_base | (static_cast<uint32_t>(j) << 29) | (static_cast<uint32_t>(j) << 4);
                        umma_mxf8(tmem_u, desc_words(a_lo + ((j * 32) >> 4), smem_desc_hi(1024)), desc_words(b_lo + j * b_step, smem_desc_hi(1024)), idesc,
                                  (kb | j) != 0 ? 1u : 0u, sf_tmem, sf_tmem + 4);
                    }
                }
                if (leader) umma_commit(empty_bar(stage));
                if (++stage == kStages) { stage = 0; phase ^= 1; }
            }
            if (leader) umma_commit(acc_full_bar);  // arrives even after a failed wait so the epilogue never hangs
        }
    } else if (warp < 6) {
        // ---- epilogue ----
        const int quadrant = warp & 3;
        const int row = quadrant * 32 + lane;
        bool ok = true;
        int local = 0;
        MxScalars scalars{};
        if (args.descale_a != nullptr) {
            scalars.on = true;
            scalars.descale_a = *args.descale_a;
            scalars.descale_b = *args.descale_b;
            scalars.scale_c = *args.scale_c;
        }
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
            int m_tile, n0, width;
            decode_item(tile, m_tile, n0, width);
            if (ok) ok = mbar_wait(acc_full_bar, local & 1, 404);
            tc_fence_after();
            const bool healthy = ok && g_device_status == 0;
            const int64_t out_row = static_cast<int64_t>(m_tile) * kTileM + row;
            mx_store_row(args, tmem_base + (static_cast<uint32_t>(quadrant * 32) << 16), out_row, n0, width, healthy, scalars);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar);
        }
        if (scalars.on && args.amax_bits != nullptr) {
            unsigned int bits = scalars.magnitude != scalars.magnitude ? 0x7fc00000u : __float_as_uint(scalars.magnitude);
            bits = __reduce_max_sync(0xffffffffu, bits);
            if (lane == 0 && bits != 0u && ok) atomicMax(args.amax_bits, bits);
        }
    } else {
        // ---- scale loaders: warp 6 + q owns ring slot q ----
        const int slot = warp - 6;
        uint32_t phase = 1;
        bool ok = true;
        int it = 0;  // ring events of this CTA, in the loader's order
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            int m_tile, n0, width;
            decode_item(tile, m_tile, n0, width);
            for (int kb = 0; kb < args.k_blocks; ++kb, ++it) {
                if ((it & (kStages - 1)) != slot) continue;
                // issue the global loads first: they do not depend on the slot being free
                uint32_t a_words[4];
                uint32_t b_words[BN / 128][4];
                if (args.sfa == nullptr) {
                    // MATMUL_FP8: every block scale is 2^0
#pragma unroll
                    for (int g = 0; g < 4; ++g) a_words[g] = 0x7f7f7f7fu;
#pragma unroll
                    for (int c = 0; c < BN / 128; ++c)
#pragma unroll
                        for (int g = 0; g < 4; ++g) b_words[c][g] = c * 128 >= width ? 0u : 0x7f7f7f7fu;
                } else {
#pragma unroll
                    for (int g = 0; g < 4; ++g)
                        a_words[g] = __ldg(reinterpret_cast<const uint32_t*>(args.sfa + (static_cast<int64_t>(m_tile) * kTileM + g * 32 + lane) * args.sfa_ld + kb * 4));
#pragma unroll
                    for (int c = 0; c < BN / 128; ++c)
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            if (c * 128 >= width) {  // a half-width work item has one chunk of column scales
                                b_words[c][g] = 0;
                                continue;
                            }
                            const uint8_t* p = args.sfb + static_cast<int64_t>(kb) * 4 * args.sfb_ld + static_cast<int64_t>(n0) + c * 128 + g * 32 + lane;
                            const uint32_t b0 = __ldg(p), b1 = __ldg(p + args.sfb_ld), b2 = __ldg(p + 2 * args.sfb_ld), b3 = __ldg(p + 3 * args.sfb_ld);
                            b_words[c][g] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
                        }
                }
                ok = mbar_wait_warp(empty_bar(slot), phase, 405);
                phase ^= 1;
                if (!ok) break;
                uint8_t* stage_base = generic_base + slot * L::kStageBytes;
                *reinterpret_cast<uint4*>(stage_base + L::kSfaOffset + lane * 16) = make_uint4(a_words[0], a_words[1], a_words[2], a_words[3]);
#pragma unroll
                for (int c = 0; c < BN / 128; ++c)
                    *reinterpret_cast<uint4*>(stage_base + L::kSfbOffset + c * 512 + lane * 16) = make_uint4(b_words[c][0], b_words[c][1], b_words[c][2], b_words[c][3]);
                fence_async_shared();
                __syncwarp();
                if (leader) mbar_arrive(full_bar(slot));
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

inline int make_map_u8(CUtensorMap* map, const void* base, const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box, const char* what) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return fail(kExecutionFailed, "%s: cuTensorMapEncodeTiled is unavailable", what);
    cuuint32_t element_strides[2] = {1, 1};
    CUresult result = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), reinterpret_cast<const cuuint64_t*>(dims),
                             reinterpret_cast<const cuuint64_t*>(strides_bytes), reinterpret_cast<const cuuint32_t*>(box), element_strides,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS) return fail(kExecutionFailed, "%s: tensor map encode failed (CUresult %d)", what, static_cast<int>(result));
    return kOk;
}

bool aligned(const void* p, uintptr_t to) { return (reinterpret_cast<uintptr_t>(p) & (to - 1)) == 0; }

bool b_is_k_major(const dfgpu_tensor& b, int64_t K) {
    const int rank = b.rank;
    return b.stride[rank - 2] == 1 && b.stride[rank - 1] % 16 == 0 && b.stride[rank - 1] >= K;
}

// Tensor maps of the E4M3 operands: A as [M rows, K bytes], B as [N rows, K bytes] (K-major) or [K rows, N bytes].
int make_operand_maps(const dfgpu_tensor& a, const dfgpu_tensor& b, const void* a_data, const void* b_data, int64_t M, int64_t N, int64_t K,
                      CUtensorMap* map_a, CUtensorMap* map_b) {
    const int rank = a.rank;
    {
        uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
        uint64_t strides[1] = {static_cast<uint64_t>(a.stride[rank - 2])};
        uint32_t box[2] = {kBlockK, kTileM};
        int status = make_map_u8(map_a, a_data, dims, strides, box, "MATMUL A (E4M3)");
        if (status) return status;
    }
    if (b_is_k_major(b, K)) {
        uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
        uint64_t strides[1] = {static_cast<uint64_t>(b.stride[rank - 1])};
        uint32_t box[2] = {kBlockK, 128};
        return make_map_u8(map_b, b_data, dims, strides, box, "MATMUL B (E4M3)");
    }
    uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    uint64_t strides[1] = {static_cast<uint64_t>(b.stride[rank - 2])};
    uint32_t box[2] = {128, kBlockK};
    return make_map_u8(map_b, b_data, dims, strides, box, "MATMUL B (E4M3)");
}

// The fused steps this kernel applies: ReLU, a per-column ADD operand, a full [M, N] ADD operand.
bool translate_steps(const dfgpu_matmul_params& p, void* const* tensors, MxArgs* args) {
    if (p.epilogue_count < 0 || p.epilogue_count > kMaxSteps) return false;
    const int rank = p.c.rank;
    if (args) args->step_count = p.epilogue_count;
    for (int i = 0; i < p.epilogue_count; ++i) {
        const dfgpu_epilogue_step& step = p.epilogue[i];
        if (step.op == DFGPU_EPI_RELU) {
            if (args) {
                args->step_kind[i] = kStepRelu;
                args->relu_lower[i] = step.relu_lower;
                args->relu_upper[i] = step.relu_upper;
                args->relu_slope[i] = step.relu_slope;
            }
            continue;
        }
        if (step.op != DFGPU_EPI_ADD || step.operand < 0 || step.operand > 1) return false;
        const dfgpu_tensor& t = p.extra[step.operand];
        if (t.rank < 1 || t.rank > rank || (t.dtype != DFGPU_BF16 && t.dtype != DFGPU_F32)) return false;
        // operand axes align with the trailing axes of C: [.., 1 or M, N]
        for (int axis = 0; axis < t.rank - 2; ++axis)
            if (t.dim[axis] != 1) return false;
        if (t.dim[t.rank - 1] != p.c.dim[rank - 1] || t.stride[t.rank - 1] != 1) return false;
        const bool per_column = t.rank == 1 || t.dim[t.rank - 2] == 1;
        if (!per_column && t.dim[t.rank - 2] != p.c.dim[rank - 2]) return false;
        if (args) {
            args->step_kind[i] = per_column ? kStepBias : kStepFull;
            args->step_data[i] = tensors[5 + step.operand];
            args->step_dtype[i] = t.dtype;
            args->step_ld[i] = per_column ? 0 : t.stride[t.rank - 2];
        }
    }
    return true;
}

// One-SM form: grid, tail split and launch.
int launch_one_sm(const CUtensorMap& map_a, const CUtensorMap& map_b, MxArgs args, int bn, cudaStream_t stream) {
    const int64_t tiles = static_cast<int64_t>(args.m_tiles) * args.n_tiles;
    const int grid = tiles < sm_count() ? static_cast<int>(tiles) : sm_count();
    // The tiles left over after the last full round over the SMs are cut into halves when the halves still fit one
    // round: 4096^3 is 512 tiles on 148 SMs, i.e. three full rounds and 68 tiles, which become 136 half tiles.
    const int remainder = static_cast<int>(tiles % grid);
    args.whole_items = static_cast<int>(tiles);
    args.total_items = static_cast<int>(tiles);
    if (bn == 256 && remainder > 0 && 2 * remainder <= grid) {
        args.whole_items = static_cast<int>(tiles - remainder);
        args.total_items = args.whole_items + 2 * remainder;
    }
    auto run = [&](auto kernel, int dynamic) -> int {
        cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dynamic);
        if (error != cudaSuccess) return fail(kExecutionFailed, "MATMUL: cannot reserve %d bytes of shared memory: %s", dynamic, cudaGetErrorString(error));
        error = launch_chained(kernel, dim3(grid), dim3(kMxThreads), dynamic, stream, map_a, map_b, args);
        if (error != cudaSuccess) return fail(kExecutionFailed, "MATMUL (tcgen05, MXFP8 block scaled): launch failed: %s", cudaGetErrorString(error));
        return check_launch("MATMUL (tcgen05, MXFP8 block scaled)");
    };
    if (bn == 256) return run(umma_mxf8_kernel<256>, MxSmem<256>::kDynamic);
    return run(umma_mxf8_kernel<128>, MxSmem<128>::kDynamic);
}

}  // namespace

bool matmul_mxf8_supported(const dfgpu_matmul_params& p) {
    if (p.a.dtype != DFGPU_E4M3 || p.b.dtype != DFGPU_E4M3 || p.a_scale.dtype != DFGPU_E8M0 || p.b_scale.dtype != DFGPU_E8M0) return false;
    if (p.c.dtype != DFGPU_BF16 && p.c.dtype != DFGPU_F32) return false;
    const int rank = p.c.rank;
    if (rank < 2 || p.a.rank != rank || p.b.rank != rank || p.a_scale.rank != rank || p.b_scale.rank != rank) return false;
    for (int i = 0; i < rank - 2; ++i)
        if (p.c.dim[i] != 1 || p.a.dim[i] != 1 || p.b.dim[i] != 1 || p.a_scale.dim[i] != 1 || p.b_scale.dim[i] != 1) return false;
    const int64_t M = p.c.dim[rank - 2], N = p.c.dim[rank - 1], K = p.a.dim[rank - 1];
    if (M % kTileM != 0 || N % 128 != 0 || K % kBlockK != 0 || M < kTileM || N < 128 || K < kBlockK) return false;
    if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 30)) return false;
    if (p.b.dim[rank - 2] != K || p.b.dim[rank - 1] != N || p.a.dim[rank - 2] != M) return false;
    // scales: one per 32 elements along K, plain layout, densely indexed
    if (p.a_block[0] != 1 || p.a_block[1] != 32 || p.b_block[0] != 32 || p.b_block[1] != 1) return false;
    if (p.a_scale.reorder != DFGPU_REORDER_NONE || p.b_scale.reorder != DFGPU_REORDER_NONE) return false;
    if (p.a_scale.dim[rank - 2] != M || p.a_scale.dim[rank - 1] != K / 32 || p.a_scale.stride[rank - 1] != 1 || p.a_scale.stride[rank - 2] % 4 != 0) return false;
    if (p.b_scale.dim[rank - 2] != K / 32 || p.b_scale.dim[rank - 1] != N || p.b_scale.stride[rank - 1] != 1) return false;
    if (p.a.stride[rank - 1] != 1 || p.a.stride[rank - 2] % 16 != 0 || p.a.stride[rank - 2] < K) return false;
    const bool b_k_major = p.b.stride[rank - 2] == 1 && p.b.stride[rank - 1] % 16 == 0 && p.b.stride[rank - 1] >= K;
    const bool b_n_major = p.b.stride[rank - 1] == 1 && p.b.stride[rank - 2] % 16 == 0 && p.b.stride[rank - 2] >= N;
    if (!b_k_major && !b_n_major) return false;
    if (p.c.stride[rank - 1] != 1 || p.c.stride[rank - 2] % 8 != 0 || p.c.stride[rank - 2] < N) return false;
    return translate_steps(p, nullptr, nullptr);
}

int launch_matmul_mxf8(const dfgpu_matmul_params& p, void* const* tensors, cudaStream_t stream) {
    const int rank = p.c.rank;
    const int64_t M = p.c.dim[rank - 2], N = p.c.dim[rank - 1], K = p.a.dim[rank - 1];
    if (!aligned(tensors[0], 16) || !aligned(tensors[1], 16) || !aligned(tensors[2], 16) || !aligned(tensors[3], 4))
        return fail(kInvalidArgument, "MATMUL: the MXFP8 kernel needs 16-byte aligned A, B and C and a 4-byte aligned A scale");
    const bool b_k_major = b_is_k_major(p.b, K);
    const int bn = N % 256 == 0 ? 256 : 128;
    CUtensorMap map_a, map_b;
    {
        int status = make_operand_maps(p.a, p.b, tensors[0], tensors[1], M, N, K, &map_a, &map_b);
        if (status) return status;
    }
    MxArgs args{};
    args.sfa = static_cast<const uint8_t*>(tensors[3]);
    args.sfb = static_cast<const uint8_t*>(tensors[4]);
    args.sfa_ld = p.a_scale.stride[rank - 2];
    args.sfb_ld = p.b_scale.stride[rank - 2];
    args.out = tensors[2];
    args.out_ld = p.c.stride[rank - 2];
    args.out_dtype = p.c.dtype;
    args.m_tiles = static_cast<int>(M / kTileM);
    args.n_tiles = static_cast<int>(N / bn);
    args.k_blocks = static_cast<int>(K / kBlockK);
    args.b_mn_major = b_k_major ? 0 : 1;
    if (!translate_steps(p, tensors, &args)) return fail(kUnsupported, "MATMUL: the fused epilogue is not one the MXFP8 kernel applies");
    return launch_one_sm(map_a, map_b, args, bn, stream);
}

bool matmul_fp8_umma_supported(const dfgpu_matmul_fp8_params& p) {
    if ((p.a.dtype != DFGPU_E4M3 && p.a.dtype != DFGPU_E5M2) || (p.b.dtype != DFGPU_E4M3 && p.b.dtype != DFGPU_E5M2)) return false;
    if (p.c.dtype != DFGPU_BF16 && p.c.dtype != DFGPU_F32 && p.c.dtype != DFGPU_E4M3) return false;
    const int rank = p.c.rank;
    if (rank < 2 || p.a.rank != rank || p.b.rank != rank) return false;
    for (int i = 0; i < rank - 2; ++i)
        if (p.c.dim[i] != 1 || p.a.dim[i] != 1 || p.b.dim[i] != 1) return false;
    const int64_t M = p.c.dim[rank - 2], N = p.c.dim[rank - 1], K = p.a.dim[rank - 1];
    if (M % kTileM != 0 || N % 128 != 0 || K % kBlockK != 0 || M < kTileM || N < 128 || K < kBlockK) return false;
    if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 30)) return false;
    if (p.b.dim[rank - 2] != K || p.b.dim[rank - 1] != N || p.a.dim[rank - 2] != M) return false;
    if (p.a.stride[rank - 1] != 1 || p.a.stride[rank - 2] % 16 != 0 || p.a.stride[rank - 2] < K) return false;
    const bool b_n_major = p.b.stride[rank - 1] == 1 && p.b.stride[rank - 2] % 16 == 0 && p.b.stride[rank - 2] >= N;
    if (!b_is_k_major(p.b, K) && !b_n_major) return false;
    // 32 output columns leave a thread as 16-byte vectors
    const int64_t row_multiple = p.c.dtype == DFGPU_E4M3 ? 16 : (p.c.dtype == DFGPU_BF16 ? 8 : 4);
    if (p.c.stride[rank - 1] != 1 || p.c.stride[rank - 2] % row_multiple != 0 || p.c.stride[rank - 2] < N) return false;
    return true;
}

int launch_matmul_fp8_umma(const dfgpu_matmul_fp8_params& p, void* const* tensors, cudaStream_t stream) {
    const int rank = p.c.rank;
    const int64_t M = p.c.dim[rank - 2], N = p.c.dim[rank - 1], K = p.a.dim[rank - 1];
    if (!aligned(tensors[0], 16) || !aligned(tensors[1], 16) || !aligned(tensors[2], 16))
        return fail(kInvalidArgument, "MATMUL_FP8: the tcgen05 kernel needs 16-byte aligned A, B and C");
    const int bn = N % 256 == 0 ? 256 : 128;
    CUtensorMap map_a, map_b;
    int status = make_operand_maps(p.a, p.b, tensors[0], tensors[1], M, N, K, &map_a, &map_b);
    if (status) return status;
    MxArgs args{};
    args.sfa = nullptr;  // unit block scales
    args.sfb = nullptr;
    args.out = tensors[2];
    args.out_ld = p.c.stride[rank - 2];
    args.out_dtype = p.c.dtype;
    args.m_tiles = static_cast<int>(M / kTileM);
    args.n_tiles = static_cast<int>(N / bn);
    args.k_blocks = static_cast<int>(K / kBlockK);
    args.b_mn_major = b_is_k_major(p.b, K) ? 0 : 1;
    args.a_format = p.a.dtype == DFGPU_E5M2 ? 1 : 0;
    args.b_format = p.b.dtype == DFGPU_E5M2 ? 1 : 0;
    args.amax_bits = static_cast<unsigned int*>(tensors[3]);
    args.descale_a = static_cast<const float*>(tensors[4]);
    args.descale_b = static_cast<const float*>(tensors[5]);
    args.scale_c = static_cast<const float*>(tensors[6]);
    return launch_one_sm(map_a, map_b, args, bn, stream);
}

int mxf8_device_status(int* status) { return read_and_clear_device_status(status); }

}  // namespace dfgpu

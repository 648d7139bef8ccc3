// Two convolutions in one persistent kernel: a filter wider than one tap whose output, after its per-channel
// ADD / RELU steps, feeds a 1 x 1 convolution without leaving the SM.
//
//   T = relu(conv_a(X, Wa) + bias_a)          K1 = 64 channels, f32 in tensor memory
//   Y = conv_b(T, Wb) [+ bias_b] [relu] [+ R]  1 x 1, K2 = 128 or 256 channels, bf16 out
//
// The intermediate T never reaches global memory, nor shared memory: the first epilogue group splits every f32 value
// into a (hi, lo) bf16 pair and stores both halves back into TENSOR memory, over accumulator columns it has just read;
// the second product takes its A operand from there and multiplies both halves by the same filter, so T keeps
// f32-grade precision (2^-17 relative) through the bf16 tensor-core product.
//
// One tile = `rows_per_tile` output rows of one image with their padded columns: GEMM row m is the padded position
// (m / pitch, m % pitch), pitch = Q + S - 1, and positions with m % pitch >= Q are computed and never stored. The
// input WINDOW of a tile (rows_per_tile + R - 1 input rows, padded columns included) is loaded once per 64-channel
// block as one TMA box; filter tap (r, s) reads it from row r * pitch + s on, so every tap is a start address into
// the same slot and an input element crosses L2 -> shared memory once per tile (the 128-byte swizzle is a function
// of the absolute shared-memory address, as TMA wrote it, so a start at any 128-byte row needs no descriptor offset).
// The last taps read up to (R - 1) * pitch + S - 1 rows past the 128th row of the window: whatever lies there only
// reaches GEMM rows that are never stored.
//
// Roles (23 warps, one CTA per SM; the epilogues are chains of dependent tensor-memory loads, conversions and
// shared-memory stores, so they get most of the warps):
//   warp 0       loader: both filters once, then one window box per 64-channel block of every tile (ring of slots)
//   warp 1       issues the products of the hi blocks of conv_a (tile j + 1 first), then conv_b of tile j
//   warp 2       issues the products of the lo blocks of a split input into a second accumulator (a lone lane issues a
//                128 x 64 x 16 product in about twice the time the tensor pipe needs to run it)
//   warps 3-6    epilogue A: accumulator(s) -> bias / ReLU -> (hi, lo) -> tensor memory (the T operand of conv_b)
//   warps 7-22   epilogue B, two groups of eight warps, each half of the K2 output channels in chunks of 64 (a thread
//                owns 32 columns of one row), two staging boxes per group used alternately: accumulator -> steps (the
//                residual operand waits in the box) -> bf16 -> the same box -> TMA store
//   warp 23      residual loader: the residual box of a chunk by TMA, as soon as the box's last store has been read
// Tensor memory (512 columns): conv_a accumulators [buffer b: hi products at 128 b, lo products at 128 b + 64], conv_b
// accumulator at 256. T of a tile overwrites the lo-product columns of its buffer as packed bf16 pairs, per 32 channels
// [16 columns of hi words | 16 columns of lo words].
// Every wait is bounded (~2 s): on expiry the waiter records a code in g_device_status, every role falls through to
// the common exit and tensor memory is freed.
#include "umma_ptx.cuh"

namespace dfgpu {
namespace {

constexpr int kTileM = 128;
constexpr int kBlockK = 64;
constexpr int kK1 = 64;                  // channels of the intermediate
constexpr int kPairThreads = 24 * 32;    // 3 control warps, 4 for epilogue A, 2 x 8 for epilogue B, the residual loader
constexpr int kMaxStages = 6;
constexpr int kAccAColumns = 64;         // per conv_a accumulator: [buffer 0 hi, buffer 0 lo, buffer 1 hi, buffer 1 lo]
constexpr int kAccBColumn0 = 4 * kAccAColumns;
constexpr int kTmemColumns = 512;

enum { kStepBias = 1, kStepFull = 2, kStepRelu = 3 };

struct StepList {
    int32_t count;
    int32_t kind[DFGPU_MAX_EPILOGUE];
    const void* data[DFGPU_MAX_EPILOGUE];
    int32_t dtype[DFGPU_MAX_EPILOGUE];
    float lower[DFGPU_MAX_EPILOGUE], upper[DFGPU_MAX_EPILOGUE], slope[DFGPU_MAX_EPILOGUE];
};

struct PairArgs {
    // first convolution
    int32_t a_blocks;           // 64-channel activation blocks (2 * C / 64 for a split input: hi blocks, then lo blocks)
    int32_t w_blocks_per_tap;   // C / 64
    int32_t split_in;
    int32_t filter_r, filter_s, pad_h, pad_w;
    int32_t rows_per_tile, window_rows, tiles_per_image, out_p, out_q, pitch;
    int32_t total_tiles;
    int32_t stages, slot_bytes, window_bytes;
    int32_t k2;                 // output channels of the second convolution: 128 or 256
    int32_t box_rows;           // rows_per_tile * Q: rows of the output / residual boxes
    int32_t box_bytes;          // bytes between staging boxes (two per epilogue B group)
    int32_t has_residual;
    int32_t early_static;       // filters are written by no kernel that may still be running
    StepList steps_a, steps_b;
    // shared-memory layout (bytes from the 1024-aligned base)
    int32_t wa_offset, wb_offset, stage_offset, ring_offset, bias_offset, barrier_offset;
    int32_t wa_bytes, wb_bytes;
};

__device__ __forceinline__ void tmem_store_32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]),
          "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (bf16 pairs, one row per lane, 8 columns per 16-deep K step) is read
// from tensor memory.
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ float split_remainder(float x, uint32_t hi_bits) {
    return (hi_bits & 0x7f800000u) == 0x7f800000u ? 0.0f : x - __uint_as_float(hi_bits);
}

// RELU_FWD, same results as relu_forward(): below `lower` the sloped branch (NaN for -inf with slope 0, as the separate
// multiply and add give), otherwise min(x, upper) -- max(x, lower) is x there -- with NaN passed through by min.NaN.
__device__ __forceinline__ float relu_step(float x, float lower, float upper, float slope) {
    float clipped;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(clipped) : "f"(x), "f"(upper));
    return x < lower ? fmaf(slope, x - lower, lower) : clipped;
}

__global__ void __launch_bounds__(kPairThreads, 1)
umma_conv_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_wa, const __grid_constant__ CUtensorMap map_wb,
                      const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_res, PairArgs args) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t wa_base = smem_base + args.wa_offset;
    const uint32_t wb_base = smem_base + args.wb_offset;
    const uint32_t stage_base = smem_base + args.stage_offset;  // two boxes per epilogue B group
    const uint32_t ring_base = smem_base + args.ring_offset;
    const uint32_t bar_base = smem_base + args.barrier_offset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
    const uint32_t w_full_bar = bar_base + 8u * (2 * kMaxStages);
    auto acc_a_full = [&](int a) { return bar_base + 8u * (2 * kMaxStages + 1 + a); };
    auto acc_a_empty = [&](int a) { return bar_base + 8u * (2 * kMaxStages + 3 + a); };
    const uint32_t t_full_bar = bar_base + 8u * (2 * kMaxStages + 5);
    auto t_done_bar = [&](int b) { return bar_base + 8u * (2 * kMaxStages + 10 + b); };  // conv_b has read the T of buffer b
    const uint32_t acc_b_full = bar_base + 8u * (2 * kMaxStages + 7);
    const uint32_t acc_b_empty = bar_base + 8u * (2 * kMaxStages + 8);
    const uint32_t tmem_slot = bar_base + 8u * (2 * kMaxStages + 9);
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(generic_base + args.barrier_offset + 8 * (2 * kMaxStages + 9));
    auto res_full = [&](int box) { return bar_base + 8u * (2 * kMaxStages + 12 + box); };   // four staging boxes
    auto res_free = [&](int box) { return bar_base + 8u * (2 * kMaxStages + 16 + box); };

    const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
    const bool leader = elect_one();
    const int issuers = args.split_in ? 2 : 1;
    chain_release();
    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_x);
        prefetch_tensormap(&map_wa);
        prefetch_tensormap(&map_wb);
        prefetch_tensormap(&map_out);
        if (args.has_residual) prefetch_tensormap(&map_res);
    }
    const int chunks = args.k2 / 128;  // 64-channel chunks per epilogue B group and tile
    int my_tiles = 0;
    for (int tile = blockIdx.x; tile < args.total_tiles; tile += gridDim.x) ++my_tiles;

    auto tile_origin = [&](int tile, int& image, int& h0, int& out_row0) {
        image = tile / args.tiles_per_image;
        h0 = (tile - image * args.tiles_per_image) * args.rows_per_tile;
        out_row0 = (image * args.out_p + h0) * args.out_q;
    };

    if (warp == 0) {
        if (leader) {
            for (int s = 0; s < args.stages; ++s) {
                mbar_init(full_bar(s), 1);
                mbar_init(empty_bar(s), 1);
            }
            mbar_init(w_full_bar, 1);
            for (int a = 0; a < 2; ++a) {
                mbar_init(acc_a_full(a), issuers);
                mbar_init(acc_a_empty(a), 4);
            }
            mbar_init(t_full_bar, 4);
            mbar_init(t_done_bar(0), 1);
            mbar_init(t_done_bar(1), 1);
            for (int box = 0; box < 4; ++box) {
                mbar_init(res_full(box), 1);
                mbar_init(res_free(box), 1);
            }
            mbar_init(acc_b_full, 1);
            mbar_init(acc_b_empty, 16);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            mbar_expect_tx(w_full_bar, static_cast<uint32_t>(args.wa_bytes + args.wb_bytes));
        }
        __syncwarp();
        if (!args.early_static) chain_wait();
        // filters: conv_a as [tap][64-channel block] slices of 64 rows x 128 B, conv_b as one K2 x 128 B block
        const int wa_slices = args.filter_r * args.filter_s * args.w_blocks_per_tap;
        for (int kb = 0; kb < wa_slices; ++kb)
            if (leader) tma_load_2d(wa_base + kb * (kK1 * 128), &map_wa, kb * kBlockK, 0, w_full_bar);
        if (leader) tma_load_2d(wb_base, &map_wb, 0, 0, w_full_bar);
        if (args.early_static) chain_wait();
    } else {
        chain_wait();
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemColumns);
        tmem_relinquish();
        tc_fence_before();
    }
    {
        // per-channel ADD operands -> f32 in shared memory: conv_a's first (K1 floats each), then conv_b's (K2 floats each)
        float* bias_stage = reinterpret_cast<float*>(generic_base + args.bias_offset);
        int at = 0;
        for (int e = 0; e < args.steps_a.count; ++e) {
            if (args.steps_a.kind[e] != kStepBias) continue;
            for (int c = threadIdx.x; c < kK1; c += blockDim.x) bias_stage[at + c] = load_as_f32(args.steps_a.data[e], args.steps_a.dtype[e], c);
            at += kK1;
        }
        for (int e = 0; e < args.steps_b.count; ++e) {
            if (args.steps_b.kind[e] != kStepBias) continue;
            for (int c = threadIdx.x; c < args.k2; c += blockDim.x) bias_stage[at + c] = load_as_f32(args.steps_b.data[e], args.steps_b.dtype[e], c);
            at += args.k2;
        }
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        // ---- loader: one window box per activation block of every tile ----
        int stage = 0;
        uint32_t phase = 1;
        bool ok = true;
        for (int tile = blockIdx.x; tile < args.total_tiles && ok; tile += gridDim.x) {
            int image, h0, out_row0;
            tile_origin(tile, image, h0, out_row0);
            for (int cb = 0; cb < args.a_blocks; ++cb) {
                ok = mbar_wait_warp(empty_bar(stage), phase, 201);
                if (!ok) break;
                if (leader) {
                    mbar_expect_tx(full_bar(stage), static_cast<uint32_t>(args.window_bytes));
                    tma_load_4d(ring_base + stage * args.slot_bytes, &map_x, cb * kBlockK, -args.pad_w, h0 - args.pad_h, image, full_bar(stage));
                }
                if (++stage == args.stages) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ---- product issuers ----
        const int me = warp == 1 ? 0 : 1;
        const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
        const uint32_t idesc_a = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kK1 >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
        const uint32_t idesc_b = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(args.k2 >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
        const uint32_t row_step = static_cast<uint32_t>(args.pitch * 128) >> 4;  // descriptor units per filter row
        const uint32_t w_tap_step = static_cast<uint32_t>(args.w_blocks_per_tap * (kK1 * 128)) >> 4;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = me < issuers && mbar_wait_warp(w_full_bar, 0, 202);
        auto issue_a = [&](int j) {
            const int buffer = j & 1;
            if (ok) ok = mbar_wait_warp(acc_a_empty(buffer), ((j >> 1) & 1) ^ 1, 203);
            // the lo products land in the columns where the T of tile j - 2 lives until conv_b of that tile has run
            if (ok && me == 1 && j >= 2) ok = mbar_wait_warp(t_done_bar(buffer), ((j >> 1) & 1) ^ 1, 212);
            tc_fence_after();
            const uint32_t tmem_acc = tmem_u + static_cast<uint32_t>((2 * buffer + me) * kAccAColumns);
            uint32_t accumulate = 0;
            for (int cb = 0; cb < args.a_blocks; ++cb) {
                const bool lo_block = cb >= args.w_blocks_per_tap;
                const bool mine = args.split_in ? (lo_block == (me == 1)) : true;
                if (mine && ok) {
                    ok = mbar_wait_warp(full_bar(stage), phase, 204);
                    if (ok) {
                        const uint32_t a_lo = smem_desc_lo(ring_base + stage * args.slot_bytes, 16);
                        const int wc = lo_block ? cb - args.w_blocks_per_tap : cb;  // the lo half meets the same filter slices
                        const uint32_t b_block = smem_desc_lo(wa_base + wc * (kK1 * 128), 16);
                        if (leader) {
                            for (int r = 0; r < args.filter_r; ++r) {
                                const uint32_t a_row = a_lo + r * row_step;
                                const uint32_t b_row = b_block + r * args.filter_s * w_tap_step;
                                if (args.filter_s == 3) {
#pragma unroll
                                    for (int tap = 0; tap < 3; ++tap)
#pragma unroll
                                        for (int k = 0; k < kBlockK / 16; ++k) {
                                            umma_bf16(tmem_acc, desc_words(a_row + ((tap * 128 + k * 32) >> 4), smem_desc_hi(1024)),
                                                      desc_words(b_row + tap * w_tap_step + ((k * 32) >> 4), smem_desc_hi(1024)), idesc_a, accumulate);
                                            accumulate = 1;
                                        }
                                } else {
                                    for (int tap = 0; tap < args.filter_s; ++tap)
#pragma unroll
                                        for (int k = 0; k < kBlockK / 16; ++k) {
                                            umma_bf16(tmem_acc, desc_words(a_row + ((tap * 128 + k * 32) >> 4), smem_desc_hi(1024)),
                                                      desc_words(b_row + tap * w_tap_step + ((k * 32) >> 4), smem_desc_hi(1024)), idesc_a, accumulate);
                                            accumulate = 1;
                                        }
                                }
                            }
                            umma_commit(empty_bar(stage));
                        }
                    }
                }
                if (++stage == args.stages) { stage = 0; phase ^= 1; }
            }
            if (leader) umma_commit(acc_a_full(buffer));  // arrives even after a failed wait, so the epilogue never hangs on it
        };
        auto issue_b = [&](int j) {
            if (ok) ok = mbar_wait_warp(t_full_bar, j & 1, 205);
            if (ok) ok = mbar_wait_warp(acc_b_empty, (j & 1) ^ 1, 206);
            tc_fence_after();
            if (leader) {
                if (ok) {
                    const uint32_t tmem_acc = tmem_u + kAccBColumn0;
                    const uint32_t t_tmem = tmem_u + static_cast<uint32_t>((2 * (j & 1) + 1) * kAccAColumns);
                    const uint32_t b_lo = smem_desc_lo(wb_base, 16);
                    // per 32 channels: hi words (2 K steps of 8 columns), then lo words; both against the same filter slices
#pragma unroll
                    for (int chunk = 0; chunk < kK1 / 32; ++chunk)
#pragma unroll
                        for (int part = 0; part < 2; ++part)
#pragma unroll
                            for (int kk = 0; kk < 2; ++kk)
                                umma_bf16_a_tmem(tmem_acc, t_tmem + chunk * 32 + part * 16 + kk * 8, desc_words(b_lo + (((chunk * 2 + kk) * 32) >> 4), smem_desc_hi(1024)), idesc_b,
                                                 (chunk | part | kk) != 0 ? 1u : 0u);
                }
                umma_commit(t_done_bar(j & 1));
                umma_commit(acc_b_full);
            }
        };
        if (me < issuers) {
            issue_a(0);
            for (int j = 0; j < my_tiles; ++j) {
                if (j + 1 < my_tiles) issue_a(j + 1);
                if (me == 0) issue_b(j);
            }
        }
    } else if (warp >= 3 && warp <= 6) {
        // ---- epilogue A: conv_a accumulator(s) -> steps -> (hi, lo) bf16 -> the T tile, 32 channels at a time ----
        const int quadrant = warp & 3;
        const float* bias_smem = reinterpret_cast<const float*>(generic_base + args.bias_offset);
        bool ok = true;
        for (int j = 0; j < my_tiles; ++j) {
            const int buffer = j & 1;
            if (ok) ok = mbar_wait(acc_a_full(buffer), (j >> 1) & 1, 207);
            tc_fence_after();
            const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quadrant * 32) << 16) + 2 * buffer * kAccAColumns;
#pragma unroll 1
            for (int chunk = 0; chunk < kK1 / 32; ++chunk) {
                float v[32];
                {
                    uint32_t raw[32];
                    tmem_load_32(lane_base + chunk * 32, raw);
                    if (args.split_in) {  // the lo blocks' share of the sum, from the second issuing warp's accumulator
                        uint32_t more[32];
                        tmem_load_32(lane_base + kAccAColumns + chunk * 32, more);
                        tmem_load_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) v[e] = __fadd_rn(__uint_as_float(raw[e]), __uint_as_float(more[e]));
                    } else {
                        tmem_load_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(raw[e]);
                    }
                }
                if (chunk == kK1 / 32 - 1) {  // the accumulators are in registers: hand them back before the arithmetic
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_a_empty(buffer));
                }
                int bias_at = 0;
                for (int e = 0; e < args.steps_a.count; ++e) {
                    if (args.steps_a.kind[e] == kStepRelu) {
                        const float lower = args.steps_a.lower[e], upper = args.steps_a.upper[e], slope = args.steps_a.slope[e];
#pragma unroll
                        for (int t = 0; t < 32; ++t) v[t] = relu_step(v[t], lower, upper, slope);
                    } else {
                        const float4* p = reinterpret_cast<const float4*>(bias_smem + bias_at + chunk * 32);
                        bias_at += kK1;
#pragma unroll
                        for (int q4 = 0; q4 < 8; ++q4) {
                            const float4 q = p[q4];
                            v[4 * q4] = __fadd_rn(v[4 * q4], q.x);
                            v[4 * q4 + 1] = __fadd_rn(v[4 * q4 + 1], q.y);
                            v[4 * q4 + 2] = __fadd_rn(v[4 * q4 + 2], q.z);
                            v[4 * q4 + 3] = __fadd_rn(v[4 * q4 + 3], q.w);
                        }
                    }
                }
                // (hi, lo) words of these 32 channels over the lo-product columns just read: 16 hi words, then 16 lo words
                uint32_t words[32];
                uint32_t not_finite = 0;  // bit 15 / 31 set when a hi half has an all-ones exponent (infinity or NaN)
#pragma unroll
                for (int t = 0; t < 16; ++t) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * t], v[2 * t + 1]);
                    words[t] = *reinterpret_cast<uint32_t*>(&h);
                    not_finite |= (words[t] & 0x7f807f80u) + 0x00800080u;
                }
                if (__any_sync(0xffffffffu, (not_finite & 0x80008000u) != 0)) {
#pragma unroll
                    for (int t = 0; t < 16; ++t) {
                        __nv_bfloat162 l = __floats2bfloat162_rn(split_remainder(v[2 * t], words[t] << 16), split_remainder(v[2 * t + 1], words[t] & 0xffff0000u));
                        words[16 + t] = *reinterpret_cast<uint32_t*>(&l);
                    }
                } else {  // every hi half is finite: the remainders need no guard
#pragma unroll
                    for (int t = 0; t < 16; ++t) {
                        __nv_bfloat162 l = __floats2bfloat162_rn(v[2 * t] - __uint_as_float(words[t] << 16), v[2 * t + 1] - __uint_as_float(words[t] & 0xffff0000u));
                        words[16 + t] = *reinterpret_cast<uint32_t*>(&l);
                    }
                }
                tmem_store_32(lane_base + kAccAColumns + chunk * 32, words);
            }
            tmem_store_wait();
            tc_fence_before();  // tensor-memory stores -> ordered before the product that the arrival below releases
            __syncwarp();
            if (lane == 0) mbar_arrive(t_full_bar);
        }
    } else if (warp >= 7 && warp <= 22) {
        // ---- epilogue B: conv_b accumulator -> steps -> bf16 -> staging box -> TMA store ----
        const int group = (warp - 7) >> 3;
        const int member = threadIdx.x - (7 + 8 * group) * 32;  // 0..255 inside the group
        const int half = ((warp - 7) >> 2) & 1;                 // which 32 of a chunk's 64 columns this warp owns
        const int quadrant = warp & 3;
        const int gemm_row = quadrant * 32 + lane;
        const int line = gemm_row / args.pitch, column = gemm_row - line * args.pitch;
        const bool row_is_output = column < args.out_q && line < args.rows_per_tile;
        const int row = row_is_output ? line * args.out_q + column : 0;  // rows compacted for the store
        const bool store_thread = member == 0;
        const int barrier_id = 1 + group;
        auto group_barrier = [&] { asm volatile("bar.sync %0, 256;" ::"r"(barrier_id) : "memory"); };
        const float* bias_smem = reinterpret_cast<const float*>(generic_base + args.bias_offset);
        int bias_a_floats = 0;
        for (int e = 0; e < args.steps_a.count; ++e) bias_a_floats += args.steps_a.kind[e] == kStepBias ? kK1 : 0;
        int image, h0, out_row0, next_row0 = 0;
        if (my_tiles > 0) tile_origin(blockIdx.x, image, h0, next_row0);
        bool ok = true;
        int n = 0;  // chunks handled: chunk n uses box n & 1 of the group
        for (int j = 0, tile = blockIdx.x; j < my_tiles; ++j, tile += gridDim.x) {
            out_row0 = next_row0;
            if (j + 1 < my_tiles) tile_origin(tile + gridDim.x, image, h0, next_row0);
            for (int c = 0; c < chunks; ++c, ++n) {
                const int col0 = group * (args.k2 / 2) + c * 64;
                const int box_index = 2 * group + (n & 1);
                uint8_t* box = generic_base + args.stage_offset + box_index * args.box_bytes;
                uint8_t* row_smem = box + row * 128;
                // (this box's previous store, two chunks back, has been read: see the end of the previous chunk; with a
                // residual operand the loader refilled it after that and the wait below sees its bytes arrive)
                if (c == 0) {
                    if (ok) ok = mbar_wait(acc_b_full, j & 1, 209);
                    tc_fence_after();
                }
                if (args.has_residual && ok) ok = mbar_wait(res_full(box_index), (n >> 1) & 1, 210);
                const bool healthy = ok;
                uint32_t raw[32];
                tmem_load_32(tmem_base + (static_cast<uint32_t>(quadrant * 32) << 16) + kAccBColumn0 + col0 + half * 32, raw);
                tmem_load_wait();
                if (c == chunks - 1) {  // this warp's columns have all left tensor memory
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_b_empty);
                }
                float v[32];
#pragma unroll
                for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(raw[e]);
                int bias_at = bias_a_floats;
                for (int e = 0; e < args.steps_b.count; ++e) {
                    const int kind = args.steps_b.kind[e];
                    if (kind == kStepRelu) {
                        const float lower = args.steps_b.lower[e], upper = args.steps_b.upper[e], slope = args.steps_b.slope[e];
#pragma unroll
                        for (int t = 0; t < 32; ++t) v[t] = relu_step(v[t], lower, upper, slope);
                    } else if (kind == kStepBias) {
                        const float4* p = reinterpret_cast<const float4*>(bias_smem + bias_at + col0 + half * 32);
                        bias_at += args.k2;
#pragma unroll
                        for (int q4 = 0; q4 < 8; ++q4) {
                            const float4 q = p[q4];
                            v[4 * q4] = __fadd_rn(v[4 * q4], q.x);
                            v[4 * q4 + 1] = __fadd_rn(v[4 * q4 + 1], q.y);
                            v[4 * q4 + 2] = __fadd_rn(v[4 * q4 + 2], q.z);
                            v[4 * q4 + 3] = __fadd_rn(v[4 * q4 + 3], q.w);
                        }
                    } else {  // the residual box staged above
#pragma unroll
                        for (int c16 = 0; c16 < 4; ++c16) {
                            const uint4 q = *reinterpret_cast<const uint4*>(row_smem + (((half * 4 + c16) ^ (row & 7)) << 4));
                            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                v[8 * c16 + 2 * t] = __fadd_rn(v[8 * c16 + 2 * t], __uint_as_float(w[t] << 16));
                                v[8 * c16 + 2 * t + 1] = __fadd_rn(v[8 * c16 + 2 * t + 1], __uint_as_float(w[t] & 0xffff0000u));
                            }
                        }
                    }
                }
#pragma unroll
                for (int c16 = 0; c16 < 4; ++c16) {
                    uint32_t w[4];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        __nv_bfloat162 pair = __floats2bfloat162_rn(v[8 * c16 + 2 * t], v[8 * c16 + 2 * t + 1]);
                        w[t] = *reinterpret_cast<uint32_t*>(&pair);
                    }
                    if (row_is_output) *reinterpret_cast<uint4*>(row_smem + (((half * 4 + c16) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                fence_async_shared();
                // The other box of the group is written next (by the residual loader, or by this group's next chunk): its
                // last store (the previous chunk's) must have read it first.
                if (store_thread) {
                    tma_store_wait_read<0>();
                    if (args.has_residual && n >= 1) mbar_arrive(res_free(box_index ^ 1));
                }
                group_barrier();
                if (store_thread) {
                    if (healthy) tma_store_2d(&map_out, stage_base + box_index * args.box_bytes, col0, out_row0);
                    tma_store_commit();
                }
            }
        }
        if (store_thread) tma_store_wait_all();
    }

    if (warp == 23 && args.has_residual) {
        // ---- residual loader: chunk n of group g goes to box 2 g + (n & 1), once the store of chunk n - 2 has been read ----
        bool ok = true;
        int n = 0;
        for (int tile = blockIdx.x; tile < args.total_tiles && ok; tile += gridDim.x) {
            int image, h0, out_row0;
            tile_origin(tile, image, h0, out_row0);
            for (int c = 0; c < chunks && ok; ++c, ++n)
                for (int g = 0; g < 2; ++g) {
                    const int box = 2 * g + (n & 1);
                    // the box's (n >> 1)-th use: free once its previous use, chunk n - 2, has been stored and read
                    ok = mbar_wait_warp(res_free(box), ((n >> 1) & 1) ^ 1, 211);
                    if (!ok) break;
                    if (leader) {
                        mbar_expect_tx(res_full(box), static_cast<uint32_t>(args.box_rows) * 128u);
                        tma_load_2d(stage_base + box * args.box_bytes, &map_res, g * (args.k2 / 2) + c * 64, out_row0, res_full(box));
                    }
                }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemColumns);
    }
}

}  // namespace
}  // namespace dfgpu

namespace dfgpu {
namespace {

constexpr int kPairSmemBudget = 227 * 1024;

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// The per-channel / full classification of one fused ADD operand (the rule of translate_epilogue in umma_gemm.cu).
bool classify_steps(const dfgpu_conv_params& p, void* const* extra_pointers, StepList* out, int* bias_steps, int* full_steps, int* residual_operand) {
    if (p.epilogue_count < 0 || p.epilogue_count > DFGPU_MAX_EPILOGUE) return false;
    *bias_steps = *full_steps = 0;
    *residual_operand = -1;
    if (out) out->count = p.epilogue_count;
    for (int i = 0; i < p.epilogue_count; ++i) {
        const dfgpu_epilogue_step& step = p.epilogue[i];
        if (step.op == DFGPU_EPI_RELU) {
            if (out) {
                out->kind[i] = kStepRelu;
                out->lower[i] = step.relu_lower;
                out->upper[i] = step.relu_upper;
                out->slope[i] = step.relu_slope;
            }
            continue;
        }
        if (step.op != DFGPU_EPI_ADD || step.operand < 0 || step.operand > 1) return false;
        const dfgpu_tensor& t = p.extra[step.operand];
        if (t.rank < 1 || t.rank > p.y.rank || (t.dtype != DFGPU_BF16 && t.dtype != DFGPU_F32)) return false;
        const int shift = p.y.rank - t.rank;
        bool per_channel = shift <= 1, full = t.rank == p.y.rank;
        for (int axis = 0; axis < t.rank; ++axis) {
            const int out_axis = axis + shift;
            if (out_axis == 1) per_channel = per_channel && t.dim[axis] == p.y.dim[1] && t.stride[axis] == 1;
            else per_channel = per_channel && t.dim[axis] == 1;
            full = full && t.dim[axis] == p.y.dim[out_axis] && t.stride[axis] == p.y.stride[out_axis];
        }
        if (!per_channel && !full) return false;
        if (per_channel) ++*bias_steps;
        else {
            if (t.dtype != DFGPU_BF16) return false;
            ++*full_steps;
            *residual_operand = step.operand;
        }
        if (out) {
            out->kind[i] = per_channel ? kStepBias : kStepFull;
            out->data[i] = extra_pointers ? extra_pointers[step.operand] : nullptr;
            out->dtype[i] = t.dtype;
        }
    }
    return true;
}

struct PairForm {
    ConvForm a;
    int64_t k2;
    int bias_a, bias_b, full_b, residual_operand;
    int window_rows, window_bytes, stages, slot_bytes, box_rows, box_bytes;
    int wa_bytes, wb_bytes, bias_bytes;
};

int round_up_1k(int64_t bytes) { return static_cast<int>((bytes + 1023) & ~int64_t{1023}); }

bool pair_form(const dfgpu_conv_params& first, const dfgpu_conv_params& second, PairForm& f) {
    // the intermediate must keep f32-grade values: FLOAT as the graph declares it, or the (hi, lo) pair type
    if (first.y.dtype != DFGPU_F32 && first.y.dtype != DFGPU_BF16X2) return false;
    if (second.x.dtype != first.y.dtype || second.y.dtype != DFGPU_BF16 || second.w.dtype != DFGPU_BF16) return false;
    dfgpu_conv_params probe = first;
    probe.y.dtype = DFGPU_BF16X2;
    probe.reserved &= ~1;
    if (!conv_umma_form(probe, f.a) || !f.a.persistent || !f.a.halo || f.a.K != kK1) return false;
    for (int axis = 0; axis < 4; ++axis)
        if (second.x.dim[axis] != first.y.dim[axis] || second.x.stride[axis] != first.y.stride[axis]) return false;
    if (second.w.rank != 4 || second.w.dim[1] != kK1 || second.w.dim[2] != 1 || second.w.dim[3] != 1 || second.w.stride[1] != 1 || second.w.stride[0] != kK1) return false;
    for (int axis = 0; axis < 2; ++axis)
        if (second.pre_pad[axis] != 0 || second.post_pad[axis] != 0 || second.stride[axis] != 1 || second.dilation[axis] != 1) return false;
    if (second.reverse_filter) return false;
    f.k2 = second.y.dim[1];
    if (f.k2 != 128 && f.k2 != 256) return false;
    if (second.y.rank != 4 || second.y.dim[0] != f.a.N || second.y.dim[2] != f.a.P || second.y.dim[3] != f.a.Q) return false;
    // packed NHWC output
    if (second.y.stride[1] != 1 || second.y.stride[3] != f.k2 || second.y.stride[2] != f.a.Q * f.k2 || second.y.stride[0] != f.a.P * f.a.Q * f.k2) return false;
    if (f.a.N * f.a.P * f.a.Q >= (1ll << 31) / 256) return false;  // byte offsets of the output stay inside 32 bits times the row pitch
    int full_a = 0, unused = -1;
    if (!classify_steps(first, nullptr, nullptr, &f.bias_a, &full_a, &unused) || full_a != 0) return false;
    if (!classify_steps(second, nullptr, nullptr, &f.bias_b, &f.full_b, &f.residual_operand) || f.full_b > 1) return false;
    const int64_t pitch = f.a.Q + f.a.S - 1;
    f.window_rows = f.a.halo_rows + static_cast<int>(f.a.R) - 1;
    if (f.window_rows > 256 || pitch > 256) return false;  // TMA box extents
    f.window_bytes = static_cast<int>(f.window_rows * pitch * 128);
    f.slot_bytes = round_up_1k(f.window_bytes);
    f.box_rows = f.a.halo_rows * static_cast<int>(f.a.Q);
    f.box_bytes = round_up_1k(f.box_rows * 128);
    f.wa_bytes = static_cast<int>(kK1 * f.a.R * f.a.S * f.a.C * 2);
    f.wb_bytes = static_cast<int>(f.k2 * kK1 * 2);
    f.bias_bytes = round_up_1k((f.bias_a * kK1 + f.bias_b * f.k2) * 4 + 256);  // staged bias vectors, then the barriers
    const int fixed = round_up_1k(f.wa_bytes) + round_up_1k(f.wb_bytes) + 4 * f.box_bytes + f.bias_bytes + 1024;
    f.stages = (kPairSmemBudget - fixed) / f.slot_bytes;
    if (f.stages > kMaxStages) f.stages = kMaxStages;
    // the last taps read past the window's rows (into rows no stored GEMM row uses): that must stay inside the allocation,
    // i.e. inside what follows the last slot
    const int64_t rows_read = kTileM + (f.a.R - 1) * pitch + f.a.S - 1;
    if (rows_read * 128 - f.slot_bytes > 4 * f.box_bytes + f.bias_bytes) return false;
    return f.stages >= 2;
}

}  // namespace

bool conv_pair_umma_supported(const dfgpu_conv_params& first, const dfgpu_conv_params& second) {
    PairForm form;
    return pair_form(first, second, form);
}

// tensors: {X, Wa, Wb, Y, first.extra0, first.extra1, second.extra0, second.extra1}
int launch_conv_pair_umma(const dfgpu_conv_params& first, const dfgpu_conv_params& second, void* const* tensors, cudaStream_t stream) {
    PairForm f;
    if (!pair_form(first, second, f)) return fail(kUnsupported, "CONV_FPROP pair: the fused tcgen05 kernel does not take these convolutions");
    for (int i = 0; i < 4; ++i)
        if (!tensors[i] || !aligned16(tensors[i])) return fail(kInvalidArgument, "CONV_FPROP pair: X, both filters and Y must be non-null and 16-byte aligned");
    const ConvForm& a = f.a;
    const int64_t Ca = a.split_in ? 2 * a.C : a.C;
    PairArgs args{};
    args.a_blocks = static_cast<int>(Ca / kBlockK);
    args.w_blocks_per_tap = static_cast<int>(a.C / kBlockK);
    args.split_in = a.split_in ? 1 : 0;
    args.filter_r = static_cast<int>(a.R);
    args.filter_s = static_cast<int>(a.S);
    args.pad_h = static_cast<int>(first.pre_pad[0]);
    args.pad_w = static_cast<int>(first.pre_pad[1]);
    args.rows_per_tile = a.halo_rows;
    args.window_rows = f.window_rows;
    args.tiles_per_image = static_cast<int>(a.P / a.halo_rows);
    args.out_p = static_cast<int>(a.P);
    args.out_q = static_cast<int>(a.Q);
    args.pitch = static_cast<int>(a.Q + a.S - 1);
    args.total_tiles = static_cast<int>(a.N) * args.tiles_per_image;
    args.stages = f.stages;
    args.slot_bytes = f.slot_bytes;
    args.window_bytes = f.window_bytes;
    args.k2 = static_cast<int>(f.k2);
    args.box_rows = f.box_rows;
    args.box_bytes = f.box_bytes;
    args.has_residual = f.full_b;
    args.early_static = ((first.reserved & 2) && (second.reserved & 2)) ? 1 : 0;  // both filters are static operands
    int bias = 0, full = 0, operand = -1;
    if (!classify_steps(first, tensors + 4, &args.steps_a, &bias, &full, &operand) || !classify_steps(second, tensors + 6, &args.steps_b, &bias, &full, &operand))
        return fail(kUnsupported, "CONV_FPROP pair: the fused epilogues are not ones the kernel applies");
    for (const StepList* list : {&args.steps_a, &args.steps_b})
        for (int e = 0; e < list->count; ++e)
            if (list->kind[e] != kStepRelu && (!list->data[e] || !aligned16(list->data[e])))
                return fail(kInvalidArgument, "CONV_FPROP pair: ADD operands must be non-null and 16-byte aligned");
    args.wa_bytes = f.wa_bytes;
    args.wb_bytes = f.wb_bytes;
    args.wa_offset = 0;
    args.wb_offset = round_up_1k(f.wa_bytes);
    args.ring_offset = args.wb_offset + round_up_1k(f.wb_bytes);
    args.stage_offset = args.ring_offset + f.stages * f.slot_bytes;  // right behind the ring: the taps' reads past the last slot land here
    args.bias_offset = args.stage_offset + 4 * f.box_bytes;
    args.barrier_offset = args.bias_offset + f.bias_bytes - 256;
    const int dynamic = args.bias_offset + f.bias_bytes + 1024;
    if (dynamic > kPairSmemBudget) return fail(kUnsupported, "CONV_FPROP pair: shared-memory layout does not fit");

    CUtensorMap map_x, map_wa, map_wb, map_out, map_res;
    int status;
    {
        uint64_t dims[4] = {static_cast<uint64_t>(Ca), static_cast<uint64_t>(a.W), static_cast<uint64_t>(a.H), static_cast<uint64_t>(a.N)};
        uint64_t strides[3] = {static_cast<uint64_t>(Ca) * 2, static_cast<uint64_t>(a.W * Ca) * 2, static_cast<uint64_t>(a.H * a.W * Ca) * 2};
        uint32_t box[4] = {kBlockK, static_cast<uint32_t>(args.pitch), static_cast<uint32_t>(f.window_rows), 1};
        if ((status = make_map(&map_x, tensors[0], 4, dims, strides, box, "CONV_FPROP pair X"))) return status;
    }
    {
        uint64_t dims[2] = {static_cast<uint64_t>(a.R * a.S * a.C), static_cast<uint64_t>(kK1)};
        uint64_t strides[1] = {static_cast<uint64_t>(a.R * a.S * a.C) * 2};
        uint32_t box[2] = {kBlockK, kK1};
        if ((status = make_map(&map_wa, tensors[1], 2, dims, strides, box, "CONV_FPROP pair W (first)"))) return status;
    }
    {
        uint64_t dims[2] = {static_cast<uint64_t>(kK1), static_cast<uint64_t>(f.k2)};
        uint64_t strides[1] = {static_cast<uint64_t>(kK1) * 2};
        uint32_t box[2] = {kBlockK, static_cast<uint32_t>(f.k2)};
        if ((status = make_map(&map_wb, tensors[2], 2, dims, strides, box, "CONV_FPROP pair W (second)"))) return status;
    }
    {
        uint64_t dims[2] = {static_cast<uint64_t>(f.k2), static_cast<uint64_t>(a.N * a.P * a.Q)};
        uint64_t strides[1] = {static_cast<uint64_t>(f.k2) * 2};
        uint32_t box[2] = {64, static_cast<uint32_t>(f.box_rows)};
        if ((status = make_map(&map_out, tensors[3], 2, dims, strides, box, "CONV_FPROP pair Y"))) return status;
        const void* residual = tensors[3];
        for (int e = 0; e < args.steps_b.count; ++e)
            if (args.steps_b.kind[e] == kStepFull) residual = args.steps_b.data[e];
        if ((status = make_map(&map_res, residual, 2, dims, strides, box, "CONV_FPROP pair residual"))) return status;
    }
    static bool configured = false;
    if (!configured) {
        cudaError_t error = cudaFuncSetAttribute(umma_conv_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBudget);
        if (error != cudaSuccess) return fail(kExecutionFailed, "CONV_FPROP pair: cannot reserve %d bytes of shared memory: %s", kPairSmemBudget, cudaGetErrorString(error));
        configured = true;
    }
    // even shares of the tile list (see launch_persistent in umma_gemm.cu)
    const int sms = sm_count();
    int grid = args.total_tiles < sms ? args.total_tiles : sms;
    if (args.total_tiles > sms) {
        const int rounds = (args.total_tiles + sms - 1) / sms;
        grid = (args.total_tiles + rounds - 1) / rounds;
    }
    cudaError_t launched = launch_chained(umma_conv_pair_kernel, dim3(grid), dim3(kPairThreads), dynamic, stream, map_x, map_wa, map_wb, map_out, map_res, args);
    if (launched != cudaSuccess) return fail(kExecutionFailed, "CONV_FPROP pair: launch failed: %s", cudaGetErrorString(launched));
    return check_launch("CONV_FPROP pair");
}

int conv_pair_device_status(int* status) { return read_and_clear_device_status(status); }

}  // namespace dfgpu

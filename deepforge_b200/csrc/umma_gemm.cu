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
#include "umma_ptx.cuh"

namespace dfgpu {
namespace {

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
    // K split (one-tile kernel only): blockIdx.z takes K slices [z * k_per_split, ...) and stores its raw f32 sums at
    // partial + z * partial_stride (same row/column indexing as `out`, leading dimension n_total); no epilogue runs,
    // whoever adds the partial sums applies it. k_split <= 1: the whole K loop in one CTA, the result goes to `out`.
    int32_t k_split, k_per_split;
    float* partial;
    int64_t partial_stride;
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
    const bool split_k = args.k_split > 1;
    const int kb_begin = split_k ? static_cast<int>(blockIdx.z) * args.k_per_split : 0;
    const int kb_count = split_k ? min(args.k_per_split, args.k_blocks - kb_begin) : args.k_blocks;

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
            for (int i = 0; i < kb_count; ++i) {
                const int kb = kb_begin + i;
                const int s = i % STAGES;
                const uint32_t parity = ((i / STAGES) & 1) ^ 1;
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
            for (int i = 0; i < kb_count && ok; ++i) {
                const int s = i % STAGES;
                const uint32_t parity = (i / STAGES) & 1;
                ok = mbar_wait(full_bar(s), parity, 102);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_src = smem_base + s * L::kStageBytes;
                const uint32_t b_src = a_src + L::kABytes;
                const uint32_t a_lo = smem_desc_lo(a_src, 16);
                const uint32_t b_lo = args.b_mn_major ? smem_desc_lo(b_src, kBlockK * 128) : smem_desc_lo(b_src, 16);
                const uint32_t b_step = args.b_mn_major ? (2048u >> 4) : (32u >> 4);
#pragma unroll
                for (int k = 0; k < kBlockK / 16; ++k)
                    umma_bf16(tmem_base, desc_words(a_lo + ((k * 32) >> 4), smem_desc_hi(1024)), desc_words(b_lo + k * b_step, smem_desc_hi(1024)), idesc, (i | k) != 0 ? 1u : 0u);
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
                if (split_k) {
                    float4* dst = reinterpret_cast<float4*>(args.partial + static_cast<int64_t>(blockIdx.z) * args.partial_stride + out_row * args.n_total + col0);
#pragma unroll
                    for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    continue;
                }
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

// ---- persistent variant for the bandwidth-bound convolutions ------------------------------
//
// One CTA per SM walks a static list of output tiles. These convolutions have tiny K loops and
// almost no math per byte, so what matters is bytes in flight per SM and cycles per handshake:
//   * the whole filter (all taps, all output-channel tiles) is loaded into shared memory ONCE per
//     CTA and stays there; the ring then carries only activation tiles, as many slots as the
//     remaining shared memory allows, filled by the TMA loader warp across tile borders;
//   * filters wider than one tap use the halo form (see PersistentArgs): one slot per filter row,
//     the taps of that row read it from shifted start rows;
//   * the issuing warp (two of them for many-tap tiles, alternating tiles) rotates over four TMEM
//     accumulators, so the next tiles are multiplied while the two epilogue warpgroups drain
//     finished ones: tcgen05.ld -> bias / ReLU / residual -> bf16 -> swizzled shared-memory tile
//     -> one TMA store per 64 output channels;
//   * a residual operand is prefetched by TMA into one of four epilogue buffers (two per epilogue
//     group) and the result is written over it in place, so the same buffer is the source of the
//     TMA store; it goes back to the loader as soon as that store has read it.
// Every global access is a full-line TMA transfer; nothing is read from HBM twice.

constexpr int kMaxRingStages = 12;
constexpr int kPersistentThreads = 352;  // loader warp, issuing warp, two epilogue warpgroups, second issuing warp
constexpr int kAccumulators = 4;          // TMEM accumulators in flight: hides the commit -> epilogue -> release round trip
constexpr int kMaxBiasFloats = 2048;    // per-channel ADD operands staged in shared memory as f32

struct PersistentArgs {
    GemmArgs gemm;
    int32_t n_tiles;       // tiles along the output-channel axis
    int32_t total_tiles;
    int32_t box_rows;      // rows of the output / residual TMA boxes (valid rows of a tile)
    int32_t stages;        // activation ring depth (slots)
    int32_t group_k;       // 64-deep K slices per ring slot: one full/empty handshake moves group_k * 16 KiB
    int32_t filter_bytes;  // resident filter: n_tiles * k_blocks * BN * 128
    int32_t w_offset, epi_offset, ring_offset, bias_offset, barrier_offset;  // shared-memory layout (bytes from the aligned base)
    int32_t bias_stride;   // output channels (floats per staged bias vector)
    // Halo form (filters wider than one tap): one ring slot holds the input rows one FILTER ROW needs, padded
    // columns included (pitch = Q + S - 1 pixels per row); the S taps of that filter row are the same slot
    // read from S starting rows, so the activations cross L2 -> shared memory R times instead of R * S times.
    // GEMM row m is then the padded position (m / pitch, m % pitch) and the positions with m % pitch >= Q are
    // computed but never stored.
    int32_t halo;          // 0 = one slot per tap (or plain GEMM rows)
    int32_t pitch;         // Q + S - 1
    int32_t slot_bytes;    // bytes between ring slots
    int32_t early_static;  // filter and bias may be fetched before the wait on the previous kernel
    int32_t issuers;       // 1, or 2: warp 10 issues the odd tiles of this CTA (a lone lane issues ~60 cycles per product,
                           // twice what a 128 x 64 x 16 product takes to run, so many-tap tiles are issue-bound with one)
    // Split storage (DFGPU_BF16X2): an f32 value kept as hi = bf16(x) and lo = bf16(x - hi), per pixel C hi values
    // followed by C lo values. A split INPUT is a 2C-channel bf16 activation tensor whose two halves meet the same
    // filter (gemm.k_blocks / k_blocks_per_tap count activation slices, w_k_blocks / w_blocks_per_tap filter slices);
    // a split OUTPUT stages and stores the hi boxes at channel n0 and the lo boxes at channel K + n0.
    int32_t split_in, split_out;
    int32_t w_k_blocks;        // 64-deep K slices of the resident filter (per N tile)
    int32_t w_blocks_per_tap;  // C / 64
    int32_t epi_bytes;         // bytes of one epilogue staging buffer
    int32_t epi_per_group;     // staging buffers per epilogue group: 2, or 1 when a buffer holds hi and lo boxes
};

// x - hi for the lo half of a split (hi, lo) pair; 0 when hi is not finite (an infinite or NaN value lives in hi alone,
// so that hi + lo reproduces it instead of inf - inf). x - hi is exact: hi holds the leading 8 significant bits of x.
__device__ __forceinline__ float split_remainder(float x, uint32_t hi_bits) {
    return (hi_bits & 0x7f800000u) == 0x7f800000u ? 0.0f : x - __uint_as_float(hi_bits);
}

template <int BN, bool HAS_RES>
__global__ void __launch_bounds__(kPersistentThreads, 1)
umma_conv_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                            const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_res,
                            PersistentArgs pargs) {
    constexpr int kABytes = kTileM * kBlockK * 2;
    constexpr int kBTileBytes = BN * 128;                 // one 64-deep slice of the filter for this N tile
    constexpr int kEpiBytes = (BN / 64) * kTileM * 128;   // one epilogue buffer
    const GemmArgs& args = pargs.gemm;
    const int STAGES = pargs.stages;
    const int G = pargs.group_k;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t w_base = smem_base + pargs.w_offset;
    const uint32_t epi_base = smem_base + pargs.epi_offset;
    const uint32_t ring_base = smem_base + pargs.ring_offset;
    const uint32_t bar_base = smem_base + pargs.barrier_offset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxRingStages + s); };
    auto acc_full_bar = [&](int a) { return bar_base + 8u * (2 * kMaxRingStages + a); };
    auto acc_empty_bar = [&](int a) { return bar_base + 8u * (2 * kMaxRingStages + 4 + a); };
    auto res_full_bar = [&](int b) { return bar_base + 8u * (2 * kMaxRingStages + 8 + b); };
    auto res_empty_bar = [&](int b) { return bar_base + 8u * (2 * kMaxRingStages + 12 + b); };
    const uint32_t w_full_bar = bar_base + 8u * (2 * kMaxRingStages + 16);
    const uint32_t tmem_slot = bar_base + 8u * (2 * kMaxRingStages + 17);
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(generic_base + pargs.barrier_offset + 8 * (2 * kMaxRingStages + 17));

    const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
    chain_release();  // the next kernel of the plan may start taking SMs as this one's CTAs leave
    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_a);
        prefetch_tensormap(&map_b);
        prefetch_tensormap(&map_out);
        if (HAS_RES) prefetch_tensormap(&map_res);
    }

    auto tile_geometry = [&](int tile, int& m_tile, int& n_tile, int& image, int& h0, int64_t& out_row0) {
        m_tile = tile / pargs.n_tiles;
        n_tile = tile - m_tile * pargs.n_tiles;
        image = 0;
        h0 = 0;
        if (args.is_conv) {
            image = m_tile / args.tiles_per_image;
            h0 = (m_tile - image * args.tiles_per_image) * args.rows_per_tile;
            out_row0 = (static_cast<int64_t>(image) * args.out_p + h0) * args.out_q;
        } else {
            out_row0 = static_cast<int64_t>(m_tile) * kTileM;
        }
    };
    const uint32_t a_bytes = args.is_conv ? static_cast<uint32_t>(args.rows_per_tile * args.out_q * kBlockK * 2) : kABytes;

    // ---- loader state (warp 0). The loop below runs on all 32 lanes with warp-uniform control flow and
    // only the TMA instructions are predicated on one elected lane: a loop that runs inside a single-lane
    // branch pays hundreds of cycles per copy for address arithmetic on the vector pipe. No divisions per
    // copy either: the filter tap and channel block advance as counters.
    struct Loader {
        int tile, index;          // current tile and its position in this CTA's list
        int kb0;                  // next K slice of the tile
        int tap_r, tap_s, cblk;   // filter tap and 64-channel block of that slice
        int stage;                // ring slot to fill next
        uint32_t phase;           // parity of that slot's "free" wait
        uint32_t filled;          // slots filled so far
        int m_tile, n_tile, image, h0;
        int64_t out_row0;
        bool open;                // geometry computed (and residual requested) for `tile`
        bool ok;
    } ld{};
    const bool leader = elect_one();  // per warp: the lane that issues this warp's asynchronous instructions
    // Fills ring slots until the tile list ends or, with `bounded`, until the first ring-full is in flight
    // (nothing in that part can wait on another warp, so it runs ahead of the CTA-wide barrier).
    auto run_loader = [&](bool bounded) {
        const uint32_t res_bytes = static_cast<uint32_t>(pargs.box_rows) * 128u * (BN / 64);
        while (ld.ok && ld.tile < pargs.total_tiles) {
            if (!ld.open) {
                if (bounded && HAS_RES && ld.index >= 4) return;
                tile_geometry(ld.tile, ld.m_tile, ld.n_tile, ld.image, ld.h0, ld.out_row0);
                if (HAS_RES) {
                    const int i = ld.index;
                    const int b = (i & 1) * 2 + ((i >> 1) & 1);  // the owning epilogue group's next buffer
                    ld.ok = mbar_wait_warp(res_empty_bar(b), ((i >> 2) & 1) ^ 1, 111);
                    if (!ld.ok) return;
                    if (leader) {
                        mbar_expect_tx(res_full_bar(b), res_bytes);
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(epi_base + b * pargs.epi_bytes + j * (kTileM * 128), &map_res, ld.n_tile * BN + 64 * j, static_cast<int>(ld.out_row0), res_full_bar(b));
                    }
                }
                ld.open = true;
            }
            if (bounded && ld.filled >= static_cast<uint32_t>(STAGES)) return;
            ld.ok = mbar_wait_warp(empty_bar(ld.stage), ld.phase, 112);
            if (!ld.ok) return;
            if (pargs.halo) {
                // one slot = the rows of filter row tap_r for channel block cblk: box (64 ch, pitch, rows, 1)
                if (leader) {
                    mbar_expect_tx(full_bar(ld.stage), static_cast<uint32_t>(args.rows_per_tile * pargs.pitch * kBlockK * 2));
                    tma_load_4d(ring_base + ld.stage * pargs.slot_bytes, &map_a, ld.cblk * kBlockK, -args.pad_w, ld.h0 + ld.tap_r - args.pad_h, ld.image, full_bar(ld.stage));
                }
                if (++ld.cblk == args.k_blocks_per_tap) { ld.cblk = 0; ++ld.tap_r; }
            } else {
            if (leader) mbar_expect_tx(full_bar(ld.stage), a_bytes * G);
            for (int g = 0; g < G; ++g) {
                const uint32_t a_dst = ring_base + ld.stage * pargs.slot_bytes + g * kABytes;
                if (args.is_conv) {
                    if (leader) tma_load_4d(a_dst, &map_a, ld.cblk * kBlockK, ld.tap_s - args.pad_w, ld.h0 + ld.tap_r - args.pad_h, ld.image, full_bar(ld.stage));
                } else {
                    if (leader) tma_load_2d(a_dst, &map_a, (ld.kb0 + g) * kBlockK, ld.m_tile * kTileM, full_bar(ld.stage));
                }
                if (++ld.cblk == args.k_blocks_per_tap) {
                    ld.cblk = 0;
                    if (++ld.tap_s == args.filter_s) { ld.tap_s = 0; ++ld.tap_r; }
                }
            }
            }
            ++ld.filled;
            if (++ld.stage == STAGES) { ld.stage = 0; ld.phase ^= 1; }
            ld.kb0 += pargs.halo ? args.filter_s : G;  // K slices this slot covers
            if (ld.kb0 >= args.k_blocks) {
                ld.tile += gridDim.x;
                ++ld.index;
                ld.kb0 = 0;
                ld.tap_r = ld.tap_s = ld.cblk = 0;
                ld.open = false;
            }
        }
    };

    if (warp == 0) {
        if (leader) {
            for (int s = 0; s < STAGES; ++s) {
                mbar_init(full_bar(s), 1);
                mbar_init(empty_bar(s), 1);
            }
            for (int a = 0; a < kAccumulators; ++a) {
                mbar_init(acc_full_bar(a), 1);
                mbar_init(acc_empty_bar(a), 4);  // one arrival per warp of the group that drained it
            }
            for (int b = 0; b < 4; ++b) {
                mbar_init(res_full_bar(b), 1);
                mbar_init(res_empty_bar(b), 1);  // the thread that issues that group's TMA stores
            }
            mbar_init(w_full_bar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            mbar_expect_tx(w_full_bar, static_cast<uint32_t>(pargs.filter_bytes));
        }
        __syncwarp();
        // Everything up to chain_wait() is private to the CTA or reads operands no running kernel writes; the loads
        // after it read the previous kernel's output.
        if (!pargs.early_static) chain_wait();
        // Start streaming right away: the filter and the first ring-full of activations are in flight
        // while the other warps allocate tensor memory and stage the bias vectors.
        for (int nt = 0; nt < pargs.n_tiles; ++nt)
            for (int kb = 0; kb < pargs.w_k_blocks; ++kb)
                if (leader) tma_load_2d(w_base + (nt * pargs.w_k_blocks + kb) * kBTileBytes, &map_b, kb * kBlockK, nt * BN, w_full_bar);
        if (pargs.early_static) chain_wait();
        ld.tile = blockIdx.x;
        ld.phase = 1;
        ld.ok = true;
        run_loader(true);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kAccumulators * BN);
        tmem_relinquish();
        tc_fence_before();
    }
    if (warp != 0 && !pargs.early_static) chain_wait();  // warp 0 waited before its first load
    {
        // per-channel ADD operands -> f32 in shared memory, once per CTA
        float* bias_stage = reinterpret_cast<float*>(generic_base + pargs.bias_offset);
        int slot = 0;
        for (int e = 0; e < args.epi_count; ++e) {
            if (args.epi_kind[e] != kEpiBias) continue;
            for (int c = threadIdx.x; c < pargs.bias_stride; c += blockDim.x)
                bias_stage[slot * pargs.bias_stride + c] = load_as_f32(args.epi_data[e], args.epi_dtype[e], c);
            ++slot;
        }
    }
    if (warp != 0 && pargs.early_static) chain_wait();  // the bias vectors above are static operands
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 0) {
        run_loader(false);
    } else if (warp == 1 || warp == 10) {
        // All 32 lanes walk the schedule; the elected lane issues the products and their commits.
        const int me = warp == 1 ? 0 : 1;
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) |
                               (static_cast<uint32_t>(kTileM >> 4) << 24);
        const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
        const int slots_per_tile = pargs.halo ? args.k_blocks / args.filter_s : args.k_blocks / G;
        int stage = 0;
        uint32_t phase = 0, it = 0;
        bool ok = me < pargs.issuers && mbar_wait_warp(w_full_bar, 0, 117);
        for (int tile = blockIdx.x, i = 0; tile < pargs.total_tiles && me < pargs.issuers; tile += gridDim.x, ++i) {
            if (pargs.issuers == 2 && (i & 1) != me) {
                // the other issuing warp's tile: step over its ring slots
                for (int n = 0; n < slots_per_tile; ++n, ++it)
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                continue;
            }
            const int acc = i % kAccumulators;
            const int n_tile = tile % pargs.n_tiles;
            if (ok) ok = mbar_wait_warp(acc_empty_bar(acc), ((i / kAccumulators) & 1) ^ 1, 113);
            tc_fence_after();
            const uint32_t tmem_acc = tmem_u + static_cast<uint32_t>(acc * BN);
            int halo_r = 0, halo_c = 0;  // filter row and channel block of the next slot (halo form)
            for (int kb0 = 0; kb0 < args.k_blocks && ok; kb0 += (pargs.halo ? args.filter_s : G), ++it) {
                ok = mbar_wait_warp(full_bar(stage), phase, 114);
                if (!ok) break;  // (the slot was filled by TMA: no tcgen05 fence needed before the products read it)
                const uint32_t a_lo = smem_desc_lo(ring_base + stage * pargs.slot_bytes, 16);
                if (pargs.halo) {
                    // tap s of this filter row reads the slot from row s on: only the start address moves, by s * 128 bytes.
                    // The 128-byte swizzle is a function of the absolute shared-memory address (TMA wrote the slot that
                    // way), so a start in the middle of an 8-row swizzle atom needs no base offset in the descriptor.
                    const int w_c = halo_c >= pargs.w_blocks_per_tap ? halo_c - pargs.w_blocks_per_tap : halo_c;  // the lo half meets the same filter slices
                    const uint32_t b_first = smem_desc_lo(w_base + ((n_tile * pargs.w_k_blocks + halo_r * args.filter_s * pargs.w_blocks_per_tap + w_c) * kBTileBytes), 16);
                    const uint32_t b_tap_step = static_cast<uint32_t>(pargs.w_blocks_per_tap * kBTileBytes) >> 4;
                    if (leader) {
                        const uint32_t first = kb0 != 0 ? 1u : 0u;
                        if (args.filter_s == 3) {
                            // straight-line code: a branch between products costs more than the product itself takes to run
#pragma unroll
                            for (int tap = 0; tap < 3; ++tap)
#pragma unroll
                                for (int k = 0; k < kBlockK / 16; ++k)
                                    umma_bf16(tmem_acc, desc_words(a_lo + ((tap * 128 + k * 32) >> 4), smem_desc_hi(1024)),
                                              desc_words(b_first + tap * b_tap_step + ((k * 32) >> 4), smem_desc_hi(1024)), idesc, (tap | k) != 0 ? 1u : first);
                        } else {
                            for (int tap = 0; tap < args.filter_s; ++tap) {
#pragma unroll
                                for (int k = 0; k < kBlockK / 16; ++k)
                                    umma_bf16(tmem_acc, desc_words(a_lo + ((tap * 128 + k * 32) >> 4), smem_desc_hi(1024)),
                                              desc_words(b_first + tap * b_tap_step + ((k * 32) >> 4), smem_desc_hi(1024)), idesc, (tap | k) != 0 ? 1u : first);
                            }
                        }
                    }
                    if (++halo_c == args.k_blocks_per_tap) { halo_c = 0; ++halo_r; }
                } else if (leader) {
                    // filter slice of activation slice kb0 (they differ for a split input: both halves of a tap's channels
                    // meet that tap's filter slices; a group of G slices never straddles a half)
                    const int tap = kb0 / args.k_blocks_per_tap, c = kb0 - tap * args.k_blocks_per_tap;
                    const int w_kb0 = tap * pargs.w_blocks_per_tap + (c >= pargs.w_blocks_per_tap ? c - pargs.w_blocks_per_tap : c);
                    const uint32_t b_lo = smem_desc_lo(w_base + (n_tile * pargs.w_k_blocks + w_kb0) * kBTileBytes, 16);
                    for (int g = 0; g < G; ++g) {
#pragma unroll
                        for (int k = 0; k < kBlockK / 16; ++k)
                            umma_bf16(tmem_acc, desc_words(a_lo + ((g * kABytes + k * 32) >> 4), smem_desc_hi(1024)),
                                      desc_words(b_lo + ((g * kBTileBytes + k * 32) >> 4), smem_desc_hi(1024)), idesc, (kb0 | g | k) != 0 ? 1u : 0u);
                    }
                }
                if (leader) umma_commit(empty_bar(stage));
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            if (leader) umma_commit(acc_full_bar(acc));  // arrives even after a failed wait so the epilogue never hangs
        }
    } else {
        // two epilogue warpgroups: group g drains accumulator g, i.e. every other tile
        const int group = (warp - 2) >> 2;
        const int quadrant = warp & 3;
        const int gemm_row = quadrant * 32 + lane;
        // halo form: GEMM row = padded position; only columns < Q of each row are outputs, compacted for the store
        int row = gemm_row;
        bool row_is_output = true;
        if (pargs.halo) {
            const int line = gemm_row / pargs.pitch, column = gemm_row - line * pargs.pitch;
            row_is_output = column < args.out_q && line < args.rows_per_tile;
            row = row_is_output ? line * args.out_q + column : 0;
        }
        const bool store_thread = ((warp - 2) & 3) == 0 && lane == 0;
        const float* bias_smem = reinterpret_cast<const float*>(generic_base + pargs.bias_offset);
        bool ok = true;
        for (int tile = blockIdx.x + group * gridDim.x, j = 0; tile < pargs.total_tiles; tile += 2 * gridDim.x, ++j) {
            int m_tile, n_tile, image, h0;
            int64_t out_row0;
            tile_geometry(tile, m_tile, n_tile, image, h0, out_row0);
            const int n0 = n_tile * BN;
            const int i = group + 2 * j;  // position of this tile in the CTA's tile list
            const int acc = i % kAccumulators;
            const int buf = pargs.epi_per_group == 2 ? group * 2 + (j & 1) : group;  // two staging buffers per epilogue group, used alternately (or one)
            if (HAS_RES && store_thread && j >= 1) {
                // The store of this group's previous tile has had a whole wait to read its buffer: hand the
                // buffer back now, so that its next residual tile streams in while this tile is worked on.
                tma_store_wait_read<0>();
                mbar_arrive(res_empty_bar(group * 2 + ((j - 1) & 1)));
            }
            if (ok) ok = mbar_wait(acc_full_bar(acc), (i / kAccumulators) & 1, 115);
            if (HAS_RES) {
                if (ok) ok = mbar_wait(res_full_bar(buf), (j >> 1) & 1, 116);
            } else {
                // this staging buffer was last read by the TMA store of this group's tile before last: at most the
                // previous tile's store may still be reading (the other buffer)
                if (store_thread) {
                    if (pargs.epi_per_group == 2) tma_store_wait_read<1>();
                    else tma_store_wait_read<0>();
                }
                epilogue_barrier(1 + group);
            }
            tc_fence_after();
            const bool healthy = ok && g_device_status == 0;
            uint8_t* tile_smem = generic_base + pargs.epi_offset + buf * pargs.epi_bytes;
#pragma unroll 1
            for (int chunk = 0; chunk < BN / 32; ++chunk) {
                uint32_t raw[32];
                tmem_load_32(tmem_base + (static_cast<uint32_t>(quadrant * 32) << 16) + acc * BN + chunk * 32, raw);
                tmem_load_wait();
                float v[32];
#pragma unroll
                for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(raw[e]);
                const int region = chunk >> 1;        // which 64-channel box
                const int chunk16 = (chunk & 1) * 4;  // first 16-byte unit inside the 128-byte row
                uint8_t* row_smem = tile_smem + region * (kTileM * 128) + row * 128;
                int bias_slot = 0;
                for (int e = 0; e < args.epi_count; ++e) {
                    const int kind = args.epi_kind[e];
                    if (kind == kEpiRelu) {
                        const float lower = args.epi_lower[e], upper = args.epi_upper[e], slope = args.epi_slope[e];
#pragma unroll
                        for (int t = 0; t < 32; ++t) v[t] = relu_fast(v[t], lower, upper, slope);
                    } else if (kind == kEpiBias) {
                        const float4* p = reinterpret_cast<const float4*>(bias_smem + bias_slot * pargs.bias_stride + n0 + chunk * 32);
                        ++bias_slot;
#pragma unroll
                        for (int q4 = 0; q4 < 8; ++q4) {
                            const float4 q = p[q4];
                            v[4 * q4] = __fadd_rn(v[4 * q4], q.x);
                            v[4 * q4 + 1] = __fadd_rn(v[4 * q4 + 1], q.y);
                            v[4 * q4 + 2] = __fadd_rn(v[4 * q4 + 2], q.z);
                            v[4 * q4 + 3] = __fadd_rn(v[4 * q4 + 3], q.w);
                        }
                    } else if (HAS_RES) {  // the residual tile the producer staged in this buffer
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            const uint4 q = *reinterpret_cast<const uint4*>(row_smem + (((chunk16 + q4) ^ (row & 7)) << 4));
                            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                v[8 * q4 + 2 * t] = __fadd_rn(v[8 * q4 + 2 * t], __uint_as_float(w[t] << 16));
                                v[8 * q4 + 2 * t + 1] = __fadd_rn(v[8 * q4 + 2 * t + 1], __uint_as_float(w[t] & 0xffff0000u));
                            }
                        }
                    }
                }
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint32_t w[4];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        __nv_bfloat162 pair = __floats2bfloat162_rn(v[8 * q4 + 2 * t], v[8 * q4 + 2 * t + 1]);
                        w[t] = *reinterpret_cast<uint32_t*>(&pair);
                    }
                    if (row_is_output) *reinterpret_cast<uint4*>(row_smem + (((chunk16 + q4) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                if (!HAS_RES && pargs.split_out) {
                    uint8_t* lo_smem = row_smem + (BN / 64) * (kTileM * 128);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint32_t w[4];
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            const float a = v[8 * q4 + 2 * t], b = v[8 * q4 + 2 * t + 1];
                            __nv_bfloat162 hi = __floats2bfloat162_rn(a, b);
                            const uint32_t hi_bits = *reinterpret_cast<uint32_t*>(&hi);
                            __nv_bfloat162 pair = __floats2bfloat162_rn(split_remainder(a, hi_bits << 16), split_remainder(b, hi_bits & 0xffff0000u));
                            w[t] = *reinterpret_cast<uint32_t*>(&pair);
                        }
                        if (row_is_output) *reinterpret_cast<uint4*>(lo_smem + (((chunk16 + q4) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
            // release the accumulator, then publish the finished tile
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty_bar(acc));
            fence_async_shared();
            epilogue_barrier(1 + group);
            if (store_thread) {
                if (healthy) {
#pragma unroll
                    for (int q = 0; q < BN / 64; ++q)
                        tma_store_2d(&map_out, epi_base + buf * pargs.epi_bytes + q * (kTileM * 128), n0 + 64 * q, static_cast<int>(out_row0));
                    if (!HAS_RES && pargs.split_out) {
#pragma unroll
                        for (int q = 0; q < BN / 64; ++q)
                            tma_store_2d(&map_out, epi_base + buf * pargs.epi_bytes + (BN / 64 + q) * (kTileM * 128), static_cast<int>(args.n_total) + n0 + 64 * q, static_cast<int>(out_row0));
                    }
                }
                tma_store_commit();
            }
        }
        if (store_thread) tma_store_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kAccumulators * BN);
    }
}

// ---- host side ----------------------------------------------------------------------------

template <int BN, int STAGES>
int launch(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmArgs& args, dim3 grid, cudaStream_t stream, bool chained) {
    using L = SmemLayout<BN, STAGES>;
    static bool configured = false;
    if (!configured) {
        cudaError_t error = cudaFuncSetAttribute(umma_gemm_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
        if (error != cudaSuccess) return fail(kExecutionFailed, "tcgen05 GEMM: cannot reserve %d bytes of shared memory: %s", L::kDynamic, cudaGetErrorString(error));
        configured = true;
    }
    if (chained) {
        cudaError_t error = launch_chained(umma_gemm_kernel<BN, STAGES>, grid, dim3(kThreads), L::kDynamic, stream, map_a, map_b, args);
        if (error != cudaSuccess) return fail(kExecutionFailed, "tcgen05 GEMM: launch failed: %s", cudaGetErrorString(error));
    } else {
        umma_gemm_kernel<BN, STAGES><<<grid, kThreads, L::kDynamic, stream>>>(map_a, map_b, args);
    }
    return check_launch("tcgen05 GEMM");
}

// Ring depth: shallow K loops (the 1x1 convolutions) get short rings so that several CTAs fit on
// one SM and overlap each other's load / MMA / epilogue phases; deep K loops (matmul) get 4 stages.
int dispatch(int bn, int k_blocks, const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmArgs& args, dim3 grid, cudaStream_t stream, bool chained = false) {
    const int stages = k_blocks <= 1 ? 1 : (k_blocks <= 12 ? 2 : 4);
    if (bn == 64) {
        if (stages == 1) return launch<64, 1>(map_a, map_b, args, grid, stream, chained);
        if (stages == 2) return launch<64, 2>(map_a, map_b, args, grid, stream, chained);
        return launch<64, 4>(map_a, map_b, args, grid, stream, chained);
    }
    if (bn == 128) {
        if (stages == 1) return launch<128, 1>(map_a, map_b, args, grid, stream, chained);
        if (stages == 2) return launch<128, 2>(map_a, map_b, args, grid, stream, chained);
        return launch<128, 4>(map_a, map_b, args, grid, stream, chained);
    }
    if (stages <= 2) return launch<256, 2>(map_a, map_b, args, grid, stream, chained);
    return launch<256, 4>(map_a, map_b, args, grid, stream, chained);
}

constexpr int kSmemBudget = 227 * 1024;

template <int BN, bool HAS_RES>
int launch_persistent(const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_out, const CUtensorMap& map_res,
                      PersistentArgs args, cudaStream_t stream) {
    constexpr int kBarrierBytes = (2 * kMaxRingStages + 18) * 8;
    int bias_vectors = 0;
    for (int e = 0; e < args.gemm.epi_count; ++e) bias_vectors += args.gemm.epi_kind[e] == kEpiBias;
    const int bias_bytes = (bias_vectors * args.bias_stride * 4 + 1023) & ~1023;
    // staging: two buffers per epilogue group (a tile is staged while the previous tile's TMA store still reads), or one
    // per group when a buffer holds the hi and the lo boxes of a split output
    args.epi_per_group = args.split_out ? 1 : 2;
    args.epi_bytes = (BN / 64) * kTileM * 128 * (args.split_out ? 2 : 1);
    args.w_offset = 0;
    args.epi_offset = (args.filter_bytes + 1023) & ~1023;
    args.ring_offset = args.epi_offset + 2 * args.epi_per_group * args.epi_bytes;
    int room = kSmemBudget - 1024 - kBarrierBytes - bias_bytes - args.ring_offset;
    // K slices per handshake: the largest divisor of the K loop (<= 4) that still leaves >= 2 ring slots
    int group = 1;
    if (args.halo) {
        // a slot holds 128 + S - 1 rows of 128 bytes: the last tap reads S - 1 rows past the 128th GEMM row
        args.slot_bytes = ((kTileM + args.gemm.filter_s - 1) * 128 + 1023) & ~1023;
    } else {
        for (int candidate = 4; candidate >= 2; --candidate)
            if (args.gemm.k_blocks % candidate == 0 && (!args.split_in || args.w_blocks_per_tap % candidate == 0) && room / (candidate * kTileM * kBlockK * 2) >= 2) {
                group = candidate;
                break;
            }
        args.slot_bytes = group * kTileM * kBlockK * 2;
    }
    int stages = room / args.slot_bytes;
    if (stages > kMaxRingStages) stages = kMaxRingStages;
    if (stages < 2) return fail(kUnsupported, "tcgen05 conv: the filter does not leave room for an activation ring");
    args.stages = stages;
    args.group_k = group;
    args.bias_offset = args.ring_offset + stages * args.slot_bytes;
    args.barrier_offset = args.bias_offset + bias_bytes;
    const int dynamic = args.barrier_offset + kBarrierBytes + 1024;
    // two issuing warps when a tile is many products (filters wider than one tap) and the ring holds two tiles
    args.issuers = (args.halo && args.gemm.k_blocks / args.gemm.filter_s + 2 <= stages) ? 2 : 1;
    static int configured = 0;
    if (configured < dynamic) {
        cudaError_t error = cudaFuncSetAttribute(umma_conv_persistent_kernel<BN, HAS_RES>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
        if (error != cudaSuccess) return fail(kExecutionFailed, "tcgen05 conv: cannot reserve %d bytes of shared memory: %s", kSmemBudget, cudaGetErrorString(error));
        configured = kSmemBudget;
    }
    // Even shares: every CTA walks ceil(tiles / SMs) tiles or one fewer. These launches are bandwidth-bound and a
    // handful of tiles per CTA long, so a last round that only a few CTAs run costs more than the SMs left idle.
    const int sms = sm_count();
    int grid = args.total_tiles < sms ? args.total_tiles : sms;
    if (args.total_tiles > sms) {
        const int rounds = (args.total_tiles + sms - 1) / sms;
        grid = (args.total_tiles + rounds - 1) / rounds;
    }
    cudaError_t launched = launch_chained(umma_conv_persistent_kernel<BN, HAS_RES>, dim3(grid), dim3(kPersistentThreads), dynamic, stream, map_a, map_b, map_out, map_res, args);
    if (launched != cudaSuccess) return fail(kExecutionFailed, "tcgen05 conv (persistent): launch failed: %s", cudaGetErrorString(launched));
    return check_launch("tcgen05 conv (persistent)");
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

bool conv_umma_form(const dfgpu_conv_params& p, ConvForm& f) {
    const bool x_ok = p.x.dtype == DFGPU_BF16 || p.x.dtype == DFGPU_BF16X2;
    const bool y_ok = p.y.dtype == DFGPU_BF16 || p.y.dtype == DFGPU_F32 || p.y.dtype == DFGPU_BF16X2;
    if (!x_ok || p.w.dtype != DFGPU_BF16 || !y_ok) return false;
    if (!nhwc_packed(p.x) || !nhwc_packed(p.w) || !nhwc_packed(p.y)) return false;
    if (p.x.dim[1] != p.w.dim[1]) return false;  // groups == 1
    f.N = p.x.dim[0]; f.C = p.x.dim[1]; f.H = p.x.dim[2]; f.W = p.x.dim[3];
    f.K = p.y.dim[1]; f.P = p.y.dim[2]; f.Q = p.y.dim[3]; f.R = p.w.dim[2]; f.S = p.w.dim[3];
    f.split_in = p.x.dtype == DFGPU_BF16X2;
    f.split_out = p.y.dtype == DFGPU_BF16X2;
    if (f.C % 64 != 0 || f.K % 64 != 0 || f.Q > 128 || f.Q < 1) return false;
    if (p.stride[0] != 1 || p.stride[1] != 1 || p.dilation[0] != 1 || p.dilation[1] != 1 || p.reverse_filter) return false;
    if (f.R * f.S > 49 || f.N * f.P > (1 << 22)) return false;
    if (f.H > 65535 || f.W > 65535 || p.pre_pad[0] > 64 || p.pre_pad[1] > 64) return false;
    if (!translate_epilogue(p.epilogue_count, p.epilogue, p.extra, p.y, 1, true, f.K, nullptr, nullptr)) return false;
    f.pointwise = f.R == 1 && f.S == 1 && p.pre_pad[0] == 0 && p.pre_pad[1] == 0 && p.post_pad[0] == 0 && p.post_pad[1] == 0;
    f.bn = pick_bn(f.K, f.R * f.S * (f.C / kBlockK));
    f.rows_per_tile = static_cast<int>(kTileM / f.Q);
    // persistent form
    int full_steps = 0, bias_steps = 0;
    bool residual_bf16 = true;
    for (int e = 0; e < p.epilogue_count; ++e) {
        if (p.epilogue[e].op != DFGPU_EPI_ADD) continue;
        const dfgpu_tensor& t = p.extra[p.epilogue[e].operand];
        bool per_channel = true;  // same classification as translate_epilogue: anything that is not one value per channel is a full tensor
        const int shift = p.y.rank - t.rank;
        for (int axis = 0; axis < t.rank; ++axis) {
            if (axis + shift == 1) per_channel = per_channel && t.dim[axis] == p.y.dim[1] && t.stride[axis] == 1;
            else per_channel = per_channel && t.dim[axis] == 1;
        }
        if (shift > 1) per_channel = false;
        if (per_channel) ++bias_steps;
        else {
            ++full_steps;
            residual_bf16 = residual_bf16 && t.dtype == DFGPU_BF16;
        }
    }
    // halo form: a tile is `halo_rows` output rows with their padded columns, halo_rows the largest divisor of P that fits
    f.halo = false;
    f.halo_rows = 0;
    const int64_t pitch = f.Q + f.S - 1;
    if (!f.pointwise && f.S > 1 && f.S <= 8 && pitch <= kTileM) {
        int halo_rows = static_cast<int>(kTileM / pitch);
        while (halo_rows > 1 && f.P % halo_rows != 0) --halo_rows;
        f.halo = true;
        f.halo_rows = halo_rows;
    }
    const bool whole_tiles = f.pointwise || f.halo || f.P % f.rows_per_tile == 0;
    const bool residual_ok = full_steps == 0 || (full_steps == 1 && residual_bf16 && !f.split_out);
    const int64_t filter_bytes = f.K * f.R * f.S * f.C * 2;
    const int epilogue_bytes = (f.split_out ? 2 * 2 : 4) * (f.bn / 64) * kTileM * 128;
    const bool filter_fits = bias_steps * f.K <= kMaxBiasFloats &&
                             filter_bytes + epilogue_bytes + 3 * kTileM * kBlockK * 2 + bias_steps * f.K * 4 + 6144 <= kSmemBudget;
    f.persistent = (p.reserved & 1) == 0 && p.y.dtype != DFGPU_F32 && whole_tiles && residual_ok && filter_fits && f.N * f.P * f.Q < (1ll << 31) && f.bn <= 128;
    if (!f.persistent) f.halo = false;
    // split tensors exist only in the persistent kernel
    if ((f.split_in || f.split_out) && !f.persistent) return false;
    return true;
}

bool conv_umma_supported(const dfgpu_conv_params& p) {
    ConvForm form;
    return conv_umma_form(p, form);
}

int launch_conv_umma(const dfgpu_conv_params& p, void* const* tensors, cudaStream_t stream, const ConvKSplit* k_split) {
    ConvForm f;
    if (!conv_umma_form(p, f)) return fail(kUnsupported, "CONV_FPROP: the tcgen05 kernel does not take this convolution");
    const int64_t N = f.N, C = f.C, H = f.H, W = f.W, K = f.K, P = f.P, Q = f.Q, R = f.R, S = f.S;
    const int64_t Ca = f.split_in ? 2 * C : C;    // bf16 channels per activation pixel in storage
    const int64_t Kout = f.split_out ? 2 * K : K;  // bf16 channels per output pixel in storage
    if (!aligned16(tensors[0]) || !aligned16(tensors[1]) || !aligned16(tensors[2]))
        return fail(kInvalidArgument, "CONV_FPROP: the tcgen05 kernel needs 16-byte aligned X, W and Y");
    GemmArgs args{};
    const bool pointwise = f.pointwise;
    const int bn = f.bn;
    CUtensorMap map_a, map_b;
    int status;
    int64_t m_tiles;
    if (pointwise) {
        const int64_t M = N * H * W;
        uint64_t dims[2] = {static_cast<uint64_t>(Ca), static_cast<uint64_t>(M)};
        uint64_t strides[1] = {static_cast<uint64_t>(Ca) * 2};
        uint32_t box[2] = {kBlockK, kTileM};
        status = make_map(&map_a, tensors[0], 2, dims, strides, box, "CONV_FPROP X");
        if (status) return status;
        args.is_conv = 0;
        args.m_total = M;
        m_tiles = (M + kTileM - 1) / kTileM;
    } else {
        const int rows = f.rows_per_tile;
        uint64_t dims[4] = {static_cast<uint64_t>(Ca), static_cast<uint64_t>(W), static_cast<uint64_t>(H), static_cast<uint64_t>(N)};
        uint64_t strides[3] = {static_cast<uint64_t>(Ca) * 2, static_cast<uint64_t>(W * Ca) * 2, static_cast<uint64_t>(H * W * Ca) * 2};
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
    args.k_blocks_per_tap = static_cast<int>(Ca / kBlockK);
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
    // Persistent kernel (TMA-store epilogue) when its preconditions hold; else one tile per CTA.
    int residual_step = -1, full_steps = 0;
    for (int e = 0; e < args.epi_count; ++e)
        if (args.epi_kind[e] == kEpiFull) {
            residual_step = e;
            ++full_steps;
        }
    if (f.persistent) {
        PersistentArgs pargs{};
        pargs.gemm = args;
        pargs.early_static = (p.reserved & 2) ? 1 : 0;
        pargs.split_in = f.split_in;
        pargs.split_out = f.split_out;
        pargs.w_blocks_per_tap = static_cast<int>(C / kBlockK);
        pargs.w_k_blocks = static_cast<int>(R * S * (C / kBlockK));
        int out_box_rows = pointwise ? kTileM : args.rows_per_tile * static_cast<int>(Q);
        // filters wider than one tap: load each filter row's input rows once, padded columns included
        if (f.halo) {
            const int64_t pitch = Q + S - 1;
            pargs.halo = 1;
            pargs.pitch = static_cast<int>(pitch);
            pargs.gemm.rows_per_tile = f.halo_rows;
            pargs.gemm.tiles_per_image = static_cast<int>(P / f.halo_rows);
            m_tiles = N * pargs.gemm.tiles_per_image;
            uint64_t dims4[4] = {static_cast<uint64_t>(Ca), static_cast<uint64_t>(W), static_cast<uint64_t>(H), static_cast<uint64_t>(N)};
            uint64_t strides3[3] = {static_cast<uint64_t>(Ca) * 2, static_cast<uint64_t>(W * Ca) * 2, static_cast<uint64_t>(H * W * Ca) * 2};
            uint32_t box4[4] = {kBlockK, static_cast<uint32_t>(pitch), static_cast<uint32_t>(f.halo_rows), 1};
            status = make_map(&map_a, tensors[0], 4, dims4, strides3, box4, "CONV_FPROP X (halo)");
            if (status) return status;
            out_box_rows = f.halo_rows * static_cast<int>(Q);
        }
        pargs.n_tiles = static_cast<int>(K / bn);
        pargs.total_tiles = static_cast<int>(m_tiles) * pargs.n_tiles;
        pargs.box_rows = out_box_rows;
        pargs.filter_bytes = static_cast<int>(K * R * S * C * 2);
        pargs.bias_stride = static_cast<int>(K);
        CUtensorMap map_out, map_res;
        uint64_t dims[2] = {static_cast<uint64_t>(Kout), static_cast<uint64_t>(N * P * Q)};
        uint64_t strides[1] = {static_cast<uint64_t>(Kout) * 2};
        uint32_t box[2] = {64, static_cast<uint32_t>(out_box_rows)};
        status = make_map(&map_out, tensors[2], 2, dims, strides, box, "CONV_FPROP Y");
        if (status) return status;
        const void* residual = full_steps ? args.epi_data[residual_step] : tensors[2];
        status = make_map(&map_res, residual, 2, dims, strides, box, "CONV_FPROP residual");
        if (status) return status;
        if (bn == 64) {
            if (full_steps) return launch_persistent<64, true>(map_a, map_b, map_out, map_res, pargs, stream);
            return launch_persistent<64, false>(map_a, map_b, map_out, map_res, pargs, stream);
        }
        if (full_steps) return launch_persistent<128, true>(map_a, map_b, map_out, map_res, pargs, stream);
        return launch_persistent<128, false>(map_a, map_b, map_out, map_res, pargs, stream);
    }
    dim3 grid(static_cast<unsigned>(m_tiles), static_cast<unsigned>(K / bn));
    if (k_split && k_split->splits > 1) {
        args.k_split = k_split->splits;
        args.k_per_split = k_split->k_blocks_per_split;
        args.partial = k_split->partial;
        args.partial_stride = N * P * Q * K;
        grid.z = static_cast<unsigned>(k_split->splits);
        return dispatch(bn, args.k_blocks, map_a, map_b, args, grid, stream);  // (ring depth as for the whole K loop: the loads are the launch)
    }
    return dispatch(bn, args.k_blocks, map_a, map_b, args, grid, stream);
}

ConvKSplit conv_umma_k_split(const dfgpu_conv_params& p) {
    ConvKSplit split{1, 0, nullptr};
    ConvForm f;
    if (!conv_umma_form(p, f) || f.persistent) return split;
    const int64_t m_tiles = f.pointwise ? (f.N * f.H * f.W + kTileM - 1) / kTileM : f.N * ((f.P + f.rows_per_tile - 1) / f.rows_per_tile);
    const int64_t tiles = m_tiles * (f.K / f.bn);
    const int k_blocks = static_cast<int>(f.R * f.S * (f.C / kBlockK));
    // (a function of the shape alone, so that a plan made on one machine sizes the scratch for every other: 148 SMs)
    const int wanted = static_cast<int>(148 / tiles);  // CTAs per tile that the tiles alone leave idle SMs for
    if (wanted < 2 || k_blocks < 4) return split;
    split.k_blocks_per_split = (k_blocks + wanted - 1) / wanted;
    if (split.k_blocks_per_split < 2) split.k_blocks_per_split = 2;
    if (split.k_blocks_per_split * kMaxKSplits < k_blocks) split.k_blocks_per_split = (k_blocks + kMaxKSplits - 1) / kMaxKSplits;
    split.splits = (k_blocks + split.k_blocks_per_split - 1) / split.k_blocks_per_split;
    return split;
}

bool matmul_umma_supported(const dfgpu_matmul_params& p, int kernel) {
    if (kernel == DFGPU_MATMUL_UMMA_MXF8) return matmul_mxf8_supported(p);
    if (kernel != DFGPU_MATMUL_UMMA_BF16) return false;
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
    if (kernel == DFGPU_MATMUL_UMMA_MXF8) return launch_matmul_mxf8(p, tensors, stream);
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

}  // namespace dfgpu

// Reads and clears the device-side status words the bounded waits write (0 = none).
// Synchronises the device; meant for tests and for the runtime's post-mortem path.
extern "C" int dfgpu_device_status(int* status) {
    using namespace dfgpu;
    if (!status) return fail(kInvalidArgument, "device_status: null pointer");
    int gemm = 0, sdpa = 0, decode = 0, mxf8 = 0, pair = 0;
    int code = read_and_clear_device_status(&gemm);
    if (code) return code;
    code = conv_pair_device_status(&pair);
    if (code) return code;
    if (!gemm) gemm = pair;
    int cluster = 0;
    code = conv_f32_device_status(&cluster);
    if (code) return code;
    if (!gemm) gemm = cluster;
    code = mxf8_device_status(&mxf8);
    if (code) return code;
    if (!gemm) gemm = mxf8;
    code = sdpa_umma_device_status(&sdpa);
    if (code) return code;
    code = decode_umma_device_status(&decode);
    if (code) return code;
    int prefix = 0;
    code = sdpa_device_status(&prefix);
    if (code) return code;
    if (!decode) decode = prefix;
    *status = gemm ? gemm : (sdpa ? sdpa : decode);
    return kOk;
}

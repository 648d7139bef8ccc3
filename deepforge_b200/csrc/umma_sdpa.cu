// SDPA forward on the 5th-generation tensor cores (bf16, head dim 128, contiguous K/V).
//
// One CTA owns a 128-row query tile of one (batch, head) and walks the key/value tiles of 128:
//   warp 0     TMA producer: Q once, then K_0, V_0, K_1, V_1, ... into a ring of 32 KiB slots
//   warp 1     one lane issues S_j = Q K_j^T into one of two TMEM score buffers (so S_{j+1} is
//              multiplied while the softmax warps work on S_j) and O += P_j V_j into the TMEM
//              output accumulator
//   warps 2-5  softmax, one query row per thread: tcgen05.ld the scores, running max / sum in the
//              exp2 domain, P_j as bf16 into a swizzled shared-memory tile (the A operand of the
//              second product), final 1/sum, O and Stats stores.
// The running maximum is only raised when it grows by more than 2^8 (the accumulator is rescaled
// in TMEM then, which is rare); Stats = ln2 * (m + log2(l)) is exact whichever reference m is
// in use. Causal graphs skip tiles above the diagonal and mask inside the diagonal tile.
// Scores are scaled after the f32 dot product, invalid positions are -inf, as in the reference's
// emit_sdpa_forward (lib/Compiler/SequenceGraph.cpp:2135-2341).
#include "umma_ptx.cuh"

namespace dfgpu {
namespace {

constexpr int kRows = 128;      // query rows per CTA
constexpr int kKeys = 128;      // keys per tile
constexpr int kHeadDim = 128;
constexpr int kTileBytes = kRows * kHeadDim * 2;  // 32 KiB: one Q / K / V / P tile (two 64-column halves)
constexpr int kHalfBytes = kTileBytes / 2;
constexpr int kSlots = 3;       // K/V ring
constexpr int kSdpaThreads = 192;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct SdpaUmmaArgs {
    int32_t heads_q, heads_kv, seq_q, seq_kv;
    int32_t q_tiles;
    int32_t causal;
    float scale_log2;  // attn_scale * log2(e)
    float* stats;      // [B, Hq, Sq] or null
    int64_t stats_batch_stride, stats_head_stride, stats_row_stride;
    // Max and Sum_exp rows (two-tile kernel only), or null; element strides like Stats
    float* row_max;
    float* row_sum;
    int64_t max_stride[3], sum_stride[3];
    float attn_scale;  // natural-log units: Max = attn_scale * largest dot product
    int32_t batch_heads;  // two-tile kernel: batch * query heads
};

struct Smem {
    static constexpr int kQ = 0;
    static constexpr int kRing = kTileBytes;
    static constexpr int kP = kRing + kSlots * kTileBytes;
    static constexpr int kBarriers = kP + 2 * kTileBytes;
    // q_full, kv_full[3], kv_empty[3], s_full[2], s_empty[2], p_full[2], pv_done[2]
    static constexpr int kBarrierCount = 1 + 2 * kSlots + 8;
    static constexpr int kTotal = kBarriers + kBarrierCount * 8 + 16;
    static constexpr int kDynamic = kTotal + 1024;
};

__device__ __forceinline__ void tmem_store_32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_store_16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(kSdpaThreads, 1)
sdpa_umma_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o, SdpaUmmaArgs args) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + Smem::kBarriers;
    const uint32_t q_full = bar_base;
    auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
    auto kv_empty = [&](int s) { return bar_base + 8u * (1 + kSlots + s); };
    auto s_full = [&](int b) { return bar_base + 8u * (1 + 2 * kSlots + b); };
    auto s_empty = [&](int b) { return bar_base + 8u * (3 + 2 * kSlots + b); };
    auto p_full = [&](int b) { return bar_base + 8u * (5 + 2 * kSlots + b); };
    auto pv_done = [&](int b) { return bar_base + 8u * (7 + 2 * kSlots + b); };
    const uint32_t tmem_slot = bar_base + 8u * Smem::kBarrierCount;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(generic_base + Smem::kBarriers + 8 * Smem::kBarrierCount);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // heavy (late) causal tiles first
    const int q_tile = args.q_tiles - 1 - static_cast<int>(blockIdx.x);
    const int bh = blockIdx.y;
    const int batch = bh / args.heads_q, head = bh - batch * args.heads_q;
    const int kv_head = head / (args.heads_q / args.heads_kv);
    const int q_row0 = (batch * args.heads_q + head) * args.seq_q + q_tile * kRows;
    const int kv_row0 = (batch * args.heads_kv + kv_head) * args.seq_kv;
    const int total_kv_tiles = args.seq_kv / kKeys;
    const int kv_tiles = args.causal ? min(total_kv_tiles, q_tile + 1) : total_kv_tiles;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kSlots; ++s) {
            mbar_init(kv_full(s), 1);
            mbar_init(kv_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(s_full(b), 1);
            mbar_init(s_empty(b), 4);
            mbar_init(p_full(b), 4);
            mbar_init(pv_done(b), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    const uint32_t tmem_o = tmem_base + 256;  // S0 at +0, S1 at +128, O at +256

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(q_full, kTileBytes);
            tma_load_2d(smem_base + Smem::kQ, &map_q, 0, q_row0, q_full);
            tma_load_2d(smem_base + Smem::kQ + kHalfBytes, &map_q, 64, q_row0, q_full);
            for (int t = 0; t < 2 * kv_tiles; ++t) {
                const int slot = t % kSlots;
                if (!mbar_wait(kv_empty(slot), ((t / kSlots) & 1) ^ 1, 201)) break;
                const CUtensorMap* map = (t & 1) ? &map_v : &map_k;
                const int row = kv_row0 + (t >> 1) * kKeys;
                const uint32_t dst = smem_base + Smem::kRing + slot * kTileBytes;
                mbar_expect_tx(kv_full(slot), kTileBytes);
                tma_load_2d(dst, map, 0, row, kv_full(slot));
                tma_load_2d(dst + kHalfBytes, map, 64, row, kv_full(slot));
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // D f32, A/B bf16, M = 128, N = 128; the second product reads V as an MN-major B operand
            const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kKeys >> 3) << 17) | (static_cast<uint32_t>(kRows >> 4) << 24);
            const uint32_t idesc_pv = idesc_qk | (1u << 16);
            const uint32_t q_smem = smem_base + Smem::kQ;
            bool ok = mbar_wait(q_full, 0, 202);
            auto issue_scores = [&](int j) {
                const int t = 2 * j, slot = t % kSlots, b = j & 1;
                if (ok) ok = mbar_wait(kv_full(slot), (t / kSlots) & 1, 203);
                if (ok) ok = mbar_wait(s_empty(b), ((j >> 1) & 1) ^ 1, 204);
                tc_fence_after();
                if (ok) {
                    const uint32_t q_lo = smem_desc_lo(q_smem, 16), k_lo = smem_desc_lo(smem_base + Smem::kRing + slot * kTileBytes, 16);
#pragma unroll
                    for (int k = 0; k < kHeadDim / 16; ++k) {
                        const uint32_t offset = ((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;
                        umma_bf16(tmem_base + b * 128, desc_words(q_lo + offset, smem_desc_hi(1024)), desc_words(k_lo + offset, smem_desc_hi(1024)), idesc_qk, k != 0 ? 1u : 0u);
                    }
                }
                umma_commit(kv_empty(slot));
                umma_commit(s_full(b));
            };
            issue_scores(0);
            for (int j = 0; j < kv_tiles; ++j) {
                if (j + 1 < kv_tiles) issue_scores(j + 1);
                const int t = 2 * j + 1, slot = t % kSlots, b = j & 1;
                if (ok) ok = mbar_wait(p_full(b), (j >> 1) & 1, 205);
                if (ok) ok = mbar_wait(kv_full(slot), (t / kSlots) & 1, 206);
                tc_fence_after();
                if (ok) {
                    const uint32_t p_lo = smem_desc_lo(smem_base + Smem::kP + b * kTileBytes, 16);
                    const uint32_t v_lo = smem_desc_lo(smem_base + Smem::kRing + slot * kTileBytes, kHalfBytes);
#pragma unroll
                    for (int k = 0; k < kKeys / 16; ++k)
                        umma_bf16(tmem_o, desc_words(p_lo + (((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4), smem_desc_hi(1024)),
                                  desc_words(v_lo + ((k * 2048) >> 4), smem_desc_hi(1024)), idesc_pv, (j | k) != 0 ? 1u : 0u);
                }
                umma_commit(kv_empty(slot));
                umma_commit(pv_done(b));
            }
        }
    } else {
        const int quadrant = warp & 3;
        const int row = quadrant * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quadrant * 32) << 16;
        const int q_index = q_tile * kRows + row;  // query position inside the sequence
        float m_ref = -INFINITY;  // reference maximum (scaled, log2 domain)
        float l_sum = 0.0f;
        bool ok = true;
        for (int j = 0; j < kv_tiles; ++j) {
            const int b = j & 1;
            if (ok) ok = mbar_wait(s_full(b), (j >> 1) & 1, 207);
            tc_fence_after();
            float s[128];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t raw[32];
                tmem_load_32(tmem_base + lane_base + b * 128 + c * 32, raw);
                tmem_load_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) s[c * 32 + e] = __uint_as_float(raw[e]) * args.scale_log2;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty(b));
            if (args.causal && j == q_tile) {
                const int limit = q_index - j * kKeys;  // keys 0..limit of this tile are visible
#pragma unroll
                for (int e = 0; e < 128; ++e)
                    if (e > limit) s[e] = -INFINITY;
            }
            float tile_max = s[0];
#pragma unroll
            for (int e = 1; e < 128; ++e) tile_max = fmaxf(tile_max, s[e]);
            // raise the reference only when it would grow by more than the threshold (or on the first tile)
            const bool raise = tile_max > m_ref + kRescaleThreshold;
            const bool any_raise = __any_sync(0xffffffffu, raise) != 0;
            if (any_raise) {
                const float m_new = fmaxf(m_ref, tile_max);
                const float alpha = m_ref == -INFINITY ? 0.0f : exp2f(m_ref - m_new);
                l_sum *= alpha;
                m_ref = m_new;
                if (j > 0) {
                    // the accumulator holds P V up to tile j-1: wait for that product, then rescale it in TMEM
                    if (ok) ok = mbar_wait(pv_done((j - 1) & 1), ((j - 1) >> 1) & 1, 208);
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < 4; ++c) {
                        uint32_t raw[32];
                        tmem_load_32(tmem_o + lane_base + c * 32, raw);
                        tmem_load_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) raw[e] = __float_as_uint(__uint_as_float(raw[e]) * alpha);
                        tmem_store_32(tmem_o + lane_base + c * 32, raw);
                    }
                    tmem_store_wait();
                    tc_fence_before();
                }
            }
            // P buffer b was last read by the product of tile j-2
            if (ok) ok = mbar_wait(pv_done(b), ((j >> 1) & 1) ^ 1, 209);
            uint8_t* p_row = generic_base + Smem::kP + b * kTileBytes + row * 128;
            float tile_sum = 0.0f;
#pragma unroll
            for (int c = 0; c < 16; ++c) {  // 16-byte units: 8 keys each
                uint32_t w[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const float p0 = exp2f(s[c * 8 + 2 * t] - m_ref);
                    const float p1 = exp2f(s[c * 8 + 2 * t + 1] - m_ref);
                    tile_sum += p0 + p1;
                    __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
                    w[t] = *reinterpret_cast<uint32_t*>(&pair);
                }
                const int half = c >> 3, unit = c & 7;
                *reinterpret_cast<uint4*>(p_row + half * kHalfBytes + ((unit ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            l_sum += tile_sum;
            fence_async_shared();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(b));
        }
        // last product done -> normalise, store O through shared memory and the TMA unit
        const int last = kv_tiles - 1;
        if (ok) ok = mbar_wait(pv_done(last & 1), (last >> 1) & 1, 210);
        tc_fence_after();
        const float inverse = l_sum > 0.0f ? 1.0f / l_sum : 0.0f;
        uint8_t* o_row = generic_base + Smem::kP + row * 128;  // P buffer 0 doubles as the output staging tile
        // P buffer 0 may still be the operand of the last product only if last is even: that product is done (waited above)
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            uint32_t raw[32];
            tmem_load_32(tmem_o + lane_base + c * 32, raw);
            tmem_load_wait();
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                uint32_t w[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    __nv_bfloat162 pair = __floats2bfloat162_rn(__uint_as_float(raw[u * 8 + 2 * t]) * inverse, __uint_as_float(raw[u * 8 + 2 * t + 1]) * inverse);
                    w[t] = *reinterpret_cast<uint32_t*>(&pair);
                }
                const int unit16 = c * 4 + u;  // 16-byte unit inside the 256-byte output row
                const int half = unit16 >> 3, unit = unit16 & 7;
                *reinterpret_cast<uint4*>(o_row + half * kHalfBytes + ((unit ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        if (args.stats != nullptr && ok)
            args.stats[batch * args.stats_batch_stride + head * args.stats_head_stride + static_cast<int64_t>(q_index) * args.stats_row_stride] =
                l_sum > 0.0f ? 0.6931471805599453f * (m_ref + log2f(l_sum)) : -INFINITY;
        tc_fence_before();
        fence_async_shared();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
            if (ok && g_device_status == 0) {
                tma_store_2d(&map_o, smem_base + Smem::kP, 0, q_row0);
                tma_store_2d(&map_o, smem_base + Smem::kP + kHalfBytes, 64, q_row0);
            }
            tma_store_commit();
            tma_store_wait_all();
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- two query tiles per CTA ------------------------------------------------------
// The softmax of one tile costs about as many cycles as its two products, so a CTA that owns two
// 128-row query tiles (A and B) lets the tensor pipe work on one while the other is in its softmax:
//   warp 16     TMA: Q_A, Q_B once, then K_0, V_0, K_1, ... into a ring of 32 KiB slots
//   warp 17     one lane issues, per key tile j:  O_A += P_A(j) V_j ; S_A(j+1) = Q_A K_{j+1}^T ;
//                                                 O_B += P_B(j) V_j ; S_B(j+1) = Q_B K_{j+1}^T
//   warps 0-7   softmax of tile A, warps 8-15 softmax of tile B (four whole warpgroups, which take the registers the
//               loader and issuing warps give up): two threads per query row, each with 64 of the
//               tile's 128 keys (the two warps that share a lane quarter trade row maxima through shared memory)
// TMEM: S_A at +0, S_B at +128, O_A at +256, O_B at +384. P never goes through shared memory: each
// thread overwrites the front of its own score row with the bf16 probabilities (two per 32-bit
// column) and the second product takes its A operand from tensor memory. The tensor pipe runs the
// products of one CTA in issue order, so S_X(j+1) may be issued right behind the product that reads P_X(j).
// Under a causal mask tile A (the earlier rows) has one key tile fewer than tile B.

constexpr int kPairSlots = 4;
constexpr int kPolyEvery = 4;  // one pair of exponentials in kPolyEvery goes to the FMA pipe (0: none)
constexpr int kPairThreads = 608;  // 2 x 8 softmax warps (two threads per query row), loader, issuer and output-store warps

struct PairSmem {
    static constexpr int kQ = 0;                       // Q_A, Q_B
    static constexpr int kRing = 2 * kTileBytes;
    static constexpr int kStage = kRing + kPairSlots * kTileBytes;  // one output tile on its way to global memory
    // 128 bytes per (tile, lane quarter): during the key loop the half-row maxima [half][lane] as bf16, after it the row sum
    // [lane] as f32. 1 KiB in all: with two Q tiles, four 32 KiB ring slots and the output tile this is what the 227 KiB leave.
    static constexpr int kExchange = kStage + kTileBytes;
    static constexpr int kBarriers = kExchange + 1024;
    // stage_free, q_full[2], q_empty[2], kv_full[S], kv_empty[S], s_full[2], p_full[2], o_full[2], o_empty[2], staged[2]
    static constexpr int kBarrierCount = 5 + 2 * kPairSlots + 10;
    static constexpr int kTotal = kBarriers + kBarrierCount * 8 + 16;
    static constexpr int kDynamic = kTotal + 1024;
};

// D[tmem] (+)= A[tmem] * B[smem]: the A operand (bf16 pairs, one row per lane) is read from tensor memory.
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Packed pairs of f32 (one 64-bit register): Blackwell's FMA pipe takes two lanes per instruction, which
// halves the instruction count of the scale-and-subtract and of the row sums in the softmax loop.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
    return v;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// 2^x on the FMA and integer pipes: round x to the nearest integer n with the 1.5 * 2^23 trick, evaluate a
// cubic for 2^(x - n) on [-0.5, 0.5] (relative error 7.5e-5, far below the bf16 rounding of P) and add n
// to the exponent field. The special-function unit runs 16 ex2 per clock per SM: 1024 cycles for a 128 x 128
// score tile, as long as its two tensor-core products take, so part of the exponentials go this way.
__device__ __forceinline__ float exp2_poly(float x) {
    x = fmaxf(x, -125.0f);  // masked scores (-inf) end as 2^-125: nothing in a sum that holds a term >= 2^-8
    const float magic = 12582912.0f;
    const float t = x + magic;
    const float f = x - (t - magic);
    const float p = fmaf(fmaf(fmaf(0.0551716685f, f, 0.2426111251f), f, 0.6932609677f), f, 0.9999280572f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}

// The same on a packed pair: the range reduction and the cubic run as f32x2 instructions (6 per pair), only the clamp
// and the exponent insertion are per element.
__device__ __forceinline__ void exp2_poly_pair(uint64_t x2, float& p0, float& p1) {
    float x0, x1;
    unpack2(x2, x0, x1);
    x2 = pack2(fmaxf(x0, -125.0f), fmaxf(x1, -125.0f));
    const uint64_t magic2 = pack2(12582912.0f, 12582912.0f);
    const uint64_t t2 = add2(x2, magic2);
    const uint64_t n2 = add2(t2, pack2(-12582912.0f, -12582912.0f));
    const uint64_t f2 = fma2(n2, pack2(-1.0f, -1.0f), x2);
    uint64_t q2 = fma2(pack2(0.0551716685f, 0.0551716685f), f2, pack2(0.2426111251f, 0.2426111251f));
    q2 = fma2(q2, f2, pack2(0.6932609677f, 0.6932609677f));
    q2 = fma2(q2, f2, pack2(0.9999280572f, 0.9999280572f));
    float q0, q1, t0, t1;
    unpack2(q2, q0, q1);
    unpack2(t2, t0, t1);
    p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
    p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
}

__device__ __forceinline__ void tmem_load_16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
// Wait for the tensor-memory loads in flight. The registers of the load that is about to be used pass through the
// statement, so that nothing that reads them can be scheduled above the wait while a later load is already in flight.
__device__ __forceinline__ void tmem_load_wait_for(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :: "memory");
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// Largest of 16 scores folded into `running`: eight three-input maxima.
__device__ __forceinline__ float max_of_16(const uint32_t (&raw)[16], float running) {
    float part[4];
#pragma unroll
    for (int g = 0; g < 4; ++g)
        part[g] = max3(__uint_as_float(raw[4 * g]), __uint_as_float(raw[4 * g + 1]), max3(__uint_as_float(raw[4 * g + 2]), __uint_as_float(raw[4 * g + 3]), running));
    return fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
}
// Sixteen scores -> probabilities 2^(s * scale + bias) as eight bf16 pairs, their sum added to two packed partial sums.
__device__ __forceinline__ void probabilities_of_16(const uint32_t (&raw)[16], uint64_t scale2, uint64_t bias2, uint64_t (&sums)[2], uint32_t* packed) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const uint64_t v = fma2(pack2(__uint_as_float(raw[2 * e]), __uint_as_float(raw[2 * e + 1])), scale2, bias2);
        float p0, p1;
        if (kPolyEvery > 0 && e % (kPolyEvery > 0 ? kPolyEvery : 1) == 0) {
            exp2_poly_pair(v, p0, p1);  // this pair on the FMA pipe
        } else {
            float x0, x1;
            unpack2(v, x0, x1);
            p0 = ex2_fast(x0);
            p1 = ex2_fast(x1);
        }
        sums[e & 1] = add2(sums[e & 1], pack2(p0, p1));
        __nv_bfloat162 two = __floats2bfloat162_rn(p0, p1);
        packed[e] = *reinterpret_cast<uint32_t*>(&two);
    }
}

// One (batch, head, query pair) of the two-tile kernel's work list.
struct PairItem {
    int batch, head;
    int q_tile_a;        // index of the first of the two 128-row query tiles
    int q_row_a;         // its first row in the [B * Hq * Sq, D] view of Q and O
    int kv_row0;         // first row of this head in the [B * Hkv * Skv, D] view of K and V
    int tiles_a, tiles_b;  // key tiles the two query tiles walk (causal: up to their diagonals)
};

__device__ __forceinline__ PairItem pair_item(const SdpaUmmaArgs& args, int bh, int pair) {
    PairItem item;
    item.batch = bh / args.heads_q;
    item.head = bh - item.batch * args.heads_q;
    const int kv_head = item.head / (args.heads_q / args.heads_kv);
    item.q_tile_a = 2 * pair;
    item.q_row_a = bh * args.seq_q + item.q_tile_a * kRows;
    item.kv_row0 = (item.batch * args.heads_kv + kv_head) * args.seq_kv;
    const int total_kv_tiles = args.seq_kv / kKeys;
    item.tiles_a = args.causal ? min(total_kv_tiles, item.q_tile_a + 1) : total_kv_tiles;
    item.tiles_b = args.causal ? min(total_kv_tiles, item.q_tile_a + 2) : total_kv_tiles;
    return item;
}

// The work list of one CTA, the same in every warp role. A head's P query pairs form units: under a causal mask unit i
// is the heavy pair P-1-i followed by the light pair i, so that every unit walks 2P+2 key tiles and equal numbers of
// units are equal work; otherwise each pair is a unit. CTA c takes units c, c + gridDim.x, ...; neighbouring CTAs
// thus work on the same head at the same time and share its K and V in L2. `body(bh, pair)` returns false to stop.
struct PairWalker {
    int k = 0;
    __device__ __forceinline__ bool next(const SdpaUmmaArgs& args, int& bh, int& pair) {
        const int pairs = args.q_tiles >> 1;
        const int units_per_head = args.causal ? (pairs + 1) >> 1 : pairs;
        const int units = units_per_head * args.batch_heads;
        for (;; ++k) {
            const int unit = static_cast<int>(blockIdx.x) + (k >> 1) * static_cast<int>(gridDim.x);
            if (unit >= units) return false;
            bh = unit / units_per_head;
            const int i = unit - bh * units_per_head;
            pair = i;
            if (args.causal) {
                pair = (k & 1) ? i : pairs - 1 - i;
                if ((k & 1) && 2 * i == pairs - 1) continue;  // the middle pair of an odd count stands alone
            } else if (k & 1) {
                continue;
            }
            ++k;
            return true;
        }
    }
};
template <class Body>
__device__ __forceinline__ void for_each_pair_item(const SdpaUmmaArgs& args, Body&& body) {
    PairWalker walker;
    int bh, pair;
    while (walker.next(args, bh, pair))  // one call site of the body: it is a whole warp role
        if (!body(bh, pair)) return;
}

// Persistent form: one CTA per SM walks its work list, and the prologue of an item (Q and the first K/V tiles, the
// first score products) runs under the tail of the previous one. 19 warps:
//   warps 0-15  softmax, two threads per query row (8 warps per query tile); they also normalise O into a staging tile
//   warp 16     TMA producer: Q_A and Q_B of an item as soon as the previous item's last score product has read the
//               old ones, then K_0, V_0, K_1, ... through a ring of 32 KiB slots that runs on across items
//   warp 17     issues the products; one elected lane issues, all lanes walk the schedule
//   warp 18     sends staged output tiles to global memory by TMA (row-per-thread global stores of 16 bytes at a
//               256-byte stride kept the load/store unit busy for ~5000 cycles per tile)
__global__ void __launch_bounds__(kPairThreads, 1)
sdpa_umma_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o, SdpaUmmaArgs args) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + PairSmem::kBarriers;
    const uint32_t stage_free = bar_base;
    auto q_full = [&](int x) { return bar_base + 8u * (1 + x); };
    auto q_empty = [&](int x) { return bar_base + 8u * (3 + x); };
    auto kv_full = [&](int s) { return bar_base + 8u * (5 + s); };
    auto kv_empty = [&](int s) { return bar_base + 8u * (5 + kPairSlots + s); };
    auto s_full = [&](int x) { return bar_base + 8u * (5 + 2 * kPairSlots + x); };
    auto p_full = [&](int x) { return bar_base + 8u * (7 + 2 * kPairSlots + x); };
    auto o_full = [&](int x) { return bar_base + 8u * (9 + 2 * kPairSlots + x); };
    auto o_empty = [&](int x) { return bar_base + 8u * (11 + 2 * kPairSlots + x); };
    auto staged = [&](int x) { return bar_base + 8u * (13 + 2 * kPairSlots + x); };
    const uint32_t tmem_slot = bar_base + 8u * PairSmem::kBarrierCount;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(generic_base + PairSmem::kBarriers + 8 * PairSmem::kBarrierCount);

    const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
        prefetch_tensormap(&map_o);
        mbar_init(stage_free, 1);
        for (int s = 0; s < kPairSlots; ++s) {
            mbar_init(kv_full(s), 1);
            mbar_init(kv_empty(s), 1);
        }
        for (int x = 0; x < 2; ++x) {
            mbar_init(s_full(x), 1);
            mbar_init(p_full(x), 8);
            mbar_init(o_full(x), 1);
            mbar_init(q_full(x), 1);
            mbar_init(q_empty(x), 1);
            mbar_init(o_empty(x), 8);
            mbar_init(staged(x), 8);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 17) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;

    if (warp == 16) {
        const bool leader = elect_one();
        int slot = 0;
        uint32_t phase = 1;  // parity of the "slot is free" wait
        uint32_t n = 0;      // items started
        for_each_pair_item(args, [&](int bh, int pair) {
            const PairItem item = pair_item(args, bh, pair);
            // a Q buffer is free once the previous item's last score product of that query tile has completed; tile A's
            // (which under a causal mask ends a key tile earlier) and the first K tile go first, so that the issuing warp
            // can start this item's tile A under the previous item's last round
            auto load_q = [&](int x) {
                if (!mbar_wait_warp(q_empty(x), (n & 1) ^ 1, 220 + x)) return false;
                if (leader) {
                    mbar_expect_tx(q_full(x), kTileBytes);
                    tma_load_2d(smem_base + PairSmem::kQ + x * kTileBytes, &map_q, 0, item.q_row_a + x * kRows, q_full(x));
                    tma_load_2d(smem_base + PairSmem::kQ + x * kTileBytes + kHalfBytes, &map_q, 64, item.q_row_a + x * kRows, q_full(x));
                }
                return true;
            };
            if (!load_q(0)) return false;
            for (int t = 0; t < 2 * item.tiles_b; ++t) {
                if (t == 1 && !load_q(1)) return false;
                if (!mbar_wait_warp(kv_empty(slot), phase, 215)) return false;
                const int row = item.kv_row0 + (t >> 1) * kKeys;
                const uint32_t dst = smem_base + PairSmem::kRing + slot * kTileBytes;
                if (leader) {
                    const CUtensorMap* map = (t & 1) ? &map_v : &map_k;
                    mbar_expect_tx(kv_full(slot), kTileBytes);
                    tma_load_2d(dst, map, 0, row, kv_full(slot));
                    tma_load_2d(dst + kHalfBytes, map, 64, row, kv_full(slot));
                }
                if (++slot == kPairSlots) { slot = 0; phase ^= 1; }
            }
            ++n;
            return true;
        });
    } else if (warp == 17) {
        // All 32 lanes walk the schedule; the elected lane issues the products and their commits.
        const bool leader = elect_one();
        const uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kKeys >> 3) << 17) | (static_cast<uint32_t>(kRows >> 4) << 24);
        const uint32_t idesc_pv = idesc_qk | (1u << 16);  // B = V read MN-major
        const uint32_t tmem_u = __shfl_sync(0xffffffffu, tmem_base, 0);
        bool ok = true;
        int slot = 0;         // ring slot of the next K or V tile to consume
        uint32_t phase = 0;
        uint32_t n = 0;       // items started
        uint32_t p_count[2] = {0, 0};  // probability tiles consumed per query tile (parity of p_full)
        // (no tcgen05 fence after a slot wait: the slot was filled by TMA, not by tensor-memory traffic of other threads)
        auto wait_slot = [&](int code) {
            if (ok) ok = mbar_wait_warp(kv_full(slot), phase, code);
        };
        auto next_slot = [&]() { if (++slot == kPairSlots) { slot = 0; phase ^= 1; } };
        auto commit = [&](uint32_t bar) { if (leader) umma_commit(bar); };
        constexpr uint32_t kDescHi = smem_desc_hi(1024);
        auto scores = [&](int x, int k_slot) {  // S_x = Q_x K^T
            if (!ok) return;
            const uint32_t q_lo = smem_desc_lo(smem_base + PairSmem::kQ + x * kTileBytes, 16);
            const uint32_t k_lo = smem_desc_lo(smem_base + PairSmem::kRing + k_slot * kTileBytes, 16);
            const uint32_t d_tmem = tmem_u + x * 128;
            if (leader) {
#pragma unroll
                for (int k = 0; k < kHeadDim / 16; ++k) {
                    const uint32_t offset = ((k >> 2) * kHalfBytes + (k & 3) * 32) >> 4;  // in 16-byte units
                    umma_bf16(d_tmem, desc_words(q_lo + offset, kDescHi), desc_words(k_lo + offset, kDescHi), idesc_qk, k != 0 ? 1u : 0u);
                }
            }
        };
        // O_x += P_x V_j. P_x lies as bf16 pairs over the scores: keys 0..63 in columns 0..31 of S_x, keys 64..127 in columns
        // 64..95 (each softmax thread overwrites columns that held its own scores only). The first product of an item
        // overwrites O_x, which the softmax warps must have read out for the previous item.
        auto product = [&](int x, int j, int v_slot) {
            if (ok && j == 0) ok = mbar_wait_warp(o_empty(x), (n & 1) ^ 1, 218 + x);
            if (ok) ok = mbar_wait_warp(p_full(x), p_count[x] & 1, 223 + x);
            ++p_count[x];
            tc_fence_after();
            if (!ok) return;
            const uint32_t v_lo = smem_desc_lo(smem_base + PairSmem::kRing + v_slot * kTileBytes, kHalfBytes);
            const uint32_t d_tmem = tmem_u + 256 + x * 128, p_tmem = tmem_u + x * 128;
            if (leader) {
#pragma unroll
                for (int k = 0; k < kKeys / 16; ++k)
                    umma_bf16_a_tmem(d_tmem, p_tmem + (k >> 2) * 64 + (k & 3) * 8, desc_words(v_lo + ((k * 2048) >> 4), kDescHi), idesc_pv, (j | k) != 0 ? 1u : 0u);
            }
        };
        PairWalker walker;
        int bh = 0, pair = 0, next_bh = 0, next_pair = 0;
        bool have = walker.next(args, bh, pair);
        bool early = false;  // S_A of the current item was issued in the previous item's last round
        int early_slot = 0;  // the ring slot of its K tile
        while (have && ok) {
            const PairItem item = pair_item(args, bh, pair);
            const int tiles_a = item.tiles_a, tiles_b = item.tiles_b;
            const bool have_next = walker.next(args, next_bh, next_pair);
            const int next_tiles_a = have_next ? pair_item(args, next_bh, next_pair).tiles_a : 0;
            int k0_slot = early_slot;
            if (!early) {
                if (ok) ok = mbar_wait_warp(q_full(0), n & 1, 222);
                wait_slot(225);
                k0_slot = slot;
                next_slot();
                scores(0, k0_slot);
                commit(s_full(0));
                if (tiles_a == 1) commit(q_empty(0));
            }
            early = false;
            if (ok) ok = mbar_wait_warp(q_full(1), n & 1, 214);
            scores(1, k0_slot);
            commit(s_full(1));
            commit(kv_empty(k0_slot));
            if (tiles_b == 1) commit(q_empty(1));
            for (int j = 0; j < tiles_b; ++j) {
                wait_slot(226);
                const int v_slot = slot;
                next_slot();
                if (j < tiles_a) {
                    product(0, j, v_slot);
                    if (j == tiles_a - 1) commit(o_full(0));
                } else if (have_next && ok && j == tiles_b - 1) {
                    // Tile A has no key tile in this item's last round (causal mask): if the next item's Q_A and first K
                    // tile have landed, its first scores go out now and its softmax runs under tile B's last round.
                    const bool landed = __all_sync(0xffffffffu, mbar_test_wait(q_full(0), (n + 1) & 1)) && __all_sync(0xffffffffu, mbar_test_wait(kv_full(slot), phase));
                    if (landed) {
                        early = true;
                        early_slot = slot;
                        next_slot();
                        scores(0, early_slot);
                        commit(s_full(0));
                        if (next_tiles_a == 1) commit(q_empty(0));
                    }
                }
                const bool more = j + 1 < tiles_b;
                int k_slot = 0;
                if (more) {
                    wait_slot(227);
                    k_slot = slot;
                    next_slot();
                }
                if (j + 1 < tiles_a) {
                    scores(0, k_slot);
                    commit(s_full(0));
                    if (j + 2 == tiles_a) commit(q_empty(0));  // the item's last read of Q_A
                }
                product(1, j, v_slot);
                commit(kv_empty(v_slot));
                if (more) {
                    scores(1, k_slot);
                    commit(s_full(1));
                    commit(kv_empty(k_slot));
                    if (j + 2 == tiles_b) commit(q_empty(1));  // the item's last read of Q_B
                }
            }
            commit(o_full(1));
            ++n;
            bh = next_bh;
            pair = next_pair;
            have = have_next;
        }
    } else if (warp == 18) {
        // Output stores: a query tile's softmax warps leave the normalised tile in the staging buffer; this warp sends it
        // off and hands the buffer to the next tile once the copy engine has read it.
        const bool leader = elect_one();
        uint32_t n = 0;
        bool ok = true;
        for_each_pair_item(args, [&](int bh, int pair) {
            const PairItem item = pair_item(args, bh, pair);
            for (int x = 0; x < 2; ++x) {
                if (ok) ok = mbar_wait_warp(staged(x), n & 1, 216 + x);
                if (leader) {
                    if (ok && g_device_status == 0) {
                        tma_store_2d(&map_o, smem_base + PairSmem::kStage, 0, item.q_row_a + x * kRows);
                        tma_store_2d(&map_o, smem_base + PairSmem::kStage + kHalfBytes, 64, item.q_row_a + x * kRows);
                    }
                    tma_store_commit();
                    tma_store_wait_read<0>();
                    mbar_arrive(stage_free);
                }
                __syncwarp();
            }
            ++n;
            return true;
        });
        if (leader) tma_store_wait_all();
    } else {
        const int sw = warp;
        const int x = sw >> 3;           // 0: tile A, 1: tile B
        const int half = (sw >> 2) & 1;  // which 64 of the tile's 128 keys (and of the 128 output columns) this thread owns
        const int quadrant = warp & 3;   // tensor-memory lane quarter of this warp; warps w and w + 4 share it
        const int row = quadrant * 32 + lane;
        const uint32_t lane_base = static_cast<uint32_t>(quadrant * 32) << 16;
        const uint32_t tmem_s = tmem_base + lane_base + x * 128;
        const uint32_t tmem_o = tmem_base + lane_base + 256 + x * 128 + half * 64;
        const float scale = args.scale_log2;
        const int pair_barrier = 1 + x * 4 + quadrant;  // the 64 threads that share these 32 rows
        uint16_t* exchange = reinterpret_cast<uint16_t*>(generic_base + PairSmem::kExchange) + ((x * 4 + quadrant) * 2) * 32;  // [half][lane]
        float* sum_exchange = reinterpret_cast<float*>(generic_base + PairSmem::kExchange) + (x * 4 + quadrant) * 32;
        const bool stamp = blockIdx.x == 0 && (threadIdx.x & 255) == 0;
        (void)stamp;
        uint32_t n = 0;        // items started
        uint32_t s_count = 0;  // score tiles consumed (parity of s_full)
        bool ok = true;
        for_each_pair_item(args, [&](int bh, int pair) {
        const PairItem item = pair_item(args, bh, pair);
        const int q_tile = item.q_tile_a + x;
        const int q_index = q_tile * kRows + row;
        const int my_tiles = x ? item.tiles_b : item.tiles_a;
        float m_ref = -INFINITY;  // reference maximum, scaled, log2 domain (identical in both threads of a row)
        float l_sum = 0.0f;       // this thread's half of the row sum
        float raw_max = -INFINITY;  // exact largest dot product among this thread's keys (for the Max / Sum_exp outputs)
        for (int j = 0; j < my_tiles; ++j, ++s_count) {
            if (ok) ok = mbar_wait(s_full(x), s_count & 1, 228 + x);
            tc_fence_after();
            // One pass over this thread's 64 scores, 16 at a time with the next load in flight: each chunk gives its part
            // of the half-row maximum and, from the second key tile on, its probabilities against the reference maximum
            // of the earlier tiles. Only a tile that raises the reference (rare after the first) is read a second time.
            const bool diagonal = args.causal && j == q_tile;
            const int limit = q_index - j * kKeys - half * 64;  // diagonal tile: keys 0..limit of this thread's 64 are visible
            const bool speculative = j > 0;
            const uint64_t scale2 = pack2(scale, scale);
            uint64_t bias2 = pack2(-m_ref, -m_ref);
            uint64_t sums[2] = {0, 0};  // two independent chains of packed partial sums
            uint32_t packed[32];        // this thread's 64 probabilities as bf16 pairs
            float mine = -INFINITY;
            {
                uint32_t raw[4][16];
                tmem_load_16(tmem_s + half * 64, raw[0]);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    tmem_load_wait_for(raw[c]);
                    if (c < 3) tmem_load_16(tmem_s + half * 64 + (c + 1) * 16, raw[c + 1]);
                    if (diagonal) {
#pragma unroll
                        for (int e = 0; e < 16; ++e)
                            if (c * 16 + e > limit) raw[c][e] = 0xff800000u;  // -inf
                    }
                    mine = max_of_16(raw[c], mine);
                    if (speculative) probabilities_of_16(raw[c], scale2, bias2, sums, packed + c * 8);
                }
            }
            raw_max = fmaxf(raw_max, mine);
            // Trade the half-row maxima with the warp that owns the other 64 keys of these rows, as bf16 rounded towards
            // +inf: any reference not below the true maximum by more than the threshold serves, and both threads must
            // arrive at the same value, so each uses the rounded form of its own half too. (One buffer suffices: the next
            // scores of this tile, which precede the next write, need the probabilities of all eight warps, and a warp
            // hands those over after this read.)
            const uint32_t mine_bits = __float_as_uint(mine);
            const uint32_t mine_up = (mine_bits & 0x80000000u) ? (mine_bits & 0xffff0000u) : ((mine_bits + 0xffffu) & 0xffff0000u);
            exchange[half * 32 + lane] = static_cast<uint16_t>(mine_up >> 16);
            asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
            const float other = __uint_as_float(static_cast<uint32_t>(exchange[(half ^ 1) * 32 + lane]) << 16);
            const float tile_max = fmaxf(__uint_as_float(mine_up), other) * scale;
            // raise the reference only when it would grow by more than the threshold (or on the first tile); the two
            // warps of these rows see the same maxima, so they take the same branches
            const bool raise = tile_max > m_ref + kRescaleThreshold;
            bool again = !speculative;
            if (__any_sync(0xffffffffu, raise)) {
                again = true;
                const float m_new = fmaxf(m_ref, tile_max);
                const float alpha = m_ref == -INFINITY ? 0.0f : ex2_fast(m_ref - m_new);
                l_sum *= alpha;
                m_ref = m_new;
                if (j > 0) {
                    // O_x holds P V up to tile j-1; that product was issued ahead of S_x(j), which has completed.
                    // This thread rescales its 64 columns of the row.
#pragma unroll 1
                    for (int c = 0; c < 2; ++c) {
                        uint32_t acc[32];
                        tmem_load_32(tmem_o + c * 32, acc);
                        tmem_load_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) acc[e] = __float_as_uint(__uint_as_float(acc[e]) * alpha);
                        tmem_store_32(tmem_o + c * 32, acc);
                    }
                }
            }
            if (again) {
                // the scores are still in place (no probabilities stored yet): form them against the new reference
                bias2 = pack2(-m_ref, -m_ref);
#pragma unroll
                for (int g = 0; g < 2; ++g) sums[g] = 0;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t raw[16];
                    tmem_load_16(tmem_s + half * 64 + c * 16, raw);
                    tmem_load_wait_for(raw);
                    if (diagonal) {
#pragma unroll
                        for (int e = 0; e < 16; ++e)
                            if (c * 16 + e > limit) raw[e] = 0xff800000u;
                    }
                    probabilities_of_16(raw, scale2, bias2, sums, packed + c * 8);
                }
            }
            tmem_store_32(tmem_s + half * 64, packed);
            {
                float lo, hi;
                unpack2(add2(sums[0], sums[1]), lo, hi);
                l_sum += lo + hi;
            }
            tmem_store_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(x));
        }
        // last product done -> read O out of tensor memory (which frees it for the next item), normalise, store
        if (ok) ok = mbar_wait(o_full(x), n & 1, 230 + x);
        tc_fence_after();
        // row sum = this thread's half + the other thread's: two hand-overs through one f32 word per row
        if (half == 1) sum_exchange[lane] = l_sum;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
        float total = l_sum;
        if (half == 0) {
            total += sum_exchange[lane];
            sum_exchange[lane] = total;
        }
        asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
        if (half == 1) total = sum_exchange[lane];
        if (args.row_max != nullptr || args.row_sum != nullptr) {
            // exact row maximum: the same two hand-overs with the f32 half-row maxima
            asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
            if (half == 1) sum_exchange[lane] = raw_max;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
            if (half == 0) {
                const float row_raw_max = fmaxf(raw_max, sum_exchange[lane]);
                const int64_t b64 = item.batch, h64 = item.head, q64 = q_index;
                const bool any = total > 0.0f;
                if (ok && args.row_max != nullptr)
                    args.row_max[b64 * args.max_stride[0] + h64 * args.max_stride[1] + q64 * args.max_stride[2]] = any ? row_raw_max * args.attn_scale : -INFINITY;
                if (ok && args.row_sum != nullptr)  // the sum was accumulated against m_ref; re-express it against the true maximum
                    args.row_sum[b64 * args.sum_stride[0] + h64 * args.sum_stride[1] + q64 * args.sum_stride[2]] = any ? total * exp2f(m_ref - row_raw_max * scale) : 0.0f;
            }
        }
        // the hand-over words double as the next item's maxima: every read above must precede those writes
        asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
        const float inverse = total > 0.0f ? 1.0f / total : 0.0f;
        // the staging tile serves the query tiles in turn: A, B, the next item's A, ...
        {
            const uint32_t turn = 2 * n + x;
            if (ok) ok = mbar_wait(stage_free, (turn & 1) ^ 1, 232 + x);
        }
        uint8_t* o_row = generic_base + PairSmem::kStage + half * kHalfBytes + row * 128;  // this thread's 64 output columns
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
            uint32_t acc[32];
            tmem_load_32(tmem_o + c * 32, acc);
            tmem_load_wait();
            if (c == 1) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(o_empty(x));
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                uint32_t w[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    __nv_bfloat162 two = __floats2bfloat162_rn(__uint_as_float(acc[u * 8 + 2 * t]) * inverse, __uint_as_float(acc[u * 8 + 2 * t + 1]) * inverse);
                    w[t] = *reinterpret_cast<uint32_t*>(&two);
                }
                const int unit = c * 4 + u;  // 16-byte unit inside this thread's 128 bytes of the output row
                *reinterpret_cast<uint4*>(o_row + ((unit ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        fence_async_shared();
        __syncwarp();
        if (lane == 0) mbar_arrive(staged(x));
        if (args.stats != nullptr && ok && half == 0)
            args.stats[item.batch * args.stats_batch_stride + item.head * args.stats_head_stride + static_cast<int64_t>(q_index) * args.stats_row_stride] =
                total > 0.0f ? 0.6931471805599453f * (m_ref + log2f(total)) : -INFINITY;
        ++n;
        return true;  // also after a wait gave up: the two warps of a row pair must meet at the same barriers to the end
        });
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 17) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

bool packed_bhsd(const dfgpu_tensor& t) {
    return t.rank == 4 && t.stride[3] == 1 && t.stride[2] == t.dim[3] && t.stride[1] == t.dim[2] * t.dim[3] &&
           t.stride[0] == t.dim[1] * t.dim[2] * t.dim[3];
}

}  // namespace

bool sdpa_umma_supported(const dfgpu_sdpa_params& p) {
    if (p.q.dtype != DFGPU_BF16 || p.k.dtype != DFGPU_BF16 || p.v.dtype != DFGPU_BF16 || p.o.dtype != DFGPU_BF16) return false;
    if (p.q.rank != 4 || p.k.rank != 4 || p.v.rank != 4 || p.o.rank != 4) return false;
    if (p.q.dim[3] != kHeadDim || p.v.dim[3] != kHeadDim || p.k.dim[3] != kHeadDim) return false;
    if (p.page_table_k.rank || p.page_table_v.rank || p.padding_mask || p.has_left_bound || p.bottom_right) return false;
    if ((p.max.rank || p.sum_exp.rank) && (p.q.dim[2] % (2 * kRows) != 0 || !(p.attn_scale > 0.0f) || !(p.attn_scale < INFINITY))) return false;  // only the two-tile kernel writes them
    if ((p.max.rank && p.max.dtype != DFGPU_F32) || (p.sum_exp.rank && p.sum_exp.dtype != DFGPU_F32)) return false;
    if (!packed_bhsd(p.q) || !packed_bhsd(p.k) || !packed_bhsd(p.v) || !packed_bhsd(p.o)) return false;
    const int64_t sq = p.q.dim[2], skv = p.k.dim[2];
    if (p.s_kv != skv || p.v.dim[2] != skv || p.k.dim[1] != p.v.dim[1]) return false;
    if (sq % kRows != 0 || skv % kKeys != 0 || sq < kRows || skv < kKeys) return false;
    if (p.has_right_bound && (p.right_bound != 0 || sq != skv)) return false;  // causal, top-left aligned, square
    if (p.stats.rank && p.stats.dtype != DFGPU_F32) return false;
    const int64_t rows_q = p.q.dim[0] * p.q.dim[1] * sq, rows_kv = p.k.dim[0] * p.k.dim[1] * skv;
    if (rows_q >= (1ll << 31) || rows_kv >= (1ll << 31) || p.q.dim[0] * p.q.dim[1] > 65535) return false;
    return true;
}

int launch_sdpa_umma(const dfgpu_sdpa_params& p, void* const* tensors, void* scratch, cudaStream_t stream) {
    (void)scratch;
    for (int i = 0; i < 4; ++i)
        if ((reinterpret_cast<uintptr_t>(tensors[i]) & 15u) != 0) return fail(kInvalidArgument, "SDPA: the tcgen05 kernel needs 16-byte aligned Q, K, V and O");
    const int64_t batch = p.q.dim[0], hq = p.q.dim[1], hkv = p.k.dim[1], sq = p.q.dim[2], skv = p.k.dim[2];
    CUtensorMap map_q, map_k, map_v, map_o;
    uint32_t box[2] = {64, kRows};
    uint64_t strides[1] = {kHeadDim * 2};
    uint64_t dims_q[2] = {kHeadDim, static_cast<uint64_t>(batch * hq * sq)};
    uint64_t dims_kv[2] = {kHeadDim, static_cast<uint64_t>(batch * hkv * skv)};
    int status = make_map(&map_q, tensors[0], 2, dims_q, strides, box, "SDPA Q");
    if (!status) status = make_map(&map_k, tensors[1], 2, dims_kv, strides, box, "SDPA K");
    if (!status) status = make_map(&map_v, tensors[2], 2, dims_kv, strides, box, "SDPA V");
    if (!status) status = make_map(&map_o, tensors[3], 2, dims_q, strides, box, "SDPA O");
    if (status) return status;
    SdpaUmmaArgs args{};
    args.heads_q = static_cast<int>(hq);
    args.heads_kv = static_cast<int>(hkv);
    args.seq_q = static_cast<int>(sq);
    args.seq_kv = static_cast<int>(skv);
    args.q_tiles = static_cast<int>(sq / kRows);
    args.causal = p.has_right_bound ? 1 : 0;
    args.scale_log2 = p.attn_scale * 1.4426950408889634f;
    args.stats = p.stats.rank ? static_cast<float*>(tensors[4]) : nullptr;
    if (p.stats.rank) {
        args.stats_batch_stride = p.stats.stride[0];
        args.stats_head_stride = p.stats.stride[1];
        args.stats_row_stride = p.stats.stride[2];
    }
    args.attn_scale = p.attn_scale;
    args.row_max = p.max.rank ? static_cast<float*>(tensors[5]) : nullptr;
    args.row_sum = p.sum_exp.rank ? static_cast<float*>(tensors[6]) : nullptr;
    for (int i = 0; i < 3; ++i) {
        args.max_stride[i] = p.max.rank ? p.max.stride[i] : 0;
        args.sum_stride[i] = p.sum_exp.rank ? p.sum_exp.stride[i] : 0;
    }
    const bool pair_form = sq % (2 * kRows) == 0 && p.attn_scale > 0.0f && p.attn_scale < INFINITY;
    static bool configured = false;
    if (!configured) {
        cudaError_t error = cudaFuncSetAttribute(sdpa_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kDynamic);
        if (error == cudaSuccess) error = cudaFuncSetAttribute(sdpa_umma_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::kDynamic);
        if (error != cudaSuccess) return fail(kExecutionFailed, "SDPA: cannot reserve %d bytes of shared memory: %s", PairSmem::kDynamic, cudaGetErrorString(error));
        configured = true;
    }
    if (pair_form) {
        // persistent: one CTA per SM over the work list (see for_each_pair_item)
        static int sm_count = 0;
        if (sm_count == 0) {
            int device = 0;
            if (cudaGetDevice(&device) != cudaSuccess || cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sm_count <= 0) {
                sm_count = 0;
                return fail(kExecutionFailed, "SDPA: cannot read the number of multiprocessors");
            }
        }
        const int pairs = args.q_tiles / 2;
        const int64_t units = static_cast<int64_t>(args.causal ? (pairs + 1) / 2 : pairs) * batch * hq;
        args.batch_heads = static_cast<int>(batch * hq);
        const unsigned grid = static_cast<unsigned>(units < sm_count ? units : sm_count);
        sdpa_umma_pair_kernel<<<grid, kPairThreads, PairSmem::kDynamic, stream>>>(map_q, map_k, map_v, map_o, args);
        return check_launch("SDPA (tcgen05, two query tiles per CTA)");
    }
    dim3 grid(static_cast<unsigned>(args.q_tiles), static_cast<unsigned>(batch * hq));
    sdpa_umma_kernel<<<grid, kSdpaThreads, Smem::kDynamic, stream>>>(map_q, map_k, map_v, map_o, args);
    return check_launch("SDPA (tcgen05)");
}

int sdpa_umma_device_status(int* status) { return read_and_clear_device_status(status); }

}  // namespace dfgpu

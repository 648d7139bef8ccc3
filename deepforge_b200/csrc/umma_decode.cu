// Paged-KV decode attention (one query token per sequence) as a TMA-fed streaming kernel.
//
// The kernel is bandwidth-bound: every valid K and V byte of the pool is read exactly once, in
// whole pages, by the TMA unit straight into swizzled shared memory, many pages in flight per SM.
// The arithmetic is done on the tensor core in TRANSPOSED form so that the tile's 128 keys map to
// the 128 TMEM lanes (one key per softmax thread) and the GQA group's query heads to columns:
//     S^T[key, head] = K_tile[key, :] . Q[head, :]          M = 128 keys,  N = 16, K = 128
//     O^T[d,   head] += V_tile^T[d, key] . P[key, head]     M = 128 (d),   N = 16, K = 128 keys
// One CTA handles one (sequence, KV head) and up to kTilesPerCta key tiles; a second kernel (the
// same merge the CUDA-core decode path uses) combines the per-CTA (max, sum, partial O) triples.
// Two CTAs share an SM (three 32 KiB ring slots each): one CTA's softmax and barrier latencies are
// covered by the other's loads, which measured 1.6x the bandwidth of one CTA with a five-slot ring.
// The page ids of a CTA's 1024 keys are fetched once into shared memory.
// Semantics as the reference (lib/Compiler/SequenceGraph.cpp:1839-1889, 1988-2341): a key is
// valid iff it lies inside the sequence's [lo, hi) window; a page id outside [0, pages) reads as
// zeros (its keys score 0 and add nothing to O) and is never dereferenced.
#include "umma_ptx.cuh"

namespace dfgpu {
namespace {

constexpr int kTileKeys = 128;
constexpr int kDim = 128;
constexpr int kHeadsPadded = 16;              // N of both products (GQA group padded)
constexpr int kTilesPerCta = 8;               // 1024 keys per CTA
constexpr int kKvTileBytes = kTileKeys * kDim * 2;  // 32 KiB
constexpr int kKvHalfBytes = kKvTileBytes / 2;
constexpr int kDecodeThreads = 192;
constexpr int kPartialStride = kDim + 2;      // o[128], max, sum  (layout shared with the merge kernel)
constexpr float kRaiseThreshold = 8.0f;

struct DecodeArgs {
    int32_t heads_q, heads_kv, group;
    int32_t block;            // tokens per page
    int32_t pages_per_tile;   // 128 / block
    int32_t table_len_k, table_len_v;
    int32_t num_pages;
    int32_t max_chunks;
    int32_t has_left, has_right, bottom_right, padding;
    int64_t left, right, s_kv;
    float scale_log2;
    const int32_t* seq_q;
    const int32_t* seq_kv;
    const int32_t* table_k;
    const int32_t* table_v;
    int64_t seq_q_stride, seq_kv_stride, table_k_stride, table_v_stride, table_k_slot_stride, table_v_slot_stride;
    float* partial;
    // compact page tables (null offsets: strided [B,1,P,1]): entry (b, slot) at offsets[b] + slot * slot stride, only
    // the slots the batch's sequence length needs, and none when the prefix failed validation (prefix_ok[0 K | 1 V])
    const void* offsets_k;
    const void* offsets_v;
    int32_t offsets_k_wide, offsets_v_wide;
    int64_t offsets_k_stride, offsets_v_stride;
    const int* prefix_ok;
};

template <int kRingSlots>
struct DecodeSmemT {
    static constexpr int kQ = 0;                                  // [16 heads x 128 d] as two swizzled halves (2 x 2 KiB), padded to 4 KiB
    static constexpr int kP = 4096;                               // two buffers of [16 heads x 128 keys] (2 x 4 KiB)
    static constexpr int kRing = 4096 + 8192;
    static constexpr int kReduce = kRing + kRingSlots * kKvTileBytes;  // cross-warp max exchange: 2 x [4 warps][8 heads] floats
    static constexpr int kPages = kReduce + 512;                  // page ids of this CTA's keys: [K | V][64] int32, -1 = reads as zeros
    static constexpr int kBarriers = kReduce + 1024;
    // q_full, kv_full[S], kv_empty[S], s_full[2], s_empty[2], p_full[2], pv_done[2]
    static constexpr int kBarrierCount = 1 + 2 * kRingSlots + 8;
    static constexpr int kTotal = kBarriers + kBarrierCount * 8 + 16;
    static constexpr int kDynamic = kTotal + 1024;
};

__device__ __forceinline__ void tmem_load_16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_store_16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// Maximum of a float over the warp in one reduction instruction: floats compare like the signed
// integers obtained by flipping the magnitude bits of negative values (a NaN score ends as a NaN output either way).
__device__ __forceinline__ float warp_max_f32(float v) {
    int32_t bits = __float_as_int(v);
    bits ^= (bits >> 31) & 0x7fffffff;
    int32_t top;
    asm volatile("redux.sync.max.s32 %0, %1, 0xffffffff;" : "=r"(top) : "r"(bits));
    top ^= (top >> 31) & 0x7fffffff;
    return __int_as_float(top);
}

// Valid key window [lo, hi) of a sequence for its single query row (q index 0).
__device__ __forceinline__ void key_window(const DecodeArgs& a, int64_t batch, int64_t& lo, int64_t& hi) {
    lo = 0;
    hi = a.s_kv;
    int64_t len_q = 0, len_kv = 0;
    if (a.padding) {
        len_q = a.seq_q[batch * a.seq_q_stride];
        len_kv = a.seq_kv[batch * a.seq_kv_stride];
        if (!(0 < len_q)) { hi = 0; return; }
        if (len_kv < hi) hi = len_kv;
    }
    int64_t shift = 0;
    if (a.bottom_right) shift = a.padding ? len_kv - len_q : a.s_kv - 1;
    if (a.has_right) {
        int64_t bound = shift + a.right + 1;
        if (bound < hi) hi = bound;
    }
    if (a.has_left) {
        int64_t bound = shift - a.left + 1;
        if (bound > lo) lo = bound;
    }
    if (hi < 0) hi = 0;
}

template <int G, int kRingSlots>
__global__ void __launch_bounds__(kDecodeThreads, kRingSlots <= 3 ? 2 : 1)
sdpa_decode_umma_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, DecodeArgs args) {
    using DecodeSmem = DecodeSmemT<kRingSlots>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + DecodeSmem::kBarriers;
    const uint32_t q_full = bar_base;
    auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
    auto kv_empty = [&](int s) { return bar_base + 8u * (1 + kRingSlots + s); };
    auto s_full = [&](int b) { return bar_base + 8u * (1 + 2 * kRingSlots + b); };
    auto s_empty = [&](int b) { return bar_base + 8u * (3 + 2 * kRingSlots + b); };
    auto p_full = [&](int b) { return bar_base + 8u * (5 + 2 * kRingSlots + b); };
    auto pv_done = [&](int b) { return bar_base + 8u * (7 + 2 * kRingSlots + b); };
    const uint32_t tmem_slot = bar_base + 8u * DecodeSmem::kBarrierCount;
    volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(generic_base + DecodeSmem::kBarriers + 8 * DecodeSmem::kBarrierCount);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        prefetch_tensormap(&map_q);
        prefetch_tensormap(&map_k);
        prefetch_tensormap(&map_v);
    }
    const int chunk = blockIdx.x;
    const int kv_head = blockIdx.y;
    const int64_t batch = blockIdx.z;

    int64_t lo, hi;
    key_window(args, batch, lo, hi);
    const int64_t chunk_begin = static_cast<int64_t>(chunk) * kTilesPerCta * kTileKeys;
    const int64_t chunk_end_all = chunk_begin + kTilesPerCta * kTileKeys;
    float* my_partial = args.partial + ((batch * args.heads_q + static_cast<int64_t>(kv_head) * G) * args.max_chunks + chunk) * kPartialStride;
    if (chunk_begin >= hi || chunk_end_all <= lo) {
        if (threadIdx.x < G) {
            float* p = my_partial + static_cast<int64_t>(threadIdx.x) * args.max_chunks * kPartialStride;
            p[kDim] = -INFINITY;
            p[kDim + 1] = 0.0f;
        }
        return;
    }
    // tiles of this CTA that intersect the window
    const int first_tile = lo > chunk_begin ? static_cast<int>((lo - chunk_begin) / kTileKeys) : 0;
    const int64_t last_key = (hi < chunk_end_all ? hi : chunk_end_all) - 1;
    const int tiles = static_cast<int>((last_key - chunk_begin) / kTileKeys) + 1 - first_tile;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kRingSlots; ++s) {
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
    // Page ids of the (at most 64 + 64) table slots this CTA's 1024 keys map to, fetched once and side by side:
    // the loader and the softmax threads then read them from shared memory instead of paying a dependent
    // global load per tile. An id outside the container is stored as -1 (its rows read as zeros).
    int32_t* page_ids = reinterpret_cast<int32_t*>(generic_base + DecodeSmem::kPages);
    if (threadIdx.x < 128) {
        const bool is_v = threadIdx.x >= 64;
        const int entry = threadIdx.x & 63;
        const int64_t table_slot = chunk_begin / args.block + entry;
        int64_t page = -1;
        const void* offsets = is_v ? args.offsets_v : args.offsets_k;
        if (entry < kTilesPerCta * args.pages_per_tile && table_slot < (is_v ? args.table_len_v : args.table_len_k)) {
            if (!offsets) {
                page = is_v ? args.table_v[batch * args.table_v_stride + table_slot * args.table_v_slot_stride]
                            : args.table_k[batch * args.table_k_stride + table_slot * args.table_k_slot_stride];
            } else if (args.prefix_ok[is_v ? 1 : 0]) {
                const int64_t length = args.seq_kv[batch * args.seq_kv_stride];
                if (table_slot < (length + args.block - 1) / args.block) {
                    const int64_t at = batch * (is_v ? args.offsets_v_stride : args.offsets_k_stride);
                    const int64_t base = (is_v ? args.offsets_v_wide : args.offsets_k_wide) ? static_cast<const int64_t*>(offsets)[at]
                                                                                          : static_cast<int64_t>(static_cast<const int32_t*>(offsets)[at]);
                    page = is_v ? args.table_v[base + table_slot * args.table_v_slot_stride] : args.table_k[base + table_slot * args.table_k_slot_stride];
                }
            }
        }
        page_ids[threadIdx.x] = (page >= 0 && page < args.num_pages) ? static_cast<int32_t>(page) : -1;
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 64);
        tmem_relinquish();
        tc_fence_before();
    }
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_ptr;
    const uint32_t tmem_o = tmem_base + 32;  // S^T buffers at +0 and +16, O^T at +32

    if (warp == 0) {
        if (lane == 0) {
            // Q rows of this GQA group (the box holds 16 rows; rows past the group are other heads or zero fill and are ignored)
            mbar_expect_tx(q_full, 2 * kHeadsPadded * 128);
            const int q_row = static_cast<int>(batch * args.heads_q + kv_head * G);
            tma_load_2d(smem_base + DecodeSmem::kQ, &map_q, 0, q_row, q_full);
            tma_load_2d(smem_base + DecodeSmem::kQ + kHeadsPadded * 128, &map_q, 64, q_row, q_full);
            const uint32_t page_bytes = static_cast<uint32_t>(args.block) * 128u;  // one page, one 64-column half
            for (int t = 0; t < 2 * tiles; ++t) {
                const int slot = t % kRingSlots;
                if (!mbar_wait(kv_empty(slot), ((t / kRingSlots) & 1) ^ 1, 301)) break;
                const bool is_v = (t & 1) != 0;
                const CUtensorMap* map = is_v ? &map_v : &map_k;
                const int32_t* ids = page_ids + (is_v ? 64 : 0) + (first_tile + (t >> 1)) * args.pages_per_tile;
                const uint32_t dst = smem_base + DecodeSmem::kRing + slot * kKvTileBytes;
                uint32_t expected = 0;
                for (int pg = 0; pg < args.pages_per_tile; ++pg)
                    if (ids[pg] >= 0) expected += 2 * page_bytes;
                mbar_expect_tx(kv_full(slot), expected);  // also the arrival; 0 bytes when every page is invalid
                for (int pg = 0; pg < args.pages_per_tile; ++pg) {
                    const int64_t page = ids[pg];
                    const uint32_t page_dst = dst + pg * page_bytes;
                    if (page >= 0) {
                        const int row = static_cast<int>((page * args.heads_kv + kv_head) * args.block);
                        tma_load_2d(page_dst, map, 0, row, kv_full(slot));
                        tma_load_2d(page_dst + kKvHalfBytes, map, 64, row, kv_full(slot));
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // S^T: A = K tile (K-major), B = Q (K-major). O^T: A = V tile read MN-major (M = d), B = P (K-major).
            const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kHeadsPadded >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
            const uint32_t idesc_o = idesc_s | (1u << 15);
            const uint32_t q_smem = smem_base + DecodeSmem::kQ;
            bool ok = mbar_wait(q_full, 0, 302);
            auto issue_scores = [&](int j) {
                const int t = 2 * j, slot = t % kRingSlots, b = j & 1;
                if (ok) ok = mbar_wait(kv_full(slot), (t / kRingSlots) & 1, 303);
                if (ok) ok = mbar_wait(s_empty(b), ((j >> 1) & 1) ^ 1, 304);
                tc_fence_after();
                if (ok) {
                    const uint32_t k_smem = smem_base + DecodeSmem::kRing + slot * kKvTileBytes;
                    const uint32_t k_lo = smem_desc_lo(k_smem, 16), q_lo = smem_desc_lo(q_smem, 16);
#pragma unroll
                    for (int k = 0; k < kDim / 16; ++k)
                        umma_bf16(tmem_base + b * 16, desc_words(k_lo + (((k >> 2) * kKvHalfBytes + (k & 3) * 32) >> 4), smem_desc_hi(1024)),
                                  desc_words(q_lo + (((k >> 2) * (kHeadsPadded * 128) + (k & 3) * 32) >> 4), smem_desc_hi(1024)), idesc_s, k != 0 ? 1u : 0u);
                }
                umma_commit(kv_empty(slot));
                umma_commit(s_full(b));
            };
            issue_scores(0);
            for (int j = 0; j < tiles; ++j) {
                if (j + 1 < tiles) issue_scores(j + 1);
                const int t = 2 * j + 1, slot = t % kRingSlots, b = j & 1;
                if (ok) ok = mbar_wait(p_full(b), (j >> 1) & 1, 305);
                if (ok) ok = mbar_wait(kv_full(slot), (t / kRingSlots) & 1, 306);
                tc_fence_after();
                if (ok) {
                    const uint32_t v_smem = smem_base + DecodeSmem::kRing + slot * kKvTileBytes;
                    const uint32_t p_smem = smem_base + DecodeSmem::kP + b * 4096;
                    const uint32_t v_lo = smem_desc_lo(v_smem, kKvHalfBytes), p_lo = smem_desc_lo(p_smem, 16);
#pragma unroll
                    for (int k = 0; k < kTileKeys / 16; ++k)
                        umma_bf16(tmem_o, desc_words(v_lo + ((k * 2048) >> 4), smem_desc_hi(1024)),
                                  desc_words(p_lo + (((k >> 2) * (kHeadsPadded * 128) + (k & 3) * 32) >> 4), smem_desc_hi(1024)), idesc_o, (j | k) != 0 ? 1u : 0u);
                }
                umma_commit(kv_empty(slot));
                umma_commit(pv_done(b));
            }
        }
    } else {
        const int quadrant = warp & 3;
        const int key_lane = quadrant * 32 + lane;  // key inside the tile for S^T, head-dim index for O^T
        const uint32_t lane_base = static_cast<uint32_t>(quadrant * 32) << 16;
        float* reduce = reinterpret_cast<float*>(generic_base + DecodeSmem::kReduce);  // [2][4][8]
        // m_ref: the reference the exponentials use (raised lazily); m_true: the real running maximum,
        // which the published partial is re-expressed in so that Max and Sum_exp come out exact
        float m_ref[G], m_true[G], l_part[G];
#pragma unroll
        for (int h = 0; h < G; ++h) { m_ref[h] = -INFINITY; m_true[h] = -INFINITY; l_part[h] = 0.0f; }
        bool ok = true;
        {
            // rows of the padded heads (G..15) of both P buffers stay zero for the whole kernel
            const int half = key_lane >> 6, within = key_lane & 63;
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int h = G; h < kHeadsPadded; ++h) {
                    const uint32_t offset = half * (kHeadsPadded * 128) + h * 128 + (((within >> 3) ^ (h & 7)) << 4) + (within & 7) * 2;
                    *reinterpret_cast<uint16_t*>(generic_base + DecodeSmem::kP + b * 4096 + offset) = 0;
                }
        }
        for (int j = 0; j < tiles; ++j) {
            const int b = j & 1;
            const int64_t key = chunk_begin + static_cast<int64_t>(first_tile + j) * kTileKeys + key_lane;
            // page validity of this key (an invalid page reads as zeros: score 0, no contribution to O)
            const int entry = ((first_tile + j) * kTileKeys + key_lane) / args.block;
            const bool k_page_ok = page_ids[entry] >= 0, v_page_ok = page_ids[64 + entry] >= 0;
            const bool in_window = key >= lo && key < hi;
            if (!v_page_ok) {
                // No TMA transfer targets this key's value row (its page id is out of range): the row must
                // read as zeros, and stale shared memory could hold NaN patterns, so clear it by hand once the
                // producer owns the slot (its barrier completes even for a zero-byte transfer).
                const int tv = 2 * j + 1, slot_v = tv % kRingSlots;
                if (ok) ok = mbar_wait(kv_full(slot_v), (tv / kRingSlots) & 1, 311);
                uint8_t* v_row = generic_base + DecodeSmem::kRing + slot_v * kKvTileBytes + key_lane * 128;
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    *reinterpret_cast<uint4*>(v_row + u * 16) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4*>(v_row + kKvHalfBytes + u * 16) = make_uint4(0, 0, 0, 0);
                }
            }
            if (ok) ok = mbar_wait(s_full(b), (j >> 1) & 1, 307);
            tc_fence_after();
            uint32_t raw[16];
            tmem_load_16(tmem_base + lane_base + b * 16, raw);
            tmem_load_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_empty(b));
            float s[G];
#pragma unroll
            for (int h = 0; h < G; ++h) {
                s[h] = k_page_ok ? __uint_as_float(raw[h]) * args.scale_log2 : 0.0f;
                if (!in_window) s[h] = -INFINITY;
            }
            // tile maximum per head over the 128 keys: warp shuffle, then one exchange through shared memory
            float warp_max[G];
#pragma unroll
            for (int h = 0; h < G; ++h) {
                warp_max[h] = warp_max_f32(s[h]);
            }
            float* slot_reduce = reduce + b * 32;
            if (lane == 0) {
#pragma unroll
                for (int h = 0; h < G; ++h) slot_reduce[quadrant * 8 + h] = warp_max[h];
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            bool raise = false;
            float tile_max[G];
#pragma unroll
            for (int h = 0; h < G; ++h) {
                tile_max[h] = fmaxf(fmaxf(slot_reduce[h], slot_reduce[8 + h]), fmaxf(slot_reduce[16 + h], slot_reduce[24 + h]));
                m_true[h] = fmaxf(m_true[h], tile_max[h]);
                raise = raise || tile_max[h] > m_ref[h] + kRaiseThreshold;
            }
            if (raise) {  // uniform over the 128 threads: they all see the same maxima
                float alpha[G];
#pragma unroll
                for (int h = 0; h < G; ++h) {
                    const float m_new = fmaxf(m_ref[h], tile_max[h]);
                    alpha[h] = m_ref[h] == -INFINITY ? 0.0f : exp2f(m_ref[h] - m_new);
                    l_part[h] *= alpha[h];
                    m_ref[h] = m_new;
                }
                if (j > 0) {
                    if (ok) ok = mbar_wait(pv_done((j - 1) & 1), ((j - 1) >> 1) & 1, 308);
                    tc_fence_after();
                    uint32_t acc[16];
                    tmem_load_16(tmem_o + lane_base, acc);
                    tmem_load_wait();
#pragma unroll
                    for (int h = 0; h < G; ++h) acc[h] = __float_as_uint(__uint_as_float(acc[h]) * alpha[h]);
                    tmem_store_16(tmem_o + lane_base, acc);
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();
                }
            }
            // P buffer b was last read by the product of tile j-2
            if (ok) ok = mbar_wait(pv_done(b), ((j >> 1) & 1) ^ 1, 309);
            uint8_t* p_tile = generic_base + DecodeSmem::kP + b * 4096;
            const int half = key_lane >> 6, within = key_lane & 63;
#pragma unroll
            for (int h = 0; h < G; ++h) {
                float p = (s[h] == -INFINITY || m_ref[h] == -INFINITY) ? 0.0f : exp2f(s[h] - m_ref[h]);
                l_part[h] += p;
                if (!v_page_ok) p = 0.0f;  // the value row reads as zeros
                const uint32_t offset = half * (kHeadsPadded * 128) + h * 128 + (((within >> 3) ^ (h & 7)) << 4) + (within & 7) * 2;
                *reinterpret_cast<__nv_bfloat16*>(p_tile + offset) = __float2bfloat16_rn(p);
            }
            fence_async_shared();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full(b));
        }
        // totals: reduce the per-thread partial sums, read O^T, publish this CTA's partial
        const int last = tiles - 1;
        if (ok) ok = mbar_wait(pv_done(last & 1), (last >> 1) & 1, 310);
        tc_fence_after();
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the max-exchange slots are free again
        float total[G];
#pragma unroll
        for (int h = 0; h < G; ++h) {
            float v = l_part[h];
#pragma unroll
            for (int step = 16; step > 0; step >>= 1) v += __shfl_xor_sync(0xffffffffu, v, step);
            if (lane == 0) reduce[quadrant * 8 + h] = v;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        uint32_t acc[16];
        tmem_load_16(tmem_o + lane_base, acc);
        tmem_load_wait();
        const bool healthy = ok && g_device_status == 0;
#pragma unroll
        for (int h = 0; h < G; ++h) {
            total[h] = reduce[h] + reduce[8 + h] + reduce[16 + h] + reduce[24 + h];
            float* p = my_partial + static_cast<int64_t>(h) * args.max_chunks * kPartialStride;
            if (healthy) {
                const float factor = m_true[h] == -INFINITY ? 0.0f : exp2f(m_ref[h] - m_true[h]);
                p[key_lane] = __uint_as_float(acc[h]) * factor;  // key_lane is the head-dim index here
                if (key_lane == 0) {
                    p[kDim] = m_true[h] == -INFINITY ? -INFINITY : m_true[h] * 0.6931471805599453f;  // natural-log units for the merge
                    p[kDim + 1] = total[h] * factor;
                }
            }
        }
        tc_fence_before();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 64);
    }
}

}  // namespace

int decode_umma_chunks(const dfgpu_sdpa_params& p) { return static_cast<int>((p.s_kv + kTilesPerCta * kTileKeys - 1) / (kTilesPerCta * kTileKeys)); }

bool decode_umma_supported(const dfgpu_sdpa_params& p) {
    if (p.q.rank != 4 || p.k.rank != 4 || p.v.rank != 4) return false;
    if (p.q.dim[2] != 1 || p.q.dim[3] != kDim || p.k.dim[3] != kDim || p.v.dim[3] != kDim) return false;
    if (p.q.dtype != DFGPU_BF16 || p.k.dtype != DFGPU_BF16 || p.v.dtype != DFGPU_BF16) return false;
    if (p.page_table_k.rank != 4 || p.page_table_v.rank != 4) return false;
    const int64_t block = p.k.dim[2];
    if (p.v.dim[2] != block || block < 16 || block > kTileKeys || (block & (block - 1)) != 0) return false;
    if (p.k.dim[1] != p.v.dim[1] || p.k.dim[0] != p.v.dim[0]) return false;
    const int64_t group = p.q.dim[1] / p.k.dim[1];
    if (group != 1 && group != 2 && group != 4 && group != 8) return false;
    // packed containers [pages, Hkv, block, D] and packed Q [B, Hq, 1, D]
    auto packed = [](const dfgpu_tensor& t) {
        return t.stride[3] == 1 && t.stride[2] == t.dim[3] && t.stride[1] == t.dim[2] * t.dim[3] && t.stride[0] == t.dim[1] * t.dim[2] * t.dim[3];
    };
    if (!packed(p.k) || !packed(p.v)) return false;
    if (p.q.stride[3] != 1 || p.q.stride[1] != kDim || p.q.stride[0] != p.q.dim[1] * kDim) return false;
    if (p.k.dim[0] * p.k.dim[1] * block >= (1ll << 31)) return false;
    if (p.q.dim[0] > 65535 || p.k.dim[1] > 65535) return false;
    return true;
}

int64_t decode_umma_scratch_bytes(const dfgpu_sdpa_params& p) {
    return p.q.dim[0] * p.q.dim[1] * decode_umma_chunks(p) * kPartialStride * static_cast<int64_t>(sizeof(float));
}

int launch_decode_umma(const dfgpu_sdpa_params& p, void* const* tensors, void* scratch, const int* prefix_ok, cudaStream_t stream) {
    for (int i = 0; i < 3; ++i)
        if ((reinterpret_cast<uintptr_t>(tensors[i]) & 15u) != 0) return fail(kInvalidArgument, "SDPA: the paged decode kernel needs 16-byte aligned Q, K and V");
    const int64_t batch = p.q.dim[0], hq = p.q.dim[1], hkv = p.k.dim[1], block = p.k.dim[2], pages = p.k.dim[0];
    CUtensorMap map_q, map_k, map_v;
    uint64_t strides[1] = {kDim * 2};
    uint64_t dims_q[2] = {kDim, static_cast<uint64_t>(batch * hq)};
    uint32_t box_q[2] = {64, kHeadsPadded};
    uint64_t dims_kv[2] = {kDim, static_cast<uint64_t>(pages * hkv * block)};
    uint32_t box_kv[2] = {64, static_cast<uint32_t>(block)};
    int status = make_map(&map_q, tensors[0], 2, dims_q, strides, box_q, "SDPA decode Q");
    if (!status) status = make_map(&map_k, tensors[1], 2, dims_kv, strides, box_kv, "SDPA decode K");
    if (!status) status = make_map(&map_v, tensors[2], 2, dims_kv, strides, box_kv, "SDPA decode V");
    if (status) return status;
    DecodeArgs args{};
    args.heads_q = static_cast<int>(hq);
    args.heads_kv = static_cast<int>(hkv);
    args.group = static_cast<int>(hq / hkv);
    args.block = static_cast<int>(block);
    args.pages_per_tile = static_cast<int>(kTileKeys / block);
    args.table_len_k = static_cast<int>(p.page_table_k.dim[2]);
    args.table_len_v = static_cast<int>(p.page_table_v.dim[2]);
    args.num_pages = static_cast<int>(pages);
    args.max_chunks = decode_umma_chunks(p);
    args.has_left = p.has_left_bound;
    args.has_right = p.has_right_bound;
    args.bottom_right = p.bottom_right;
    args.padding = p.padding_mask;
    args.left = p.left_bound;
    args.right = p.right_bound;
    args.s_kv = p.s_kv;
    args.scale_log2 = p.attn_scale * 1.4426950408889634f;
    args.seq_q = static_cast<const int32_t*>(tensors[7]);
    args.seq_kv = static_cast<const int32_t*>(tensors[8]);
    args.table_k = static_cast<const int32_t*>(tensors[9]);
    args.table_v = static_cast<const int32_t*>(tensors[10]);
    args.seq_q_stride = p.seq_q.rank ? p.seq_q.stride[0] : 0;
    args.seq_kv_stride = p.seq_kv.rank ? p.seq_kv.stride[0] : 0;
    args.table_k_stride = p.page_table_k.stride[0];
    args.table_v_stride = p.page_table_v.stride[0];
    args.table_k_slot_stride = p.page_table_k.stride[2];
    args.table_v_slot_stride = p.page_table_v.stride[2];
    args.partial = static_cast<float*>(scratch);
    args.offsets_k = p.page_offsets_k.rank ? tensors[14] : nullptr;
    args.offsets_v = p.page_offsets_v.rank ? tensors[15] : nullptr;
    args.offsets_k_wide = p.page_offsets_k.dtype == DFGPU_I64;
    args.offsets_v_wide = p.page_offsets_v.dtype == DFGPU_I64;
    args.offsets_k_stride = p.page_offsets_k.rank ? p.page_offsets_k.stride[0] : 0;
    args.offsets_v_stride = p.page_offsets_v.rank ? p.page_offsets_v.stride[0] : 0;
    args.prefix_ok = prefix_ok;
    dim3 grid(static_cast<unsigned>(args.max_chunks), static_cast<unsigned>(hkv), static_cast<unsigned>(batch));
    auto run = [&](auto kernel, int dynamic) -> int {
        cudaError_t error = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dynamic);
        if (error != cudaSuccess) return fail(kExecutionFailed, "SDPA decode: cannot reserve %d bytes of shared memory: %s", dynamic, cudaGetErrorString(error));
        kernel<<<grid, kDecodeThreads, dynamic, stream>>>(map_q, map_k, map_v, args);
        return check_launch("SDPA paged decode (tcgen05)");
    };
    // three ring slots: two CTAs per SM (about 219 KiB of shared memory together) hide each other's softmax latency
#define DFGPU_DECODE_CASE(G_) return run(sdpa_decode_umma_kernel<G_, 3>, DecodeSmemT<3>::kDynamic)
    switch (args.group) {
        case 1: DFGPU_DECODE_CASE(1);
        case 2: DFGPU_DECODE_CASE(2);
        case 4: DFGPU_DECODE_CASE(4);
        default: DFGPU_DECODE_CASE(8);
    }
#undef DFGPU_DECODE_CASE
}

int decode_umma_device_status(int* status) { return read_and_clear_device_status(status); }

}  // namespace dfgpu

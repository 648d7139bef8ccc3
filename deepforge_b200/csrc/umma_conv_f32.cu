// f32 CONV_FPROP on the bf16 tensor cores in ONE launch; made for convolutions with fewer output tiles than SMs, where
// the clusters below spread one tile's reduction over several SMs, and correct for any number of tiles (one CTA per tile then).
//
// x = xh + xm + xl and w = wh + wm + wl with bf16 pieces (the leading 8 significant bits, the next 8, the last 8, each
// cut off rather than rounded, so every subtraction that forms them is exact and no piece can round past the largest
// bf16), and x * w = xm*wm + xl*wh + xh*wl + xm*wh + xh*wm + xh*wh up to 2^-23 relative: six bf16 products per 16-deep K
// step, accumulated in f32 in tensor memory.
//
// One thread-block cluster per 128-pixel x 64-channel output tile. The K loop runs over units (one filter tap x 64 input
// channels); the cluster's CTAs share the units out between them. A CTA's 512 loader threads read the f32 X rows of a tap
// (zero rows outside the image) and the f32 filter rows, split them in registers and write the three pieces of each
// straight into the 128-byte-swizzled shared-memory tiles the tcgen05 descriptors expect, two units in flight; one more
// warp issues the 24 products of a unit when its tiles are complete. Every rank owns one slice of the tile's rows: at the
// end a CTA parks its f32 partial tile in its own shared memory and sends each owner its rows with one bulk copy into the
// owner's inbox (shared memory to shared memory across the cluster, signalled on the owner's mbarrier); each CTA waits for
// its inbox to fill, adds its rows over all ranks in rank order, applies the epilogue and stores Y.
//
// Channel counts are free: a unit's missing channels and a tile's missing filter rows are written as zeros (a group of 8
// input channels that is not whole is read value by value). Stride, dilation, asymmetric padding and filter reversal only change which input pixel
// and which filter tap a loader thread reads. The tensors may have any strides: with contiguous channels on 16-byte
// boundaries (channels-last X and Y, KRSC filter) a group of 8 channels is two float4 loads; otherwise (NCHW, a
// transposed MATMUL operand, a pointer that is only 4-byte aligned) neighbouring threads take neighbouring pixels (or
// output channels) and read their channels value by value, so that a warp's loads still fall side by side. Read value by
// value, the tensors may also be f16 or bf16 (widened to f32, whose lower pieces are then zero; Y narrowed on the store),
// which gives strided, dilated and odd-sized convolutions of those types a tensor-core path too. Groups: every 64-channel
// output tile belongs to one group and reads that group's input channels. Rank-5 convolutions: an output pixel is (image,
// depth, row, column) and the units run over the depth taps as well.
//
// A product with an infinite or NaN factor does not survive the split, so the loaders also record whether they saw
// one; the ranks exchange that beside the partial tiles, and a cluster that saw one computes its tile on the CUDA cores
// instead (zero padding still multiplied, as the reference's single-node path does).
#include <cooperative_groups.h>

#include <mutex>

#include "conv_args.cuh"
#include "umma_ptx.cuh"

namespace cg = cooperative_groups;

namespace dfgpu {
namespace {

constexpr int kTileM = 128, kTileN = 64, kChunk = 64;
constexpr int kLoaders = 512, kThreads = kLoaders + 32;
constexpr int kPieceBytesA = kTileM * 128, kPieceBytesB = kTileN * 128;   // 64 bf16 = one 128-byte swizzled row per pixel
constexpr int kUnitBytes = 3 * (kPieceBytesA + kPieceBytesB);
constexpr int kBuffers = 2;
constexpr int kMaxRanks = 8;
constexpr int kMaxUnitsPerRank = 64;
constexpr int kInboxOffset = kBuffers * kUnitBytes;                        // the rows this rank owns, one chunk per sending rank
constexpr int kRowBytes = kTileN * 4;
constexpr int kInboxBytes = (kTileM + kMaxRanks) * kRowBytes + kMaxRanks * 16;   // ranks * (ceil(128 / ranks) rows + a 16-byte trailer)
static_assert(kInboxBytes <= kUnitBytes, "the outgoing chunks are parked in the first operand buffer");
constexpr int kControlOffset = kInboxOffset + kInboxBytes;
constexpr int kSmemBytes = kControlOffset + 128 + 1024;                    // (+ the slack that aligns the tiles to 1024 bytes)
constexpr int kAccumulatorColumns = 64;

struct ClusterConvArgs {
    const void* x;
    const void* w;
    void* y;
    int x_type, w_type, y_type;                   // DFGPU_F32, DFGPU_F16 or DFGPU_BF16 (the float4 accesses are for f32 only)
    int m_total, units, units_per_rank, chunks;   // chunks: 64-channel slices per filter tap
    int tiles_per_image;                          // 0: tiles run over all pixels of all images; else over one image each, and the
    int32_t w_n;                                  // filter of image n starts w_n elements further on (a batched MATMUL's B)
    FastDivisor by_tiles;                         // tiles_per_image
    // strides in floats; 32 bits are enough, and cheaper in the loaders: every element lies within 2^31 floats of the first
    int32_t x_n, x_c, x_h, x_w;                   // X by image, channel, row, column
    int32_t w_k, w_c, w_r, w_s;                   // the filter by output channel, input channel, tap row, tap column
    int32_t y_n, y_k, y_p, y_q;                   // Y by image, channel, row, column
    int P, Q, H, W, R, S;                         // output and input rows and columns, filter rows and columns
    int depth_out, depth_in, depth_taps;          // a rank-5 convolution's third spatial axis (1, 1, 1 otherwise): an output pixel is (image, depth, row, column)
    int32_t x_d, w_t, y_d;                        // ... and its strides
    FastDivisor by_depth, by_plane;               // depth_out; R * S
    int x_quads, w_quads, y_quads;                // channels are contiguous and every other stride and the pointer a multiple of 16 bytes: float4 accesses
    int w_along_k;                                // output channels are contiguous in the filter (a MATMUL's row-major B): neighbouring threads take neighbouring output channels
    FastDivisor by_q, by_p, by_chunks, by_s;      // output width and height, chunks, filter width
};

__device__ __forceinline__ uint32_t map_to_rank(uint32_t cta_address, uint32_t rank) {
    uint32_t cluster_address;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(cluster_address) : "r"(cta_address), "r"(rank));
    return cluster_address;
}
// `bytes` (a multiple of 16) from this CTA's shared memory into another CTA's, counted on that CTA's mbarrier.
__device__ __forceinline__ void bulk_copy_to_rank(uint32_t cluster_destination, uint32_t cta_source, uint32_t bytes, uint32_t cluster_barrier) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(cluster_destination), "r"(cta_source), "r"(bytes), "r"(cluster_barrier) : "memory");
}

__device__ __forceinline__ uint64_t pair_of(uint32_t first, uint32_t second) {
    uint64_t pair;
    asm("mov.b64 %0, {%1, %2};" : "=l"(pair) : "r"(first), "r"(second));
    return pair;
}
__device__ __forceinline__ uint64_t add_pairs(uint64_t a, uint64_t b) {   // two f32 additions in one instruction
    uint64_t sum;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(sum) : "l"(a), "l"(b));
    return sum;
}
__device__ __forceinline__ void halves_of(uint64_t pair, uint32_t& first, uint32_t& second) {
    asm("mov.b64 {%0, %1}, %2;" : "=r"(first), "=r"(second) : "l"(pair));
}
// The leading bf16 of an f32 bit pattern (cut off, not rounded), negated: what to add to take it away.
__device__ __forceinline__ uint32_t minus_leading_bf16(uint32_t bits) { return (bits & 0xffff0000u) ^ 0x80000000u; }

// One value of an f32, f16 or bf16 tensor.
__device__ __forceinline__ float load_value(const void* data, int type, int offset) {
    if (type == DFGPU_F32) return __ldg(static_cast<const float*>(data) + offset);
    const uint16_t bits = __ldg(static_cast<const uint16_t*>(data) + offset);
    return type == DFGPU_BF16 ? __uint_as_float(static_cast<uint32_t>(bits) << 16) : __half2float(__ushort_as_half(bits));
}

// Two consecutive f32 quads as three 16-byte groups of bf16 pieces (high, middle, low); false when a value is infinite or NaN.
__device__ __forceinline__ bool split_eight(const float4& a, const float4& b, uint4 (&piece)[3]) {
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t h[4], m[4], l[4];
    bool finite = true;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t v0 = __float_as_uint(v[2 * i]), v1 = __float_as_uint(v[2 * i + 1]);
        finite = finite && fabsf(v[2 * i]) <= 3.4028234663852886e38f && fabsf(v[2 * i + 1]) <= 3.4028234663852886e38f;
        uint32_t r0, r1, l0, l1;
        const uint64_t rest = add_pairs(pair_of(v0, v1), pair_of(minus_leading_bf16(v0), minus_leading_bf16(v1)));   // (exact)
        halves_of(rest, r0, r1);
        halves_of(add_pairs(rest, pair_of(minus_leading_bf16(r0), minus_leading_bf16(r1))), l0, l1);   // (at most 8 significant bits are left)
        h[i] = __byte_perm(v0, v1, 0x7632);   // the upper halves of two words side by side
        m[i] = __byte_perm(r0, r1, 0x7632);
        l[i] = __byte_perm(l0, l1, 0x7632);
    }
    piece[0] = make_uint4(h[0], h[1], h[2], h[3]);
    piece[1] = make_uint4(m[0], m[1], m[2], m[3]);
    piece[2] = make_uint4(l[0], l[1], l[2], l[3]);
    return finite;
}

// FAST: X, W and Y all take float4 accesses (the flags in the arguments are then not looked at).
template <bool FAST>
__global__ void __launch_bounds__(kThreads, 1)
umma_conv_f32_kernel(const __grid_constant__ ClusterConvArgs g, const __grid_constant__ ConvArgs a) {
    const bool x_quads = FAST || g.x_quads != 0, w_quads = FAST || g.w_quads != 0, y_quads = FAST || g.y_quads != 0;
    const bool w_along_k = !FAST && g.w_along_k != 0;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = static_cast<int>(cluster.block_rank()), ranks = static_cast<int>(cluster.num_blocks());
    const int tid = threadIdx.x, warp = uniform_warp_index(), lane = tid & 31;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t full_bar = smem_base + kControlOffset, empty_bar = full_bar + 8 * kBuffers;
    const uint32_t inbox_bar = empty_bar + 8 * kBuffers;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kControlOffset + 16 * kBuffers + 8);

    // The tile's first row as a pixel index over all images, and how many of its 128 rows exist.
    // Along z: the 64-channel tiles of the output, group by group (a group's output channels meet its own input channels only).
    int n0 = blockIdx.z * kTileN, K = static_cast<int>(a.y.dim[1]), C = static_cast<int>(a.x.dim[1]), x_group = 0;
    if (!FAST && a.groups > 1) {   // (the all-float4 instantiation is for one group)
        const int per_group = static_cast<int>(a.k_per_group), tiles_per_group = (per_group + kTileN - 1) / kTileN;
        const int group = static_cast<int>(blockIdx.z) / tiles_per_group;
        n0 = group * per_group + (static_cast<int>(blockIdx.z) - group * tiles_per_group) * kTileN;
        K = (group + 1) * per_group;                       // (the end of this group's output channels)
        C = static_cast<int>(a.c_per_group);
        x_group = group * C * g.x_c;                       // (where the group's input channels start in X; the filter holds C per output channel)
    }
    int m0 = blockIdx.y * kTileM, rows_live = min(kTileM, g.m_total - m0), filter_first = 0;
    if (!FAST && g.tiles_per_image > 0) {   // (the all-float4 instantiation is for unbatched problems)
        const int image = static_cast<int>(fast_divide(blockIdx.y, g.by_tiles)), first = (static_cast<int>(blockIdx.y) - image * g.tiles_per_image) * kTileM;
        const int pixels = g.P * g.Q;
        m0 = image * pixels + first;
        rows_live = min(kTileM, pixels - first);
        filter_first = image * g.w_n;
    }
    const int first_unit = rank * g.units_per_rank;
    const int my_units = max(0, min(g.units - first_unit, g.units_per_rank));
    const int P = g.P, Q = g.Q, H = g.H, W = g.W, R = g.R, S = g.S;
    const bool volume = !FAST && g.depth_taps * g.depth_in * g.depth_out > 1;   // (a depth axis: the general instantiation only)

    // Loader threads: which rows of the operand tiles this thread fills (the issuing warp computes them too, and loads nothing).
    // X with contiguous channels: a thread takes one group of 8 channels (16 bytes of bf16) of two pixels, as two float4 loads each.
    // Any other X (channels strided, as in NCHW): neighbouring threads take neighbouring pixels, so that their loads of one
    // channel fall side by side, and a thread reads two groups of 8 channels of one pixel value by value.
    const int row[2] = {x_quads ? tid >> 3 : tid & 127, x_quads ? 64 + (tid >> 3) : tid & 127};
    const int x_unit[2] = {x_quads ? tid & 7 : (tid >> 7) & 3, x_quads ? tid & 7 : 4 + ((tid >> 7) & 3)};
    int ih0[2], iw0[2], id0[2];
    int x_image[2];   // element offsets (everything lies within 2^31 elements of the first)
    bool live[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = m0 + row[i];
        live[i] = row[i] < rows_live;
        const int mm = live[i] ? m : 0;
        const int line = static_cast<int>(fast_divide(mm, g.by_q)), q = mm - line * Q;
        const int plane = static_cast<int>(fast_divide(line, g.by_p)), p = line - plane * P;
        const int n = volume ? static_cast<int>(fast_divide(plane, g.by_depth)) : plane;
        ih0[i] = p * a.stride_h - a.pad_h;
        iw0[i] = q * a.stride_w - a.pad_w;
        id0[i] = volume ? (plane - n * g.depth_out) * a.stride_d - a.pad_d : 0;
        x_image[i] = n * g.x_n + x_group + x_unit[i] * 8 * g.x_c;
    }
    // The filter tile: 64 output channels x 8 groups of 8 input channels. Stored with input channels contiguous, a thread
    // reads its group as two quads; stored with output channels contiguous, neighbouring threads take neighbouring output
    // channels and each reads its 8 input channels one by one.
    const int w_channel = w_along_k ? tid & 63 : tid >> 3, w_unit = w_along_k ? (tid >> 6) & 7 : tid & 7;
    const int w_row = filter_first + (n0 + w_channel < K ? (n0 + w_channel) * g.w_k + w_unit * 8 * g.w_c : 0);   // (rows past the last filter are never read)
    auto eight = [](const void* data, int type, int first, int stride, int count, float4 (&v)[2]) {   // `count` (of eight) values `stride` elements apart, zeros behind them
        float value[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) value[j] = j < count ? load_value(data, type, first + j * stride) : 0.0f;
        v[0] = make_float4(value[0], value[1], value[2], value[3]);
        v[1] = make_float4(value[4], value[5], value[6], value[7]);
    };
    const float4 zero = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    auto fetch = [&](int u, float4 (&xv)[2][2], float4 (&wv)[2]) {
        const int unit = first_unit + u;
        const int tap = static_cast<int>(fast_divide(unit, g.by_chunks)), c0 = (unit - tap * g.chunks) * kChunk;
        const int t = volume ? static_cast<int>(fast_divide(tap, g.by_plane)) : 0, in_plane = tap - t * R * S;
        const int r = static_cast<int>(fast_divide(in_plane, g.by_s)), s = in_plane - r * S;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int ih = ih0[i] + r * a.dilation_h, iw = iw0[i] + s * a.dilation_w, id = id0[i] + t * a.dilation_d;
            xv[i][0] = xv[i][1] = zero;
            if (live[i] && ih >= 0 && ih < H && iw >= 0 && iw < W && (!volume || (id >= 0 && id < g.depth_in)) && c0 + x_unit[i] * 8 < C) {
                const int source = x_image[i] + ih * g.x_h + iw * g.x_w + c0 * g.x_c + (volume ? id * g.x_d : 0);
                if (x_quads) {
                    xv[i][0] = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(g.x) + source));
                    xv[i][1] = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(g.x) + source) + 1);
                } else {
                    eight(g.x, g.x_type, source, g.x_c, C - (c0 + x_unit[i] * 8), xv[i]);
                }
            }
        }
        wv[0] = wv[1] = zero;
        if (n0 + w_channel >= K || c0 + w_unit * 8 >= C) {
            // (a filter row or a channel group past the end: zeros, which add nothing)
        } else {
            // (a reversed filter meets input tap (r, s) with its tap (R-1-r, S-1-s))
            const int source = w_row + (a.reverse ? R - 1 - r : r) * g.w_r + (a.reverse ? S - 1 - s : s) * g.w_s + c0 * g.w_c +
                               (volume ? (a.reverse ? g.depth_taps - 1 - t : t) * g.w_t : 0);
            if (w_quads) {
                wv[0] = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(g.w) + source));
                wv[1] = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(g.w) + source) + 1);
            } else {
                eight(g.w, g.w_type, source, g.w_c, C - (c0 + w_unit * 8), wv);
            }
        }
    };
    float4 xv[2][2], wv[2];
    if (tid < kLoaders && my_units > 0) fetch(0, xv, wv);   // in flight while the barriers and tensor memory are set up

    if (tid == 0) {
        for (int b = 0; b < kBuffers; ++b) {
            mbar_init(full_bar + 8 * b, kLoaders);
            mbar_init(empty_bar + 8 * b, 1);
        }
        mbar_init(inbox_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        mbar_expect_tx(inbox_bar, static_cast<uint32_t>(ranks) * (((kTileM + ranks - 1) / ranks) * kRowBytes + 16));   // one chunk from every rank
    }
    if (warp == kLoaders / 32) {
        tmem_alloc(smem_u32(tmem_slot), kAccumulatorColumns);
        tmem_relinquish();
    }
    cluster.barrier_arrive();   // (waited for before the first copy into another CTA's shared memory: its inbox barrier is armed by then)
    // The CTA meets once, for the barriers and the tensor memory address: the loaders after they have written their first
    // unit (that needs neither), the issuing warp at once.
    auto meet = [&] {
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
    };

    bool ok = true, finite = true;
    if (tid < kLoaders) {
        // ---- loaders: f32 rows -> three bf16 pieces in the swizzled operand tiles ----------------------------------
#pragma unroll 1
        for (int u = 0; u < my_units; ++u) {
            const int buffer = u & 1;
            float4 xn[2][2], wn[2];
            if (u + 1 < my_units) fetch(u + 1, xn, wn);   // the next unit's loads are in flight while this one is split
            if (u >= kBuffers) ok = mbar_wait(empty_bar + 8 * buffer, ((u >> 1) - 1) & 1, 131) && ok;
            uint8_t* tiles = smem + buffer * kUnitBytes;
            uint4 piece[3];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                finite = split_eight(xv[i][0], xv[i][1], piece) && finite;
                uint8_t* target = tiles + row[i] * 128 + ((x_unit[i] ^ (row[i] & 7)) << 4);
#pragma unroll
                for (int j = 0; j < 3; ++j) *reinterpret_cast<uint4*>(target + j * kPieceBytesA) = piece[j];
            }
            finite = split_eight(wv[0], wv[1], piece) && finite;
            uint8_t* target = tiles + 3 * kPieceBytesA + w_channel * 128 + ((w_unit ^ (w_channel & 7)) << 4);
#pragma unroll
            for (int j = 0; j < 3; ++j) *reinterpret_cast<uint4*>(target + j * kPieceBytesB) = piece[j];
            fence_async_shared();
            if (u == 0) meet();
            mbar_arrive(full_bar + 8 * buffer);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                xv[i][0] = xn[i][0];
                xv[i][1] = xn[i][1];
                wv[i] = wn[i];
            }
        }
        if (my_units == 0) meet();
    } else {
        // ---- issuing warp: the 24 products of every unit --------------------------------------------------------------
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(kTileN >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
        meet();
        const uint32_t tmem_u = __shfl_sync(0xffffffffu, *tmem_slot, 0);
#pragma unroll 1
        for (int u = 0; u < my_units; ++u) {
            const int buffer = u & 1;
            ok = mbar_wait_warp(full_bar + 8 * buffer, (u >> 1) & 1, 132) && ok;
            tc_fence_after();
            if (ok) {
                const uint32_t a_lo = smem_desc_lo(smem_base + buffer * kUnitBytes, 16);
                const uint32_t b_lo = smem_desc_lo(smem_base + buffer * kUnitBytes + 3 * kPieceBytesA, 16);
                if (elect_one()) {
                    // smallest products first: middle*middle, low*high, high*low, middle*high, high*middle, high*high
                    constexpr int piece_a[6] = {1, 2, 0, 1, 0, 0}, piece_b[6] = {1, 0, 2, 0, 1, 0};
#pragma unroll
                    for (int product = 0; product < 6; ++product)
#pragma unroll
                        for (int k = 0; k < kChunk / 16; ++k)
                            umma_bf16(tmem_u, desc_words(a_lo + ((piece_a[product] * kPieceBytesA + k * 32) >> 4), smem_desc_hi(1024)),
                                      desc_words(b_lo + ((piece_b[product] * kPieceBytesB + k * 32) >> 4), smem_desc_hi(1024)), idesc, (u | product | k) != 0 ? 1u : 0u);
                    umma_commit(empty_bar + 8 * buffer);
                }
                __syncwarp();
            }
        }
    }

    // ---- this CTA's partial tile: tensor memory -> its own shared memory, one chunk per owner -> the owners' inboxes ---
    const int rows_per_rank = (kTileM + ranks - 1) / ranks;
    const int chunk_bytes = rows_per_rank * kRowBytes + 16;   // an owner's rows, then 16 bytes that say whether the sender met an infinity or a NaN
    if (warp < 8) {
        const int quadrant = warp & 3, half = warp >> 2;   // lanes 32 * quadrant.. of tensor memory, 32 of the 64 columns
        const int row = quadrant * 32 + lane;
        uint32_t r[32];
        if (my_units > 0) {
            ok = mbar_wait(empty_bar + 8 * ((my_units - 1) & 1), ((my_units - 1) >> 1) & 1, 133) && ok;   // the last commit covers every product
            tc_fence_after();
            tmem_load_32(*tmem_slot + (static_cast<uint32_t>(quadrant * 32) << 16) + half * 32, r);
            tmem_load_wait();
            tc_fence_before();
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        const int owner = row / rows_per_rank;
        uint8_t* parked = smem + owner * chunk_bytes + (row - owner * rows_per_rank) * kRowBytes;   // (over the first operand buffer: every product is done)
#pragma unroll
        for (int j = 0; j < 8; ++j)
            *reinterpret_cast<uint4*>(parked + (((half * 8 + j) ^ (row & 7)) << 4)) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
    }
    const int unsplittable = __syncthreads_or(finite ? 0 : 1);
    if (tid < ranks) *reinterpret_cast<uint4*>(smem + tid * chunk_bytes + rows_per_rank * kRowBytes) = make_uint4(static_cast<uint32_t>(unsplittable), 0u, 0u, 0u);
    fence_async_shared();
    __syncthreads();
    cluster.barrier_wait();
    if (tid < ranks)
        bulk_copy_to_rank(map_to_rank(smem_base + kInboxOffset + rank * chunk_bytes, tid), smem_base + tid * chunk_bytes, chunk_bytes, map_to_rank(inbox_bar, tid));
    ok = mbar_wait(inbox_bar, 0, 134) && ok;
    // Waited for before leaving: a CTA whose inbox is full has been read by every copy aimed at it, so when all have arrived
    // no copy still reads any CTA's shared memory. (Relaxed: nothing is published with it, and the releasing form waits
    // more than a thousand cycles here.)
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    // ---- this rank's rows: the sum over all ranks' partial tiles, the epilogue, Y --------------------------------------
    const uint8_t* inbox = smem + kInboxOffset;
    int any_unsplittable = 0;
#pragma unroll
    for (int z = 0; z < kMaxRanks; ++z) any_unsplittable |= z < ranks ? *reinterpret_cast<const int*>(inbox + z * chunk_bytes + rows_per_rank * kRowBytes) : 0;
    const int row_begin = rank * rows_per_rank, row_end = min(kTileM, row_begin + rows_per_rank);
    if (!any_unsplittable) {
        // Y with contiguous channels: 16 neighbouring threads store one pixel's 64 channels as float4s. Any other Y (NCHW):
        // neighbouring threads take neighbouring pixels and store their four channels one by one.
        const int rows = row_end - row_begin;
        for (int item = tid; item < rows * 16; item += kThreads) {
            const int row = row_begin + (y_quads ? item >> 4 : item % rows), unit = y_quads ? item & 15 : item / rows;
            const int m = m0 + row, k = n0 + unit * 4;
            if (row >= rows_live || k >= K) continue;
            const int offset = (row - row_begin) * kRowBytes + ((unit ^ (row & 7)) << 4);
            float4 part[kMaxRanks];
#pragma unroll
            for (int z = 0; z < kMaxRanks; ++z)   // every load in flight before the first sum
                part[z] = z < ranks ? *reinterpret_cast<const float4*>(inbox + z * chunk_bytes + offset) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            float4 sum = part[0];
#pragma unroll
            for (int z = 1; z < kMaxRanks; ++z) {
                if (z >= ranks) break;
                sum.x = __fadd_rn(sum.x, part[z].x);
                sum.y = __fadd_rn(sum.y, part[z].y);
                sum.z = __fadd_rn(sum.z, part[z].z);
                sum.w = __fadd_rn(sum.w, part[z].w);
            }
            const int line = static_cast<int>(fast_divide(m, g.by_q)), q = m - line * Q;
            const int plane = static_cast<int>(fast_divide(line, g.by_p)), p = line - plane * P;
            const int n = volume ? static_cast<int>(fast_divide(plane, g.by_depth)) : plane, d = volume ? plane - n * g.depth_out : 0;
            if (a.epilogue.count > 0) {
                sum.x = apply_epilogue(sum.x, a, n, k, p, q, d);
                sum.y = apply_epilogue(sum.y, a, n, k + 1, p, q, d);
                sum.z = apply_epilogue(sum.z, a, n, k + 2, p, q, d);
                sum.w = apply_epilogue(sum.w, a, n, k + 3, p, q, d);
            }
            const int target = n * g.y_n + p * g.y_p + q * g.y_q + k * g.y_k + d * g.y_d;
            if (y_quads) {
                *reinterpret_cast<float4*>(static_cast<float*>(g.y) + target) = sum;
            } else {
                store_from_f32(g.y, g.y_type, target, sum.x);
                if (k + 1 < K) store_from_f32(g.y, g.y_type, target + g.y_k, sum.y);
                if (k + 2 < K) store_from_f32(g.y, g.y_type, target + 2 * g.y_k, sum.z);
                if (k + 3 < K) store_from_f32(g.y, g.y_type, target + 3 * g.y_k, sum.w);
            }
        }
    } else {
        // An infinity or a NaN among this tile's inputs: the same rows on the CUDA cores, every tap multiplied (zero
        // padding included), channels innermost.
        for (int item = tid; item < (row_end - row_begin) * kTileN; item += kThreads) {
            const int row = row_begin + item / kTileN, k = n0 + item % kTileN;
            const int m = m0 + row;
            if (row >= rows_live || k >= K) continue;
            const int q = m % Q, p = (m / Q) % P, plane = m / (P * Q), n = plane / g.depth_out, d = plane % g.depth_out;
            const int filter = filter_first + k * g.w_k;
            float sum = 0.0f;
            for (int t = 0; t < g.depth_taps; ++t)
                for (int r = 0; r < R; ++r)
                    for (int s = 0; s < S; ++s) {
                        const int ih = p * a.stride_h - a.pad_h + r * a.dilation_h, iw = q * a.stride_w - a.pad_w + s * a.dilation_w;
                        const int id = d * a.stride_d - a.pad_d + t * a.dilation_d;
                        const bool inside = ih >= 0 && ih < H && iw >= 0 && iw < W && id >= 0 && id < g.depth_in;
                        const int pixel = n * g.x_n + x_group + (inside ? ih * g.x_h + iw * g.x_w + id * g.x_d : 0);
                        const int tap = filter + (a.reverse ? R - 1 - r : r) * g.w_r + (a.reverse ? S - 1 - s : s) * g.w_s +
                                        (a.reverse ? g.depth_taps - 1 - t : t) * g.w_t;
                        for (int c = 0; c < C; ++c)
                            sum = fmaf(inside ? load_value(g.x, g.x_type, pixel + c * g.x_c) : 0.0f, load_value(g.w, g.w_type, tap + c * g.w_c), sum);
                    }
            store_from_f32(g.y, g.y_type, n * g.y_n + p * g.y_p + q * g.y_q + k * g.y_k + d * g.y_d, apply_epilogue(sum, a, n, k, p, q, d));
        }
    }
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    if (warp == kLoaders / 32) {
        tc_fence_after();
        tmem_dealloc(*tmem_slot, kAccumulatorColumns);
    }
}

}  // namespace

namespace {

struct ClusterForm {
    int tiles_m, tiles_n, units, chunks, ranks, units_per_rank;
};

void share_units(ClusterForm& form, int ranks) {
    form.units_per_rank = (form.units + ranks - 1) / ranks;
    form.ranks = (form.units + form.units_per_rank - 1) / form.units_per_rank;   // (no rank without a unit)
}

bool cluster_form(const dfgpu_conv_params& p, ClusterForm& form) {
    auto plain_float = [](int type) { return type == DFGPU_F32 || type == DFGPU_F16 || type == DFGPU_BF16; };
    if (!plain_float(p.x.dtype) || !plain_float(p.w.dtype) || !plain_float(p.y.dtype)) return false;
    const int rank = p.x.rank;   // 4, or 5 with a depth axis in front of the rows
    if ((rank != 4 && rank != 5) || p.w.rank != rank || p.y.rank != rank) return false;
    // any strides (channels-last, NCHW, padded rows ...), as long as every element lies within 2^31 floats of the first
    auto reach = [](const dfgpu_tensor& t) {
        int64_t last = 0;
        for (int i = 0; i < t.rank; ++i) {
            if (t.stride[i] < 0 || t.dim[i] <= 0) return int64_t{1} << 62;
            last += (t.dim[i] - 1) * t.stride[i];
        }
        return last;
    };
    if (reach(p.x) >= (1ll << 31) || reach(p.w) >= (1ll << 31) || reach(p.y) >= (1ll << 31)) return false;
    if (p.w.dim[1] <= 0 || p.x.dim[1] % p.w.dim[1] != 0 || p.w.dim[0] != p.y.dim[1]) return false;
    const int64_t groups = p.x.dim[1] / p.w.dim[1];
    if (p.y.dim[1] % groups != 0) return false;
    int64_t m_total = p.y.dim[0], taps = 1;
    for (int axis = 2; axis < rank; ++axis) m_total *= p.y.dim[axis], taps *= p.w.dim[axis];
    if (m_total >= (1ll << 31)) return false;
    const int64_t chunks = (p.w.dim[1] + kChunk - 1) / kChunk, tiles_n = groups * ((p.y.dim[1] / groups + kTileN - 1) / kTileN);
    const int64_t tiles = (m_total + kTileM - 1) / kTileM * tiles_n;
    const int64_t units = taps * chunks;
    constexpr int kSms = 148;   // (a query has no device: the count this library is built for)
    if ((m_total + kTileM - 1) / kTileM > 65535 || tiles_n > 65535) return false;   // (grid extents)
    form.tiles_m = static_cast<int>((m_total + kTileM - 1) / kTileM);
    form.tiles_n = static_cast<int>(tiles_n);
    form.units = static_cast<int>(units);
    form.chunks = static_cast<int>(chunks);
    share_units(form, static_cast<int>(std::min<int64_t>(std::min<int64_t>(kMaxRanks, units), std::max<int64_t>(1, kSms / tiles))));
    return form.units_per_rank <= kMaxUnitsPerRank;
}

// How many clusters of each size the device runs at once (index = cluster size).
struct ClusterCapacity {
    int clusters[kMaxRanks + 1];
    cudaError_t error;
};

// Worked out once per device (the shared-memory attribute of the kernel is a per-device setting too).
constexpr int kMaxDevices = 64;
const ClusterCapacity& cluster_capacity() {
    static ClusterCapacity table[kMaxDevices];
    static std::once_flag once[kMaxDevices];
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
        static const ClusterCapacity unknown = [] { ClusterCapacity c{}; c.error = cudaErrorInvalidDevice; return c; }();
        return unknown;
    }
    std::call_once(once[device], [device] {
        ClusterCapacity& c = table[device];
        c = ClusterCapacity{};
        c.error = cudaFuncSetAttribute(umma_conv_f32_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (c.error == cudaSuccess) c.error = cudaFuncSetAttribute(umma_conv_f32_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        for (int ranks = 1; ranks <= kMaxRanks && c.error == cudaSuccess; ++ranks) {
            cudaLaunchConfig_t config{};
            config.gridDim = dim3(ranks, 148, 1);
            config.blockDim = dim3(kThreads);
            config.dynamicSmemBytes = kSmemBytes;
            cudaLaunchAttribute attribute{};
            attribute.id = cudaLaunchAttributeClusterDimension;
            attribute.val.clusterDim.x = ranks;
            attribute.val.clusterDim.y = attribute.val.clusterDim.z = 1;
            config.attrs = &attribute;
            config.numAttrs = 1;
            c.error = cudaOccupancyMaxActiveClusters(&c.clusters[ranks], umma_conv_f32_kernel<false>, &config);   // (the same threads, registers bound and shared memory for both)
        }
    });
    return table[device];
}

}  // namespace

// The launch itself: all tiles' clusters at once, with fewer ranks per tile when the device cannot co-schedule that many
// clusters of the first size.
static int launch_clusters(ClusterForm form, ClusterConvArgs g, const ConvArgs& a, const char* what, cudaStream_t stream) {
    const ClusterCapacity& capacity = cluster_capacity();
    if (capacity.error != cudaSuccess) return fail(kExecutionFailed, "%s: cluster launch set-up failed: %s", what, cudaGetErrorString(capacity.error));
    const int tiles = form.tiles_m * form.tiles_n;
    while (form.ranks > 1 && capacity.clusters[form.ranks] < tiles) share_units(form, form.ranks - 1);
    if (capacity.clusters[form.ranks] < 1) return fail(kExecutionFailed, "%s: the device cannot run a cluster of %d CTAs with %d bytes of shared memory", what, form.ranks, kSmemBytes);
    // float4 accesses where the channels are contiguous and everything else falls on 16-byte boundaries
    auto quads = [](const void* pointer, int type, int64_t channels, int group, int32_t channel_stride, int32_t s0, int32_t s1, int32_t s2, int32_t s3) {
        return type == DFGPU_F32 && channels % group == 0 && channel_stride == 1 && s0 % 4 == 0 && s1 % 4 == 0 && s2 % 4 == 0 && s3 % 4 == 0 &&
               (reinterpret_cast<uintptr_t>(pointer) & 15u) == 0;
    };
    g.x_quads = quads(g.x, g.x_type, a.c_per_group, 8, g.x_c, g.x_n, g.x_h, g.x_w, 0);
    g.w_quads = quads(g.w, g.w_type, a.c_per_group, 8, g.w_c, g.w_k, g.w_r, g.w_s, g.w_n);
    g.y_quads = quads(g.y, g.y_type, a.k_per_group, 4, g.y_k, g.y_n, g.y_p, g.y_q, 0);
    g.w_along_k = !g.w_quads && g.w_k == 1;
    g.units = form.units;
    g.units_per_rank = form.units_per_rank;
    g.chunks = form.chunks;
    g.by_q = make_fast_divisor(static_cast<uint32_t>(g.Q));
    g.by_p = make_fast_divisor(static_cast<uint32_t>(g.P));
    g.by_depth = make_fast_divisor(static_cast<uint32_t>(g.depth_out));
    g.by_plane = make_fast_divisor(static_cast<uint32_t>(g.R * g.S));
    g.by_chunks = make_fast_divisor(static_cast<uint32_t>(form.chunks));
    g.by_s = make_fast_divisor(static_cast<uint32_t>(g.S));
    g.by_tiles = make_fast_divisor(static_cast<uint32_t>(std::max(1, g.tiles_per_image)));
    cudaLaunchConfig_t config{};
    config.gridDim = dim3(form.ranks, form.tiles_m, form.tiles_n);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = form.ranks;
    attribute.val.clusterDim.y = attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    const bool fast = g.x_quads && g.w_quads && g.y_quads && a.groups == 1 && g.tiles_per_image == 0 && g.depth_out * g.depth_in * g.depth_taps == 1;
    cudaError_t error = fast ? cudaLaunchKernelEx(&config, umma_conv_f32_kernel<true>, g, a) : cudaLaunchKernelEx(&config, umma_conv_f32_kernel<false>, g, a);
    if (error != cudaSuccess) return fail(kExecutionFailed, "%s: cluster launch failed: %s", what, cudaGetErrorString(error));
    return check_launch(what);
}

bool conv_f32_cluster_supported(const dfgpu_conv_params& p) {
    ClusterForm form;
    return cluster_form(p, form);
}

int launch_conv_f32_cluster(const dfgpu_conv_params& p, const ConvArgs& a, void* const* tensors, cudaStream_t stream) {
    ClusterForm form;
    if (!cluster_form(p, form)) return fail(kUnsupported, "CONV_FPROP: the one-launch tcgen05 form needs FLOAT, HALF or BFLOAT16 X, W and Y and at most 64 reduction units (64 channels x one tap) per CTA");
    ClusterConvArgs g{};
    g.x = tensors[0], g.w = tensors[1], g.y = tensors[2];
    g.x_type = p.x.dtype, g.w_type = p.w.dtype, g.y_type = p.y.dtype;
    auto stride = [](const dfgpu_tensor& t, int axis) { return static_cast<int32_t>(t.dim[axis] == 1 ? 0 : t.stride[axis]); };   // (< 2^31: cluster_form)
    const int rows = p.x.rank - 2, columns = p.x.rank - 1;   // the axes of the last two spatial extents
    g.P = static_cast<int>(p.y.dim[rows]), g.Q = static_cast<int>(p.y.dim[columns]);
    g.H = static_cast<int>(p.x.dim[rows]), g.W = static_cast<int>(p.x.dim[columns]);
    g.R = static_cast<int>(p.w.dim[rows]), g.S = static_cast<int>(p.w.dim[columns]);
    g.depth_out = g.depth_in = g.depth_taps = 1;
    if (p.x.rank == 5) {
        g.depth_out = static_cast<int>(p.y.dim[2]), g.depth_in = static_cast<int>(p.x.dim[2]), g.depth_taps = static_cast<int>(p.w.dim[2]);
        g.x_d = stride(p.x, 2), g.w_t = stride(p.w, 2), g.y_d = stride(p.y, 2);
    }
    g.m_total = static_cast<int>(p.y.dim[0] * g.depth_out * g.P * g.Q);
    g.x_n = stride(p.x, 0), g.x_c = stride(p.x, 1), g.x_h = stride(p.x, rows), g.x_w = stride(p.x, columns);
    g.w_k = stride(p.w, 0), g.w_c = stride(p.w, 1), g.w_r = stride(p.w, rows), g.w_s = stride(p.w, columns);
    g.y_n = stride(p.y, 0), g.y_k = stride(p.y, 1), g.y_p = stride(p.y, rows), g.y_q = stride(p.y, columns);
    return launch_clusters(form, g, a, "CONV_FPROP", stream);
}

// ---- MATMUL through the same kernel: C[M, N] = A[M, K] B[K, N] is the 1 x 1 convolution of M pixels with K input and N
// output channels, B its filter stored either way round ------------------------------------------------------------------
namespace {
struct MatmulAsConv {
    ClusterForm form;
    int64_t m, n, k, batch;
    int batch_axis;                          // the one batch axis of extent > 1 (-1: none)
    int64_t a_m, a_k, b_k, b_n, c_m, c_n;   // strides in elements
    int64_t a_b, b_b, c_b;                  // ... of the batch axis (0 where the operand is broadcast)
};

bool matmul_cluster_form(const dfgpu_matmul_params& p, MatmulAsConv& f) {
    auto plain_float = [](int type) { return type == DFGPU_F32 || type == DFGPU_F16 || type == DFGPU_BF16; };
    if (!plain_float(p.a.dtype) || !plain_float(p.b.dtype) || !plain_float(p.c.dtype) || p.a_scale.rank || p.b_scale.rank) return false;
    const int rank = p.c.rank;
    if (rank < 2 || p.a.rank != rank || p.b.rank != rank) return false;
    f.batch = 1, f.batch_axis = -1, f.a_b = f.b_b = f.c_b = 0;
    for (int i = 0; i < rank - 2; ++i) {
        if (p.c.dim[i] == 1) continue;
        if (f.batch_axis >= 0) return false;   // (one batch axis: each image of the convolution is one matrix)
        f.batch_axis = i;
        f.batch = p.c.dim[i];
        f.a_b = p.a.dim[i] == 1 ? 0 : p.a.stride[i];
        f.b_b = p.b.dim[i] == 1 ? 0 : p.b.stride[i];
        f.c_b = p.c.stride[i];
    }
    f.m = p.c.dim[rank - 2], f.n = p.c.dim[rank - 1], f.k = p.a.dim[rank - 1];
    if (f.m >= (1ll << 24) || f.m <= 0 || f.n <= 0 || f.k <= 0) return false;
    f.a_m = p.a.stride[rank - 2], f.a_k = p.a.stride[rank - 1];
    f.b_k = p.b.stride[rank - 2], f.b_n = p.b.stride[rank - 1];
    f.c_m = p.c.stride[rank - 2], f.c_n = p.c.stride[rank - 1];
    // any strides (either operand transposed, padded rows), every element within 2^31 elements of the first
    for (int64_t stride : {f.a_m, f.a_k, f.b_k, f.b_n, f.c_m, f.c_n, f.a_b, f.b_b, f.c_b})
        if (stride < 0) return false;
    if ((f.batch - 1) * f.a_b + (f.m - 1) * f.a_m + (f.k - 1) * f.a_k >= (1ll << 31) || (f.batch - 1) * f.b_b + (f.k - 1) * f.b_k + (f.n - 1) * f.b_n >= (1ll << 31) ||
        (f.batch - 1) * f.c_b + (f.m - 1) * f.c_m + (f.n - 1) * f.c_n >= (1ll << 31) || f.batch * f.m >= (1ll << 31))
        return false;
    const int64_t tiles_m = f.batch * ((f.m + kTileM - 1) / kTileM), tiles_n = (f.n + kTileN - 1) / kTileN, units = (f.k + kChunk - 1) / kChunk;
    const int64_t tiles = tiles_m * tiles_n;
    constexpr int kSms = 148;
    if (tiles_m > 65535 || tiles_n > 65535) return false;
    f.form.tiles_m = static_cast<int>(tiles_m);
    f.form.tiles_n = static_cast<int>(tiles_n);
    f.form.units = f.form.chunks = static_cast<int>(units);
    share_units(f.form, static_cast<int>(std::min<int64_t>(std::min<int64_t>(kMaxRanks, units), std::max<int64_t>(1, kSms / tiles))));
    return f.form.units_per_rank <= kMaxUnitsPerRank;
}
}  // namespace

bool matmul_f32_cluster_supported(const dfgpu_matmul_params& p) {
    MatmulAsConv f;
    return matmul_cluster_form(p, f);
}

int launch_matmul_f32_cluster(const dfgpu_matmul_params& p, void* const* tensors, cudaStream_t stream) {
    MatmulAsConv f;
    if (!matmul_cluster_form(p, f)) return fail(kUnsupported, "MATMUL: the one-launch tcgen05 form needs FLOAT, HALF or BFLOAT16 A, B and C and at most one batch axis");
    // The convolution's view of the problem: one image of 1 x M pixels with K channels in and N out; an epilogue operand
    // [.., M, N] becomes [1, N, 1, M].
    ConvArgs a{};
    auto image = [](int64_t channels, int64_t pixels) {
        View v{};
        v.dtype = DFGPU_F32;
        v.rank = 4;
        v.dim[0] = 1, v.dim[1] = channels, v.dim[2] = 1, v.dim[3] = pixels;
        return v;
    };
    a.x = image(f.k, f.m);
    a.y = image(f.n, f.m);
    a.x.dim[0] = a.y.dim[0] = f.batch;   // (one image per matrix of the batch)
    a.w = image(f.k, 1);
    a.w.dim[0] = f.n;
    a.epilogue = make_epilogue(p.epilogue_count, p.epilogue);
    for (int i = 0; i < 2; ++i) {
        const dfgpu_tensor& t = p.extra[i];
        View v{};
        v.dtype = t.dtype;
        v.rank = 4;
        for (int d = 0; d < 4; ++d) v.dim[d] = 1;
        if (t.rank >= 1) v.dim[1] = t.dim[t.rank - 1], v.stride[1] = t.stride[t.rank - 1];
        if (t.rank >= 2) v.dim[3] = t.dim[t.rank - 2], v.stride[3] = t.stride[t.rank - 2];
        const int own_axis = f.batch_axis - (p.c.rank - t.rank);   // the operand's axis under C's batch axis
        if (f.batch_axis >= 0 && own_axis >= 0) v.dim[0] = t.dim[own_axis], v.stride[0] = t.stride[own_axis];
        a.extra[i] = v;
        a.extra_data[i] = tensors[5 + i];
    }
    a.stride_h = a.stride_w = a.dilation_h = a.dilation_w = 1;
    a.groups = 1;
    a.c_per_group = f.k;
    a.k_per_group = f.n;
    ClusterConvArgs g{};
    g.x = tensors[0], g.w = tensors[1], g.y = tensors[2];
    g.x_type = p.a.dtype, g.w_type = p.b.dtype, g.y_type = p.c.dtype;
    g.P = g.H = g.R = g.S = 1;
    g.Q = g.W = static_cast<int>(f.m);
    g.depth_out = g.depth_in = g.depth_taps = 1;
    g.m_total = static_cast<int>(f.batch * f.m);
    if (f.batch > 1) {
        g.tiles_per_image = static_cast<int>((f.m + kTileM - 1) / kTileM);
        g.x_n = static_cast<int32_t>(f.a_b), g.y_n = static_cast<int32_t>(f.c_b), g.w_n = static_cast<int32_t>(f.b_b);
    }
    auto stride = [](int64_t extent, int64_t step) { return static_cast<int32_t>(extent == 1 ? 0 : step); };   // (< 2^31: matmul_cluster_form)
    g.x_w = stride(f.m, f.a_m), g.x_c = stride(f.k, f.a_k);   // (one image, one row of pixels: the other strides are never multiplied by anything but 0)
    g.w_k = stride(f.n, f.b_n), g.w_c = stride(f.k, f.b_k);
    g.y_q = stride(f.m, f.c_m), g.y_k = stride(f.n, f.c_n);
    return launch_clusters(f.form, g, a, "MATMUL", stream);
}

int conv_f32_device_status(int* status) { return read_and_clear_device_status(status); }

}  // namespace dfgpu

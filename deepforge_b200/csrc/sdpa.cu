// SDPA forward on CUDA cores.
//
//  * sdpa_rowwise_kernel: one warp per (batch, head, query) row; covers every case
//    the launcher accepts (f32/f16/bf16, any strides with unit head-dim stride, GQA,
//    padding mask, left/right bounds with either diagonal alignment, paged K/V,
//    Stats/Max/Sum_exp). It is the general kernel and the one small graphs use.
//  * sdpa_paged_decode_kernel (+ merge): the bandwidth-bound decode case -- one query
//    token per sequence, bf16, head dim 128, K/V in a paged pool. Split-KV: a CTA
//    streams 256 tokens of one (sequence, kv head) for all query heads of the GQA
//    group, so each K/V byte is read from HBM exactly once; a second kernel merges
//    the per-chunk (max, sum, partial O) triples.
//
// Semantics follow the reference: score = attn_scale * dot(q, k); a score is valid
// iff padding/bounds allow it; max and sum run over valid scores only; a row with
// no valid score gives O = 0, Stats = Max = -inf, Sum_exp = 0; an out-of-range page
// id reads as zeros without touching memory.
#include <atomic>
#include <cmath>
#include "common.cuh"
#include "umma.cuh"

namespace dfgpu {
namespace {

struct SdpaArgs {
    View q, k, v, o, stats, max, sum_exp, seq_q, seq_kv, table_k, table_v, bias;
    const void* bias_data;
    View sink;
    const float* sink_data;
    View block_mask;
    const uint8_t* block_mask_data;
    int32_t alibi;
    float alibi_slope_scale;  // -8 / n, n the largest power of two not above the head count
    int32_t alibi_n;
    const void* q_data;
    const void* k_data;
    const void* v_data;
    void* o_data;
    void* stats_data;
    void* max_data;
    void* sum_exp_data;
    const int32_t* seq_q_data;
    const int32_t* seq_kv_data;
    const int32_t* table_k_data;
    const int32_t* table_v_data;
    // compact page tables: per-batch element offsets into the table's storage (null: the table is strided [B,1,P,1])
    const void* offsets_k_data;
    const void* offsets_v_data;
    int32_t offsets_k_wide, offsets_v_wide;      // INT64 offsets
    int64_t offsets_k_stride, offsets_v_stride;  // elements between consecutive batch entries
    const int* prefix_ok;                        // [2] written by the validation kernel: K table, V table
    float scale;
    int32_t padding, has_left, has_right, bottom_right;
    int64_t left, right, s_kv;
    // dropout on the probabilities that weight V: 0 none, 1 the counter-based Bernoulli stream, 2 the caller's mask
    int32_t dropout_kind;
    uint32_t keep_threshold;       // floor((1 - probability) * 2^24): a 24-bit sample below it keeps the element
    float dropout_scale;           // kind 1: 1 / (1 - probability)
    View dropout_mask, rng_dump;
    const float* dropout_mask_data;
    const float* dropout_scale_data;
    const int64_t* seed_data;
    const int64_t* offset_data;
    float* rng_dump_data;
};

// The reference's Bernoulli stream (lib/Compiler/SequenceGraph.cpp:1413-1456): a splitmix64 round over seed + offset + the flat index of
// the score, whose top 24 bits are compared with the threshold.
__device__ __forceinline__ float bernoulli_keep(int64_t seed, int64_t offset, int64_t linear, uint32_t threshold) {
    uint64_t z = static_cast<uint64_t>(seed) + static_cast<uint64_t>(offset) + static_cast<uint64_t>(linear) + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (z >> 40) < threshold ? 1.0f : 0.0f;
}

__device__ __forceinline__ int64_t off4(const View& t, int64_t a, int64_t b, int64_t c, int64_t d) {
    return a * t.stride[0] + b * t.stride[1] + c * t.stride[2] + d * t.stride[3];
}

// Key range [lo, hi) that is valid for query row iq of batch ib (empty if lo >= hi).
__device__ __forceinline__ void valid_range(const SdpaArgs& a, int64_t ib, int64_t iq, int64_t& lo, int64_t& hi) {
    lo = 0;
    hi = a.s_kv;
    int64_t len_q = 0, len_kv = 0;
    if (a.padding) {
        len_q = a.seq_q_data[ib * a.seq_q.stride[0]];
        len_kv = a.seq_kv_data[ib * a.seq_kv.stride[0]];
        if (!(iq < len_q)) { hi = 0; return; }
        if (len_kv < hi) hi = len_kv;
    }
    int64_t shift = 0;
    if (a.bottom_right) shift = a.padding ? len_kv - len_q : a.s_kv - a.q.dim[2];
    if (a.has_right) {
        int64_t bound = iq + shift + a.right + 1;  // kv - q <= shift + right
        if (bound < hi) hi = bound;
    }
    if (a.has_left) {
        int64_t bound = iq + shift - a.left + 1;  // kv - q > shift - left
        if (bound > lo) lo = bound;
    }
    if (hi < 0) hi = 0;
}

__device__ __forceinline__ int64_t load_offset(const void* data, int wide, int64_t index) {
    return wide ? static_cast<const int64_t*>(data)[index] : static_cast<int64_t>(static_cast<const int32_t*>(data)[index]);
}

// Page id of (batch ib, table slot), or -1 where the table holds none: a strided table has dim[2] slots per batch; a
// compact one (which = 0 K, 1 V) has the slots its batch's sequence length needs, at offsets[ib] + slot * stride[2],
// and none at all when its prefix failed validation.
__device__ __forceinline__ int64_t page_of_slot(const SdpaArgs& a, int which, int64_t ib, int64_t slot) {
    const View& table = which ? a.table_v : a.table_k;
    const int32_t* data = which ? a.table_v_data : a.table_k_data;
    const void* offsets = which ? a.offsets_v_data : a.offsets_k_data;
    if (!offsets) return slot < table.dim[2] ? static_cast<int64_t>(data[off4(table, ib, 0, slot, 0)]) : -1;
    if (!a.prefix_ok[which]) return -1;
    const int64_t block = which ? a.v.dim[2] : a.k.dim[2];
    const int64_t length = a.seq_kv_data[ib * a.seq_kv.stride[0]];
    if (slot >= (length + block - 1) / block) return -1;
    const int64_t base = load_offset(offsets, which ? a.offsets_v_wide : a.offsets_k_wide, ib * (which ? a.offsets_v_stride : a.offsets_k_stride));
    return data[base + slot * table.stride[2]];
}

// Base offset of the row (token ikv, head) of a K/V container (which = 0 K, 1 V), or -1 for an invalid page.
__device__ __forceinline__ int64_t kv_row_offset(const SdpaArgs& a, int which, int64_t ib, int64_t head, int64_t ikv) {
    const View& t = which ? a.v : a.k;
    const View& table = which ? a.table_v : a.table_k;
    if (table.rank == 0) return off4(t, ib, head, ikv, 0);
    int64_t block = t.dim[2];
    int64_t slot = ikv / block, within = ikv - slot * block;
    int64_t page = page_of_slot(a, which, ib, slot);
    if (page < 0 || page >= t.dim[0]) return -1;
    return off4(t, page, head, within, 0);
}

// Validation of a compact page table's batch prefix, one CTA per table (blockIdx.x = 0 K, 1 V): the rules of the
// reference's host-side check (lib/Runtime/Executable.cpp:619-716), applied where the offsets live. Writes
// prefix_ok[table] and, on failure, a status code the host reads through dfgpu_device_status().
__device__ int g_sdpa_status = 0;

__global__ void __launch_bounds__(256)
validate_page_prefix_kernel(SdpaArgs a, int* prefix_ok) {
    const int which = blockIdx.x;
    const void* offsets = which ? a.offsets_v_data : a.offsets_k_data;
    if (!offsets) {
        if (threadIdx.x == 0) prefix_ok[which] = 1;
        return;
    }
    const View& table = which ? a.table_v : a.table_k;
    const int wide = which ? a.offsets_v_wide : a.offsets_k_wide;
    const int64_t stride = which ? a.offsets_v_stride : a.offsets_k_stride;
    const int64_t batches = table.dim[0], block = which ? a.v.dim[2] : a.k.dim[2];
    const int64_t bound = batches * ((table.dim[2] - 1) * table.stride[2] + 1);  // the compiled storage bound, in entries
    bool bad = load_offset(offsets, wide, 0) != 0;
    for (int64_t b = threadIdx.x; b < batches; b += blockDim.x) {
        const int64_t start = load_offset(offsets, wide, b * stride), end = load_offset(offsets, wide, (b + 1) * stride);
        const int64_t length = a.seq_kv_data[b * a.seq_kv.stride[0]];
        if (start < 0 || end < start || end > bound) bad = true;
        if (length < 0 || length > table.dim[2] * block) bad = true;
        const int64_t slots = (length + block - 1) / block;
        const int64_t needed = slots > 0 ? 1 + (slots - 1) * table.stride[2] : 0;
        if (end - start < needed) bad = true;
    }
    const int any_bad = __syncthreads_or(bad ? 1 : 0);
    if (threadIdx.x == 0) {
        prefix_ok[which] = any_bad ? 0 : 1;
        if (any_bad) atomicCAS(&g_sdpa_status, 0, 601 + which);
    }
}

constexpr int kRowwiseMaxD = 256;
constexpr int kPrefixScratchBytes = 256;  // the two validation results of compact page tables, ahead of a kernel's own scratch

__global__ void __launch_bounds__(128)
sdpa_rowwise_kernel(SdpaArgs a, int64_t rows) {
    __shared__ float q_shared[4][kRowwiseMaxD];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + warp;
    if (row >= rows) return;
    const int64_t sq = a.q.dim[2], hq = a.q.dim[1];
    const int64_t iq = row % sq;
    const int64_t ih = (row / sq) % hq;
    const int64_t ib = row / (sq * hq);
    const int64_t kh = ih / (hq / a.k.dim[1]);
    const int64_t vh = ih / (hq / a.v.dim[1]);
    const int dqk = static_cast<int>(a.q.dim[3]);
    const int dv = static_cast<int>(a.v.dim[3]);
    float* qs = q_shared[warp];
    for (int d = lane; d < dqk; d += 32) qs[d] = load_as_f32(a.q_data, a.q.dtype, off4(a.q, ib, ih, iq, d));
    __syncwarp();

    int64_t lo, hi;
    valid_range(a, ib, iq, lo, hi);
    float dropout_scale = 1.0f;
    int64_t seed = 0, stream_offset = 0;
    const int64_t linear_row = ((ib * hq + ih) * sq + iq) * a.s_kv;   // flat index of this row's first score in [B, Hq, Sq, Skv]
    if (a.dropout_kind == 1) {
        dropout_scale = a.dropout_scale;
        seed = a.seed_data[0];
        stream_offset = a.offset_data[0];
        if (a.rng_dump.rank)   // the mask of every position of the row, masked ones too
            for (int64_t ikv = lane; ikv < a.s_kv; ikv += 32)
                a.rng_dump_data[off4(a.rng_dump, ib, ih, iq, ikv)] = bernoulli_keep(seed, stream_offset, linear_row + ikv, a.keep_threshold);
    } else if (a.dropout_kind == 2) {
        dropout_scale = a.dropout_scale_data[0];
    }
    float running_max = -INFINITY, running_sum = 0.0f;
    if (a.sink.rank) {  // the sink logit takes part in the maximum and the sum, not in O
        running_max = a.sink_data[ih * a.sink.stride[1]];
        running_sum = 1.0f;
    }
    float acc[kRowwiseMaxD / 32];
#pragma unroll
    for (int i = 0; i < kRowwiseMaxD / 32; ++i) acc[i] = 0.0f;

    for (int64_t base = lo; base < hi; base += 32) {
        int64_t ikv = base + lane;
        float score = -INFINITY;
        bool enabled = ikv < hi;
        if (enabled && a.block_mask.rank) {
            const int64_t key_tile = ikv >> 7;
            const uint32_t byte = a.block_mask_data[off4(a.block_mask, ib, ih, iq >> 7, key_tile >> 3)];
            enabled = ((byte >> (key_tile & 7)) & 1u) != 0u;
        }
        if (enabled) {
            int64_t offset = kv_row_offset(a, 0, ib, kh, ikv);
            float dot = 0.0f;
            if (offset >= 0) {
                if (a.k.dtype == DFGPU_BF16 && (dqk & 7) == 0 && (offset & 7) == 0 &&
                    (reinterpret_cast<uintptr_t>(a.k_data) & 15u) == 0) {
                    const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(a.k_data) + offset);
                    for (int d = 0; d < dqk; d += 8) {
                        uint4 raw = __ldg(p + (d >> 3));
                        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            dot = fmaf(qs[d + 2 * i], __uint_as_float(w[i] << 16), dot);
                            dot = fmaf(qs[d + 2 * i + 1], __uint_as_float(w[i] & 0xffff0000u), dot);
                        }
                    }
                } else {
                    for (int d = 0; d < dqk; ++d) dot = fmaf(qs[d], load_as_f32(a.k_data, a.k.dtype, offset + d), dot);
                }
            }
            score = __fmul_rn(a.scale, dot);
            if (a.bias.rank) {
                const int64_t offset = (a.bias.dim[0] == 1 ? 0 : ib) * a.bias.stride[0] + (a.bias.dim[1] == 1 ? 0 : ih) * a.bias.stride[1] +
                                       (a.bias.dim[2] == 1 ? 0 : iq) * a.bias.stride[2] + (a.bias.dim[3] == 1 ? 0 : ikv) * a.bias.stride[3];
                score = __fadd_rn(score, load_as_f32(a.bias_data, a.bias.dtype, offset));
            }
            if (a.alibi) {
                // slope of head h: 2^(-8 (h+1) / n) for h < n, else 2^(-8 (2 (h-n) + 1) / 2 / n)
                const float position = ih < a.alibi_n ? static_cast<float>(ih + 1) : (static_cast<float>(2 * (ih - a.alibi_n) + 1) * 0.5f);
                const float slope = exp2f(__fmul_rn(a.alibi_slope_scale, position));
                score = __fadd_rn(score, __fmul_rn(static_cast<float>(ikv - iq), slope));
            }
        }
        float chunk_max = score;
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) chunk_max = fmaxf(chunk_max, __shfl_xor_sync(0xffffffffu, chunk_max, s));
        float new_max = fmaxf(running_max, chunk_max);
        float correction = running_max == -INFINITY ? 0.0f : expf(running_max - new_max);
        float probability = (enabled && new_max != -INFINITY) ? expf(score - new_max) : 0.0f;
        float chunk_sum = probability;
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) chunk_sum += __shfl_xor_sync(0xffffffffu, chunk_sum, s);
        running_sum = running_sum * correction + chunk_sum;
        running_max = new_max;
#pragma unroll
        for (int i = 0; i < kRowwiseMaxD / 32; ++i) acc[i] *= correction;
        // what weights V: (p * mask) * scale; the maximum and the sum above are those without dropout
        float weight = probability;
        if (a.dropout_kind != 0 && enabled) {
            float mask;
            if (a.dropout_kind == 1) {
                mask = bernoulli_keep(seed, stream_offset, linear_row + ikv, a.keep_threshold);
            } else {
                const View& t = a.dropout_mask;
                mask = a.dropout_mask_data[(t.dim[0] == 1 ? 0 : ib) * t.stride[0] + (t.dim[1] == 1 ? 0 : ih) * t.stride[1] +
                                           (t.dim[2] == 1 ? 0 : iq) * t.stride[2] + (t.dim[3] == 1 ? 0 : ikv) * t.stride[3]];
            }
            weight = __fmul_rn(__fmul_rn(probability, mask), dropout_scale);
        }
        int count = static_cast<int>(hi - base < 32 ? hi - base : 32);
        for (int j = 0; j < count; ++j) {
            float pj = __shfl_sync(0xffffffffu, weight, j);
            int64_t offset = kv_row_offset(a, 1, ib, vh, base + j);
            if (offset < 0) continue;
#pragma unroll
            for (int i = 0; i < kRowwiseMaxD / 32; ++i) {
                int d = lane + 32 * i;
                if (d < dv) acc[i] = fmaf(pj, load_as_f32(a.v_data, a.v.dtype, offset + d), acc[i]);
            }
        }
    }
    float inverse = running_sum > 0.0f ? 1.0f / running_sum : 0.0f;
#pragma unroll
    for (int i = 0; i < kRowwiseMaxD / 32; ++i) {
        int d = lane + 32 * i;
        if (d < dv) store_from_f32(a.o_data, a.o.dtype, off4(a.o, ib, ih, iq, d), acc[i] * inverse);
    }
    if (lane == 0) {
        if (a.stats.rank) store_from_f32(a.stats_data, a.stats.dtype, off4(a.stats, ib, ih, iq, 0), running_max + logf(running_sum));
        if (a.max.rank) store_from_f32(a.max_data, a.max.dtype, off4(a.max, ib, ih, iq, 0), running_max);
        if (a.sum_exp.rank) store_from_f32(a.sum_exp_data, a.sum_exp.dtype, off4(a.sum_exp, ib, ih, iq, 0), running_sum);
    }
}

// ---- paged decode ------------------------------------------------------------------

constexpr int kDecodeChunk = 256;   // tokens per CTA
constexpr int kDecodeD = 128;       // head dim
constexpr int kDecodeMaxGroup = 8;  // query heads per kv head
constexpr int kPartialStride = kDecodeD + 2;  // o[128], max, sum

__device__ __forceinline__ void unpack8(const uint4& raw, float (&out)[8]) {
    uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        out[2 * i] = __uint_as_float(w[i] << 16);
        out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <int G>
__global__ void __launch_bounds__(256)
sdpa_paged_decode_kernel(SdpaArgs a, float* __restrict__ partial, int max_chunks) {
    __shared__ float scores[G][kDecodeChunk];
    __shared__ float reduce[8][G][kDecodeD / 4 + 1];  // staged in 4 passes of 32 columns
    __shared__ int64_t page_base_k[kDecodeChunk / 16];
    __shared__ int64_t page_base_v[kDecodeChunk / 16];
    __shared__ float head_max[G], head_sum[G];

    const int chunk = blockIdx.x;
    const int64_t hkv = blockIdx.y;
    const int64_t ib = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t hq = a.q.dim[1];

    int64_t lo, hi;
    valid_range(a, ib, 0, lo, hi);
    const int64_t chunk_begin = static_cast<int64_t>(chunk) * kDecodeChunk;
    float* my_partial = partial + ((ib * hq + hkv * G) * max_chunks + chunk) * kPartialStride;
    if (chunk_begin >= hi || chunk_begin + kDecodeChunk <= lo) {
        // nothing valid here: publish an empty partial so the merge can skip it
        if (tid < G) {
            float* p = my_partial + static_cast<int64_t>(tid) * max_chunks * kPartialStride;
            p[kDecodeD] = -INFINITY;
            p[kDecodeD + 1] = 0.0f;
        }
        return;
    }

    // page bases for this chunk (block sizes are powers of two between 16 and 256)
    const int64_t block = a.k.dim[2];
    const int pages_in_chunk = static_cast<int>(kDecodeChunk / block) > 0 ? static_cast<int>(kDecodeChunk / block) : 1;
    if (tid < pages_in_chunk) {
        int64_t slot = chunk_begin / block + tid;
        int64_t kb = -1, vb = -1;
        {
            int64_t page = page_of_slot(a, 0, ib, slot);
            if (page >= 0 && page < a.k.dim[0]) kb = page * a.k.stride[0] + hkv * a.k.stride[1];
        }
        {
            int64_t page = page_of_slot(a, 1, ib, slot);
            if (page >= 0 && page < a.v.dim[0]) vb = page * a.v.stride[0] + hkv * a.v.stride[1];
        }
        page_base_k[tid] = kb;
        page_base_v[tid] = vb;
    }

    // phase 1: scores. 8 lanes per token, each lane owns 16 of the 128 head-dim elements.
    const int part = lane & 7, token_in_warp = lane >> 3;
    float qreg[G][16];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const uint16_t* qp = static_cast<const uint16_t*>(a.q_data) + off4(a.q, ib, hkv * G + g, 0, part * 16);
        uint4 r0 = __ldg(reinterpret_cast<const uint4*>(qp));
        uint4 r1 = __ldg(reinterpret_cast<const uint4*>(qp) + 1);
        float lo8[8], hi8[8];
        unpack8(r0, lo8);
        unpack8(r1, hi8);
#pragma unroll
        for (int i = 0; i < 8; ++i) { qreg[g][i] = lo8[i]; qreg[g][8 + i] = hi8[i]; }
    }
    __syncthreads();

    const uint16_t* kdata = static_cast<const uint16_t*>(a.k_data);
#pragma unroll 2
    for (int step = 0; step < kDecodeChunk / 32; ++step) {
        int token = step * 32 + warp * 4 + token_in_warp;
        int64_t ikv = chunk_begin + token;
        int64_t base = page_base_k[token / block];
        bool in_range = ikv >= lo && ikv < hi;
        float dot[G];
#pragma unroll
        for (int g = 0; g < G; ++g) dot[g] = 0.0f;
        if (in_range && base >= 0) {
            const uint4* kp = reinterpret_cast<const uint4*>(kdata + base + (ikv % block) * a.k.stride[2] + part * 16);
            uint4 r0 = __ldg(kp), r1 = __ldg(kp + 1);
            float kv[16];
            {
                float lo8[8], hi8[8];
                unpack8(r0, lo8);
                unpack8(r1, hi8);
#pragma unroll
                for (int i = 0; i < 8; ++i) { kv[i] = lo8[i]; kv[8 + i] = hi8[i]; }
            }
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int i = 0; i < 16; ++i) dot[g] = fmaf(qreg[g][i], kv[i], dot[g]);
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            dot[g] += __shfl_xor_sync(0xffffffffu, dot[g], 1);
            dot[g] += __shfl_xor_sync(0xffffffffu, dot[g], 2);
            dot[g] += __shfl_xor_sync(0xffffffffu, dot[g], 4);
        }
        if (part == 0) {
#pragma unroll
            for (int g = 0; g < G; ++g) scores[g][token] = in_range ? __fmul_rn(a.scale, dot[g]) : -INFINITY;
        }
    }
    __syncthreads();

    // phase 2: per-head max / exp / sum over the chunk; warp g owns head g.
    if (warp < G) {
        float local_max = -INFINITY;
#pragma unroll
        for (int i = 0; i < kDecodeChunk / 32; ++i) local_max = fmaxf(local_max, scores[warp][lane + 32 * i]);
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) local_max = fmaxf(local_max, __shfl_xor_sync(0xffffffffu, local_max, s));
        float local_sum = 0.0f;
#pragma unroll
        for (int i = 0; i < kDecodeChunk / 32; ++i) {
            float s = scores[warp][lane + 32 * i];
            float p = (s == -INFINITY) ? 0.0f : expf(s - local_max);
            scores[warp][lane + 32 * i] = p;
            local_sum += p;
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) local_sum += __shfl_xor_sync(0xffffffffu, local_sum, s);
        if (lane == 0) { head_max[warp] = local_max; head_sum[warp] = local_sum; }
    }
    __syncthreads();

    // phase 3: partial O. 16 lanes per token row, 8 head-dim elements per lane.
    const int column = (lane & 15) * 8, row_in_warp = lane >> 4;
    float acc[G][8];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = 0.0f;
    const uint16_t* vdata = static_cast<const uint16_t*>(a.v_data);
#pragma unroll 4
    for (int step = 0; step < kDecodeChunk / 16; ++step) {
        int token = step * 16 + warp * 2 + row_in_warp;
        int64_t ikv = chunk_begin + token;
        int64_t base = page_base_v[token / block];
        if (ikv >= lo && ikv < hi && base >= 0) {
            uint4 raw = __ldg(reinterpret_cast<const uint4*>(vdata + base + (ikv % block) * a.v.stride[2] + column));
            float vv[8];
            unpack8(raw, vv);
#pragma unroll
            for (int g = 0; g < G; ++g) {
                float p = scores[g][token];
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(p, vv[i], acc[g][i]);
            }
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] += __shfl_xor_sync(0xffffffffu, acc[g][i], 16);

    // cross-warp reduction, 32 columns at a time to keep shared memory small
    for (int pass = 0; pass < 4; ++pass) {
        __syncthreads();
        if (lane < 16 && (column >> 5) == pass) {
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int i = 0; i < 8; ++i) reduce[warp][g][(column & 31) + i] = acc[g][i];
        }
        __syncthreads();
        for (int e = tid; e < G * 32; e += 256) {
            int g = e >> 5, c = e & 31;
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) sum += reduce[w][g][c];
            my_partial[static_cast<int64_t>(g) * max_chunks * kPartialStride + pass * 32 + c] = sum;
        }
    }
    if (tid < G) {
        float* p = my_partial + static_cast<int64_t>(tid) * max_chunks * kPartialStride;
        p[kDecodeD] = head_max[tid];
        p[kDecodeD + 1] = head_sum[tid];
    }
}

// One CTA of 128 threads per (batch, query head): combine the chunk partials.
__global__ void __launch_bounds__(128)
sdpa_decode_merge_kernel(SdpaArgs a, const float* __restrict__ partial, int max_chunks, int chunk_keys) {
    const int64_t row = blockIdx.x;  // b * Hq + h
    const int64_t hq = a.q.dim[1];
    const int64_t ib = row / hq, ih = row % hq;
    const int d = threadIdx.x;
    int64_t lo, hi;
    valid_range(a, ib, 0, lo, hi);
    int chunks = hi > 0 ? static_cast<int>((hi + chunk_keys - 1) / chunk_keys) : 0;
    if (chunks > max_chunks) chunks = max_chunks;
    const float* base = partial + row * max_chunks * kPartialStride;
    float total_max = -INFINITY;
    for (int c = 0; c < chunks; ++c) total_max = fmaxf(total_max, base[c * kPartialStride + kDecodeD]);
    float total_sum = 0.0f, value = 0.0f;
    for (int c = 0; c < chunks; ++c) {
        float m = base[c * kPartialStride + kDecodeD];
        if (m == -INFINITY) continue;
        float weight = expf(m - total_max);
        total_sum = fmaf(base[c * kPartialStride + kDecodeD + 1], weight, total_sum);
        value = fmaf(base[c * kPartialStride + d], weight, value);
    }
    float result = total_sum > 0.0f ? value / total_sum : 0.0f;
    store_from_f32(a.o_data, a.o.dtype, off4(a.o, ib, ih, 0, d), result);
    if (d == 0) {
        if (a.stats.rank) store_from_f32(a.stats_data, a.stats.dtype, off4(a.stats, ib, ih, 0, 0), total_max + logf(total_sum));
        if (a.max.rank) store_from_f32(a.max_data, a.max.dtype, off4(a.max, ib, ih, 0, 0), total_max);
        if (a.sum_exp.rank) store_from_f32(a.sum_exp_data, a.sum_exp.dtype, off4(a.sum_exp, ib, ih, 0, 0), total_sum);
    }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int build_args(const dfgpu_sdpa_params& p, void* const* tensors, SdpaArgs& a) {
    if (!valid_tensor(p.q) || !valid_tensor(p.k) || !valid_tensor(p.v) || !valid_tensor(p.o))
        return fail(kInvalidShape, "SDPA: tensor rank or extent out of range");
    if (p.q.rank != 4 || p.k.rank != 4 || p.v.rank != 4 || p.o.rank != 4)
        return fail(kInvalidShape, "SDPA: Q, K, V and O must have rank 4");
    if (p.q.stride[3] != 1 || p.k.stride[3] != 1 || p.v.stride[3] != 1 || p.o.stride[3] != 1)
        return fail(kInvalidLayout, "SDPA: the head dimension must have unit stride");
    auto float_type = [](int t) { return t == DFGPU_F32 || t == DFGPU_F16 || t == DFGPU_BF16; };
    if (!float_type(p.q.dtype) || !float_type(p.k.dtype) || !float_type(p.v.dtype) || !float_type(p.o.dtype))
        return fail(kUnsupported, "SDPA: Q, K, V and O must be FLOAT, HALF or BFLOAT16");
    int64_t hq = p.q.dim[1], hk = p.k.dim[1], hv = p.v.dim[1];
    if (hk <= 0 || hv <= 0 || hq % hk != 0 || hq % hv != 0) return fail(kInvalidShape, "SDPA: query heads must be a multiple of K and V heads");
    if (p.k.dim[3] != p.q.dim[3]) return fail(kInvalidShape, "SDPA: Q and K head dimensions differ");
    if (p.o.dim[0] != p.q.dim[0] || p.o.dim[1] != hq || p.o.dim[2] != p.q.dim[2] || p.o.dim[3] != p.v.dim[3])
        return fail(kInvalidShape, "SDPA: O must be [B, Hq, Sq, Dv]");
    bool paged_k = p.page_table_k.rank != 0, paged_v = p.page_table_v.rank != 0;
    const dfgpu_tensor* tables[2] = {&p.page_table_k, &p.page_table_v};
    const dfgpu_tensor* containers[2] = {&p.k, &p.v};
    for (int i = 0; i < 2; ++i) {
        const dfgpu_tensor& table = *tables[i];
        if (table.rank == 0) {
            if (containers[i]->dim[0] != p.q.dim[0] || containers[i]->dim[2] < p.s_kv)
                return fail(kInvalidShape, "SDPA: K/V batch or sequence extent is inconsistent");
            continue;
        }
        if (table.rank != 4 || table.dtype != DFGPU_I32 || table.dim[0] != p.q.dim[0] || table.dim[1] != 1 || table.dim[3] != 1)
            return fail(kInvalidShape, "SDPA: page table must be INT32 [B,1,P,1]");
        if (table.dim[2] * containers[i]->dim[2] < p.s_kv) return fail(kInvalidShape, "SDPA: page table capacity is below the key/value length");
        const dfgpu_tensor& offsets = i == 0 ? p.page_offsets_k : p.page_offsets_v;
        if (offsets.rank != 0) {
            if (offsets.rank != 4 || (offsets.dtype != DFGPU_I32 && offsets.dtype != DFGPU_I64) || offsets.dim[0] != p.q.dim[0] + 1 || offsets.dim[1] != 1 ||
                offsets.dim[2] != 1 || offsets.dim[3] != 1)
                return fail(kInvalidShape, "SDPA: page table offsets must be INT32 or INT64 [B+1,1,1,1]");
            if (table.stride[2] <= 0) return fail(kInvalidLayout, "SDPA: a compact page table needs a positive slot stride");
        }
    }
    if ((p.page_offsets_k.rank && !paged_k) || (p.page_offsets_v.rank && !paged_v)) return fail(kInvalidArgument, "SDPA: page table offsets without a page table");
    if ((paged_k || paged_v) && !p.padding_mask) return fail(kInvalidArgument, "SDPA: paged K/V requires the padding mask and sequence lengths");
    if (p.padding_mask) {
        if (p.seq_q.rank == 0 || p.seq_kv.rank == 0 || p.seq_q.dtype != DFGPU_I32 || p.seq_kv.dtype != DFGPU_I32)
            return fail(kInvalidArgument, "SDPA: padding mask needs INT32 SEQ_LEN_Q and SEQ_LEN_KV");
        if (p.seq_q.dim[0] != p.q.dim[0] || p.seq_kv.dim[0] != p.q.dim[0]) return fail(kInvalidShape, "SDPA: sequence length tensors must be [B,1,1,1]");
    }
    if (p.s_kv <= 0) return fail(kInvalidShape, "SDPA: key/value length must be positive");
    const dfgpu_tensor* row_outputs[3] = {&p.stats, &p.max, &p.sum_exp};
    for (const dfgpu_tensor* t : row_outputs) {
        if (t->rank == 0) continue;
        if (t->rank != 4 || t->dim[0] != p.q.dim[0] || t->dim[1] != hq || t->dim[2] != p.q.dim[2] || t->dim[3] != 1 || !float_type(t->dtype))
            return fail(kInvalidShape, "SDPA: row outputs must be [B, Hq, Sq, 1]");
    }
    a.q = make_view(p.q); a.k = make_view(p.k); a.v = make_view(p.v); a.o = make_view(p.o);
    a.stats = make_view(p.stats); a.max = make_view(p.max); a.sum_exp = make_view(p.sum_exp);
    a.seq_q = make_view(p.seq_q); a.seq_kv = make_view(p.seq_kv);
    a.table_k = make_view(p.page_table_k); a.table_v = make_view(p.page_table_v);
    if (tensors) {
        a.q_data = tensors[0]; a.k_data = tensors[1]; a.v_data = tensors[2]; a.o_data = tensors[3];
        a.stats_data = tensors[4]; a.max_data = tensors[5]; a.sum_exp_data = tensors[6];
        a.seq_q_data = static_cast<const int32_t*>(tensors[7]);
        a.seq_kv_data = static_cast<const int32_t*>(tensors[8]);
        a.table_k_data = static_cast<const int32_t*>(tensors[9]);
        a.table_v_data = static_cast<const int32_t*>(tensors[10]);
        if (!a.q_data || !a.k_data || !a.v_data || !a.o_data) return fail(kInvalidArgument, "SDPA: null Q/K/V/O pointer");
        if ((p.stats.rank && !a.stats_data) || (p.max.rank && !a.max_data) || (p.sum_exp.rank && !a.sum_exp_data))
            return fail(kInvalidArgument, "SDPA: null row-output pointer");
        if (p.padding_mask && (!a.seq_q_data || !a.seq_kv_data)) return fail(kInvalidArgument, "SDPA: null sequence length pointer");
        if ((paged_k && !a.table_k_data) || (paged_v && !a.table_v_data)) return fail(kInvalidArgument, "SDPA: null page table pointer");
    }
    a.offsets_k_data = (tensors && p.page_offsets_k.rank) ? tensors[14] : nullptr;  // (read only when declared: shorter pointer lists stay valid)
    a.offsets_v_data = (tensors && p.page_offsets_v.rank) ? tensors[15] : nullptr;
    if (tensors && ((p.page_offsets_k.rank && !a.offsets_k_data) || (p.page_offsets_v.rank && !a.offsets_v_data)))
        return fail(kInvalidArgument, "SDPA: null page table offsets pointer");
    a.offsets_k_wide = p.page_offsets_k.dtype == DFGPU_I64;
    a.offsets_v_wide = p.page_offsets_v.dtype == DFGPU_I64;
    a.offsets_k_stride = p.page_offsets_k.rank ? p.page_offsets_k.stride[0] : 0;
    a.offsets_v_stride = p.page_offsets_v.rank ? p.page_offsets_v.stride[0] : 0;
    a.prefix_ok = nullptr;
    a.bias = make_view(p.bias);
    a.bias_data = (tensors && p.bias.rank) ? tensors[11] : nullptr;  // callers without a bias may pass 11 pointers
    if (p.bias.rank) {
        if (!valid_tensor(p.bias) || p.bias.rank != 4 || !float_type(p.bias.dtype)) return fail(kInvalidShape, "SDPA: bias must be a rank-4 FLOAT, HALF or BFLOAT16 tensor");
        const int64_t extent[4] = {p.q.dim[0], hq, p.q.dim[2], p.s_kv};
        for (int i = 0; i < 4; ++i)
            if (p.bias.dim[i] != 1 && p.bias.dim[i] != extent[i]) return fail(kInvalidShape, "SDPA: bias is not broadcast-compatible with attention scores");
        if (tensors && !a.bias_data) return fail(kInvalidArgument, "SDPA: null bias pointer");
    }
    a.sink = make_view(p.sink);
    a.sink_data = (tensors && p.sink.rank) ? static_cast<const float*>(tensors[12]) : nullptr;
    if (p.sink.rank) {
        if (p.sink.rank != 4 || p.sink.dtype != DFGPU_F32 || p.sink.dim[0] != 1 || p.sink.dim[1] != hq || p.sink.dim[2] != 1 || p.sink.dim[3] != 1)
            return fail(kInvalidShape, "SDPA: sink token must have dimensions [1,Hq,1,1] and type FLOAT");
        if (tensors && !a.sink_data) return fail(kInvalidArgument, "SDPA: null sink token pointer");
    }
    a.block_mask = make_view(p.block_mask);
    a.block_mask_data = (tensors && p.block_mask.rank) ? static_cast<const uint8_t*>(tensors[13]) : nullptr;
    if (p.block_mask.rank) {
        const int64_t query_tiles = (p.q.dim[2] - 1) / 128 + 1, key_tiles = (p.s_kv - 1) / 128 + 1;
        if (p.block_mask.rank != 4 || p.block_mask.dtype != DFGPU_U8 || p.block_mask.dim[0] != p.q.dim[0] || p.block_mask.dim[1] != hq ||
            p.block_mask.dim[2] != query_tiles || p.block_mask.dim[3] != (key_tiles + 7) / 8)
            return fail(kInvalidShape, "SDPA: block mask must be UINT8 with dimensions [B,Hq,ceil(Sq/128),ceil(ceil(Skv/128)/8)]");
        if (tensors && !a.block_mask_data) return fail(kInvalidArgument, "SDPA: null block mask pointer");
    }
    a.dropout_kind = p.dropout_kind;
    a.keep_threshold = 0;
    a.dropout_scale = 1.0f;
    a.dropout_mask = make_view(p.dropout_mask);
    a.rng_dump = make_view(p.rng_dump);
    a.dropout_mask_data = nullptr; a.dropout_scale_data = nullptr; a.seed_data = nullptr; a.offset_data = nullptr; a.rng_dump_data = nullptr;
    if (p.dropout_kind < 0 || p.dropout_kind > 2) return fail(kInvalidArgument, "SDPA: unknown dropout kind %d", p.dropout_kind);
    auto one_element = [](const dfgpu_tensor& t, int dtype) {
        if (t.rank < 1 || t.dtype != dtype) return false;
        for (int i = 0; i < t.rank; ++i)
            if (t.dim[i] != 1) return false;
        return true;
    };
    if (p.dropout_kind == 1) {
        if (!(p.dropout_probability >= 0.0 && p.dropout_probability < 1.0)) return fail(kInvalidArgument, "SDPA: dropout probability must be in [0, 1)");
        if (!one_element(p.seed, DFGPU_I64) || !one_element(p.offset, DFGPU_I64)) return fail(kInvalidShape, "SDPA: Seed and Offset must be one INT64 element each");
        const double keep = 1.0 - p.dropout_probability;
        a.keep_threshold = static_cast<uint32_t>(static_cast<int64_t>(std::floor(keep * static_cast<double>(1u << 24))));
        a.dropout_scale = static_cast<float>(1.0 / keep);
        if (p.rng_dump.rank) {
            if (p.rng_dump.rank != 4 || p.rng_dump.dtype != DFGPU_F32 || p.rng_dump.dim[0] != p.q.dim[0] || p.rng_dump.dim[1] != hq || p.rng_dump.dim[2] != p.q.dim[2] ||
                p.rng_dump.dim[3] != p.s_kv)
                return fail(kInvalidShape, "SDPA: RNG_DUMP must be FLOAT [B, Hq, Sq, Skv]");
        }
        if (tensors) {
            a.seed_data = static_cast<const int64_t*>(tensors[18]);
            a.offset_data = static_cast<const int64_t*>(tensors[19]);
            a.rng_dump_data = p.rng_dump.rank ? static_cast<float*>(tensors[20]) : nullptr;
            if (!a.seed_data || !a.offset_data || (p.rng_dump.rank && !a.rng_dump_data)) return fail(kInvalidArgument, "SDPA: null Seed, Offset or RNG_DUMP pointer");
        }
    } else if (p.dropout_kind == 2) {
        if (p.dropout_mask.rank != 4 || p.dropout_mask.dtype != DFGPU_F32 || !valid_tensor(p.dropout_mask)) return fail(kInvalidShape, "SDPA: Dropout_mask must be a rank-4 FLOAT tensor");
        const int64_t extent[4] = {p.q.dim[0], hq, p.q.dim[2], p.s_kv};
        for (int i = 0; i < 4; ++i)
            if (p.dropout_mask.dim[i] != 1 && p.dropout_mask.dim[i] != extent[i]) return fail(kInvalidShape, "SDPA: Dropout_mask is not broadcast-compatible with attention scores");
        if (!one_element(p.dropout_scale, DFGPU_F32)) return fail(kInvalidShape, "SDPA: Dropout_scale must be one FLOAT element");
        if (p.rng_dump.rank) return fail(kInvalidArgument, "SDPA: RNG_DUMP requires probability dropout");
        if (tensors) {
            a.dropout_mask_data = static_cast<const float*>(tensors[16]);
            a.dropout_scale_data = static_cast<const float*>(tensors[17]);
            if (!a.dropout_mask_data || !a.dropout_scale_data) return fail(kInvalidArgument, "SDPA: null Dropout_mask or Dropout_scale pointer");
        }
    } else if (p.rng_dump.rank) {
        return fail(kInvalidArgument, "SDPA: RNG_DUMP requires probability dropout");
    }
    a.alibi = p.alibi_mask;
    a.alibi_n = 1;
    while (2 * static_cast<int64_t>(a.alibi_n) <= hq) a.alibi_n *= 2;
    a.alibi_slope_scale = -8.0f / static_cast<float>(a.alibi_n);
    a.scale = p.attn_scale;
    a.padding = p.padding_mask;
    a.has_left = p.has_left_bound;
    a.has_right = p.has_right_bound;
    a.bottom_right = p.bottom_right;
    a.left = p.left_bound;
    a.right = p.right_bound;
    a.s_kv = p.s_kv;
    return kOk;
}

bool decode_supported(const dfgpu_sdpa_params& p) {
    if (p.q.dim[2] != 1 || p.q.dim[3] != kDecodeD || p.v.dim[3] != kDecodeD) return false;
    if (p.q.dtype != DFGPU_BF16 || p.k.dtype != DFGPU_BF16 || p.v.dtype != DFGPU_BF16) return false;
    if (p.page_table_k.rank == 0 || p.page_table_v.rank == 0) return false;
    int64_t block = p.k.dim[2];
    if (p.v.dim[2] != block || block < 16 || block > kDecodeChunk || (block & (block - 1)) != 0) return false;
    if (p.k.dim[1] != p.v.dim[1]) return false;
    int64_t group = p.q.dim[1] / p.k.dim[1];
    if (group != 1 && group != 2 && group != 4 && group != 8) return false;
    if (p.k.stride[2] % 8 != 0 || p.v.stride[2] % 8 != 0 || p.k.stride[1] % 8 != 0 || p.v.stride[1] % 8 != 0 ||
        p.k.stride[0] % 8 != 0 || p.v.stride[0] % 8 != 0 || p.q.stride[0] % 8 != 0 || p.q.stride[1] % 8 != 0)
        return false;
    if (p.q.dim[0] > 65535 || p.k.dim[1] > 65535) return false;
    return true;
}

int decode_chunks(const dfgpu_sdpa_params& p) { return static_cast<int>((p.s_kv + kDecodeChunk - 1) / kDecodeChunk); }

int choose_kernel(const dfgpu_sdpa_params& p, int& kernel) {
    int automatic = DFGPU_SDPA_ROWWISE;
    const bool plain_scores = p.bias.rank == 0 && !p.alibi_mask && p.sink.rank == 0 && p.block_mask.rank == 0 && p.dropout_kind == 0;  // bias, ALiBi, sink token, block mask, dropout: general kernel only
    if (!plain_scores) automatic = DFGPU_SDPA_ROWWISE;
    else if (decode_umma_supported(p)) automatic = DFGPU_SDPA_PAGED_DECODE_UMMA;
    else if (decode_supported(p)) automatic = DFGPU_SDPA_PAGED_DECODE;
    else if (sdpa_umma_supported(p)) automatic = DFGPU_SDPA_UMMA;
    kernel = p.kernel == DFGPU_SDPA_AUTO ? automatic : p.kernel;
    if (!plain_scores && kernel != DFGPU_SDPA_ROWWISE) return fail(kUnsupported, "SDPA: bias, ALiBi, the sink token, the block mask and dropout run on the general kernel only");
    if (kernel == DFGPU_SDPA_ROWWISE) {
        if (p.q.dim[3] > kRowwiseMaxD || p.v.dim[3] > kRowwiseMaxD) return fail(kUnsupported, "SDPA: head dimension above %d", kRowwiseMaxD);
        return kOk;
    }
    if (kernel == DFGPU_SDPA_PAGED_DECODE) {
        if (!decode_supported(p)) return fail(kUnsupported, "SDPA: the paged decode kernel needs Sq=1, bf16, D=128, paged K and V, group size 1/2/4/8");
        return kOk;
    }
    if (kernel == DFGPU_SDPA_UMMA) {
        if (!sdpa_umma_supported(p)) return fail(kUnsupported, "SDPA: the tcgen05 kernel does not cover this shape, layout or mask");
        return kOk;
    }
    if (kernel == DFGPU_SDPA_PAGED_DECODE_UMMA) {
        if (!decode_umma_supported(p)) return fail(kUnsupported, "SDPA: the TMA paged decode kernel needs Sq=1, bf16, D=128, packed paged K and V, page size 16..128, group size 1/2/4/8");
        return kOk;
    }
    return fail(kInvalidArgument, "SDPA: unknown kernel id %d", kernel);
}

}  // namespace
}  // namespace dfgpu

using namespace dfgpu;

extern "C" int dfgpu_query_sdpa_forward(const dfgpu_sdpa_params* p, dfgpu_plan_info* info) {
    if (!p || !info) return fail(kInvalidArgument, "SDPA: null params");
    SdpaArgs a;
    int status = build_args(*p, nullptr, a);
    if (status) return status;
    int kernel;
    status = choose_kernel(*p, kernel);
    if (status) return status;
    info->kernel = kernel;
    info->launches = 1;
    info->scratch_bytes = 0;
    if (kernel == DFGPU_SDPA_PAGED_DECODE) {
        info->launches = 2;
        info->scratch_bytes = p->q.dim[0] * p->q.dim[1] * decode_chunks(*p) * kPartialStride * static_cast<int64_t>(sizeof(float));
    }
    if (kernel == DFGPU_SDPA_PAGED_DECODE_UMMA) {
        info->launches = 2;
        info->scratch_bytes = decode_umma_scratch_bytes(*p);
    }
    if (p->page_offsets_k.rank || p->page_offsets_v.rank) {  // compact page tables: the validation launch and its two result words
        info->launches += 1;
        info->scratch_bytes += kPrefixScratchBytes;
    }
    return kOk;
}

extern "C" int dfgpu_sdpa_forward(const dfgpu_sdpa_params* p, void* const* tensors, void* scratch, void* stream_handle) {
    if (!p || !tensors) return fail(kInvalidArgument, "SDPA: null params");
    SdpaArgs a;
    int status = build_args(*p, tensors, a);
    if (status) return status;
    int kernel;
    status = choose_kernel(*p, kernel);
    if (status) return status;
    cudaStream_t stream = as_stream(stream_handle);
    if (p->page_offsets_k.rank || p->page_offsets_v.rank) {
        // compact page tables: validate the prefixes on the device first; the attention kernels read the verdict
        if (!scratch || !aligned16(scratch)) return fail(kInvalidArgument, "SDPA: compact page tables need the 16-byte aligned scratch dfgpu_query_sdpa_forward reports");
        int* prefix_ok = static_cast<int*>(scratch);
        scratch = static_cast<uint8_t*>(scratch) + kPrefixScratchBytes;
        validate_page_prefix_kernel<<<2, 256, 0, stream>>>(a, prefix_ok);
        status = check_launch("SDPA page table prefix validation");
        if (status) return status;
        a.prefix_ok = prefix_ok;
    }
    if (kernel == DFGPU_SDPA_UMMA) return launch_sdpa_umma(*p, tensors, scratch, stream);
    if (kernel == DFGPU_SDPA_PAGED_DECODE_UMMA) {
        if (!scratch || !aligned16(scratch)) return fail(kInvalidArgument, "SDPA: the paged decode kernel needs its 16-byte aligned scratch buffer");
        status = launch_decode_umma(*p, tensors, scratch, a.prefix_ok, stream);
        if (status) return status;
        const int chunks = decode_umma_chunks(*p);
        sdpa_decode_merge_kernel<<<static_cast<unsigned>(p->q.dim[0] * p->q.dim[1]), kDecodeD, 0, stream>>>(a, static_cast<const float*>(scratch), chunks, 1024);
        return check_launch("SDPA decode merge");
    }
    if (kernel == DFGPU_SDPA_PAGED_DECODE) {
        if (!scratch) return fail(kInvalidArgument, "SDPA: the paged decode kernel needs its scratch buffer");
        if (!aligned16(a.q_data) || !aligned16(a.k_data) || !aligned16(a.v_data) || !aligned16(scratch))
            return fail(kInvalidArgument, "SDPA: the paged decode kernel needs 16-byte aligned Q, K, V and scratch");
        int chunks = decode_chunks(*p);
        int group = static_cast<int>(p->q.dim[1] / p->k.dim[1]);
        dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(p->k.dim[1]), static_cast<unsigned>(p->q.dim[0]));
        float* partial = static_cast<float*>(scratch);
        switch (group) {
            case 1: sdpa_paged_decode_kernel<1><<<grid, 256, 0, stream>>>(a, partial, chunks); break;
            case 2: sdpa_paged_decode_kernel<2><<<grid, 256, 0, stream>>>(a, partial, chunks); break;
            case 4: sdpa_paged_decode_kernel<4><<<grid, 256, 0, stream>>>(a, partial, chunks); break;
            default: sdpa_paged_decode_kernel<8><<<grid, 256, 0, stream>>>(a, partial, chunks); break;
        }
        status = check_launch("SDPA paged decode");
        if (status) return status;
        sdpa_decode_merge_kernel<<<static_cast<unsigned>(p->q.dim[0] * p->q.dim[1]), kDecodeD, 0, stream>>>(a, partial, chunks, kDecodeChunk);
        return check_launch("SDPA decode merge");
    }
    int64_t rows = p->q.dim[0] * p->q.dim[1] * p->q.dim[2];
    sdpa_rowwise_kernel<<<static_cast<unsigned>((rows + 3) / 4), 128, 0, stream>>>(a, rows);
    return check_launch("SDPA");
}

namespace dfgpu {
int sdpa_device_status(int* status) {
    int zero = 0;
    cudaError_t error = cudaMemcpyFromSymbol(status, g_sdpa_status, sizeof(int));
    if (error == cudaSuccess) error = cudaMemcpyToSymbol(g_sdpa_status, &zero, sizeof(int));
    if (error != cudaSuccess) return fail(kExecutionFailed, "device_status: %s", cudaGetErrorString(error));
    return kOk;
}
}  // namespace dfgpu

// ---- paged decode for callers that cannot allocate ---------------------------------------
//
// Some hosts of this library are not allowed to call cudaMalloc on the path that runs the
// decode step: a serving loop that pre-reserved all device memory at start-up and runs with
// allocation disabled, a plugin called while the framework above it holds its allocator
// lock, a real-time thread that must not enter the driver's allocator. For those callers the
// split-KV partial results live in the fixed device array below instead of a caller-provided
// scratch buffer. The price is a size limit and shared state:
//   * the partials of one call must fit kStaticDecodeScratchBytes (8 MiB): batch * query
//     heads * ceil(s_kv / 256) chunks * 520 bytes; larger requests are refused with a message,
//   * every GPU that loads this library keeps the 8 MiB resident until the process exits,
//   * all calls on one device share the array: it still holds the previous call's partials
//     when the next call starts. Nothing in it has to be zero beforehand, because a call
//     rewrites every slot it later reads (chunks without valid tokens are marked empty by
//     the first kernel), but two calls whose kernels overlap on the GPU (different streams
//     or threads) race on it; callers must serialise them.
// The array's device address is looked up with cudaGetSymbolAddress the first time the entry
// point runs on a device (with that device current) and remembered per device; make that
// first call before any stream capture begins.
constexpr size_t kStaticDecodeScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_static_decode_scratch[kStaticDecodeScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
// One address per device, written once; atomic because two host threads may make their first call at the same time
// (both resolve the same value).
std::atomic<void*> g_static_decode_scratch_address[kMaxDevices];

int static_decode_scratch(void** address, cudaStream_t stream) {
    int device = 0;
    cudaError_t error = cudaGetDevice(&device);
    if (error != cudaSuccess) return dfgpu::fail(dfgpu::kExecutionFailed, "SDPA static decode: cudaGetDevice failed: %s", cudaGetErrorString(error));
    if (device < 0 || device >= kMaxDevices) return dfgpu::fail(dfgpu::kUnsupported, "SDPA static decode: device ordinal %d is above %d", device, kMaxDevices - 1);
    // The array belongs to the CURRENT device: a stream of another device would run the kernels there with this
    // device's array. The legacy default stream (null) and the per-thread default stream follow the current device.
    if (stream != nullptr && stream != cudaStreamLegacy && stream != cudaStreamPerThread) {
        int stream_device = device;
        if (cudaStreamGetDevice(stream, &stream_device) == cudaSuccess && stream_device != device)
            return dfgpu::fail(dfgpu::kInvalidArgument, "SDPA static decode: the stream belongs to device %d but device %d is current", stream_device, device);
        (void)cudaGetLastError();
    }
    if (g_static_decode_scratch_address[device].load(std::memory_order_acquire) == nullptr) {
        // In host code the array's name is only a handle for the runtime, not a device pointer:
        // the address a kernel can use has to come from the runtime, for the current device.
        void* resolved = nullptr;
        error = cudaGetSymbolAddress(&resolved, g_static_decode_scratch);
        if (error != cudaSuccess || resolved == nullptr)
            return dfgpu::fail(dfgpu::kExecutionFailed, "SDPA static decode: cudaGetSymbolAddress failed: %s", cudaGetErrorString(error));
        g_static_decode_scratch_address[device].store(resolved, std::memory_order_release);
    }
    *address = g_static_decode_scratch_address[device].load(std::memory_order_acquire);
    return dfgpu::kOk;
}
}  // namespace

extern "C" int dfgpu_sdpa_paged_decode_static(const dfgpu_sdpa_params* p, void* const* tensors, void* stream_handle) {
    if (!p || !tensors) return fail(kInvalidArgument, "SDPA static decode: null params");
    SdpaArgs a;
    int status = build_args(*p, tensors, a);
    if (status) return status;
    if (!decode_supported(*p) || p->bias.rank != 0 || p->alibi_mask || p->sink.rank != 0 || p->block_mask.rank != 0 || p->page_offsets_k.rank != 0 ||
        p->page_offsets_v.rank != 0 || p->dropout_kind != 0)
        return fail(kUnsupported, "SDPA static decode: needs Sq=1, bf16, D=128, strided page tables for K and V, group size 1/2/4/8, no bias or ALiBi");
    if (!aligned16(a.q_data) || !aligned16(a.k_data) || !aligned16(a.v_data))
        return fail(kInvalidArgument, "SDPA static decode: needs 16-byte aligned Q, K and V");
    const int chunks = decode_chunks(*p);
    const size_t needed = static_cast<size_t>(p->q.dim[0]) * static_cast<size_t>(p->q.dim[1]) * static_cast<size_t>(chunks) * kPartialStride * sizeof(float);
    if (needed > kStaticDecodeScratchBytes)
        return fail(kInvalidShape, "SDPA static decode: this call needs %zu bytes of split-KV partials, the built-in scratch holds %zu (batch * query heads * ceil(s_kv/256) * 520 must not exceed it)",
                    needed, kStaticDecodeScratchBytes);
    void* scratch = nullptr;
    cudaStream_t stream = as_stream(stream_handle);
    status = static_decode_scratch(&scratch, stream);
    if (status) return status;
    const int group = static_cast<int>(p->q.dim[1] / p->k.dim[1]);
    dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(p->k.dim[1]), static_cast<unsigned>(p->q.dim[0]));
    float* partial = static_cast<float*>(scratch);
    switch (group) {
        case 1: sdpa_paged_decode_kernel<1><<<grid, 256, 0, stream>>>(a, partial, chunks); break;
        case 2: sdpa_paged_decode_kernel<2><<<grid, 256, 0, stream>>>(a, partial, chunks); break;
        case 4: sdpa_paged_decode_kernel<4><<<grid, 256, 0, stream>>>(a, partial, chunks); break;
        default: sdpa_paged_decode_kernel<8><<<grid, 256, 0, stream>>>(a, partial, chunks); break;
    }
    status = check_launch("SDPA static decode");
    if (status) return status;
    sdpa_decode_merge_kernel<<<static_cast<unsigned>(p->q.dim[0] * p->q.dim[1]), kDecodeD, 0, stream>>>(a, partial, chunks, kDecodeChunk);
    return check_launch("SDPA static decode merge");
}

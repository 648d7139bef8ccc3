// BLOCK_SCALE_QUANTIZE / BLOCK_SCALE_DEQUANTIZE for MXFP8 (E4M3 codes, E8M0 scales).
//
// Bandwidth-bound kernels: 16-byte loads, integer amax, integer exponent math for
// the scale, the hardware e4m3x2 convert with the two fix-ups that make it equal
// to the reference's candidate search (lib/Compiler/Numeric.cpp:504-632):
//   * a non-zero negative that rounds to zero encodes as 0x00 (only an exact -0.0
//     input gives 0x80), because the search visits +0 first and -0 never wins a tie;
//   * NaN encodes as 0x7f whatever its sign.
// The scale rule is 2^ceil(log2(amax/448)) (lib/Compiler/SpecializedGraph.cpp:810-838),
// amax == 0 -> 1.0, NaN -> 0xff, and the codes are x / decode(stored scale).
#include "common.cuh"

namespace dfgpu {
namespace {

// ---- scalar building blocks ---------------------------------------------------

// |x| bit patterns order like unsigned integers, and every NaN pattern is larger
// than +Inf, so an unsigned max over (bits & 0x7fffffff) is arith.maximumf over
// |x| with NaN propagation.
// `largest`: the largest finite value of the code type (448 for E4M3, 57344 for E5M2; SpecializedGraph.cpp:795-808).
__device__ __forceinline__ uint32_t scale_code_from_amax_bits(uint32_t amax_bits, float largest = 448.0f) {
    if (amax_bits > 0x7f800000u) return 0xffu;  // NaN block
    float desired = __fdiv_rn(__uint_as_float(amax_bits), largest);
    uint32_t bits = __float_as_uint(desired);
    if (bits == 0u) return 127u;            // desired > 0 is false -> scale 1.0
    if (bits == 0x7f800000u) return 0xfeu;  // +Inf saturates
    int exponent = static_cast<int>(bits >> 23);
    uint32_t mantissa = bits & 0x7fffffu;
    int n;  // ceil(log2(desired))
    if (exponent == 0) {
        int top = 31 - __clz(mantissa);
        n = top - 149 + ((mantissa & (mantissa - 1u)) != 0u ? 1 : 0);
    } else {
        n = exponent - 127 + (mantissa != 0u ? 1 : 0);
    }
    int code = n + 127;
    // 2^n below 2^-127 is nearest (in the linear distance the search uses) to code 0.
    return static_cast<uint32_t>(code < 0 ? 0 : (code > 254 ? 254 : code));
}


// The reference's search, literally (used only by the self-check kernel).
__device__ uint32_t encode_e4m3_search(float value) {
    uint32_t best = 0;
    float best_difference = fabsf(__fsub_rn(value, decode_e4m3(0)));
    for (uint32_t candidate = 0; candidate < 256; ++candidate) {
        float difference = fabsf(__fsub_rn(value, decode_e4m3(candidate)));
        bool better = difference < best_difference;
        bool equal = difference == best_difference;
        bool valid = (candidate & 0x7fu) < 127u;
        if (valid && (better || (equal && (candidate & 1u) == 0u && (best & 1u) != 0u))) {
            best = candidate;
            best_difference = difference;
        }
    }
    bool negative = (__float_as_uint(value) & 0x80000000u) != 0u;
    float absolute = fabsf(value);
    uint32_t result = best;
    if (absolute == 0.0f) result = negative ? 0x80u : 0x00u;
    if (absolute > 448.0f) result = 0x7eu | (negative ? 0x80u : 0u);
    if (value != value) result = 0x7fu;
    return result;
}

__global__ void selfcheck_e4m3_kernel(uint32_t first_bits, uint64_t count, unsigned long long* result) {
    uint64_t index = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    uint64_t step = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    unsigned long long bad = 0;
    unsigned long long witness = 0;
    for (; index < count; index += step) {
        uint32_t bits = first_bits + static_cast<uint32_t>(index);
        float v = __uint_as_float(bits);
        if (encode_e4m3_scalar(v) != encode_e4m3_search(v)) {
            ++bad;
            witness = static_cast<unsigned long long>(bits) + 1ull;
        }
    }
    if (bad) {
        atomicAdd(&result[0], bad);
        atomicExch(&result[1], witness);
    }
}

__global__ void debug_scale_codes_kernel(const float* amax, uint8_t* codes, int64_t count) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) codes[i] = static_cast<uint8_t>(scale_code_from_amax_bits(__float_as_uint(amax[i]) & 0x7fffffffu));
}

__global__ void debug_encode_kernel(const float* values, uint8_t* codes, int64_t count) {
    int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) codes[i] = static_cast<uint8_t>(encode_e4m3_scalar(values[i]));
}

// ---- scale addressing -----------------------------------------------------------

struct ScaleLayout {
    int32_t reordered;  // F8_128x4
    int32_t m_axis, k_axis;
};

// F8_128x4 (lib/Compiler/Numeric.cpp:240-308): 512-byte tiles of 128 M x 4 K.
__device__ __forceinline__ int64_t f8_128x4_offset(int64_t leading, int64_t m, int64_t k,
                                                   int64_t m_extent, int64_t k_extent) {
    int64_t m_blocks = m_extent >> 7, k_blocks = k_extent >> 2;
    return (((leading * m_blocks + (m >> 7)) * k_blocks + (k >> 2)) << 9) + ((m & 31) << 4) +
           (((m >> 5) & 3) << 2) + (k & 3);
}

__device__ __forceinline__ int64_t scale_offset(const View& scale, const ScaleLayout& layout,
                                                const int64_t* index) {
    if (layout.reordered) {
        int64_t leading = 0;
        for (int axis = 0; axis + 2 < scale.rank; ++axis) leading = leading * scale.dim[axis] + index[axis];
        return f8_128x4_offset(leading, index[layout.m_axis], index[layout.k_axis],
                               scale.dim[layout.m_axis], scale.dim[layout.k_axis]);
    }
    int64_t offset = 0;
    for (int i = 0; i < scale.rank; ++i) offset += index[i] * scale.stride[i];
    return offset;
}

// Same rule as the reference's layout check (lib/Compiler/Numeric.cpp:38-87).
bool resolve_reorder(const dfgpu_tensor& t, ScaleLayout& layout) {
    layout = ScaleLayout{0, 0, 0};
    if (t.reorder == DFGPU_REORDER_NONE) return true;
    if (t.reorder != DFGPU_REORDER_F8_128x4 || t.rank < 2) return false;
    int first = t.rank - 2;
    for (int attempt = 0; attempt < 2; ++attempt) {
        int ma = first + attempt;
        int ka = attempt == 0 ? first + 1 : first;
        int64_t m = t.dim[ma], k = t.dim[ka];
        if (m <= 0 || k <= 0 || m % 128 != 0 || k % 4 != 0) continue;
        if (t.stride[ka] != 1 || t.stride[ma] != k) continue;
        int64_t expected = m * k;
        bool packed = true;
        for (int axis = first; axis > 0; --axis) {
            if (t.stride[axis - 1] != expected) { packed = false; break; }
            expected *= t.dim[axis - 1];
        }
        if (packed) {
            layout = ScaleLayout{1, ma, ka};
            return true;
        }
    }
    return false;
}

// ---- scale initialisation: every slot <- encode(1.0) = 0x7f --------------------

__global__ void fill_bytes_kernel(uint8_t* data, int64_t count, uint8_t value) {
    int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 16;
    if (i + 16 <= count && (reinterpret_cast<uintptr_t>(data + i) & 15u) == 0) {
        uint32_t w = value * 0x01010101u;
        *reinterpret_cast<uint4*>(data + i) = make_uint4(w, w, w, w);
    } else {
        for (int64_t j = i; j < count && j < i + 16; ++j) data[j] = value;
    }
}

__global__ void fill_strided_kernel(uint8_t* data, View view, int64_t count, uint8_t value) {
    int64_t flat = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (flat >= count) return;
    int64_t offset = 0;
    for (int i = view.rank - 1; i >= 0; --i) {
        offset += (flat % view.dim[i]) * view.stride[i];
        flat /= view.dim[i];
    }
    data[offset] = value;
}

// ---- generic quantize: one thread per block, any strides -----------------------

__global__ void bsq_generic_kernel(const void* x, uint8_t* y, uint8_t* scale, View xv, View yv, View sv,
                                   ScaleLayout layout, int axis, int64_t block, int64_t block_total) {
    int64_t flat = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (flat >= block_total) return;
    int64_t index[DFGPU_MAX_RANK];
    for (int i = xv.rank - 1; i >= 0; --i) {
        int64_t extent = i == axis ? xv.dim[i] / block : xv.dim[i];
        index[i] = flat % extent;
        flat /= extent;
    }
    int64_t x_base = 0, y_base = 0;
    for (int i = 0; i < xv.rank; ++i) {
        int64_t position = i == axis ? index[i] * block : index[i];
        x_base += position * xv.stride[i];
        y_base += position * yv.stride[i];
    }
    uint32_t amax_bits = 0;
    for (int64_t j = 0; j < block; ++j) {
        float value = load_as_f32(x, xv.dtype, x_base + j * xv.stride[axis]);
        uint32_t bits = __float_as_uint(value) & 0x7fffffffu;
        amax_bits = bits > amax_bits ? bits : amax_bits;
    }
    if (yv.dtype == DFGPU_FP4) {
        // FP4 codes take an E4M3 scale that is not made a power of two (lib/Compiler/SpecializedGraph.cpp:810-838): amax / 6, 1 when that
        // is not positive, NaN kept; every value is divided by the STORED scale (:927-931) and packed two codes to a byte
        const float desired = __fdiv_rn(__uint_as_float(amax_bits), 6.0f);
        float guarded = desired > 0.0f ? desired : 1.0f;
        if (desired != desired) guarded = desired;
        const uint32_t scale_code = encode_e4m3_scalar(guarded);
        scale[scale_offset(sv, layout, index)] = static_cast<uint8_t>(scale_code);
        const float stored = decode_e4m3(scale_code);
        for (int64_t j = 0; j < block; ++j) {
            const float value = __fdiv_rn(load_as_f32(x, xv.dtype, x_base + j * xv.stride[axis]), stored);
            store_nibble(y, y_base + j * yv.stride[axis], encode_e2m1_scalar(value));
        }
        return;
    }
    const bool e5m2 = yv.dtype == DFGPU_E5M2;
    uint32_t code = scale_code_from_amax_bits(amax_bits, e5m2 ? 57344.0f : 448.0f);
    scale[scale_offset(sv, layout, index)] = static_cast<uint8_t>(code);
    float reciprocal = reciprocal_e8m0(code);
    for (int64_t j = 0; j < block; ++j) {
        float value = __fmul_rn(load_as_f32(x, xv.dtype, x_base + j * xv.stride[axis]), reciprocal);
        y[y_base + j * yv.stride[axis]] = static_cast<uint8_t>(e5m2 ? encode_e5m2_scalar(value) : encode_e4m3_scalar(value));
    }
}

// ---- row kernel: block of 32 along the contiguous axis --------------------------
// Each thread owns 8 consecutive elements (one 16-byte load for 16-bit inputs, two
// for f32); 4 neighbouring lanes form one block and share the amax with two
// shuffles. A warp therefore covers 8 blocks = 256 elements per step.

template <typename T>
struct Load8;

template <>
struct Load8<float> {
    __device__ static void load(const void* base, int64_t element, float (&out)[8]) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + element);
        float4 a = __ldg(p), b = __ldg(p + 1);
        out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
        out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
    }
};
template <>
struct Load8<__nv_bfloat16> {
    __device__ static void load(const void* base, int64_t element, float (&out)[8]) {
        uint4 raw = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + element));
        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};
template <>
struct Load8<__half> {
    __device__ static void load(const void* base, int64_t element, float (&out)[8]) {
        uint4 raw = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + element));
        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            out[2 * i] = f.x;
            out[2 * i + 1] = f.y;
        }
    }
};

__device__ __forceinline__ uint2 quantize8(const float (&v)[8], uint32_t code) {
    if (code == 0xffu) return make_uint2(0x7f7f7f7fu, 0x7f7f7f7fu);
    float reciprocal = reciprocal_e8m0(code);
    uint32_t p0 = encode_e4m3_pair(__fmul_rn(v[0], reciprocal), __fmul_rn(v[1], reciprocal));
    uint32_t p1 = encode_e4m3_pair(__fmul_rn(v[2], reciprocal), __fmul_rn(v[3], reciprocal));
    uint32_t p2 = encode_e4m3_pair(__fmul_rn(v[4], reciprocal), __fmul_rn(v[5], reciprocal));
    uint32_t p3 = encode_e4m3_pair(__fmul_rn(v[6], reciprocal), __fmul_rn(v[7], reciprocal));
    return make_uint2(p0 | (p1 << 16), p2 | (p3 << 16));
}

template <typename T>
__global__ void __launch_bounds__(256)
bsq_row32_kernel(const void* __restrict__ x, uint8_t* __restrict__ y, uint8_t* __restrict__ scale,
                 int64_t rows, int64_t cols, int reordered, int64_t scale_k_extent) {
    // A thread owns kChunks groups of 8 consecutive elements, kChunks * 2048 elements apart, so that each
    // load instruction of a warp is one contiguous 512-byte (16-bit input) segment and all of a thread's
    // loads are in flight before the first amax. 4 neighbouring lanes form one 32-element block.
    constexpr int kChunks = 4;
    chain_release();
    chain_wait();
    const int64_t total = rows * cols;
    const int64_t tile0 = static_cast<int64_t>(blockIdx.x) * (256 * 8 * kChunks);
    float v[kChunks][8];
    bool live[kChunks];
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const int64_t element = tile0 + (static_cast<int64_t>(c) * 256 + threadIdx.x) * 8;
        live[c] = element < total;
        Load8<T>::load(x, live[c] ? element : 0, v[c]);  // a dead chunk re-reads element 0 and is discarded
    }
    const int64_t k_blocks = cols >> 5;
#pragma unroll
    for (int c = 0; c < kChunks; ++c) {
        const int64_t element = tile0 + (static_cast<int64_t>(c) * 256 + threadIdx.x) * 8;
        uint32_t amax_bits = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint32_t bits = __float_as_uint(v[c][i]) & 0x7fffffffu;
            amax_bits = bits > amax_bits ? bits : amax_bits;
        }
        // blocks are 4 whole lanes and the element count is a multiple of 32, so the 4 lanes of a block are live together
        uint32_t other = __shfl_xor_sync(0xffffffffu, amax_bits, 1);
        amax_bits = other > amax_bits ? other : amax_bits;
        other = __shfl_xor_sync(0xffffffffu, amax_bits, 2);
        amax_bits = other > amax_bits ? other : amax_bits;
        const uint32_t code = scale_code_from_amax_bits(amax_bits);
        const uint2 packed = quantize8(v[c], code);
        if (live[c]) *reinterpret_cast<uint2*>(y + element) = packed;
        if (live[c] && (threadIdx.x & 3) == 0) {
            const int64_t block_index = element >> 5;
            if (reordered) {
                const int64_t row = block_index / k_blocks, kb = block_index - row * k_blocks;
                scale[f8_128x4_offset(0, row, kb, rows, scale_k_extent)] = static_cast<uint8_t>(code);
            } else {
                scale[block_index] = static_cast<uint8_t>(code);
            }
        }
    }
}

// ---- column kernel: block of 32 along the second-to-last axis -------------------
// X is [batch, K, N] packed; a thread owns 8 rows x VEC columns and keeps the raw
// 16-byte loads in registers (VEC = 8 for 16-bit inputs, 4 for f32), so X is read
// from HBM exactly once and the amax runs on the raw bit patterns.

template <typename T>
struct ColumnTraits;

template <>
struct ColumnTraits<float> {
    static constexpr int VEC = 4;
    __device__ static void amax(const uint4& raw, uint32_t (&acc)[4]) {
        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] = max(acc[i], w[i] & 0x7fffffffu);
    }
    __device__ static uint32_t amax_f32_bits(uint32_t pattern) { return pattern; }
    __device__ static void values(const uint4& raw, float (&out)[4]) {
        out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y);
        out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
    }
};

template <>
struct ColumnTraits<__nv_bfloat16> {
    static constexpr int VEC = 8;
    __device__ static void amax(const uint4& raw, uint32_t (&acc)[8]) {
        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            acc[2 * i] = max(acc[2 * i], w[i] & 0x7fffu);
            acc[2 * i + 1] = max(acc[2 * i + 1], (w[i] >> 16) & 0x7fffu);
        }
    }
    __device__ static uint32_t amax_f32_bits(uint32_t pattern) { return pattern << 16; }
    __device__ static void values(const uint4& raw, float (&out)[8]) {
        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

template <>
struct ColumnTraits<__half> {
    static constexpr int VEC = 8;
    __device__ static void amax(const uint4& raw, uint32_t (&acc)[8]) { ColumnTraits<__nv_bfloat16>::amax(raw, acc); }
    __device__ static uint32_t amax_f32_bits(uint32_t pattern) {
        return __float_as_uint(__half2float(__ushort_as_half(static_cast<unsigned short>(pattern))));
    }
    __device__ static void values(const uint4& raw, float (&out)[8]) {
        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            out[2 * i] = f.x;
            out[2 * i + 1] = f.y;
        }
    }
};

template <typename T>
__global__ void __launch_bounds__(128)
bsq_col32_kernel(const void* __restrict__ x, uint8_t* __restrict__ y, uint8_t* __restrict__ scale,
                 int64_t k_extent, int64_t n_extent, int reordered, int64_t scale_k_extent) {
    // One CTA = one 32-row block over 32 * VEC columns: warp g holds rows 8g..8g+7 (8 raw 16-byte loads per
    // thread, 512 contiguous bytes per warp instruction) and the four partial column maxima meet in shared memory.
    using Traits = ColumnTraits<T>;
    constexpr int VEC = Traits::VEC;
    constexpr int kRows = 8;
    __shared__ uint32_t partial[4][VEC][32];
    chain_release();
    chain_wait();
    const int lane = threadIdx.x & 31, group = threadIdx.x >> 5;
    const int64_t column = (static_cast<int64_t>(blockIdx.x) * 32 + lane) * VEC;
    const bool live = column < n_extent;
    const int64_t kb = blockIdx.y;
    const int64_t batch = blockIdx.z;
    const int64_t base = (batch * k_extent + kb * 32 + group * kRows) * n_extent + (live ? column : 0);
    const T* xp = static_cast<const T*>(x) + base;
    uint4 raw[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) raw[r] = __ldg(reinterpret_cast<const uint4*>(xp + r * n_extent));
    uint32_t pattern[VEC];
#pragma unroll
    for (int c = 0; c < VEC; ++c) pattern[c] = 0;
#pragma unroll
    for (int r = 0; r < kRows; ++r) Traits::amax(raw[r], pattern);
#pragma unroll
    for (int c = 0; c < VEC; ++c) partial[group][c][lane] = pattern[c];
    __syncthreads();
    if (!live) return;
    uint32_t code[VEC];
    float reciprocal[VEC];
    const int64_t k_blocks = k_extent >> 5;
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
        uint32_t m = max(max(partial[0][c][lane], partial[1][c][lane]), max(partial[2][c][lane], partial[3][c][lane]));
        code[c] = scale_code_from_amax_bits(Traits::amax_f32_bits(m));
        reciprocal[c] = reciprocal_e8m0(code[c]);
    }
    if (group == 0) {
        if (reordered) {
            // scale dims [batch, K/32, N] with N as the 128-row axis of the tile
#pragma unroll
            for (int c = 0; c < VEC; ++c)
                scale[f8_128x4_offset(batch, column + c, kb, n_extent, scale_k_extent)] = static_cast<uint8_t>(code[c]);
        } else {
            uint8_t* out = scale + (batch * k_blocks + kb) * n_extent + column;
            if constexpr (VEC == 8) {
                *reinterpret_cast<uint2*>(out) =
                    make_uint2(code[0] | (code[1] << 8) | (code[2] << 16) | (code[3] << 24),
                               code[4] | (code[5] << 8) | (code[6] << 16) | (code[7] << 24));
            } else {
                *reinterpret_cast<uint32_t*>(out) = code[0] | (code[1] << 8) | (code[2] << 16) | (code[3] << 24);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        float v[VEC];
        Traits::values(raw[r], v);
        uint32_t bytes[VEC];
#pragma unroll
        for (int c = 0; c < VEC; c += 2) {
            uint32_t pair = encode_e4m3_pair(__fmul_rn(v[c], reciprocal[c]), __fmul_rn(v[c + 1], reciprocal[c + 1]));
            bytes[c] = code[c] == 0xffu ? 0x7fu : (pair & 0xffu);
            bytes[c + 1] = code[c + 1] == 0xffu ? 0x7fu : (pair >> 8);
        }
        uint8_t* out = y + base + r * n_extent;
        if constexpr (VEC == 8) {
            *reinterpret_cast<uint2*>(out) =
                make_uint2(bytes[0] | (bytes[1] << 8) | (bytes[2] << 16) | (bytes[3] << 24),
                           bytes[4] | (bytes[5] << 8) | (bytes[6] << 16) | (bytes[7] << 24));
        } else {
            *reinterpret_cast<uint32_t*>(out) = bytes[0] | (bytes[1] << 8) | (bytes[2] << 16) | (bytes[3] << 24);
        }
    }
}

// ---- bf16 input: the row form, the column form and pairs of either in one kernel ---------------------------
// A CTA of 256 threads encodes one tile of 16 KB of input: 8192 consecutive elements (row form), or 32 rows x 256
// columns (column form). A grid is the tiles of one tensor, or the tiles of two independent tensors back to back
// (the two operands of a block-scaled matmul): one launch, one ramp and one tail for both.
//
// Instruction issue, not HBM, bounds these kernels (the generic kernels above spend ~13 instructions per element),
// so the encode is kept short and free of barriers and shared memory:
//   * the amax runs on packed bf16 bit patterns (max.u16x2), and the scale code comes from those bits by integer
//     arithmetic: amax = (1 + f/128) * 2^E with a 7-bit fraction f gives amax/448 = ((128 + f)/224) * 2^(E-8), whose
//     ceil(log2) is E-8 for f <= 96 and E-7 above (128+f is never close enough to 224 for the f32 rounding of the
//     quotient to matter), so code = max(0, ((bits + 31) >> 7) - 8); zero, infinity and NaN are set apart;
//   * elements are scaled as packed bf16 pairs (a product with a power of two is exact in bf16 wherever the E4M3
//     code is not zero anyway) and widened only for the hardware e4m3x2 convert;
//   * the lanes that share a block meet by shuffle, one lane derives each block's scale and the others get it by
//     shuffle again;
//   * the tiny-negative fix-up of the E4M3 encode (cvt rounds -1e-9 to -0 = 0x80, the reference's search to
//     +0 = 0x00) and the plain f32 path for blocks with an infinite or NaN amax run behind ONE warp-uniform branch per
//     tile, taken only where some packed code is 0x80 or some scale code is 0xfe/0xff, which random data almost never has.
constexpr int kTileThreads = 256;

struct BsqTask {
    const void* x;
    uint8_t* y;
    uint8_t* scale;
    int64_t rows, cols;        // row form: flattened rows x cols; column form: K x N of one batch entry
    int64_t scale_k_extent;
    int32_t reordered;
    int32_t column_form;
    uint32_t tiles_x, tiles_y;  // column form: tiles along N and K (the batch axis is the slowest)
    uint32_t tiles;
    FastDivisor k_blocks;       // row form with a reordered scale: blocks per row, when every block index is < 2^29
    int32_t narrow_blocks;
    int32_t narrow_scale;       // a scale tensor of less than 2^30 bytes: 32-bit offsets into a reordered layout
};

// f8_128x4_offset() in 32-bit arithmetic, for scale tensors below 2^30 bytes.
__device__ __forceinline__ uint32_t f8_128x4_offset32(uint32_t leading, uint32_t m, uint32_t k, uint32_t m_extent, uint32_t k_extent) {
    const uint32_t m_blocks = m_extent >> 7, k_blocks = k_extent >> 2;
    return (((leading * m_blocks + (m >> 7)) * k_blocks + (k >> 2)) << 9) + ((m & 31u) << 4) + (((m >> 5) & 3u) << 2) + (k & 3u);
}

// Bit 7 of some byte of the result is set iff a byte of `codes` is 0x80 (callers OR several of these and mask once).
__device__ __forceinline__ uint32_t marks_of_0x80(uint32_t codes) {
    const uint32_t t = codes ^ 0x80808080u;  // a byte is zero exactly where the code was 0x80
    return (t - 0x01010101u) & ~t;
}

// Scale code of a block from the bf16 bit pattern of its |x| maximum (see above); equal to
// scale_code_from_amax_bits(bits << 16) for all 32768 patterns.
__device__ __forceinline__ uint32_t scale_code_from_bf16_amax(uint32_t bits) {
    const int code = static_cast<int>((bits + 31u) >> 7) - 8;
    uint32_t result = static_cast<uint32_t>(code < 0 ? 0 : code);
    if (bits == 0u) result = 127u;
    if (bits >= 0x7f80u) result = bits > 0x7f80u ? 0xffu : 0xfeu;
    return result;
}

// Unsigned maximum of the two 16-bit halves (one instruction; the __vmaxu2 intrinsic is a software sequence here).
__device__ __forceinline__ uint32_t max_u16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Two bf16 values (one word) times their two power-of-two reciprocals (bf16 pair) -> two E4M3 codes, low element in
// the low byte. Only meaningful for finite scales below 2^127 (codes 0..253).
__device__ __forceinline__ uint32_t scale_and_cvt_pair(uint32_t word, uint32_t reciprocals) {
    const uint32_t product = mul_bf16x2(word, reciprocals);
    return cvt_e4m3_pair(__uint_as_float(product << 16), __uint_as_float(product & 0xffff0000u));
}

// The exact rule for one word, whatever the codes: NaN-scaled elements are 0x7f, tiny negatives go to +0, -0.0 stays -0.
__device__ __forceinline__ uint32_t encode_pair_exact(uint32_t word, uint32_t code_lo, uint32_t code_hi) {
    const uint32_t both = encode_e4m3_pair(__fmul_rn(__uint_as_float(word << 16), reciprocal_e8m0(code_lo)),
                                           __fmul_rn(__uint_as_float(word & 0xffff0000u), reciprocal_e8m0(code_hi)));
    const uint32_t lo = code_lo == 0xffu ? 0x7fu : (both & 0xffu), hi = code_hi == 0xffu ? 0x7fu : (both >> 8);
    return lo | (hi << 8);
}

// Row form: thread t holds chunks (c * 256 + t) of 8 elements, c = 0..3; four lanes make one block of 32.
__device__ __forceinline__ void encode_row_tile(const BsqTask& task, uint32_t tile) {
    const int lane = threadIdx.x & 31;
    const int64_t tile0 = static_cast<int64_t>(tile) * 8192, left = task.rows * task.cols - tile0;
    const uint32_t count = static_cast<uint32_t>(left < 8192 ? left : 8192);  // elements of this tile
    const uint4* const x_tile = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(task.x) + tile0);
    uint4 raw[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t chunk = static_cast<uint32_t>(c) * 256u + threadIdx.x;
        raw[c] = chunk * 8u < count ? __ldg(x_tile + chunk) : make_uint4(0, 0, 0, 0);
    }
    // |x| maxima as bf16 bit patterns (integer order = magnitude order, NaN patterns are the largest)
    uint32_t amax16[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t a = raw[c].x & 0x7fff7fffu, b = raw[c].y & 0x7fff7fffu, d = raw[c].z & 0x7fff7fffu, e = raw[c].w & 0x7fff7fffu;
        uint32_t m = max_u16x2(max_u16x2(a, b), max_u16x2(d, e));
        m = max_u16x2(m, __shfl_xor_sync(0xffffffffu, m, 1));
        m = max_u16x2(m, __shfl_xor_sync(0xffffffffu, m, 2));
        amax16[c] = max(m & 0xffffu, m >> 16);
    }
    // lane q of a block (q = lane & 3) turns chunk q's maximum into its scale code; the four lanes then exchange
    const int q = lane & 3;
    const uint32_t mine = q == 0 ? amax16[0] : (q == 1 ? amax16[1] : (q == 2 ? amax16[2] : amax16[3]));
    const uint32_t my_code = scale_code_from_bf16_amax(mine);
    uint32_t code[4], worst = 0, marks = 0;
    uint2 packed[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        code[c] = __shfl_sync(0xffffffffu, my_code, (lane & ~3) + c);
        worst = max(worst, code[c]);
        const uint32_t reciprocals = ((254u - code[c]) << 7) * 0x00010001u;  // 2^(127 - code) twice, as bf16
        const uint32_t p0 = scale_and_cvt_pair(raw[c].x, reciprocals), p1 = scale_and_cvt_pair(raw[c].y, reciprocals);
        const uint32_t p2 = scale_and_cvt_pair(raw[c].z, reciprocals), p3 = scale_and_cvt_pair(raw[c].w, reciprocals);
        packed[c] = make_uint2(p0 | (p1 << 16), p2 | (p3 << 16));
        marks |= marks_of_0x80(packed[c].x) | marks_of_0x80(packed[c].y);
    }
    const bool redo = (marks & 0x80808080u) != 0u || worst >= 0xfeu;
    if (__any_sync(0xffffffffu, redo)) {
        if (redo) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
                packed[c] = make_uint2(encode_pair_exact(raw[c].x, code[c], code[c]) | (encode_pair_exact(raw[c].y, code[c], code[c]) << 16),
                                       encode_pair_exact(raw[c].z, code[c], code[c]) | (encode_pair_exact(raw[c].w, code[c], code[c]) << 16));
        }
    }
    uint8_t* const y_tile = task.y + tile0;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t offset = (static_cast<uint32_t>(c) * 256u + threadIdx.x) * 8u;
        if (offset < count) *reinterpret_cast<uint2*>(y_tile + offset) = packed[c];
    }
    if (q == 0) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t offset = (static_cast<uint32_t>(c) * 256u + threadIdx.x) * 8u;
            if (offset >= count) continue;
            if (!task.reordered) {
                task.scale[(tile0 + offset) >> 5] = static_cast<uint8_t>(code[c]);
            } else if (task.narrow_blocks && task.narrow_scale) {
                const uint32_t block_index = tile * 256u + (offset >> 5);
                const uint32_t row = fast_divide(block_index, task.k_blocks), kb = block_index - row * task.k_blocks.divisor;
                task.scale[f8_128x4_offset32(0, row, kb, static_cast<uint32_t>(task.rows), static_cast<uint32_t>(task.scale_k_extent))] = static_cast<uint8_t>(code[c]);
            } else {
                const int64_t block_index = (tile0 + offset) >> 5, k_blocks = task.cols >> 5;
                const int64_t row = block_index / k_blocks, kb = block_index - row * k_blocks;
                task.scale[f8_128x4_offset(0, row, kb, task.rows, task.scale_k_extent)] = static_cast<uint8_t>(code[c]);
            }
        }
    }
}

// Column form: warp w holds columns 32w..32w+31 of the tile's 256, lane l rows (l >> 2) + 8j (j = 0..3) and the 8
// columns 8(l & 3).. of them. The eight row groups of a warp meet by shuffle, lane l derives the scale code of column
// (l >> 2) of its lane group's eight, and the lanes of equal (l & 3) trade the eight codes by shuffle again.
__device__ __forceinline__ void encode_column_tile(const BsqTask& task, uint32_t tile) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = lane >> 2, part = lane & 3;
    const uint32_t tile_x = tile % task.tiles_x, rest = tile / task.tiles_x;
    const uint32_t kb = rest % task.tiles_y, batch = rest / task.tiles_y;
    const int64_t column = static_cast<int64_t>(tile_x) * 256 + warp * 32 + part * 8;
    const bool live = column < task.cols;
    const int64_t row0 = static_cast<int64_t>(batch) * task.rows + static_cast<int64_t>(kb) * 32 + group;  // counted over all batch entries
    const int64_t first = row0 * task.cols + (live ? column : 0), row_step = 8 * task.cols;
    const uint16_t* const x = static_cast<const uint16_t*>(task.x) + first;
    uint4 raw[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) raw[r] = __ldg(reinterpret_cast<const uint4*>(x + r * row_step));
    uint32_t best[4];
    best[0] = raw[0].x & 0x7fff7fffu;
    best[1] = raw[0].y & 0x7fff7fffu;
    best[2] = raw[0].z & 0x7fff7fffu;
    best[3] = raw[0].w & 0x7fff7fffu;
#pragma unroll
    for (int r = 1; r < 4; ++r) {
        best[0] = max_u16x2(best[0], raw[r].x & 0x7fff7fffu);
        best[1] = max_u16x2(best[1], raw[r].y & 0x7fff7fffu);
        best[2] = max_u16x2(best[2], raw[r].z & 0x7fff7fffu);
        best[3] = max_u16x2(best[3], raw[r].w & 0x7fff7fffu);
    }
#pragma unroll
    for (int offset = 4; offset < 32; offset <<= 1) {
#pragma unroll
        for (int i = 0; i < 4; ++i) best[i] = max_u16x2(best[i], __shfl_xor_sync(0xffffffffu, best[i], offset));
    }
    // column `group` of this lane's eight: word group >> 1, low or high half
    const uint32_t word = (group >> 1) == 0 ? best[0] : ((group >> 1) == 1 ? best[1] : ((group >> 1) == 2 ? best[2] : best[3]));
    const uint32_t my_code = scale_code_from_bf16_amax((group & 1) ? (word >> 16) : (word & 0xffffu));
    uint32_t code[8], worst = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        code[c] = __shfl_sync(0xffffffffu, my_code, c * 4 + part);
        worst = max(worst, code[c]);
    }
    uint32_t reciprocals[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) reciprocals[i] = ((254u - code[2 * i]) << 7) | ((254u - code[2 * i + 1]) << 23);
    uint2 packed[4];
    uint32_t marks = 0;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const uint32_t p0 = scale_and_cvt_pair(raw[r].x, reciprocals[0]), p1 = scale_and_cvt_pair(raw[r].y, reciprocals[1]);
        const uint32_t p2 = scale_and_cvt_pair(raw[r].z, reciprocals[2]), p3 = scale_and_cvt_pair(raw[r].w, reciprocals[3]);
        packed[r] = make_uint2(p0 | (p1 << 16), p2 | (p3 << 16));
        marks |= marks_of_0x80(packed[r].x) | marks_of_0x80(packed[r].y);
    }
    const bool redo = (marks & 0x80808080u) != 0u || worst >= 0xfeu;
    if (__any_sync(0xffffffffu, redo)) {
        if (redo) {
#pragma unroll
            for (int r = 0; r < 4; ++r)
                packed[r] = make_uint2(encode_pair_exact(raw[r].x, code[0], code[1]) | (encode_pair_exact(raw[r].y, code[2], code[3]) << 16),
                                       encode_pair_exact(raw[r].z, code[4], code[5]) | (encode_pair_exact(raw[r].w, code[6], code[7]) << 16));
        }
    }
    if (!live) return;
    uint8_t* const out = task.y + first;
#pragma unroll
    for (int r = 0; r < 4; ++r) *reinterpret_cast<uint2*>(out + r * row_step) = packed[r];
    // (lane `group` == column index: every lane stores the one code it derived)
    if (task.reordered && task.narrow_scale) {
        task.scale[f8_128x4_offset32(batch, static_cast<uint32_t>(column) + group, kb, static_cast<uint32_t>(task.cols), static_cast<uint32_t>(task.scale_k_extent))] = static_cast<uint8_t>(my_code);
    } else if (task.reordered) {
        task.scale[f8_128x4_offset(batch, column + group, kb, task.cols, task.scale_k_extent)] = static_cast<uint8_t>(my_code);
    } else {
        task.scale[(static_cast<int64_t>(batch) * (task.rows >> 5) + kb) * task.cols + column + group] = static_cast<uint8_t>(my_code);
    }
}

// (five CTAs per SM: 48 registers; more warps hide the load latency better than the few spilled bytes cost)
__global__ void __launch_bounds__(kTileThreads, 5)
bsq_tile_bf16_kernel(const BsqTask first, const BsqTask second) {
    chain_release();
    chain_wait();
    const bool in_first = blockIdx.x < first.tiles;
    const BsqTask task = in_first ? first : second;
    const uint32_t tile = in_first ? blockIdx.x : blockIdx.x - first.tiles;
    if (task.column_form) encode_column_tile(task, tile);
    else encode_row_tile(task, tile);
}

// ---- dequantize -------------------------------------------------------------------

struct BlockSizes {
    int64_t per_axis[DFGPU_MAX_RANK];
};

__global__ void bsd_generic_kernel(const uint8_t* x, const uint8_t* scale, void* y, View xv, View sv, View yv,
                                   ScaleLayout layout, int block_first_axis, BlockSizes sizes, int64_t total) {
    int64_t flat = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (flat >= total) return;
    const int64_t* blocks = sizes.per_axis;  // 1 where unblocked
    int64_t index[DFGPU_MAX_RANK], scale_index[DFGPU_MAX_RANK];
    for (int i = yv.rank - 1; i >= 0; --i) {
        index[i] = flat % yv.dim[i];
        flat /= yv.dim[i];
        scale_index[i] = i >= block_first_axis ? index[i] / blocks[i] : index[i];
    }
    int64_t xo = 0, yo = 0;
    for (int i = 0; i < yv.rank; ++i) {
        xo += index[i] * xv.stride[i];
        yo += index[i] * yv.stride[i];
    }
    // codes: FP8 (a byte each) or FP4 / INT4 (two to a byte); scales: E8M0, E4M3 or a plain floating type
    float code_value = load_as_f32(x, xv.dtype, xo);
    float value = __fmul_rn(code_value, load_as_f32(scale, sv.dtype, scale_offset(sv, layout, scale_index)));
    store_from_f32(y, yv.dtype, yo, value);
}

// Packed rank-2 [R, C]: a thread turns 16 consecutive codes of one row into 16 outputs.
template <int OUT_DTYPE>
__global__ void __launch_bounds__(256)
bsd_packed_kernel(const uint8_t* __restrict__ x, const uint8_t* __restrict__ scale, void* __restrict__ y,
                  int64_t rows, int64_t cols, int64_t block_rows, int64_t block_cols) {
    int64_t thread = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    int64_t element = thread * 16;
    if (element >= rows * cols) return;
    int64_t row = element / cols, col = element - row * cols;
    int64_t scale_cols = cols / block_cols;
    uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + element));
    uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float out[16];
    const uint8_t* scale_row = scale + (row / block_rows) * scale_cols;
    if (block_cols >= 16) {
        float s = decode_e8m0(__ldg(scale_row + col / block_cols));
#pragma unroll
        for (int i = 0; i < 16; ++i) out[i] = __fmul_rn(decode_e4m3((w[i >> 2] >> ((i & 3) * 8)) & 0xffu), s);
    } else if (block_cols == 1 && ((reinterpret_cast<uintptr_t>(scale_row + col)) & 15u) == 0) {
        // one scale per column (blocks run down the rows): 16 scale bytes in one load
        uint4 sraw = __ldg(reinterpret_cast<const uint4*>(scale_row + col));
        uint32_t sw[4] = {sraw.x, sraw.y, sraw.z, sraw.w};
#pragma unroll
        for (int i = 0; i < 16; ++i)
            out[i] = __fmul_rn(decode_e4m3((w[i >> 2] >> ((i & 3) * 8)) & 0xffu), decode_e8m0((sw[i >> 2] >> ((i & 3) * 8)) & 0xffu));
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float s = decode_e8m0(__ldg(scale_row + (col + i) / block_cols));
            out[i] = __fmul_rn(decode_e4m3((w[i >> 2] >> ((i & 3) * 8)) & 0xffu), s);
        }
    }
    if (OUT_DTYPE == DFGPU_F32) {
        float4* dst = reinterpret_cast<float4*>(static_cast<float*>(y) + element);
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = make_float4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
    } else {
        uint32_t packed[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint32_t lo, hi;
            if (OUT_DTYPE == DFGPU_BF16) {
                lo = f32_to_bf16_bits(out[2 * i]);
                hi = f32_to_bf16_bits(out[2 * i + 1]);
            } else {
                lo = __half_as_ushort(__float2half_rn(out[2 * i]));
                hi = __half_as_ushort(__float2half_rn(out[2 * i + 1]));
            }
            packed[i] = lo | (hi << 16);
        }
        uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(y) + element);
        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    }
}

bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

struct BsqPlan {
    int kernel = 0;
    int axis = 0;
    bool needs_fill = false;
    ScaleLayout layout{};
    int64_t rows = 0, cols = 0, batch = 0, scale_k_extent = 0;
    int64_t scale_bytes = 0;  // (E8M0: one byte per slot, padding slots included)
};

int plan_bsq(const dfgpu_bsq_params& p, BsqPlan& plan) {
    if (!valid_tensor(p.x) || !valid_tensor(p.y) || !valid_tensor(p.scale))
        return fail(kInvalidShape, "BLOCK_SCALE_QUANTIZE: tensor rank or extent out of range");
    if (p.x.dtype != DFGPU_F32 && p.x.dtype != DFGPU_F16 && p.x.dtype != DFGPU_BF16)
        return fail(kUnsupported, "BLOCK_SCALE_QUANTIZE: X must be FLOAT, HALF or BFLOAT16");
    // lib/Compiler/SpecializedGraph.cpp:368-380
    const bool fp4 = p.y.dtype == DFGPU_FP4;
    if (fp4 ? p.scale.dtype != DFGPU_E4M3 : ((p.y.dtype != DFGPU_E4M3 && p.y.dtype != DFGPU_E5M2) || p.scale.dtype != DFGPU_E8M0))
        return fail(kUnsupported, "BLOCK_SCALE_QUANTIZE: FP8_E4M3 or FP8_E5M2 codes take FP8_E8M0 scales, FP4_E2M1 codes FP8_E4M3 scales");
    if (fp4 && p.scale.reorder != DFGPU_REORDER_NONE) return fail(kUnsupported, "BLOCK_SCALE_QUANTIZE: FP4 codes take an unreordered scale tensor");
    int rank = p.x.rank;
    if (p.y.rank != rank || p.scale.rank != rank)
        return fail(kInvalidShape, "BLOCK_SCALE_QUANTIZE: X, Y and scale ranks differ");
    int axis = p.axis < 0 ? rank - 1 : p.axis;
    if (axis >= rank || p.block_size <= 0 || p.x.dim[axis] % p.block_size != 0)
        return fail(kInvalidShape, "BLOCK_SCALE_QUANTIZE: block size does not divide the block axis");
    bool scale_matches = true;
    for (int i = 0; i < rank; ++i) {
        if (p.y.dim[i] != p.x.dim[i]) return fail(kInvalidShape, "BLOCK_SCALE_QUANTIZE: Y dims differ from X");
        int64_t logical = i == axis ? p.x.dim[i] / p.block_size : p.x.dim[i];
        if (p.scale.dim[i] < logical) return fail(kInvalidShape, "BLOCK_SCALE_QUANTIZE: scale tensor smaller than the block grid");
        if (p.scale.dim[i] != logical) scale_matches = false;
    }
    if (!resolve_reorder(p.scale, plan.layout))
        return fail(kInvalidLayout, "BLOCK_SCALE_QUANTIZE: scale is not a valid F8_128x4 layout");
    plan.axis = axis;
    plan.needs_fill = !scale_matches;
    plan.scale_bytes = element_count(p.scale);

    bool packed = is_packed_row_major(p.x) && is_packed_row_major(p.y);
    for (int i = 0; i + 2 < rank; ++i)
        if (p.scale.dim[i] != p.x.dim[i]) packed = false;  // fast kernels want an unpadded leading grid
    if (plan.layout.reordered) plan.scale_k_extent = p.scale.dim[plan.layout.k_axis];
    bool scale_ok_none = plan.layout.reordered == 0 && scale_matches && is_packed_row_major(p.scale);
    int kernel = DFGPU_BSQ_GENERIC;
    if (packed && p.block_size == 32) {
        if (axis == rank - 1) {
            bool reordered_ok = plan.layout.reordered && rank == 2 && plan.layout.m_axis == 0 &&
                                p.scale.dim[0] == p.x.dim[0];
            if (scale_ok_none || reordered_ok) {
                kernel = DFGPU_BSQ_ROW32;
                plan.cols = p.x.dim[rank - 1];
                plan.rows = element_count(p.x) / plan.cols;
            }
        } else if (axis == rank - 2 && rank >= 2) {
            int vec = p.x.dtype == DFGPU_F32 ? 4 : 8;
            bool reordered_ok = plan.layout.reordered && plan.layout.m_axis == rank - 1 &&
                                p.scale.dim[rank - 1] == p.x.dim[rank - 1];
            if ((scale_ok_none || reordered_ok) && p.x.dim[rank - 1] % vec == 0) {
                kernel = DFGPU_BSQ_COL32;
                plan.cols = p.x.dim[rank - 1];
                plan.rows = p.x.dim[rank - 2];
                plan.batch = element_count(p.x) / (plan.cols * plan.rows);
                if (plan.batch > 65535 || plan.rows / 32 > 65535) kernel = DFGPU_BSQ_GENERIC;
            }
        }
    }
    if (p.y.dtype != DFGPU_E4M3) kernel = DFGPU_BSQ_GENERIC;   // (the fast kernels are built on the hardware e4m3x2 convert)
    if (p.kernel != DFGPU_BSQ_AUTO && p.kernel != kernel) {
        if (p.kernel == DFGPU_BSQ_GENERIC) kernel = DFGPU_BSQ_GENERIC;
        else return fail(kUnsupported, "BLOCK_SCALE_QUANTIZE: requested kernel %d does not cover this layout", p.kernel);
    }
    plan.kernel = kernel;
    return kOk;
}

// The bf16 tile kernel's view of one tensor whose plan is the row or the column form.
BsqTask tile_task(const BsqPlan& plan, const void* x, uint8_t* y, uint8_t* scale) {
    BsqTask task{};
    task.x = x;
    task.y = y;
    task.scale = scale;
    task.rows = plan.rows;
    task.cols = plan.cols;
    task.scale_k_extent = plan.scale_k_extent;
    task.reordered = plan.layout.reordered;
    task.k_blocks = make_fast_divisor(1);
    task.narrow_scale = plan.scale_bytes > 0 && plan.scale_bytes < (1ll << 30) ? 1 : 0;
    if (plan.kernel == DFGPU_BSQ_ROW32) {
        task.column_form = 0;
        task.tiles = static_cast<uint32_t>((plan.rows * plan.cols + 8191) / 8192);
        const int64_t k_blocks = plan.cols / 32, blocks = plan.rows * k_blocks;
        task.narrow_blocks = blocks < (1ll << 29) ? 1 : 0;
        if (task.narrow_blocks) task.k_blocks = make_fast_divisor(static_cast<uint32_t>(k_blocks));
    } else {
        task.column_form = 1;
        task.tiles_x = static_cast<uint32_t>((plan.cols + 255) / 256);
        task.tiles_y = static_cast<uint32_t>(plan.rows / 32);
        task.tiles = task.tiles_x * task.tiles_y * static_cast<uint32_t>(plan.batch);
    }
    return task;
}

// One CTA per tile: the tiles of one launch must fit a grid.
bool tile_task_fits(const BsqPlan& plan) {
    const int64_t tiles = plan.kernel == DFGPU_BSQ_ROW32 ? (plan.rows * plan.cols + 8191) / 8192 : ((plan.cols + 255) / 256) * (plan.rows / 32) * plan.batch;
    return tiles > 0 && tiles <= (1ll << 30);
}

int launch_tiles(const BsqTask& first, const BsqTask& second, cudaStream_t stream, const char* what) {
    cudaError_t status = launch_chained(bsq_tile_bf16_kernel, dim3(first.tiles + second.tiles), dim3(kTileThreads), 0, stream, first, second);
    if (status != cudaSuccess) return fail(kExecutionFailed, "%s: launch failed: %s", what, cudaGetErrorString(status));
    return check_launch(what);
}

}  // namespace
}  // namespace dfgpu

using namespace dfgpu;

extern "C" int dfgpu_query_block_scale_quantize(const dfgpu_bsq_params* p, dfgpu_plan_info* info) {
    if (!p || !info) return fail(kInvalidArgument, "BLOCK_SCALE_QUANTIZE: null params");
    BsqPlan plan;
    int status = plan_bsq(*p, plan);
    if (status) return status;
    info->kernel = plan.kernel;
    info->launches = 1 + (plan.needs_fill ? 1 : 0);
    info->scratch_bytes = 0;
    return kOk;
}

extern "C" int dfgpu_block_scale_quantize(const dfgpu_bsq_params* p, void* const* tensors, void* scratch,
                                          void* stream_handle) {
    (void)scratch;
    if (!p || !tensors) return fail(kInvalidArgument, "BLOCK_SCALE_QUANTIZE: null params");
    BsqPlan plan;
    int status = plan_bsq(*p, plan);
    if (status) return status;
    const void* x = tensors[0];
    uint8_t* y = static_cast<uint8_t*>(tensors[1]);
    uint8_t* scale = static_cast<uint8_t*>(tensors[2]);
    if (!x || !y || !scale) return fail(kInvalidArgument, "BLOCK_SCALE_QUANTIZE: null tensor pointer");
    cudaStream_t stream = as_stream(stream_handle);

    if (plan.needs_fill) {
        // step 1 of the reference: every scale slot, padding included, <- encode(1.0)
        int64_t count = element_count(p->scale);
        const uint8_t one = p->scale.dtype == DFGPU_E4M3 ? 0x38 : 0x7f;   // 1.0 as E4M3 (FP4 codes) or E8M0
        if (plan.layout.reordered || is_packed_row_major(p->scale)) {
            int64_t threads = (count + 15) / 16;
            fill_bytes_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(scale, count, one);
        } else {
            fill_strided_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, stream>>>(
                scale, make_view(p->scale), count, one);
        }
    }

    int kernel = plan.kernel;
    if (kernel == DFGPU_BSQ_ROW32 && !(aligned(x, 16) && aligned(y, 8))) kernel = DFGPU_BSQ_GENERIC;
    if (kernel == DFGPU_BSQ_COL32 && !(aligned(x, 16) && aligned(y, 8) && aligned(scale, 8))) kernel = DFGPU_BSQ_GENERIC;
    if (p->x.dtype == DFGPU_BF16 && kernel != DFGPU_BSQ_GENERIC && !tile_task_fits(plan)) kernel = DFGPU_BSQ_GENERIC;

    if (kernel == DFGPU_BSQ_ROW32) {
        int64_t threads = (plan.rows * plan.cols / 8 + 3) / 4;  // 4 chunks of 8 elements per thread
        unsigned grid = static_cast<unsigned>((threads + 255) / 256);
        int reordered = plan.layout.reordered;
        if (p->x.dtype == DFGPU_F32) launch_chained(bsq_row32_kernel<float>, dim3(grid), dim3(256), 0, stream, x, y, scale, plan.rows, plan.cols, reordered, plan.scale_k_extent);
        else if (p->x.dtype == DFGPU_BF16) return launch_tiles(tile_task(plan, x, y, scale), BsqTask{}, stream, "BLOCK_SCALE_QUANTIZE");
        else launch_chained(bsq_row32_kernel<__half>, dim3(grid), dim3(256), 0, stream, x, y, scale, plan.rows, plan.cols, reordered, plan.scale_k_extent);
    } else if (kernel == DFGPU_BSQ_COL32) {
        int vec = p->x.dtype == DFGPU_F32 ? 4 : 8;
        int64_t lanes = plan.cols / vec;  // one lane per group of vec columns, 32 lanes (x 4 row groups) per CTA
        dim3 grid(static_cast<unsigned>((lanes + 31) / 32), static_cast<unsigned>(plan.rows / 32),
                  static_cast<unsigned>(plan.batch));
        int reordered = plan.layout.reordered;
        if (p->x.dtype == DFGPU_F32) launch_chained(bsq_col32_kernel<float>, grid, dim3(128), 0, stream, x, y, scale, plan.rows, plan.cols, reordered, plan.scale_k_extent);
        else if (p->x.dtype == DFGPU_BF16) return launch_tiles(tile_task(plan, x, y, scale), BsqTask{}, stream, "BLOCK_SCALE_QUANTIZE");
        else launch_chained(bsq_col32_kernel<__half>, grid, dim3(128), 0, stream, x, y, scale, plan.rows, plan.cols, reordered, plan.scale_k_extent);
    } else {
        int64_t block_total = element_count(p->x) / p->block_size;
        unsigned grid = static_cast<unsigned>((block_total + 127) / 128);
        bsq_generic_kernel<<<grid, 128, 0, stream>>>(x, y, scale, make_view(p->x), make_view(p->y),
                                                     make_view(p->scale), plan.layout, plan.axis, p->block_size,
                                                     block_total);
    }
    return check_launch("BLOCK_SCALE_QUANTIZE");
}

namespace {

struct BsdPlan {
    int kernel = 0;
    ScaleLayout layout{};
    int64_t blocks[DFGPU_MAX_RANK];
    int first_axis = 0;
};

int plan_bsd(const dfgpu_bsd_params& p, BsdPlan& plan) {
    if (!valid_tensor(p.x) || !valid_tensor(p.y) || !valid_tensor(p.scale))
        return fail(kInvalidShape, "BLOCK_SCALE_DEQUANTIZE: tensor rank or extent out of range");
    // lib/Compiler/SpecializedGraph.cpp:291-302
    const bool code_ok = p.x.dtype == DFGPU_E4M3 || p.x.dtype == DFGPU_E5M2 || p.x.dtype == DFGPU_FP4 || p.x.dtype == DFGPU_I4;
    const bool scale_ok = p.scale.dtype == DFGPU_E8M0 || p.scale.dtype == DFGPU_E4M3 || p.scale.dtype == DFGPU_F32 || p.scale.dtype == DFGPU_F16 || p.scale.dtype == DFGPU_BF16;
    if (!code_ok || !scale_ok)
        return fail(kUnsupported, "BLOCK_SCALE_DEQUANTIZE: X must be FP8_E4M3, FP8_E5M2, FP4_E2M1 or INT4 and the scale FP8_E8M0, FP8_E4M3, FLOAT, HALF or BFLOAT16");
    if (p.scale.dtype != DFGPU_E8M0 && p.scale.reorder != DFGPU_REORDER_NONE) return fail(kUnsupported, "BLOCK_SCALE_DEQUANTIZE: only FP8_E8M0 scales may be reordered");
    if (p.y.dtype != DFGPU_F32 && p.y.dtype != DFGPU_F16 && p.y.dtype != DFGPU_BF16)
        return fail(kUnsupported, "BLOCK_SCALE_DEQUANTIZE: Y must be FLOAT, HALF or BFLOAT16");
    int rank = p.y.rank;
    if (p.x.rank != rank || p.scale.rank != rank || p.block_count < 1 || p.block_count > rank)
        return fail(kInvalidShape, "BLOCK_SCALE_DEQUANTIZE: ranks or block_size length inconsistent");
    plan.first_axis = rank - p.block_count;
    for (int i = 0; i < DFGPU_MAX_RANK; ++i) plan.blocks[i] = 1;
    for (int i = 0; i < rank; ++i) {
        if (p.x.dim[i] != p.y.dim[i]) return fail(kInvalidShape, "BLOCK_SCALE_DEQUANTIZE: X dims differ from Y");
        int64_t block = i >= plan.first_axis ? p.block[i - plan.first_axis] : 1;
        if (block <= 0) return fail(kInvalidShape, "BLOCK_SCALE_DEQUANTIZE: non-positive block size");
        plan.blocks[i] = block;
        if (p.scale.dim[i] < (p.y.dim[i] + block - 1) / block)
            return fail(kInvalidShape, "BLOCK_SCALE_DEQUANTIZE: scale tensor smaller than the block grid");
    }
    if (!resolve_reorder(p.scale, plan.layout))
        return fail(kInvalidLayout, "BLOCK_SCALE_DEQUANTIZE: scale is not a valid F8_128x4 layout");
    int kernel = DFGPU_BSD_GENERIC;
    if (rank == 2 && !plan.layout.reordered && is_packed_row_major(p.x) && is_packed_row_major(p.y) &&
        is_packed_row_major(p.scale) && p.y.dim[1] % 16 == 0 && p.y.dim[0] % plan.blocks[0] == 0 &&
        p.y.dim[1] % plan.blocks[1] == 0 && p.scale.dim[0] == p.y.dim[0] / plan.blocks[0] &&
        p.scale.dim[1] == p.y.dim[1] / plan.blocks[1] && (plan.blocks[1] % 16 == 0 || plan.blocks[1] < 16))
        kernel = DFGPU_BSD_PACKED;
    if (p.x.dtype != DFGPU_E4M3 || p.scale.dtype != DFGPU_E8M0) kernel = DFGPU_BSD_GENERIC;
    if (p.kernel != DFGPU_BSD_AUTO && p.kernel != kernel) {
        if (p.kernel == DFGPU_BSD_GENERIC) kernel = DFGPU_BSD_GENERIC;
        else return fail(kUnsupported, "BLOCK_SCALE_DEQUANTIZE: requested kernel %d does not cover this layout", p.kernel);
    }
    plan.kernel = kernel;
    return kOk;
}

}  // namespace

// ---- two BLOCK_SCALE_QUANTIZE nodes in one launch ---------------------------------------------------

namespace {
// The task of one tensor inside the shared grid, when its plan is one of the two bf16 fast forms with nothing to
// pre-fill; false otherwise (the caller then launches the nodes separately).
bool pair_task(const dfgpu_bsq_params& p, void* const* tensors, dfgpu::BsqTask& task) {
    using namespace dfgpu;
    BsqPlan plan;
    if (plan_bsq(p, plan) != kOk || plan.needs_fill || p.x.dtype != DFGPU_BF16) return false;
    if (plan.kernel != DFGPU_BSQ_ROW32 && plan.kernel != DFGPU_BSQ_COL32) return false;
    if (!tile_task_fits(plan)) return false;
    task = tile_task(plan, tensors ? tensors[0] : nullptr, tensors ? static_cast<uint8_t*>(tensors[1]) : nullptr, tensors ? static_cast<uint8_t*>(tensors[2]) : nullptr);
    return true;
}
}  // namespace

extern "C" int dfgpu_query_block_scale_quantize_pair(const dfgpu_bsq_pair_params* p, dfgpu_plan_info* info) {
    if (!p || !info) return fail(kInvalidArgument, "BLOCK_SCALE_QUANTIZE pair: null params");
    BsqTask first, second;
    if (!pair_task(p->first, nullptr, first) || !pair_task(p->second, nullptr, second))
        return fail(kUnsupported, "BLOCK_SCALE_QUANTIZE pair: both tensors must take a bf16 32-element fast form with an unpadded scale tensor");
    info->kernel = DFGPU_BSQ_PAIR_BF16;
    info->launches = 1;
    info->scratch_bytes = 0;
    return kOk;
}

extern "C" int dfgpu_block_scale_quantize_pair(const dfgpu_bsq_pair_params* p, void* const* tensors, void* scratch, void* stream_handle) {
    (void)scratch;
    if (!p || !tensors) return fail(kInvalidArgument, "BLOCK_SCALE_QUANTIZE pair: null params");
    for (int i = 0; i < 6; ++i)
        if (!tensors[i]) return fail(kInvalidArgument, "BLOCK_SCALE_QUANTIZE pair: null tensor pointer");
    BsqTask first, second;
    if (!pair_task(p->first, tensors, first) || !pair_task(p->second, tensors + 3, second))
        return fail(kUnsupported, "BLOCK_SCALE_QUANTIZE pair: both tensors must take a bf16 32-element fast form with an unpadded scale tensor");
    for (int i = 0; i < 6; ++i)
        if (!aligned(tensors[i], i % 3 == 0 ? 16 : 8)) return fail(kInvalidArgument, "BLOCK_SCALE_QUANTIZE pair: X must be 16-byte aligned, Y and scale 8-byte aligned");
    return launch_tiles(first, second, as_stream(stream_handle), "BLOCK_SCALE_QUANTIZE pair");
}

extern "C" int dfgpu_query_block_scale_dequantize(const dfgpu_bsd_params* p, dfgpu_plan_info* info) {
    if (!p || !info) return fail(kInvalidArgument, "BLOCK_SCALE_DEQUANTIZE: null params");
    BsdPlan plan;
    int status = plan_bsd(*p, plan);
    if (status) return status;
    info->kernel = plan.kernel;
    info->launches = 1;
    info->scratch_bytes = 0;
    return kOk;
}

extern "C" int dfgpu_block_scale_dequantize(const dfgpu_bsd_params* p, void* const* tensors, void* scratch,
                                            void* stream_handle) {
    (void)scratch;
    if (!p || !tensors) return fail(kInvalidArgument, "BLOCK_SCALE_DEQUANTIZE: null params");
    BsdPlan plan;
    int status = plan_bsd(*p, plan);
    if (status) return status;
    const uint8_t* x = static_cast<const uint8_t*>(tensors[0]);
    const uint8_t* scale = static_cast<const uint8_t*>(tensors[1]);
    void* y = tensors[2];
    if (!x || !y || !scale) return fail(kInvalidArgument, "BLOCK_SCALE_DEQUANTIZE: null tensor pointer");
    cudaStream_t stream = as_stream(stream_handle);
    int kernel = plan.kernel;
    if (kernel == DFGPU_BSD_PACKED && !(aligned(x, 16) && aligned(y, 16))) kernel = DFGPU_BSD_GENERIC;
    int64_t total = element_count(p->y);
    if (kernel == DFGPU_BSD_PACKED) {
        int64_t threads = total / 16;
        unsigned grid = static_cast<unsigned>((threads + 255) / 256);
        int64_t rows = p->y.dim[0], cols = p->y.dim[1];
        if (p->y.dtype == DFGPU_F32) bsd_packed_kernel<DFGPU_F32><<<grid, 256, 0, stream>>>(x, scale, y, rows, cols, plan.blocks[0], plan.blocks[1]);
        else if (p->y.dtype == DFGPU_BF16) bsd_packed_kernel<DFGPU_BF16><<<grid, 256, 0, stream>>>(x, scale, y, rows, cols, plan.blocks[0], plan.blocks[1]);
        else bsd_packed_kernel<DFGPU_F16><<<grid, 256, 0, stream>>>(x, scale, y, rows, cols, plan.blocks[0], plan.blocks[1]);
    } else {
        unsigned grid = static_cast<unsigned>((total + 255) / 256);
        BlockSizes sizes;
        for (int i = 0; i < DFGPU_MAX_RANK; ++i) sizes.per_axis[i] = plan.blocks[i];
        bsd_generic_kernel<<<grid, 256, 0, stream>>>(x, scale, y, make_view(p->x), make_view(p->scale),
                                                     make_view(p->y), plan.layout, plan.first_axis, sizes, total);
    }
    return check_launch("BLOCK_SCALE_DEQUANTIZE");
}

extern "C" int dfgpu_selfcheck_e4m3(uint32_t first_bits, uint64_t count, void* result, void* stream_handle) {
    if (!result) return fail(kInvalidArgument, "selfcheck: null result pointer");
    selfcheck_e4m3_kernel<<<148 * 8, 256, 0, as_stream(stream_handle)>>>(
        first_bits, count, static_cast<unsigned long long*>(result));
    return check_launch("selfcheck_e4m3");
}

extern "C" int dfgpu_debug_scale_codes(const void* amax, void* codes, int64_t count, void* stream_handle) {
    if (!amax || !codes || count < 0) return fail(kInvalidArgument, "debug_scale_codes: bad arguments");
    if (count == 0) return kOk;
    debug_scale_codes_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, as_stream(stream_handle)>>>(
        static_cast<const float*>(amax), static_cast<uint8_t*>(codes), count);
    return check_launch("debug_scale_codes");
}

extern "C" int dfgpu_debug_encode_e4m3(const void* values, void* codes, int64_t count, void* stream_handle) {
    if (!values || !codes || count < 0) return fail(kInvalidArgument, "debug_encode_e4m3: bad arguments");
    if (count == 0) return kOk;
    debug_encode_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, as_stream(stream_handle)>>>(
        static_cast<const float*>(values), static_cast<uint8_t*>(codes), count);
    return check_launch("debug_encode_e4m3");
}

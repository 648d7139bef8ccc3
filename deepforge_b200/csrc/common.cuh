// Shared device/host helpers of the dfgpu kernel library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "dfgpu.h"

namespace dfgpu {

// DeepForge Status codes the launchers return.
constexpr int kOk = 0;
constexpr int kInvalidArgument = 1;
constexpr int kInvalidValue = 8;
constexpr int kInvalidLayout = 14;
constexpr int kInvalidShape = 15;
constexpr int kExecutionFailed = 19;
constexpr int kUnsupported = 20;

int fail(int code, const char* format, ...);
int check_launch(const char* what);

inline cudaStream_t as_stream(void* stream) { return static_cast<cudaStream_t>(stream); }

inline int64_t element_count(const dfgpu_tensor& t) {
    int64_t count = 1;
    for (int i = 0; i < t.rank; ++i) count *= t.dim[i];
    return count;
}

inline bool is_packed_row_major(const dfgpu_tensor& t) {
    int64_t expected = 1;
    for (int i = t.rank - 1; i >= 0; --i) {
        if (t.dim[i] != 1 && t.stride[i] != expected) return false;
        expected *= t.dim[i];
    }
    return true;
}

inline int dtype_bytes(int dtype) {
    switch (dtype) {
        case DFGPU_F32: case DFGPU_I32: case DFGPU_BF16X2: return 4;
        case DFGPU_I64: return 8;
        case DFGPU_E5M2: case DFGPU_U8: return 1;
        case DFGPU_F16: case DFGPU_BF16: return 2;
        default: return 1;
    }
}

inline bool valid_tensor(const dfgpu_tensor& t) {
    if (t.rank < 1 || t.rank > DFGPU_MAX_RANK) return false;
    for (int i = 0; i < t.rank; ++i)
        if (t.dim[i] <= 0 || t.stride[i] < 0) return false;
    return true;
}

int sm_count();

// ---- programmatic dependent launch ------------------------------------------------
// A kernel launched with launch_chained() may start while the kernel before it in the stream is still
// draining: its CTAs take SMs as the earlier kernel's CTAs leave, run their private prologue (barrier
// setup, tensor-memory allocation) and then block in chain_wait() until the earlier kernel has completed
// and its writes are visible. Every kernel launched this way must call chain_wait() before its first
// global-memory access; chain_release() at its top lets the kernel after it do the same. Both are no-ops
// when the kernel was launched the ordinary way. Captured into a CUDA graph the dependency becomes a
// programmatic edge, so the gap between the kernels of one plan shrinks to the tail of the slowest CTA.
#ifdef __CUDACC__
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <typename... Params, typename... Args>
cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t dynamic_smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t config{};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = dynamic_smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}
#endif

// ---- device-side element access -------------------------------------------------

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) {
    return __uint_as_float(bits16 << 16);
}

// Round-to-nearest-even f32 -> bf16 with NaN kept quiet (arith.truncf semantics).
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float value) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(value));
}

// E4M3 decode: exponent 0 -> m * 2^-9, 0x7f/0xff -> NaN, else (1+m/8) * 2^(e-7).
__device__ __forceinline__ float decode_e4m3(uint32_t code) {
    uint32_t magnitude = code & 0x7fu;
    float value;
    if (magnitude == 0x7fu) {
        value = __int_as_float(0x7fc00000);
    } else if ((magnitude >> 3) == 0) {
        value = static_cast<float>(magnitude) * 0.001953125f;
    } else {
        // place exponent/mantissa into an f32: bias 7 -> 127 adds 120 to the exponent
        value = __uint_as_float((magnitude << 20) + (120u << 23));
    }
    return (code & 0x80u) ? -value : value;
}

// E8M0 decode: 2^(code-127); 0xff -> NaN. Code 0 is the f32 subnormal 2^-127.
__device__ __forceinline__ float decode_e8m0(uint32_t code) {
    if (code == 0xffu) return __int_as_float(0x7fc00000);
    if (code == 0u) return __uint_as_float(0x00400000u);
    return __uint_as_float(code << 23);
}

// Exact reciprocal of an E8M0 scale as f32 (2^(127-code)); multiplying by it is
// bit-identical to the IEEE division by the scale because both are the correctly
// rounded value of the same real number. code 254 -> 2^-127 (subnormal), NaN kept.
__device__ __forceinline__ float reciprocal_e8m0(uint32_t code) {
    if (code == 0xffu) return __int_as_float(0x7fc00000);
    if (code == 254u) return __uint_as_float(0x00400000u);
    return __uint_as_float((254u - code) << 23);
}

// ---- f32 -> E4M3 with the reference's search semantics (lib/Compiler/Numeric.cpp:504-632): the hardware
// convert (round to nearest even, saturate to 448) plus two fix-ups, NaN -> 0x7f and a negative that rounds
// to zero -> +0.
// Two f32 -> two E4M3 codes (first value in the low byte).
__device__ __forceinline__ uint32_t cvt_e4m3_pair(float first, float second) {
    uint16_t packed;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(packed) : "f"(second), "f"(first));
    return packed;
}

// A negative in [-2^-10, -0) rounds to zero: the reference gives +0 for it.
__device__ __forceinline__ float flush_negative_underflow(float v) {
    uint32_t bits = __float_as_uint(v);
    return (bits - 0x80000001u) <= (0xBA800000u - 0x80000001u) ? 0.0f : v;
}

__device__ __forceinline__ uint32_t encode_e4m3_pair(float a, float b) {
    return cvt_e4m3_pair(flush_negative_underflow(a), flush_negative_underflow(b));
}

__device__ __forceinline__ uint32_t encode_e4m3_scalar(float v) {
    if (v != v) return 0x7fu;
    return encode_e4m3_pair(v, 0.0f) & 0xffu;
}

// E5M2 is the upper byte of binary16: decode through the half type (subnormals, infinity and NaN included).
__device__ __forceinline__ float decode_e5m2(uint32_t code) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(code << 8)));
}
// f32 -> E5M2 with the reference's search semantics (lib/Compiler/Numeric.cpp:396-425, 504-632): round to nearest
// even, |v| > 57344 (infinity included) -> 0x7b | sign, NaN -> 0x7f, a negative that rounds to zero -> +0.
__device__ __forceinline__ uint32_t encode_e5m2_scalar(float v) {
    if (v != v) return 0x7fu;
    const uint32_t bits = __float_as_uint(v);
    if ((bits - 0x80000001u) <= (0xB7000000u - 0x80000001u)) v = 0.0f;  // [-2^-17, -0): rounds to zero, the reference gives +0
    uint16_t packed;
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(packed) : "f"(0.0f), "f"(v));
    return packed & 0xffu;
}

// FP4 E2M1 (lib/Compiler/Numeric.cpp:155-168): the low four bits of the code.
__device__ __forceinline__ float decode_e2m1(uint32_t code) {
    const uint32_t exponent = (code >> 1) & 3u, mantissa = code & 1u;
    const float value = exponent == 0 ? 0.5f * static_cast<float>(mantissa) : ldexpf(1.0f + 0.5f * static_cast<float>(mantissa), static_cast<int>(exponent) - 1);
    return (code & 8u) ? -value : value;
}
// f32 -> FP4 E2M1 as the reference's search gives it (lib/Compiler/Numeric.cpp:396-425, 504-632): the nearest of the 16 codes, an even code
// taking a tie from an odd one, exact zero with its sign, |v| > 6 -> 0x7 | sign, NaN -> 0x7.
__device__ __forceinline__ uint32_t encode_e2m1_scalar(float v) {
    uint32_t best = 0;
    float best_difference = fabsf(__fsub_rn(v, decode_e2m1(0)));
    for (uint32_t candidate = 0; candidate < 16; ++candidate) {
        const float difference = fabsf(__fsub_rn(v, decode_e2m1(candidate)));
        if (difference < best_difference || (difference == best_difference && (candidate & 1u) == 0u && (best & 1u) != 0u)) {
            best = candidate;
            best_difference = difference;
        }
    }
    const bool negative = (__float_as_uint(v) & 0x80000000u) != 0u;
    const float absolute = fabsf(v);
    uint32_t result = best;
    if (absolute == 0.0f) result = negative ? 0x8u : 0x0u;
    if (absolute > 6.0f) result = 0x7u | (negative ? 0x8u : 0x0u);
    if (v != v) result = 0x7u;
    return result;
}
// Packed four-bit tensors: element offset e is nibble e % 2 of byte e / 2. A store keeps the byte's other nibble; neighbouring
// elements may belong to other threads, so it goes through a compare-and-swap on the aligned word that holds the byte.
__device__ __forceinline__ uint32_t load_nibble(const void* data, int64_t offset) {
    return (static_cast<const uint8_t*>(data)[offset >> 1] >> ((offset & 1) * 4)) & 0xfu;
}
__device__ __forceinline__ void store_nibble(void* data, int64_t offset, uint32_t code) {
    uint8_t* byte = static_cast<uint8_t*>(data) + (offset >> 1);
    uint32_t* word = reinterpret_cast<uint32_t*>(reinterpret_cast<uintptr_t>(byte) & ~static_cast<uintptr_t>(3));
    const uint32_t shift = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(byte) & 3u) * 8u + static_cast<uint32_t>(offset & 1) * 4u;
    uint32_t seen = *word, assumed;
    do {
        assumed = seen;
        seen = atomicCAS(word, assumed, (assumed & ~(0xfu << shift)) | ((code & 0xfu) << shift));
    } while (seen != assumed);
}

__device__ __forceinline__ float load_as_f32(const void* data, int dtype, int64_t offset) {
    switch (dtype) {
        case DFGPU_F32: return static_cast<const float*>(data)[offset];
        case DFGPU_F16: return __half2float(static_cast<const __half*>(data)[offset]);
        case DFGPU_BF16: return bf16_bits_to_f32(static_cast<const uint16_t*>(data)[offset]);
        case DFGPU_E4M3: return decode_e4m3(static_cast<const uint8_t*>(data)[offset]);
        case DFGPU_E8M0: return decode_e8m0(static_cast<const uint8_t*>(data)[offset]);
        case DFGPU_E5M2: return decode_e5m2(static_cast<const uint8_t*>(data)[offset]);
        case DFGPU_I32: return static_cast<float>(static_cast<const int32_t*>(data)[offset]);
        case DFGPU_FP4: return decode_e2m1(load_nibble(data, offset));
        case DFGPU_I4: { const int nibble = static_cast<int>(load_nibble(data, offset)); return static_cast<float>(nibble >= 8 ? nibble - 16 : nibble); }
        default: return 0.0f;
    }
}

__device__ __forceinline__ void store_from_f32(void* data, int dtype, int64_t offset, float value) {
    switch (dtype) {
        case DFGPU_F32: static_cast<float*>(data)[offset] = value; break;
        case DFGPU_F16: static_cast<__half*>(data)[offset] = __float2half_rn(value); break;
        case DFGPU_BF16: static_cast<uint16_t*>(data)[offset] = f32_to_bf16_bits(value); break;
        case DFGPU_E4M3: static_cast<uint8_t*>(data)[offset] = static_cast<uint8_t>(encode_e4m3_scalar(value)); break;
        case DFGPU_E5M2: static_cast<uint8_t*>(data)[offset] = static_cast<uint8_t>(encode_e5m2_scalar(value)); break;
        case DFGPU_FP4: store_nibble(data, offset, encode_e2m1_scalar(value)); break;
        default: break;
    }
}

// arith.maximumf / minimumf: NaN if either side is NaN (CUDA's fmaxf drops NaN), -0 below +0: one max.NaN / min.NaN.
__device__ __forceinline__ float maximum_nan(float a, float b) {
    float m;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(m) : "f"(a), "f"(b));
    return m;
}
__device__ __forceinline__ float minimum_nan(float a, float b) {
    float m;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(m) : "f"(a), "f"(b));
    return m;
}

// RELU_FWD with clips and lower slope:
//   x < lower ? lower + slope * (x - lower) : min(max(x, lower), upper), NaN propagating.
__device__ __forceinline__ float relu_forward(float x, float lower, float upper, float slope) {
    float clipped = minimum_nan(maximum_nan(x, lower), upper);
    float lower_branch = __fadd_rn(lower, __fmul_rn(slope, __fsub_rn(x, lower)));
    return x < lower ? lower_branch : clipped;
}

// Tensor view passed by value to the generic kernels.
struct View {
    int32_t dtype;
    int32_t rank;
    int64_t dim[DFGPU_MAX_RANK];
    int64_t stride[DFGPU_MAX_RANK];
};

inline View make_view(const dfgpu_tensor& t) {
    View v{};
    v.dtype = t.dtype;
    v.rank = t.rank;
    for (int i = 0; i < DFGPU_MAX_RANK; ++i) {
        v.dim[i] = i < t.rank ? t.dim[i] : 1;
        v.stride[i] = i < t.rank ? t.stride[i] : 0;
    }
    return v;
}

// The fused epilogue carried by value into contraction kernels.
struct Epilogue {
    int32_t count;
    int32_t op[DFGPU_MAX_EPILOGUE];
    int32_t operand[DFGPU_MAX_EPILOGUE];
    float lower[DFGPU_MAX_EPILOGUE];
    float upper[DFGPU_MAX_EPILOGUE];
    float slope[DFGPU_MAX_EPILOGUE];
};

inline Epilogue make_epilogue(int count, const dfgpu_epilogue_step* steps) {
    Epilogue e{};
    e.count = count;
    for (int i = 0; i < count && i < DFGPU_MAX_EPILOGUE; ++i) {
        e.op[i] = steps[i].op;
        e.operand[i] = steps[i].operand;
        e.lower[i] = steps[i].relu_lower;
        e.upper[i] = steps[i].relu_upper;
        e.slope[i] = steps[i].relu_slope;
    }
    return e;
}

int validate_epilogue(int count, const dfgpu_epilogue_step* steps, const dfgpu_tensor* extra,
                      void* const* extra_pointers, const dfgpu_tensor& out, const char* what);

// n / d for 0 <= n < 2^31 as a multiply and a shift (d >= 1): m = ceil(2^(31+L) / d) with L = ceil(log2 d).
struct FastDivisor {
    uint32_t divisor, multiplier, shift;
};

inline FastDivisor make_fast_divisor(uint32_t d) {
    if (d <= 1) return FastDivisor{1, 0, 0};
    uint32_t log = 0;
    while ((1ull << log) < d) ++log;
    const uint64_t power = 1ull << (31 + log);
    return FastDivisor{d, static_cast<uint32_t>((power + d - 1) / d), log - 1};
}

__device__ __forceinline__ uint32_t fast_divide(uint32_t n, const FastDivisor& d) {
    return d.divisor == 1 ? n : __umulhi(n, d.multiplier) >> d.shift;
}

}  // namespace dfgpu

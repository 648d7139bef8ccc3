// POINTWISE nodes that could not be fused into a contraction's epilogue.
// One thread per output element, trailing-axis NumPy broadcast, f32 math.
//
// Every mode of the reference's pointwise_result (lib/Compiler/FoundationalGraph.cpp:2581-2955) goes through
// pointwise_value below: the same expression, one separately rounded f32 operation per step, with CUDA's full-precision
// math functions (no fast-math intrinsics). Packed tensors of equal shape (f32, f16 or bf16) take the kernel of four values per
// load; anything else (broadcast, strides, mixed storage types, three inputs, GEN_INDEX) one element per thread, where
// ADD / MUL / SUB / RELU_FWD / IDENTITY keep a kernel with nothing else in it.
#include "common.cuh"

namespace dfgpu {
namespace {

__device__ __forceinline__ int64_t broadcast_offset(const View& t, int out_rank, const int64_t* index) {
    int shift = out_rank - t.rank;
    int64_t offset = 0;
    for (int i = 0; i < t.rank; ++i) offset += (t.dim[i] == 1 ? 0 : index[i + shift]) * t.stride[i];
    return offset;
}

struct PointwiseScalars {
    float relu_lower, relu_upper, relu_slope, elu_alpha, softplus_beta, swish_beta;
    int axis;
};

__host__ __device__ constexpr int input_count(int mode) {
    if (mode < 0 || mode >= DFGPU_PW_MODE_COUNT) return 0;
    if (mode == DFGPU_PW_BINARY_SELECT) return 3;
    switch (mode) {
        case DFGPU_PW_ADD: case DFGPU_PW_MUL: case DFGPU_PW_SUB: case DFGPU_PW_DIV: case DFGPU_PW_ADD_SQUARE:
        case DFGPU_PW_MIN: case DFGPU_PW_MAX: case DFGPU_PW_MOD: case DFGPU_PW_POW:
        case DFGPU_PW_LOGICAL_AND: case DFGPU_PW_LOGICAL_OR:
        case DFGPU_PW_CMP_EQ: case DFGPU_PW_CMP_NEQ: case DFGPU_PW_CMP_GT: case DFGPU_PW_CMP_GE: case DFGPU_PW_CMP_LT: case DFGPU_PW_CMP_LE:
        case DFGPU_PW_RELU_BWD: case DFGPU_PW_TANH_BWD: case DFGPU_PW_SIGMOID_BWD: case DFGPU_PW_ELU_BWD:
        case DFGPU_PW_SOFTPLUS_BWD: case DFGPU_PW_SWISH_BWD: case DFGPU_PW_GELU_BWD: case DFGPU_PW_GELU_APPROX_TANH_BWD:
            return 2;
        default: return 1;
    }
}

inline bool simple_mode(int mode) { return mode >= DFGPU_PW_ADD && mode <= DFGPU_PW_SUB; }

// 1 / (1 + exp(-v)) (FoundationalGraph.cpp:2569-2579)
__device__ __forceinline__ float sigmoid_value(float v) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v))); }

// x, y, z: IN_0, IN_1, IN_2 (0 where the mode has none). u: the activation's input (IN_1 of a _BWD mode, else IN_0).
__device__ __forceinline__ float pointwise_value(int mode, float x, float y, float z, const PointwiseScalars& s, int64_t position) {
    const float u = (mode >= DFGPU_PW_RELU_BWD && input_count(mode) == 2) ? y : x;
    switch (mode) {
        case DFGPU_PW_ADD: return __fadd_rn(x, y);
        case DFGPU_PW_MUL: return __fmul_rn(x, y);
        case DFGPU_PW_SUB: return __fsub_rn(x, y);
        case DFGPU_PW_DIV: return __fdiv_rn(x, y);
        case DFGPU_PW_ADD_SQUARE: return __fadd_rn(x, __fmul_rn(y, y));
        case DFGPU_PW_MIN: return minimum_nan(x, y);
        case DFGPU_PW_MAX: return maximum_nan(x, y);
        case DFGPU_PW_MOD: return fmodf(x, y);
        case DFGPU_PW_POW: return powf(x, y);
        case DFGPU_PW_SQRT: return __fsqrt_rn(x);
        case DFGPU_PW_RSQRT: return __fdiv_rn(1.0f, __fsqrt_rn(x));
        case DFGPU_PW_EXP: return expf(x);
        case DFGPU_PW_LOG: return logf(x);
        case DFGPU_PW_NEG: return -x;
        case DFGPU_PW_ABS: return fabsf(x);
        case DFGPU_PW_CEIL: return ceilf(x);
        case DFGPU_PW_FLOOR: return floorf(x);
        case DFGPU_PW_COS: return cosf(x);
        case DFGPU_PW_SIN: return sinf(x);
        case DFGPU_PW_TAN: return tanf(x);
        case DFGPU_PW_ERF: return erff(x);
        case DFGPU_PW_RECIPROCAL: return __fdiv_rn(1.0f, x);
        case DFGPU_PW_IDENTITY: return x;
        case DFGPU_PW_GEN_INDEX: return __ull2float_rn(static_cast<unsigned long long>(position));
        case DFGPU_PW_LOGICAL_NOT: return x == 0.0f ? 1.0f : 0.0f;
        case DFGPU_PW_LOGICAL_AND: return (x != 0.0f) && (y != 0.0f) ? 1.0f : 0.0f;
        case DFGPU_PW_LOGICAL_OR: return (x != 0.0f) || (y != 0.0f) ? 1.0f : 0.0f;
        case DFGPU_PW_BINARY_SELECT: return z != 0.0f ? y : x;
        case DFGPU_PW_CMP_EQ: return x == y ? 1.0f : 0.0f;
        case DFGPU_PW_CMP_NEQ: return x != y ? 1.0f : 0.0f;
        case DFGPU_PW_CMP_GT: return x > y ? 1.0f : 0.0f;
        case DFGPU_PW_CMP_GE: return x >= y ? 1.0f : 0.0f;
        case DFGPU_PW_CMP_LT: return x < y ? 1.0f : 0.0f;
        case DFGPU_PW_CMP_LE: return x <= y ? 1.0f : 0.0f;
        case DFGPU_PW_RELU_FWD: return relu_forward(x, s.relu_lower, s.relu_upper, s.relu_slope);
        case DFGPU_PW_RELU_BWD: return __fmul_rn(x, y < s.relu_lower ? s.relu_slope : (y > s.relu_upper ? 0.0f : 1.0f));
        case DFGPU_PW_TANH_FWD: return tanhf(u);
        case DFGPU_PW_TANH_BWD: { float t = tanhf(u); return __fmul_rn(x, __fsub_rn(1.0f, __fmul_rn(t, t))); }
        case DFGPU_PW_SIGMOID_FWD: return sigmoid_value(u);
        case DFGPU_PW_SIGMOID_BWD: { float v = sigmoid_value(u); return __fmul_rn(x, __fmul_rn(v, __fsub_rn(1.0f, v))); }
        case DFGPU_PW_ELU_FWD: { float e = expf(u); return u >= 0.0f ? u : __fmul_rn(s.elu_alpha, __fsub_rn(e, 1.0f)); }
        case DFGPU_PW_ELU_BWD: { float e = expf(u); return __fmul_rn(x, u >= 0.0f ? 1.0f : __fmul_rn(s.elu_alpha, e)); }
        case DFGPU_PW_SOFTPLUS_FWD: {
            float scaled = __fmul_rn(s.softplus_beta, u);
            float logarithm = logf(__fadd_rn(1.0f, expf(-fabsf(scaled))));
            return __fdiv_rn(__fadd_rn(maximum_nan(scaled, 0.0f), logarithm), s.softplus_beta);
        }
        case DFGPU_PW_SOFTPLUS_BWD: return __fmul_rn(x, sigmoid_value(__fmul_rn(s.softplus_beta, u)));
        case DFGPU_PW_SWISH_FWD: return __fmul_rn(u, sigmoid_value(__fmul_rn(s.swish_beta, u)));
        case DFGPU_PW_SWISH_BWD: {
            float scaled = __fmul_rn(s.swish_beta, u);
            float v = sigmoid_value(scaled);
            return __fmul_rn(x, __fadd_rn(v, __fmul_rn(scaled, __fmul_rn(v, __fsub_rn(1.0f, v)))));
        }
        case DFGPU_PW_GELU_FWD: case DFGPU_PW_GELU_BWD: {
            float cdf = __fmul_rn(0.5f, __fadd_rn(1.0f, erff(__fmul_rn(u, 0.7071067811865475f))));
            if (mode == DFGPU_PW_GELU_FWD) return __fmul_rn(u, cdf);
            float density = __fmul_rn(0.3989422804014327f, expf(__fmul_rn(-0.5f, __fmul_rn(u, u))));
            return __fmul_rn(x, __fadd_rn(cdf, __fmul_rn(u, density)));
        }
        case DFGPU_PW_GELU_APPROX_TANH_FWD: case DFGPU_PW_GELU_APPROX_TANH_BWD: {
            float square = __fmul_rn(u, u);
            float cubic = __fmul_rn(square, u);
            float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(u, __fmul_rn(0.044715f, cubic)));
            float t = tanhf(inner);
            float cdf = __fmul_rn(0.5f, __fadd_rn(1.0f, t));
            if (mode == DFGPU_PW_GELU_APPROX_TANH_FWD) return __fmul_rn(u, cdf);
            float inner_derivative = __fmul_rn(0.7978845608028654f, __fadd_rn(1.0f, __fmul_rn(0.134145f, square)));
            float tanh_derivative = __fsub_rn(1.0f, __fmul_rn(t, t));
            return __fmul_rn(x, __fadd_rn(cdf, __fmul_rn(0.5f, __fmul_rn(u, __fmul_rn(tanh_derivative, inner_derivative)))));
        }
        default: return x;
    }
}

// Any mode, any strides and storage types: one thread per output element.
__global__ void pointwise_general_kernel(const void* a, const void* b, const void* c, void* out, View av, View bv, View cv, View ov,
                                         int mode, PointwiseScalars s, int64_t total) {
    int64_t flat = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (flat >= total) return;
    int64_t index[DFGPU_MAX_RANK];
    int64_t out_offset = 0;
    for (int i = ov.rank - 1; i >= 0; --i) {
        index[i] = flat % ov.dim[i];
        flat /= ov.dim[i];
        out_offset += index[i] * ov.stride[i];
    }
    const int inputs = input_count(mode);
    float x = load_as_f32(a, av.dtype, broadcast_offset(av, ov.rank, index));
    float y = inputs >= 2 ? load_as_f32(b, bv.dtype, broadcast_offset(bv, ov.rank, index)) : 0.0f;
    float z = inputs >= 3 ? load_as_f32(c, cv.dtype, broadcast_offset(cv, ov.rank, index)) : 0.0f;
    int64_t position = mode == DFGPU_PW_GEN_INDEX ? index[s.axis] : 0;
    store_from_f32(out, ov.dtype, out_offset, pointwise_value(mode, x, y, z, s, position));
}

__global__ void pointwise_kernel(const void* a, const void* b, void* out, View av, View bv, View ov, int mode,
                                 float lower, float upper, float slope, int64_t total) {
    int64_t flat = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (flat >= total) return;
    int64_t index[DFGPU_MAX_RANK];
    int64_t out_offset = 0;
    for (int i = ov.rank - 1; i >= 0; --i) {
        index[i] = flat % ov.dim[i];
        flat /= ov.dim[i];
        out_offset += index[i] * ov.stride[i];
    }
    float x = load_as_f32(a, av.dtype, broadcast_offset(av, ov.rank, index));
    float y = 0.0f;
    if (mode == DFGPU_PW_ADD || mode == DFGPU_PW_MUL || mode == DFGPU_PW_SUB)
        y = load_as_f32(b, bv.dtype, broadcast_offset(bv, ov.rank, index));
    float result;
    switch (mode) {
        case DFGPU_PW_ADD: result = __fadd_rn(x, y); break;
        case DFGPU_PW_MUL: result = __fmul_rn(x, y); break;
        case DFGPU_PW_SUB: result = __fsub_rn(x, y); break;
        case DFGPU_PW_RELU_FWD: result = relu_forward(x, lower, upper, slope); break;
        default: result = x; break;
    }
    store_from_f32(out, ov.dtype, out_offset, result);
}

// All operands packed with identical dims: quads of four values. A quad is loaded as it is stored (16 bytes of f32, 8 of
// bf16) and widened only where it is used, so that the quads a thread has in flight cost a register per 4 bytes.
template <typename T> struct Quad;
template <> struct Quad<float> { using type = float4; };
template <> struct Quad<__nv_bfloat16> { using type = uint2; };
template <> struct Quad<__half> { using type = ushort4; };  // (a type of its own, so that widen() tells HALF from BFLOAT16)

template <typename T>
__device__ __forceinline__ typename Quad<T>::type load_quad(const void* p, int64_t i) {
    return __ldg(reinterpret_cast<const typename Quad<T>::type*>(static_cast<const T*>(p) + i));
}
__device__ __forceinline__ void widen(const float4& r, float (&v)[4]) { v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w; }
__device__ __forceinline__ void widen(const uint2& r, float (&v)[4]) {
    v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
    v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
}
__device__ __forceinline__ void widen(const ushort4& r, float (&v)[4]) {
    v[0] = __half2float(__ushort_as_half(r.x)); v[1] = __half2float(__ushort_as_half(r.y));
    v[2] = __half2float(__ushort_as_half(r.z)); v[3] = __half2float(__ushort_as_half(r.w));
}
template <typename T>
__device__ __forceinline__ void store4(void* p, int64_t i, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(void* p, int64_t i, const float (&v)[4]) {
    *reinterpret_cast<float4*>(static_cast<float*>(p) + i) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(void* p, int64_t i, const float (&v)[4]) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);  // the same rounding, two values per cvt
    *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p) + i) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

// Quads of four values a thread keeps in flight: its U quads lie one block-width apart, so that each of a warp's loads
// stays contiguous; every load is issued before the first value is used. 32 bytes per thread and operand: with 8 (bf16)
// or 16 (f32) the loads in flight of a full SM do not cover the latency of HBM.
template <>
__device__ __forceinline__ void store4<__half>(void* p, int64_t i, const float (&v)[4]) {
    __half2 lo = __floats2half2_rn(v[0], v[1]), hi = __floats2half2_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p) + i) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

template <typename T> struct QuadsInFlight;
template <> struct QuadsInFlight<float> { static constexpr int value = 2; };
template <> struct QuadsInFlight<__nv_bfloat16> { static constexpr int value = 4; };
template <> struct QuadsInFlight<__half> { static constexpr int value = 4; };

constexpr int kPackedThreads = 256;

template <typename T>
unsigned packed_grid(int64_t total) {
    const int64_t per_block = static_cast<int64_t>(kPackedThreads) * 4 * QuadsInFlight<T>::value;
    return static_cast<unsigned>((total + per_block - 1) / per_block);
}

// Every mode with one or two inputs (not GEN_INDEX, which needs the element's index). The mode is looked at once per
// thread: the switch leads into a body compiled for that mode alone. A switch per value made every mode cost ~50 us on
// 25.7 M values whatever its arithmetic, and even a five-way switch per value held bf16 RELU_FWD at 37 us (23 us here).
template <typename T, int MODE>
__device__ __forceinline__ void packed_body(const void* a, const void* b, void* out, const PointwiseScalars& s, int64_t total) {
    constexpr int U = QuadsInFlight<T>::value;
    constexpr bool binary = input_count(MODE) == 2;
    const int64_t first = (static_cast<int64_t>(blockIdx.x) * U * kPackedThreads + threadIdx.x) * 4;
    typename Quad<T>::type raw_x[U], raw_y[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t i = first + static_cast<int64_t>(u) * kPackedThreads * 4;
        if (i < total) {
            raw_x[u] = load_quad<T>(a, i);
            if (binary) raw_y[u] = load_quad<T>(b, i);
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
        const int64_t i = first + static_cast<int64_t>(u) * kPackedThreads * 4;
        if (i >= total) break;
        float x[4], y[4] = {0.0f, 0.0f, 0.0f, 0.0f}, r[4];
        widen(raw_x[u], x);
        if (binary) widen(raw_y[u], y);
#pragma unroll
        for (int j = 0; j < 4; ++j) r[j] = pointwise_value(MODE, x[j], y[j], 0.0f, s, 0);
        store4<T>(out, i, r);
    }
}

#define DFGPU_PW_EVERY_MODE(X)                                                                                              \
    X(0) X(1) X(2) X(3) X(4) X(5) X(6) X(7) X(8) X(9) X(10) X(11) X(12) X(13) X(14) X(15) X(16) X(17) X(18) X(19) X(20) X(21) \
    X(22) X(23) X(24) X(25) X(26) X(27) X(28) X(29) X(30) X(31) X(32) X(33) X(34) X(35) X(36) X(37) X(38) X(39) X(40) X(41)  \
    X(42) X(43) X(44) X(45) X(46) X(47) X(48) X(49)
static_assert(DFGPU_PW_MODE_COUNT == 50, "DFGPU_PW_EVERY_MODE lists every mode");

// One kernel for the modes with one input and one for those with two. 32 registers, a full SM of 2048 threads, cover
// the latency of HBM best (bf16 RELU_FWD: 84 % of the copy bandwidth against 76 % at 48 registers) except for two bf16
// inputs, where eight quads in flight per thread want 48 registers (92 % against 88 % when held to 32).
template <typename T, int INPUTS>
__global__ void __launch_bounds__(kPackedThreads, (sizeof(T) == 2 && INPUTS == 2) ? 5 : 2048 / kPackedThreads)
pointwise_general_packed_kernel(const void* a, const void* b, void* out, int mode, PointwiseScalars s, int64_t total) {
    switch (mode) {
#define DFGPU_PW_CASE(M) case M: if constexpr (input_count(M) == INPUTS) packed_body<T, M>(a, b, out, s, total); break;
        DFGPU_PW_EVERY_MODE(DFGPU_PW_CASE)
#undef DFGPU_PW_CASE
        default: break;
    }
}

template <typename T>
void launch_packed(int inputs, const void* a, const void* b, void* out, int mode, const PointwiseScalars& s, int64_t total, cudaStream_t stream) {
    if (inputs == 1) pointwise_general_packed_kernel<T, 1><<<packed_grid<T>(total), kPackedThreads, 0, stream>>>(a, b, out, mode, s, total);
    else pointwise_general_packed_kernel<T, 2><<<packed_grid<T>(total), kPackedThreads, 0, stream>>>(a, b, out, mode, s, total);
}

bool same_packed(const dfgpu_tensor& a, const dfgpu_tensor& b) {
    if (a.rank != b.rank) return false;
    for (int i = 0; i < a.rank; ++i)
        if (a.dim[i] != b.dim[i]) return false;
    return is_packed_row_major(a) && is_packed_row_major(b);
}

int validate(const dfgpu_pointwise_params& p, int& inputs) {
    inputs = input_count(p.mode);
    if (inputs == 0) return fail(kUnsupported, "POINTWISE: mode %d is not executable on this backend", p.mode);
    if (!valid_tensor(p.in0) || !valid_tensor(p.out) || (inputs >= 2 && !valid_tensor(p.in1)) || (inputs >= 3 && !valid_tensor(p.in2)))
        return fail(kInvalidShape, "POINTWISE: tensor rank or extent out of range");
    const dfgpu_tensor* operands[3] = {&p.in0, &p.in1, &p.in2};
    for (int n = 0; n < inputs; ++n) {
        const dfgpu_tensor& t = *operands[n];
        if (t.rank > p.out.rank) return fail(kInvalidShape, "POINTWISE: input rank exceeds output rank");
        int shift = p.out.rank - t.rank;
        for (int i = 0; i < t.rank; ++i)
            if (t.dim[i] != 1 && t.dim[i] != p.out.dim[i + shift])
                return fail(kInvalidShape, "POINTWISE: input does not broadcast onto the output");
        if (t.dtype != DFGPU_F32 && t.dtype != DFGPU_BF16 && t.dtype != DFGPU_F16)
            return fail(kUnsupported, "POINTWISE: unsupported input type");
    }
    if (p.out.dtype != DFGPU_F32 && p.out.dtype != DFGPU_BF16 && p.out.dtype != DFGPU_F16)
        return fail(kUnsupported, "POINTWISE: unsupported output type");
    if (p.mode == DFGPU_PW_GEN_INDEX && (p.axis < 0 || p.axis >= p.out.rank))
        return fail(kInvalidValue, "POINTWISE: GEN_INDEX needs an axis inside the output's rank");
    if ((p.mode == DFGPU_PW_SOFTPLUS_FWD || p.mode == DFGPU_PW_SOFTPLUS_BWD) && !(p.softplus_beta > 0.0f))
        return fail(kInvalidValue, "POINTWISE: softplus beta must be positive");
    if ((p.mode == DFGPU_PW_RELU_FWD || p.mode == DFGPU_PW_RELU_BWD) && p.relu_lower > p.relu_upper)
        return fail(kInvalidValue, "POINTWISE: ReLU lower clip exceeds upper clip");
    return kOk;
}

}  // namespace
}  // namespace dfgpu

using namespace dfgpu;

extern "C" int dfgpu_pointwise_input_count(int32_t mode) { return input_count(mode); }

extern "C" int dfgpu_query_pointwise(const dfgpu_pointwise_params* p, dfgpu_plan_info* info) {
    if (!p || !info) return fail(kInvalidArgument, "POINTWISE: null params");
    int inputs;
    int status = validate(*p, inputs);
    if (status) return status;
    info->kernel = 1;
    info->launches = 1;
    info->scratch_bytes = 0;
    return kOk;
}

extern "C" int dfgpu_pointwise(const dfgpu_pointwise_params* p, void* const* tensors, void* scratch, void* stream_handle) {
    (void)scratch;
    if (!p || !tensors) return fail(kInvalidArgument, "POINTWISE: null params");
    int inputs;
    int status = validate(*p, inputs);
    if (status) return status;
    const bool binary = inputs == 2;
    if (!tensors[0] || !tensors[2] || (inputs >= 2 && !tensors[1]) || (inputs >= 3 && !tensors[3]))
        return fail(kInvalidArgument, "POINTWISE: null tensor pointer");
    cudaStream_t stream = as_stream(stream_handle);
    int64_t total = element_count(p->out);
    auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    bool packed = same_packed(p->in0, p->out) && (!binary || same_packed(p->in1, p->out)) && total % 4 == 0 &&
                  aligned16(tensors[0]) && aligned16(tensors[2]) && (!binary || aligned16(tensors[1]));
    bool f32_all = p->in0.dtype == DFGPU_F32 && p->out.dtype == DFGPU_F32 && (!binary || p->in1.dtype == DFGPU_F32);
    bool bf16_all = p->in0.dtype == DFGPU_BF16 && p->out.dtype == DFGPU_BF16 && (!binary || p->in1.dtype == DFGPU_BF16);
    bool f16_all = p->in0.dtype == DFGPU_F16 && p->out.dtype == DFGPU_F16 && (!binary || p->in1.dtype == DFGPU_F16);
    PointwiseScalars s{p->relu_lower, p->relu_upper, p->relu_slope, p->elu_alpha, p->softplus_beta, p->swish_beta, p->axis};
    if (packed && (f32_all || bf16_all || f16_all) && inputs <= 2 && p->mode != DFGPU_PW_GEN_INDEX) {
        if (f32_all) launch_packed<float>(inputs, tensors[0], tensors[1], tensors[2], p->mode, s, total, stream);
        else if (f16_all) launch_packed<__half>(inputs, tensors[0], tensors[1], tensors[2], p->mode, s, total, stream);
        else launch_packed<__nv_bfloat16>(inputs, tensors[0], tensors[1], tensors[2], p->mode, s, total, stream);
    } else if (!simple_mode(p->mode)) {
        unsigned grid = static_cast<unsigned>((total + 255) / 256);
        pointwise_general_kernel<<<grid, 256, 0, stream>>>(tensors[0], tensors[1], inputs >= 3 ? tensors[3] : nullptr, tensors[2],
                                                           make_view(p->in0), inputs >= 2 ? make_view(p->in1) : make_view(p->in0),
                                                           inputs >= 3 ? make_view(p->in2) : make_view(p->in0), make_view(p->out),
                                                           p->mode, s, total);
    } else {
        unsigned grid = static_cast<unsigned>((total + 255) / 256);
        pointwise_kernel<<<grid, 256, 0, stream>>>(tensors[0], tensors[1], tensors[2], make_view(p->in0),
                                                   binary ? make_view(p->in1) : make_view(p->in0), make_view(p->out),
                                                   p->mode, p->relu_lower, p->relu_upper, p->relu_slope, total);
    }
    return check_launch("POINTWISE");
}

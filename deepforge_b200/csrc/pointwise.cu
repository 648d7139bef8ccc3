// POINTWISE nodes that could not be fused into a contraction's epilogue.
// One thread per output element, trailing-axis NumPy broadcast, f32 math.
#include "common.cuh"

namespace dfgpu {
namespace {

__device__ __forceinline__ int64_t broadcast_offset(const View& t, int out_rank, const int64_t* index) {
    int shift = out_rank - t.rank;
    int64_t offset = 0;
    for (int i = 0; i < t.rank; ++i) offset += (t.dim[i] == 1 ? 0 : index[i + shift]) * t.stride[i];
    return offset;
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

// All operands packed with identical dims: 4 elements per thread.
template <typename T>
__device__ __forceinline__ void load4(const void* p, int64_t i, float (&v)[4]);
template <>
__device__ __forceinline__ void load4<float>(const void* p, int64_t i, float (&v)[4]) {
    float4 r = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p) + i));
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const void* p, int64_t i, float (&v)[4]) {
    uint2 r = __ldg(reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p) + i));
    v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
    v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
}
template <typename T>
__device__ __forceinline__ void store4(void* p, int64_t i, const float (&v)[4]);
template <>
__device__ __forceinline__ void store4<float>(void* p, int64_t i, const float (&v)[4]) {
    *reinterpret_cast<float4*>(static_cast<float*>(p) + i) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(void* p, int64_t i, const float (&v)[4]) {
    uint32_t lo = f32_to_bf16_bits(v[0]) | (static_cast<uint32_t>(f32_to_bf16_bits(v[1])) << 16);
    uint32_t hi = f32_to_bf16_bits(v[2]) | (static_cast<uint32_t>(f32_to_bf16_bits(v[3])) << 16);
    *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p) + i) = make_uint2(lo, hi);
}

template <typename TA, typename TB, typename TO>
__global__ void pointwise_packed_kernel(const void* a, const void* b, void* out, int mode, float lower, float upper,
                                        float slope, int64_t total) {
    int64_t i = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (i >= total) return;
    float x[4], y[4] = {0.f, 0.f, 0.f, 0.f}, r[4];
    load4<TA>(a, i, x);
    if (mode == DFGPU_PW_ADD || mode == DFGPU_PW_MUL || mode == DFGPU_PW_SUB) load4<TB>(b, i, y);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        switch (mode) {
            case DFGPU_PW_ADD: r[j] = __fadd_rn(x[j], y[j]); break;
            case DFGPU_PW_MUL: r[j] = __fmul_rn(x[j], y[j]); break;
            case DFGPU_PW_SUB: r[j] = __fsub_rn(x[j], y[j]); break;
            case DFGPU_PW_RELU_FWD: r[j] = relu_forward(x[j], lower, upper, slope); break;
            default: r[j] = x[j]; break;
        }
    }
    store4<TO>(out, i, r);
}

bool same_packed(const dfgpu_tensor& a, const dfgpu_tensor& b) {
    if (a.rank != b.rank) return false;
    for (int i = 0; i < a.rank; ++i)
        if (a.dim[i] != b.dim[i]) return false;
    return is_packed_row_major(a) && is_packed_row_major(b);
}

int validate(const dfgpu_pointwise_params& p, bool& binary) {
    binary = p.mode == DFGPU_PW_ADD || p.mode == DFGPU_PW_MUL || p.mode == DFGPU_PW_SUB;
    if (p.mode < DFGPU_PW_ADD || p.mode > DFGPU_PW_SUB) return fail(kUnsupported, "POINTWISE: mode %d is not executable on this backend", p.mode);
    if (!valid_tensor(p.in0) || !valid_tensor(p.out) || (binary && !valid_tensor(p.in1)))
        return fail(kInvalidShape, "POINTWISE: tensor rank or extent out of range");
    const dfgpu_tensor* inputs[2] = {&p.in0, &p.in1};
    for (int n = 0; n < (binary ? 2 : 1); ++n) {
        const dfgpu_tensor& t = *inputs[n];
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
    return kOk;
}

}  // namespace
}  // namespace dfgpu

using namespace dfgpu;

extern "C" int dfgpu_query_pointwise(const dfgpu_pointwise_params* p, dfgpu_plan_info* info) {
    if (!p || !info) return fail(kInvalidArgument, "POINTWISE: null params");
    bool binary;
    int status = validate(*p, binary);
    if (status) return status;
    info->kernel = 1;
    info->launches = 1;
    info->scratch_bytes = 0;
    return kOk;
}

extern "C" int dfgpu_pointwise(const dfgpu_pointwise_params* p, void* const* tensors, void* scratch, void* stream_handle) {
    (void)scratch;
    if (!p || !tensors) return fail(kInvalidArgument, "POINTWISE: null params");
    bool binary;
    int status = validate(*p, binary);
    if (status) return status;
    if (!tensors[0] || !tensors[2] || (binary && !tensors[1])) return fail(kInvalidArgument, "POINTWISE: null tensor pointer");
    cudaStream_t stream = as_stream(stream_handle);
    int64_t total = element_count(p->out);
    auto aligned16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    bool packed = same_packed(p->in0, p->out) && (!binary || same_packed(p->in1, p->out)) && total % 4 == 0 &&
                  aligned16(tensors[0]) && aligned16(tensors[2]) && (!binary || aligned16(tensors[1]));
    bool f32_all = p->in0.dtype == DFGPU_F32 && p->out.dtype == DFGPU_F32 && (!binary || p->in1.dtype == DFGPU_F32);
    bool bf16_all = p->in0.dtype == DFGPU_BF16 && p->out.dtype == DFGPU_BF16 && (!binary || p->in1.dtype == DFGPU_BF16);
    if (packed && (f32_all || bf16_all)) {
        unsigned grid = static_cast<unsigned>((total / 4 + 255) / 256);
        if (f32_all)
            pointwise_packed_kernel<float, float, float><<<grid, 256, 0, stream>>>(tensors[0], tensors[1], tensors[2], p->mode, p->relu_lower, p->relu_upper, p->relu_slope, total);
        else
            pointwise_packed_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, stream>>>(tensors[0], tensors[1], tensors[2], p->mode, p->relu_lower, p->relu_upper, p->relu_slope, total);
    } else {
        unsigned grid = static_cast<unsigned>((total + 255) / 256);
        pointwise_kernel<<<grid, 256, 0, stream>>>(tensors[0], tensors[1], tensors[2], make_view(p->in0),
                                                   binary ? make_view(p->in1) : make_view(p->in0), make_view(p->out),
                                                   p->mode, p->relu_lower, p->relu_upper, p->relu_slope, total);
    }
    return check_launch("POINTWISE");
}

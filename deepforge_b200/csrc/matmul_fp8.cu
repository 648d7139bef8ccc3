// MATMUL_FP8: C = store((sum_k A*B) * Descale_A * Descale_B * Scale_C), Amax_C = max |value before Scale_C|.
//
// Follows the reference's emit_matmul_fp8 (lib/Compiler/SpecializedGraph.cpp:982-1090): the sum runs in f32 from
// 0.0 in k order, the two descales are separate multiplications, Amax_C folds maximumf (NaN-propagating) from 0.0
// over |value|, and C takes value * Scale_C through store_from_f32. The kernel here is the general one (any rank,
// batch broadcast over extent-1 axes, any strides; one thread per output element, so the k order is the
// reference's); large aligned problems go to the tcgen05 kernel in umma_mxf8.cu, whose f32 additions run in the
// tensor core's order. Amax_C is cleared by a memset in the stream and folded with an atomic maximum on the bits of
// the non-negative f32 (NaN, made canonical, is the largest pattern, so it sticks like maximumf's).
#include "common.cuh"
#include "umma.cuh"

namespace dfgpu {
namespace {

struct Fp8Args {
    View a, b, c;
    int rank;
    int64_t m, n, k;
    const float* descale_a;
    const float* descale_b;
    const float* scale_c;
    unsigned int* amax_bits;
};

__global__ void __launch_bounds__(256)
matmul_fp8_scalar_kernel(const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ c, Fp8Args g) {
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int64_t im = static_cast<int64_t>(blockIdx.y) * 16 + ty;
    const int64_t in = static_cast<int64_t>(blockIdx.x) * 16 + tx;
    int64_t batch = blockIdx.z;
    int64_t ao = 0, bo = 0, co = 0;
    for (int i = g.rank - 3; i >= 0; --i) {
        const int64_t position = batch % g.c.dim[i];
        batch /= g.c.dim[i];
        ao += (g.a.dim[i] == 1 ? 0 : position) * g.a.stride[i];
        bo += (g.b.dim[i] == 1 ? 0 : position) * g.b.stride[i];
        co += position * g.c.stride[i];
    }
    const int r = g.rank;
    float magnitude = 0.0f;
    if (im < g.m && in < g.n) {
        float sum = 0.0f;
        const int64_t a_row = ao + im * g.a.stride[r - 2], b_col = bo + in * g.b.stride[r - 1];
        for (int64_t ik = 0; ik < g.k; ++ik) {
            const float av = load_as_f32(a, g.a.dtype, a_row + ik * g.a.stride[r - 1]);
            const float bv = load_as_f32(b, g.b.dtype, b_col + ik * g.b.stride[r - 2]);
            sum = __fadd_rn(sum, __fmul_rn(av, bv));
        }
        float value = __fmul_rn(sum, *g.descale_a);
        value = __fmul_rn(value, *g.descale_b);
        magnitude = fabsf(value);
        store_from_f32(c, g.c.dtype, co + im * g.c.stride[r - 2] + in * g.c.stride[r - 1], __fmul_rn(value, *g.scale_c));
    }
    // fold over the block, then one atomic per warp
    unsigned int bits = magnitude != magnitude ? 0x7fc00000u : __float_as_uint(magnitude);
    bits = __reduce_max_sync(0xffffffffu, bits);
    if ((threadIdx.x & 31) == 0 && bits != 0u) atomicMax(g.amax_bits, bits);
}

int build_args(const dfgpu_matmul_fp8_params& p, void* const* tensors, Fp8Args& g) {
    const int rank = p.c.rank;
    if (rank < 2 || rank > DFGPU_MAX_RANK || p.a.rank != rank || p.b.rank != rank)
        return fail(kInvalidShape, "MATMUL_FP8: A, B, and C must have equal rank of at least two");
    if ((p.a.dtype != DFGPU_E4M3 && p.a.dtype != DFGPU_E5M2) || (p.b.dtype != DFGPU_E4M3 && p.b.dtype != DFGPU_E5M2))
        return fail(kUnsupported, "MATMUL_FP8: A and B must be FP8_E4M3 or FP8_E5M2");
    if (p.c.dtype != DFGPU_F32 && p.c.dtype != DFGPU_F16 && p.c.dtype != DFGPU_BF16 && p.c.dtype != DFGPU_E4M3 && p.c.dtype != DFGPU_E5M2)
        return fail(kUnsupported, "MATMUL_FP8: C must be FLOAT, HALF, BFLOAT16, FP8_E4M3 or FP8_E5M2");
    const int64_t m = p.c.dim[rank - 2], n = p.c.dim[rank - 1], k = p.a.dim[rank - 1];
    if (p.b.dim[rank - 2] != k || p.a.dim[rank - 2] != m || p.b.dim[rank - 1] != n)
        return fail(kInvalidShape, "MATMUL_FP8: matrix M, N, and K dimensions are inconsistent");
    for (int i = 0; i < rank; ++i)
        if (p.a.dim[i] <= 0 || p.b.dim[i] <= 0 || p.c.dim[i] <= 0) return fail(kInvalidShape, "MATMUL_FP8: extents must be positive");
    for (int i = 0; i < rank - 2; ++i)
        if ((p.a.dim[i] != 1 && p.a.dim[i] != p.c.dim[i]) || (p.b.dim[i] != 1 && p.b.dim[i] != p.c.dim[i]))
            return fail(kInvalidShape, "MATMUL_FP8: batch dimensions are not broadcast-compatible");
    g.a = make_view(p.a);
    g.b = make_view(p.b);
    g.c = make_view(p.c);
    g.rank = rank;
    g.m = m;
    g.n = n;
    g.k = k;
    g.amax_bits = tensors ? static_cast<unsigned int*>(tensors[3]) : nullptr;
    g.descale_a = tensors ? static_cast<const float*>(tensors[4]) : nullptr;
    g.descale_b = tensors ? static_cast<const float*>(tensors[5]) : nullptr;
    g.scale_c = tensors ? static_cast<const float*>(tensors[6]) : nullptr;
    return kOk;
}

int choose_kernel(const dfgpu_matmul_fp8_params& p, int& kernel) {
    const int automatic = matmul_fp8_umma_supported(p) ? DFGPU_MATMUL_FP8_UMMA : DFGPU_MATMUL_FP8_SCALAR;
    kernel = p.kernel == DFGPU_MATMUL_FP8_AUTO ? automatic : p.kernel;
    if (kernel != DFGPU_MATMUL_FP8_SCALAR && kernel != DFGPU_MATMUL_FP8_UMMA) return fail(kInvalidArgument, "MATMUL_FP8: unknown kernel id %d", kernel);
    if (kernel == DFGPU_MATMUL_FP8_UMMA && !matmul_fp8_umma_supported(p))
        return fail(kUnsupported, "MATMUL_FP8: the tcgen05 kernel does not cover this shape, layout or type");
    return kOk;
}

}  // namespace
}  // namespace dfgpu

using namespace dfgpu;

extern "C" int dfgpu_query_matmul_fp8(const dfgpu_matmul_fp8_params* p, dfgpu_plan_info* info) {
    if (!p || !info) return fail(kInvalidArgument, "MATMUL_FP8: null params");
    Fp8Args g;
    int status = build_args(*p, nullptr, g);
    if (status) return status;
    int kernel;
    status = choose_kernel(*p, kernel);
    if (status) return status;
    info->kernel = kernel;
    info->launches = 1;  // plus the 4-byte memset that clears Amax_C
    info->scratch_bytes = 0;
    return kOk;
}

extern "C" int dfgpu_matmul_fp8(const dfgpu_matmul_fp8_params* p, void* const* tensors, void* scratch, void* stream_handle) {
    (void)scratch;
    if (!p || !tensors) return fail(kInvalidArgument, "MATMUL_FP8: null params");
    for (int i = 0; i < 7; ++i)
        if (!tensors[i]) return fail(kInvalidArgument, "MATMUL_FP8: null tensor pointer (A, B, C, Amax_C, Descale_A, Descale_B, Scale_C are all required)");
    for (int i = 3; i < 7; ++i)
        if ((reinterpret_cast<uintptr_t>(tensors[i]) & 3u) != 0) return fail(kInvalidArgument, "MATMUL_FP8: the FLOAT scalars must be 4-byte aligned");
    Fp8Args g;
    int status = build_args(*p, tensors, g);
    if (status) return status;
    int kernel;
    status = choose_kernel(*p, kernel);
    if (status) return status;
    cudaStream_t stream = as_stream(stream_handle);
    cudaError_t error = cudaMemsetAsync(tensors[3], 0, sizeof(float), stream);
    if (error != cudaSuccess) return fail(kExecutionFailed, "MATMUL_FP8: clearing Amax_C failed: %s", cudaGetErrorString(error));
    if (kernel == DFGPU_MATMUL_FP8_UMMA) return launch_matmul_fp8_umma(*p, tensors, stream);
    int64_t batches = 1;
    for (int i = 0; i < g.rank - 2; ++i) batches *= p->c.dim[i];
    if (batches > 65535 || (g.m + 15) / 16 > 65535) return fail(kUnsupported, "MATMUL_FP8: more than 65535 batch matrices or row blocks");
    dim3 grid(static_cast<unsigned>((g.n + 15) / 16), static_cast<unsigned>((g.m + 15) / 16), static_cast<unsigned>(batches));
    matmul_fp8_scalar_kernel<<<grid, 256, 0, stream>>>(tensors[0], tensors[1], tensors[2], g);
    return check_launch("MATMUL_FP8");
}

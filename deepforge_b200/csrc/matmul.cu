// MATMUL on CUDA cores: batched, broadcast over leading axes, arbitrary strides,
// f32 accumulation. With block scales attached, A and/or B are E4M3 codes that are
// decoded and multiplied by their E8M0 block scale while the tile is staged, which
// absorbs the BLOCK_SCALE_DEQUANTIZE nodes in front of the MATMUL. The tcgen05
// kernels in umma_gemm.cu take over for the large bf16 / MXFP8 cases.
#include "common.cuh"
#include "umma.cuh"

namespace dfgpu {
namespace {

struct MatmulArgs {
    View a, b, c;
    View a_scale, b_scale;
    const uint8_t* a_scale_data;
    const uint8_t* b_scale_data;
    int64_t a_block[2], b_block[2];
    View extra[2];
    const void* extra_data[2];
    Epilogue epilogue;
    int rank;
    int64_t m, n, k;
};

__device__ __forceinline__ void batch_offsets(const MatmulArgs& g, int64_t batch, int64_t& ao, int64_t& bo, int64_t& co,
                                              int64_t& aso, int64_t& bso, int64_t* batch_index) {
    ao = bo = co = aso = bso = 0;
    for (int i = g.rank - 3; i >= 0; --i) {
        int64_t position = batch % g.c.dim[i];
        batch /= g.c.dim[i];
        batch_index[i] = position;
        ao += (g.a.dim[i] == 1 ? 0 : position) * g.a.stride[i];
        bo += (g.b.dim[i] == 1 ? 0 : position) * g.b.stride[i];
        co += position * g.c.stride[i];
        if (g.a_scale.rank) aso += (g.a_scale.dim[i] == 1 ? 0 : position) * g.a_scale.stride[i];
        if (g.b_scale.rank) bso += (g.b_scale.dim[i] == 1 ? 0 : position) * g.b_scale.stride[i];
    }
}

__global__ void __launch_bounds__(256)
matmul_ffma_kernel(const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ c, MatmulArgs g, const int* __restrict__ run_if_any,
                   int flag_count) {
    constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;
    __shared__ float as[BK][BM + 4];
    __shared__ float bs[BK][BN + 4];
    const int tid = threadIdx.x;
    if (run_if_any) {
        // second pass behind the split-operand tensor-core form: it only has work when one of the flags is set
        int any = 0;
        for (int i = tid; i < flag_count; i += 256) any |= run_if_any[i];
        if (!__syncthreads_or(any)) return;
    }
    const int64_t m0 = static_cast<int64_t>(blockIdx.x) * BM;
    const int64_t n0 = static_cast<int64_t>(blockIdx.y) * BN;
    int64_t batch_index[DFGPU_MAX_RANK];
    int64_t ao, bo, co, aso, bso;
    batch_offsets(g, blockIdx.z, ao, bo, co, aso, bso, batch_index);
    const int r = g.rank;
    // A is read k-fastest when its k stride is 1, else m-fastest; same idea for B.
    const bool a_k_fast = g.a.stride[r - 1] == 1;
    const bool b_n_fast = g.b.stride[r - 1] == 1;
    const int ty = tid / 16, tx = tid % 16;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int64_t k0 = 0; k0 < g.k; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int e = tid + i * 256;
            int mm = a_k_fast ? e / BK : e % BM;
            int kk = a_k_fast ? e % BK : e / BM;
            int64_t m = m0 + mm, k = k0 + kk;
            float value = 0.0f;
            if (m < g.m && k < g.k) {
                value = load_as_f32(a, g.a.dtype, ao + m * g.a.stride[r - 2] + k * g.a.stride[r - 1]);
                if (g.a_scale.rank)
                    value = __fmul_rn(value, decode_e8m0(g.a_scale_data[aso + (m / g.a_block[0]) * g.a_scale.stride[r - 2] +
                                                                           (k / g.a_block[1]) * g.a_scale.stride[r - 1]]));
            }
            as[kk][mm] = value;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int e = tid + i * 256;
            int nn = b_n_fast ? e % BN : e / BK;
            int kk = b_n_fast ? e / BN : e % BK;
            int64_t n = n0 + nn, k = k0 + kk;
            float value = 0.0f;
            if (n < g.n && k < g.k) {
                value = load_as_f32(b, g.b.dtype, bo + k * g.b.stride[r - 2] + n * g.b.stride[r - 1]);
                if (g.b_scale.rank)
                    value = __fmul_rn(value, decode_e8m0(g.b_scale_data[bso + (k / g.b_block[0]) * g.b_scale.stride[r - 2] +
                                                                           (n / g.b_block[1]) * g.b_scale.stride[r - 1]]));
            }
            bs[kk][nn] = value;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[TM], bv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = as[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) bv[j] = bs[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        int64_t m = m0 + ty * TM + i;
        if (m >= g.m) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            int64_t n = n0 + tx * TN + j;
            if (n >= g.n) continue;
            float value = acc[i][j];
            for (int step = 0; step < g.epilogue.count; ++step) {
                if (g.epilogue.op[step] == DFGPU_EPI_ADD) {
                    const View& t = g.extra[g.epilogue.operand[step]];
                    int shift = r - t.rank;
                    int64_t offset = 0;
                    for (int axis = 0; axis < t.rank; ++axis) {
                        int out_axis = axis + shift;
                        int64_t position = out_axis == r - 1 ? n : (out_axis == r - 2 ? m : batch_index[out_axis]);
                        offset += (t.dim[axis] == 1 ? 0 : position) * t.stride[axis];
                    }
                    value = __fadd_rn(value, load_as_f32(g.extra_data[g.epilogue.operand[step]], t.dtype, offset));
                } else {
                    value = relu_forward(value, g.epilogue.lower[step], g.epilogue.upper[step], g.epilogue.slope[step]);
                }
            }
            store_from_f32(c, g.c.dtype, co + m * g.c.stride[r - 2] + n * g.c.stride[r - 1], value);
        }
    }
}

int build_args(const dfgpu_matmul_params& p, void* const* tensors, MatmulArgs& g) {
    if (!valid_tensor(p.a) || !valid_tensor(p.b) || !valid_tensor(p.c))
        return fail(kInvalidShape, "MATMUL: tensor rank or extent out of range");
    int rank = p.c.rank;
    if (rank < 2 || p.a.rank != rank || p.b.rank != rank) return fail(kInvalidShape, "MATMUL: A, B and C must have equal rank >= 2");
    int64_t m = p.c.dim[rank - 2], n = p.c.dim[rank - 1], k = p.a.dim[rank - 1];
    if (p.a.dim[rank - 2] != m || p.b.dim[rank - 1] != n || p.b.dim[rank - 2] != k)
        return fail(kInvalidShape, "MATMUL: M/N/K extents are inconsistent");
    for (int i = 0; i < rank - 2; ++i) {
        if ((p.a.dim[i] != 1 && p.a.dim[i] != p.c.dim[i]) || (p.b.dim[i] != 1 && p.b.dim[i] != p.c.dim[i]))
            return fail(kInvalidShape, "MATMUL: batch axes do not broadcast");
    }
    auto float_type = [](int t) { return t == DFGPU_F32 || t == DFGPU_F16 || t == DFGPU_BF16; };
    const dfgpu_tensor* operands[2] = {&p.a, &p.b};
    const dfgpu_tensor* scales[2] = {&p.a_scale, &p.b_scale};
    const int64_t* blocks[2] = {p.a_block, p.b_block};
    for (int which = 0; which < 2; ++which) {
        const dfgpu_tensor& t = *operands[which];
        const dfgpu_tensor& s = *scales[which];
        if (s.rank == 0) {
            if (!float_type(t.dtype)) return fail(kUnsupported, "MATMUL: operand must be FLOAT, HALF or BFLOAT16 unless block scales are attached");
            continue;
        }
        if (t.dtype != DFGPU_E4M3 || s.dtype != DFGPU_E8M0 || s.reorder != DFGPU_REORDER_NONE)
            return fail(kUnsupported, "MATMUL: fused dequantize takes FP8_E4M3 codes with unreordered FP8_E8M0 scales");
        if (s.rank != rank || blocks[which][0] <= 0 || blocks[which][1] <= 0)
            return fail(kInvalidShape, "MATMUL: block scale descriptor is inconsistent");
        for (int axis = rank - 2; axis < rank; ++axis) {
            int64_t block = blocks[which][axis - (rank - 2)];
            if (s.dim[axis] < (t.dim[axis] + block - 1) / block) return fail(kInvalidShape, "MATMUL: block scale tensor smaller than the block grid");
        }
    }
    if (!float_type(p.c.dtype)) return fail(kUnsupported, "MATMUL: C must be FLOAT, HALF or BFLOAT16");
    int status = validate_epilogue(p.epilogue_count, p.epilogue, p.extra, tensors ? tensors + 5 : nullptr, p.c, "MATMUL");
    if (status) return status;
    g.a = make_view(p.a);
    g.b = make_view(p.b);
    g.c = make_view(p.c);
    g.a_scale = make_view(p.a_scale);
    g.b_scale = make_view(p.b_scale);
    g.a_scale.rank = p.a_scale.rank;
    g.b_scale.rank = p.b_scale.rank;
    g.a_scale_data = tensors ? static_cast<const uint8_t*>(tensors[3]) : nullptr;
    g.b_scale_data = tensors ? static_cast<const uint8_t*>(tensors[4]) : nullptr;
    for (int i = 0; i < 2; ++i) {
        g.a_block[i] = p.a_block[i] > 0 ? p.a_block[i] : 1;
        g.b_block[i] = p.b_block[i] > 0 ? p.b_block[i] : 1;
        g.extra[i] = make_view(p.extra[i]);
        g.extra_data[i] = tensors ? tensors[5 + i] : nullptr;
    }
    g.epilogue = make_epilogue(p.epilogue_count, p.epilogue);
    g.rank = rank;
    g.m = m;
    g.n = n;
    g.k = k;
    return kOk;
}

// ---- f32 matmul on the bf16 tensor cores (split_f32.cu) ----------------------------------------------------
struct SplitMatmul {
    dfgpu_matmul_params bf16;  // the bf16 matmul over 6K
    SplitOperand a, b;         // (pointers filled in at launch)
    int64_t as_offset, bs_offset, flags_offset, scratch_bytes;
    int flag_count;
};

// Takes unbatched f32 A [M, K] with K contiguous, f32 B with N or K contiguous and f32 C, K a multiple of 32 and the
// shape limits of the bf16 tcgen05 matmul on the 6K-deep copies.
bool f32_split_matmul(const dfgpu_matmul_params& p, SplitMatmul& form) {
    if (p.a.dtype != DFGPU_F32 || p.b.dtype != DFGPU_F32 || p.c.dtype != DFGPU_F32 || p.a_scale.rank || p.b_scale.rank) return false;
    const int rank = p.c.rank;
    if (rank < 2 || p.a.rank != rank || p.b.rank != rank) return false;
    for (int i = 0; i < rank - 2; ++i)
        if (p.c.dim[i] != 1 || p.a.dim[i] != 1 || p.b.dim[i] != 1) return false;
    const int64_t M = p.c.dim[rank - 2], N = p.c.dim[rank - 1], K = p.a.dim[rank - 1];
    if (K % 32 != 0 || N % 4 != 0 || M * K >= (1ll << 29) || K * N >= (1ll << 29)) return false;
    if (p.a.stride[rank - 1] != 1 || p.a.stride[rank - 2] % 4 != 0 || p.a.stride[rank - 2] < K) return false;
    const bool b_n_major = p.b.stride[rank - 1] == 1 && p.b.stride[rank - 2] % 4 == 0 && p.b.stride[rank - 2] >= N;
    const bool b_k_major = !b_n_major && p.b.stride[rank - 2] == 1 && p.b.stride[rank - 1] % 4 == 0 && p.b.stride[rank - 1] >= K;
    if (!b_n_major && !b_k_major) return false;
    form.bf16 = p;
    form.bf16.kernel = DFGPU_MATMUL_UMMA_BF16;
    dfgpu_tensor& a = form.bf16.a;
    dfgpu_tensor& b = form.bf16.b;
    a.dtype = b.dtype = DFGPU_BF16;
    a.dim[rank - 1] = kSplitPieces * K;
    a.stride[rank - 2] = kSplitPieces * K;
    b.dim[rank - 2] = kSplitPieces * K;
    if (b_n_major) {
        b.stride[rank - 2] = N;  // [6K, N], N contiguous
        b.stride[rank - 1] = 1;
    } else {
        b.stride[rank - 2] = 1;  // [N, 6K] seen as [6K, N] with K contiguous
        b.stride[rank - 1] = kSplitPieces * K;
    }
    if (!matmul_umma_supported(form.bf16, DFGPU_MATMUL_UMMA_BF16)) return false;
    form.a = SplitOperand{nullptr, nullptr, M * K / 4, K / 4, p.a.stride[rank - 2], kSplitPieces * K, K};
    form.b = b_n_major ? SplitOperand{nullptr, nullptr, K * N / 4, N / 4, p.b.stride[rank - 2], N, K * N}
                       : SplitOperand{nullptr, nullptr, N * K / 4, K / 4, p.b.stride[rank - 1], kSplitPieces * K, K};
    auto round_up = [](int64_t v) { return (v + 255) / 256 * 256; };
    form.flag_count = split_flag_count(form.a, form.b);
    form.as_offset = 0;
    form.bs_offset = round_up(M * K * kSplitPieces * 2);
    form.flags_offset = form.bs_offset + round_up(K * N * kSplitPieces * 2);
    form.scratch_bytes = form.flags_offset + round_up(static_cast<int64_t>(form.flag_count) * 4);
    return true;
}

int choose_kernel(const dfgpu_matmul_params& p, int& kernel) {
    int automatic = DFGPU_MATMUL_FFMA;
    SplitMatmul split;
    const bool split_ok = f32_split_matmul(p, split);
    if (matmul_umma_supported(p, DFGPU_MATMUL_UMMA_MXF8)) automatic = DFGPU_MATMUL_UMMA_MXF8;
    else if (matmul_umma_supported(p, DFGPU_MATMUL_UMMA_BF16)) automatic = DFGPU_MATMUL_UMMA_BF16;
    else {
        const int64_t macs = p.c.dim[p.c.rank - 2] * p.c.dim[p.c.rank - 1] * p.a.dim[p.a.rank - 1];
        if (split_ok && macs >= kSplitFormMinMacs) automatic = DFGPU_MATMUL_UMMA_F32X3;  // (three launches: big products only)
        // (one launch beats three where the output tiles fit one wave or all columns fit one tile)
        const int64_t row_tiles = (p.c.dim[p.c.rank - 2] + 127) / 128, column_tiles = (p.c.dim[p.c.rank - 1] + 63) / 64;
        const bool one_launch_pays = automatic != DFGPU_MATMUL_UMMA_F32X3 || row_tiles * column_tiles <= 148 || column_tiles == 1;
        if (one_launch_pays && p.a.dim[p.a.rank - 1] >= kClusterFormMinDepth && matmul_f32_cluster_supported(p)) automatic = DFGPU_MATMUL_UMMA_F32X3_CLUSTER;
    }
    kernel = p.kernel == DFGPU_MATMUL_AUTO ? automatic : p.kernel;
    if (kernel < DFGPU_MATMUL_FFMA || kernel > DFGPU_MATMUL_UMMA_F32X3_CLUSTER) return fail(kInvalidArgument, "MATMUL: unknown kernel id %d", kernel);
    if (kernel == DFGPU_MATMUL_UMMA_F32X3_CLUSTER) {
        if (!matmul_f32_cluster_supported(p))
            return fail(kUnsupported, "MATMUL: the one-launch tcgen05 form needs FLOAT, HALF or BFLOAT16 A, B and C and at most one batch axis");
        return kOk;
    }
    if (kernel == DFGPU_MATMUL_UMMA_F32X3) {
        if (!split_ok) return fail(kUnsupported, "MATMUL: the split-operand tcgen05 form needs unbatched f32 A (K contiguous), B and C, K a multiple of 32, N of 64");
        return kOk;
    }
    if (kernel != DFGPU_MATMUL_FFMA && !matmul_umma_supported(p, kernel))
        return fail(kUnsupported, "MATMUL: the requested tcgen05 kernel does not cover this shape, layout or type");
    return kOk;
}

}  // namespace
}  // namespace dfgpu

using namespace dfgpu;

extern "C" int dfgpu_query_matmul(const dfgpu_matmul_params* p, dfgpu_plan_info* info) {
    if (!p || !info) return fail(kInvalidArgument, "MATMUL: null params");
    MatmulArgs g;
    dfgpu_matmul_params copy = *p;
    copy.epilogue_count = 0;
    int status = build_args(copy, nullptr, g);
    if (status) return status;
    int kernel;
    status = choose_kernel(*p, kernel);
    if (status) return status;
    info->kernel = kernel;
    info->launches = 1;
    info->scratch_bytes = 0;
    if (kernel == DFGPU_MATMUL_UMMA_F32X3) {
        SplitMatmul split;
        f32_split_matmul(*p, split);
        info->launches = 3;
        info->scratch_bytes = split.scratch_bytes;
    }
    return kOk;
}

extern "C" int dfgpu_matmul(const dfgpu_matmul_params* p, void* const* tensors, void* scratch, void* stream_handle) {
    if (!p || !tensors) return fail(kInvalidArgument, "MATMUL: null params");
    if (!tensors[0] || !tensors[1] || !tensors[2]) return fail(kInvalidArgument, "MATMUL: null tensor pointer");
    if ((p->a_scale.rank && !tensors[3]) || (p->b_scale.rank && !tensors[4])) return fail(kInvalidArgument, "MATMUL: null block scale pointer");
    MatmulArgs g;
    int status = build_args(*p, tensors, g);
    if (status) return status;
    int kernel;
    status = choose_kernel(*p, kernel);
    if (status) return status;
    cudaStream_t stream = as_stream(stream_handle);
    if (kernel == DFGPU_MATMUL_UMMA_F32X3_CLUSTER) return launch_matmul_f32_cluster(*p, tensors, stream);  // (any f32 pointer: 4-byte alignment is enough)
    if (kernel == DFGPU_MATMUL_UMMA_F32X3) {
        SplitMatmul split;
        if (!f32_split_matmul(*p, split)) return fail(kUnsupported, "MATMUL: the split-operand tcgen05 form does not take this matmul");
        if (!scratch || (reinterpret_cast<uintptr_t>(scratch) & 15u) != 0 || (reinterpret_cast<uintptr_t>(tensors[0]) & 15u) != 0 ||
            (reinterpret_cast<uintptr_t>(tensors[1]) & 15u) != 0)
            return fail(kInvalidArgument, "MATMUL: the split-operand tcgen05 form needs 16-byte aligned A and B and its 16-byte aligned scratch (dfgpu_query_matmul gives the size)");
        uint8_t* base = static_cast<uint8_t*>(scratch);
        split.a.source = static_cast<const float*>(tensors[0]);
        split.a.pieces = reinterpret_cast<uint16_t*>(base + split.as_offset);
        split.b.source = static_cast<const float*>(tensors[1]);
        split.b.pieces = reinterpret_cast<uint16_t*>(base + split.bs_offset);
        int* flags = reinterpret_cast<int*>(base + split.flags_offset);
        status = launch_split6(split.a, split.b, flags, stream);
        if (status) return status;
        void* bf16_tensors[7] = {split.a.pieces, split.b.pieces, tensors[2], nullptr, nullptr, tensors[5], tensors[6]};
        status = launch_matmul_umma(split.bf16, bf16_tensors, DFGPU_MATMUL_UMMA_BF16, stream);
        if (status) return status;
        dim3 grid(static_cast<unsigned>((g.m + 63) / 64), static_cast<unsigned>((g.n + 63) / 64), 1);
        matmul_ffma_kernel<<<grid, 256, 0, stream>>>(tensors[0], tensors[1], tensors[2], g, flags, split.flag_count);
        return check_launch("MATMUL");
    }
    if (kernel != DFGPU_MATMUL_FFMA) return launch_matmul_umma(*p, tensors, kernel, stream);
    int64_t batches = 1;
    for (int i = 0; i < g.rank - 2; ++i) batches *= p->c.dim[i];
    if (batches > 65535) return fail(kUnsupported, "MATMUL: more than 65535 batch matrices");
    dim3 grid(static_cast<unsigned>((g.m + 63) / 64), static_cast<unsigned>((g.n + 63) / 64), static_cast<unsigned>(batches));
    matmul_ffma_kernel<<<grid, 256, 0, stream>>>(tensors[0], tensors[1], tensors[2], g, nullptr, 0);
    return check_launch("MATMUL");
}

// CONV_FPROP on CUDA cores: a direct kernel that covers every rank-4 convolution
// the generic path accepts (groups, stride, dilation, asymmetric padding, filter
// reversal, any strides, f32/f16/bf16 storage) and an f32-accumulate implicit-GEMM
// kernel for groups == 1. The tcgen05 implicit GEMM for bf16 NHWC lives in
// umma_gemm.cu; this file owns the launcher and the kernel choice.
//
// Padding: out-of-range taps read as 0 and are still multiplied, which is what the
// reference's single-node path does with its materialised zero padding; for finite
// data this equals the generic path's "skip the tap" rule.
#include "common.cuh"
#include "conv_args.cuh"
#include "umma.cuh"

namespace dfgpu {
namespace {

__global__ void conv_direct_kernel(const void* x, const void* w, void* y, ConvArgs a, int64_t total) {
    int64_t flat = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (flat >= total) return;
    int64_t q = flat % a.y.dim[3];
    int64_t rest = flat / a.y.dim[3];
    int64_t p = rest % a.y.dim[2];
    rest /= a.y.dim[2];
    int64_t k = rest % a.y.dim[1];
    int64_t n = rest / a.y.dim[1];
    int64_t group = k / a.k_per_group;
    int64_t R = a.w.dim[2], S = a.w.dim[3];
    float sum = 0.0f;
    for (int64_t c = 0; c < a.c_per_group; ++c) {
        int64_t xc = group * a.c_per_group + c;
        for (int64_t r = 0; r < R; ++r) {
            int64_t ih = p * a.stride_h + r * a.dilation_h - a.pad_h;
            if (ih < 0 || ih >= a.x.dim[2]) continue;
            for (int64_t s = 0; s < S; ++s) {
                int64_t iw = q * a.stride_w + s * a.dilation_w - a.pad_w;
                if (iw < 0 || iw >= a.x.dim[3]) continue;
                int64_t wr = a.reverse ? R - 1 - r : r, ws = a.reverse ? S - 1 - s : s;
                float xv = load_as_f32(x, a.x.dtype, n * a.x.stride[0] + xc * a.x.stride[1] + ih * a.x.stride[2] + iw * a.x.stride[3]);
                float wv = load_as_f32(w, a.w.dtype, k * a.w.stride[0] + c * a.w.stride[1] + wr * a.w.stride[2] + ws * a.w.stride[3]);
                sum = __fadd_rn(sum, __fmul_rn(xv, wv));
            }
        }
    }
    sum = apply_epilogue(sum, a, n, k, p, q);
    store_from_f32(y, a.y.dtype, n * a.y.stride[0] + k * a.y.stride[1] + p * a.y.stride[2] + q * a.y.stride[3], sum);
}

// Implicit GEMM: M = N*P*Q output pixels, N = K output channels, K = C*R*S.
// BM x 64 tile, 16-deep K slices through shared memory, 256 threads with a
// (BM/16) x 4 register tile each. CHANNELS_LAST picks the K ordering (r,s,c with c
// fastest, or c,r,s with s fastest) and the thread->element map of the X loads so
// that consecutive lanes read consecutive addresses in either layout.
template <int BM, bool CHANNELS_LAST>
__global__ void __launch_bounds__(256)
conv_igemm_ffma_kernel(const void* __restrict__ x, const void* __restrict__ w, void* __restrict__ y, ConvArgs a,
                       int64_t m_total, int64_t k_total) {
    constexpr int BN = 64, BK = 16, TM = BM / 16, TN = 4;
    constexpr int A_PER_THREAD = BM * BK / 256;
    constexpr int B_PER_THREAD = BN * BK / 256;
    __shared__ float as[BK][BM + 4];
    __shared__ float bs[BK][BN + 4];

    const int tid = threadIdx.x;
    const int64_t m0 = static_cast<int64_t>(blockIdx.x) * BM;
    const int64_t n0 = static_cast<int64_t>(blockIdx.y) * BN;
    const int64_t P = a.y.dim[2], Q = a.y.dim[3];
    const int64_t C = a.x.dim[1], R = a.w.dim[2], S = a.w.dim[3];
    const int64_t K = a.y.dim[1];

    // element -> (m, k) map of this thread's A loads
    int a_m[A_PER_THREAD], a_k[A_PER_THREAD];
    int64_t a_base[A_PER_THREAD];
    int32_t a_ih0[A_PER_THREAD], a_iw0[A_PER_THREAD];
    bool a_ok[A_PER_THREAD];
#pragma unroll
    for (int i = 0; i < A_PER_THREAD; ++i) {
        int e = tid + i * 256;
        if (CHANNELS_LAST) { a_k[i] = e % BK; a_m[i] = e / BK; }
        else { a_m[i] = e % BM; a_k[i] = e / BM; }
        int64_t m = m0 + a_m[i];
        a_ok[i] = m < m_total;
        int64_t mm = a_ok[i] ? m : 0;
        int64_t q = mm % Q, p = (mm / Q) % P, n = mm / (P * Q);
        a_base[i] = n * a.x.stride[0];
        a_ih0[i] = static_cast<int32_t>(p * a.stride_h - a.pad_h);
        a_iw0[i] = static_cast<int32_t>(q * a.stride_w - a.pad_w);
    }
    int b_n[B_PER_THREAD], b_k[B_PER_THREAD];
#pragma unroll
    for (int i = 0; i < B_PER_THREAD; ++i) {
        int e = tid + i * 256;
        b_k[i] = e % BK;
        b_n[i] = e / BK;
    }

    const int ty = tid / 16, tx = tid % 16;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int64_t k0 = 0; k0 < k_total; k0 += BK) {
#pragma unroll
        for (int i = 0; i < A_PER_THREAD; ++i) {
            int64_t kk = k0 + a_k[i];
            float value = 0.0f;
            if (a_ok[i] && kk < k_total) {
                int64_t c, r, s;
                if (CHANNELS_LAST) { c = kk % C; s = (kk / C) % S; r = kk / (C * S); }
                else { s = kk % S; r = (kk / S) % R; c = kk / (R * S); }
                int64_t ih = a_ih0[i] + r * a.dilation_h, iw = a_iw0[i] + s * a.dilation_w;
                if (ih >= 0 && ih < a.x.dim[2] && iw >= 0 && iw < a.x.dim[3])
                    value = load_as_f32(x, a.x.dtype, a_base[i] + c * a.x.stride[1] + ih * a.x.stride[2] + iw * a.x.stride[3]);
            }
            as[a_k[i]][a_m[i]] = value;
        }
#pragma unroll
        for (int i = 0; i < B_PER_THREAD; ++i) {
            int64_t kk = k0 + b_k[i];
            int64_t n = n0 + b_n[i];
            float value = 0.0f;
            if (n < K && kk < k_total) {
                int64_t c, r, s;
                if (CHANNELS_LAST) { c = kk % C; s = (kk / C) % S; r = kk / (C * S); }
                else { s = kk % S; r = (kk / S) % R; c = kk / (R * S); }
                if (a.reverse) { r = R - 1 - r; s = S - 1 - s; }
                value = load_as_f32(w, a.w.dtype, n * a.w.stride[0] + c * a.w.stride[1] + r * a.w.stride[2] + s * a.w.stride[3]);
            }
            bs[b_k[i]][b_n[i]] = value;
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
        if (m >= m_total) continue;
        int64_t q = m % Q, p = (m / Q) % P, n = m / (P * Q);
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            int64_t k = n0 + tx * TN + j;
            if (k >= K) continue;
            float value = apply_epilogue(acc[i][j], a, n, k, p, q);
            store_from_f32(y, a.y.dtype, n * a.y.stride[0] + k * a.y.stride[1] + p * a.y.stride[2] + q * a.y.stride[3], value);
        }
    }
}

// Fast form of the implicit GEMM for the common f32 case: channels-last X with C % 16 == 0, a packed KRSC filter,
// one group, no filter reversal. A 16-deep K slice then lies inside one filter tap, so the tap is decoded once
// per slice for the whole CTA (no per-element divisions), X and W come in as 16-byte loads, and the loads of
// slice k+1 are in flight (in registers) while slice k is multiplied out of shared memory.
template <int BM>
__global__ void __launch_bounds__(256)
conv_nhwc_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, void* __restrict__ y, ConvArgs a, int m_total,
                     const int* __restrict__ run_if_any, int flag_count, const float* __restrict__ partial, int partial_count) {
    constexpr int BN = 64, BK = 16, TM = BM / 16, TN = 4;
    __shared__ float as[2][BK][BM + 4];
    __shared__ float bs[2][BK][BN + 4];
    const int tid = threadIdx.x;
    if (run_if_any) {
        // Second pass behind the split-operand tensor-core form: it only convolves when one of the flags is set. With
        // the flags clear it is done at once, or, where the tensor-core launch split K over several CTAs per tile, it
        // adds their partial sums (in order) for its own outputs and applies the epilogue.
        int any = 0;
        for (int i = tid; i < flag_count; i += 256) any |= run_if_any[i];
        if (!__syncthreads_or(any)) {
            if (partial_count < 2) return;
            const int P = static_cast<int>(a.y.dim[2]), Q = static_cast<int>(a.y.dim[3]), K = static_cast<int>(a.y.dim[1]);
            const int64_t stride = static_cast<int64_t>(m_total) * K;
            const int ty = tid / 16, tx = tid % 16;
            for (int i = 0; i < TM; ++i) {
                const int m = blockIdx.x * BM + ty * TM + i;
                const int k0 = blockIdx.y * BN + tx * TN;
                if (m >= m_total || k0 >= K) continue;  // (K is a multiple of 64 in this form: whole float4s)
                const float* source = partial + static_cast<int64_t>(m) * K + k0;
                float4 part[kMaxKSplits];
#pragma unroll
                for (int z = 0; z < kMaxKSplits; ++z)  // every load in flight before the first sum
                    part[z] = z < partial_count ? __ldg(reinterpret_cast<const float4*>(source + z * stride)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                float4 sum = part[0];
#pragma unroll
                for (int z = 1; z < kMaxKSplits; ++z) {
                    if (z >= partial_count) break;
                    sum.x = __fadd_rn(sum.x, part[z].x);
                    sum.y = __fadd_rn(sum.y, part[z].y);
                    sum.z = __fadd_rn(sum.z, part[z].z);
                    sum.w = __fadd_rn(sum.w, part[z].w);
                }
                const int q = m % Q, p = (m / Q) % P, n = m / (P * Q);
                const float values[4] = {sum.x, sum.y, sum.z, sum.w};
                for (int j = 0; j < TN; ++j) {
                    const float value = apply_epilogue(values[j], a, n, k0 + j, p, q);
                    store_from_f32(y, a.y.dtype, n * a.y.stride[0] + (k0 + j) * a.y.stride[1] + p * a.y.stride[2] + q * a.y.stride[3], value);
                }
            }
            return;
        }
    }
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int P = static_cast<int>(a.y.dim[2]), Q = static_cast<int>(a.y.dim[3]);
    const int C = static_cast<int>(a.x.dim[1]), S = static_cast<int>(a.w.dim[3]);
    const int H = static_cast<int>(a.x.dim[2]), W = static_cast<int>(a.x.dim[3]);
    const int K = static_cast<int>(a.y.dim[1]);
    const int slices_per_tap = C / BK;
    const int slices = static_cast<int>(a.w.dim[2]) * S * slices_per_tap;

    // A: BM pixels x 16 channels = BM * 4 float4, one per thread for the first BM * 4 threads
    const bool a_loader = tid < BM * 4;
    const int a_m = tid >> 2, a_quad = tid & 3;
    int a_ih0 = 0, a_iw0 = 0;
    const float* a_base = x;
    bool a_valid = false;
    if (a_loader) {
        const int m = m0 + a_m;
        a_valid = m < m_total;
        const int mm = a_valid ? m : 0;
        const int q = mm % Q, p = (mm / Q) % P, n = mm / (P * Q);
        a_ih0 = p * a.stride_h - a.pad_h;
        a_iw0 = q * a.stride_w - a.pad_w;
        a_base = x + static_cast<int64_t>(n) * a.x.stride[0] + a_quad * 4;
    }
    // B: 64 output channels x 16 = 256 float4, one per thread
    const int b_n = tid >> 2, b_quad = tid & 3;
    const bool b_valid = n0 + b_n < K;
    const float* b_base = w + static_cast<int64_t>(b_valid ? n0 + b_n : 0) * a.w.stride[0] + b_quad * 4;

    auto fetch = [&](int slice, float4& av, float4& bv) {
        const int tap = slice / slices_per_tap, c0 = (slice - tap * slices_per_tap) * BK;
        const int r = tap / S, sx = tap - r * S;
        av = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (a_loader && a_valid) {
            const int ih = a_ih0 + r * a.dilation_h, iw = a_iw0 + sx * a.dilation_w;
            if (ih >= 0 && ih < H && iw >= 0 && iw < W)
                av = __ldg(reinterpret_cast<const float4*>(a_base + static_cast<int64_t>(ih) * a.x.stride[2] + static_cast<int64_t>(iw) * a.x.stride[3] + c0));
        }
        bv = b_valid ? __ldg(reinterpret_cast<const float4*>(b_base + static_cast<int64_t>(tap) * C + c0)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    };
    auto stash = [&](int buffer, const float4& av, const float4& bv) {
        if (a_loader) {
            as[buffer][a_quad * 4 + 0][a_m] = av.x;
            as[buffer][a_quad * 4 + 1][a_m] = av.y;
            as[buffer][a_quad * 4 + 2][a_m] = av.z;
            as[buffer][a_quad * 4 + 3][a_m] = av.w;
        }
        bs[buffer][b_quad * 4 + 0][b_n] = bv.x;
        bs[buffer][b_quad * 4 + 1][b_n] = bv.y;
        bs[buffer][b_quad * 4 + 2][b_n] = bv.z;
        bs[buffer][b_quad * 4 + 3][b_n] = bv.w;
    };

    const int ty = tid / 16, tx = tid % 16;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    float4 av, bv;
    fetch(0, av, bv);
    stash(0, av, bv);
    __syncthreads();
    for (int slice = 0; slice < slices; ++slice) {
        const int buffer = slice & 1;
        if (slice + 1 < slices) fetch(slice + 1, av, bv);
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a_reg[TM], b_reg[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a_reg[i] = as[buffer][kk][ty * TM + i];
            const float4 b4 = *reinterpret_cast<const float4*>(&bs[buffer][kk][tx * TN]);
            b_reg[0] = b4.x; b_reg[1] = b4.y; b_reg[2] = b4.z; b_reg[3] = b4.w;
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a_reg[i], b_reg[j], acc[i][j]);
        }
        if (slice + 1 < slices) stash(buffer ^ 1, av, bv);  // the other buffer was last read before the previous barrier
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= m_total) continue;
        const int q = m % Q, p = (m / Q) % P, n = m / (P * Q);
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int k = n0 + tx * TN + j;
            if (k >= K) continue;
            const float value = apply_epilogue(acc[i][j], a, n, k, p, q);
            store_from_f32(y, a.y.dtype, n * a.y.stride[0] + k * a.y.stride[1] + p * a.y.stride[2] + q * a.y.stride[3], value);
        }
    }
}

bool nhwc_f32_fast_form(const dfgpu_conv_params& p, void* const* tensors) {
    if (p.x.dtype != DFGPU_F32 || p.w.dtype != DFGPU_F32 || p.reverse_filter) return false;
    const int64_t C = p.x.dim[1], R = p.w.dim[2], S = p.w.dim[3];
    if (p.w.dim[1] != C || C % 16 != 0) return false;  // one group, whole 16-channel slices
    if (p.x.stride[1] != 1 || p.x.stride[3] % 4 != 0 || p.x.stride[2] % 4 != 0 || p.x.stride[0] % 4 != 0) return false;
    if (p.w.stride[1] != 1 || p.w.stride[3] != C || p.w.stride[2] != S * C || p.w.stride[0] != R * S * C) return false;
    if (element_count(p.x) >= (1ll << 31) || element_count(p.y) >= (1ll << 31) || element_count(p.w) >= (1ll << 31)) return false;
    if ((reinterpret_cast<uintptr_t>(tensors[0]) & 15u) != 0 || (reinterpret_cast<uintptr_t>(tensors[1]) & 15u) != 0) return false;
    return true;
}

// ---- f32 convolution on the bf16 tensor cores ------------------------------------------------------------
// X and W as six-piece bf16 copies (split_f32.cu), the bf16 convolution over 6C channels on tcgen05, and the CUDA-core
// kernel behind it: it adds the partial sums when the tensor-core launch split K over several CTAs per tile, or redoes
// the convolution when the split kernel flagged an infinity or a NaN in X or W (it returns at once otherwise).

struct SplitForm {
    dfgpu_conv_params bf16;   // the 6C-channel bf16 convolution
    int64_t x_quads, w_quads;
    int64_t xs_offset, ws_offset, flags_offset, partial_offset, scratch_bytes;
    int flag_count;
    ConvKSplit k_split;       // few tiles: several CTAs per tile, partial sums in scratch, added by the CUDA-core launch
};

// The split-operand form takes packed channels-last f32 X, a packed KRSC f32 filter and a packed channels-last Y, with
// the shape limits of the tcgen05 convolution (C and K multiples of 64, stride 1, dilation 1).
bool f32_split_form(const dfgpu_conv_params& p, SplitForm& form) {
    if (p.x.dtype != DFGPU_F32 || p.w.dtype != DFGPU_F32 || p.y.dtype != DFGPU_F32 || p.reverse_filter) return false;
    if (p.x.rank != 4 || p.w.rank != 4 || p.y.rank != 4) return false;
    auto packed = [](const dfgpu_tensor& t) {
        return t.stride[1] == 1 && t.stride[3] == t.dim[1] && t.stride[2] == t.dim[3] * t.dim[1] && t.stride[0] == t.dim[2] * t.dim[3] * t.dim[1];
    };
    if (!packed(p.x) || !packed(p.w) || !packed(p.y) || p.x.dim[1] != p.w.dim[1] || p.x.dim[1] % 64 != 0) return false;
    if (element_count(p.x) >= (1ll << 29) || element_count(p.w) >= (1ll << 29) || element_count(p.y) >= (1ll << 31)) return false;
    form.bf16 = p;
    form.bf16.kernel = DFGPU_CONV_UMMA_BF16;
    for (dfgpu_tensor* t : {&form.bf16.x, &form.bf16.w}) {
        t->dtype = DFGPU_BF16;
        t->dim[1] *= kSplitPieces;
        t->stride[3] = t->dim[1];
        t->stride[2] = t->dim[3] * t->dim[1];
        t->stride[0] = t->dim[2] * t->dim[3] * t->dim[1];
    }
    if (!conv_umma_supported(form.bf16)) return false;
    form.x_quads = element_count(p.x) / 4;
    form.w_quads = element_count(p.w) / 4;
    auto round_up = [](int64_t v) { return (v + 255) / 256 * 256; };
    form.flag_count = split_flag_count(SplitOperand{nullptr, nullptr, form.x_quads, 1, 0, 0, 0}, SplitOperand{nullptr, nullptr, form.w_quads, 1, 0, 0, 0});
    form.xs_offset = 0;
    form.ws_offset = round_up(element_count(p.x) * kSplitPieces * 2);
    form.flags_offset = form.ws_offset + round_up(element_count(p.w) * kSplitPieces * 2);
    form.partial_offset = form.flags_offset + round_up(static_cast<int64_t>(form.flag_count) * 4);
    form.k_split = conv_umma_k_split(form.bf16);
    form.scratch_bytes = form.partial_offset + (form.k_split.splits > 1 ? round_up(form.k_split.splits * element_count(p.y) * 4) : 0);
    return true;
}

int build_args(const dfgpu_conv_params& p, void* const* tensors, ConvArgs& a) {
    if (!valid_tensor(p.x) || !valid_tensor(p.w) || !valid_tensor(p.y))
        return fail(kInvalidShape, "CONV_FPROP: tensor rank or extent out of range");
    const int rank = p.x.rank;
    if ((rank != 4 && rank != 5) || p.w.rank != rank || p.y.rank != rank)
        return fail(kUnsupported, "CONV_FPROP: only rank-4 (2-D) and rank-5 (3-D) convolutions are executable on this backend");
    auto float_type = [](int t) { return t == DFGPU_F32 || t == DFGPU_F16 || t == DFGPU_BF16; };
    // split (hi, lo) activations exist for the tcgen05 kernel only: choose_kernel() refuses them for every other one
    if (!(float_type(p.x.dtype) || p.x.dtype == DFGPU_BF16X2) || !float_type(p.w.dtype) || !(float_type(p.y.dtype) || p.y.dtype == DFGPU_BF16X2))
        return fail(kUnsupported, "CONV_FPROP: tensors must be FLOAT, HALF or BFLOAT16");
    if (p.x.dim[0] != p.y.dim[0] || p.w.dim[0] != p.y.dim[1] || p.w.dim[1] <= 0 || p.x.dim[1] % p.w.dim[1] != 0)
        return fail(kInvalidShape, "CONV_FPROP: convolution N/K/C dimensions are inconsistent");
    int64_t groups = p.x.dim[1] / p.w.dim[1];
    if (groups <= 0 || p.y.dim[1] % groups != 0)
        return fail(kInvalidShape, "CONV_FPROP: convolution output channels are not divisible by groups");
    for (int axis = 2; axis < rank; ++axis) {
        // rank 5: axis 2 is the depth with its own attributes, the last two axes use the arrays
        const bool depth = rank == 5 && axis == 2;
        const int slot = axis - (rank - 2);
        const int64_t pre = depth ? p.depth_pre_pad : p.pre_pad[slot], post = depth ? p.depth_post_pad : p.post_pad[slot];
        const int64_t step = depth ? p.depth_stride : p.stride[slot], spread = depth ? p.depth_dilation : p.dilation[slot];
        if (pre < 0 || post < 0 || step <= 0 || spread <= 0)
            return fail(kInvalidArgument, "CONV_FPROP: padding must be non-negative and stride/dilation positive");
        int64_t dilated = spread * (p.w.dim[axis] - 1) + 1;
        int64_t padded = p.x.dim[axis] + pre + post;
        if (padded < dilated) return fail(kInvalidShape, "CONV_FPROP: effective filter exceeds padded input");
        if (p.y.dim[axis] != 1 + (padded - dilated) / step)
            return fail(kInvalidShape, "CONV_FPROP: output spatial dimensions do not match attributes");
    }
    int status = validate_epilogue(p.epilogue_count, p.epilogue, p.extra, tensors ? tensors + 3 : nullptr, p.y, "CONV_FPROP");
    if (status) return status;
    a.x = make_view(p.x);
    a.w = make_view(p.w);
    a.y = make_view(p.y);
    a.extra[0] = make_view(p.extra[0]);
    a.extra[1] = make_view(p.extra[1]);
    a.extra_data[0] = tensors ? tensors[3] : nullptr;
    a.extra_data[1] = tensors ? tensors[4] : nullptr;
    a.epilogue = make_epilogue(p.epilogue_count, p.epilogue);
    a.pad_d = rank == 5 ? static_cast<int32_t>(p.depth_pre_pad) : 0;
    a.stride_d = rank == 5 ? static_cast<int32_t>(p.depth_stride) : 1;
    a.dilation_d = rank == 5 ? static_cast<int32_t>(p.depth_dilation) : 1;
    a.pad_h = static_cast<int32_t>(p.pre_pad[0]);
    a.pad_w = static_cast<int32_t>(p.pre_pad[1]);
    a.stride_h = static_cast<int32_t>(p.stride[0]);
    a.stride_w = static_cast<int32_t>(p.stride[1]);
    a.dilation_h = static_cast<int32_t>(p.dilation[0]);
    a.dilation_w = static_cast<int32_t>(p.dilation[1]);
    a.reverse = p.reverse_filter;
    a.groups = static_cast<int32_t>(groups);
    a.c_per_group = p.w.dim[1];
    a.k_per_group = p.y.dim[1] / groups;
    return kOk;
}

int choose_kernel(const dfgpu_conv_params& p, const ConvArgs& a, int& kernel) {
    if (p.x.rank == 5) {   // 3-D: the one-launch tcgen05 kernel is the only one that walks a depth axis
        if (!conv_f32_cluster_supported(p))
            return fail(kUnsupported, "CONV_FPROP: a 3-D convolution needs FLOAT, HALF or BFLOAT16 tensors and at most 64 reduction units (64 channels x one tap) per CTA");
        if (p.kernel != DFGPU_CONV_AUTO && p.kernel != DFGPU_CONV_UMMA_F32X3_CLUSTER)
            return fail(kUnsupported, "CONV_FPROP: 3-D convolutions run on DFGPU_CONV_UMMA_F32X3_CLUSTER only");
        kernel = DFGPU_CONV_UMMA_F32X3_CLUSTER;
        return kOk;
    }
    int automatic = a.groups == 1 ? DFGPU_CONV_IGEMM_FFMA : DFGPU_CONV_DIRECT;
    if (conv_umma_supported(p)) automatic = DFGPU_CONV_UMMA_BF16;
    SplitForm split;
    const bool split_ok = f32_split_form(p, split);
    // (three launches instead of one: only where the convolution is big enough for the tensor cores to pay for them)
    const int64_t macs = p.y.dim[0] * p.y.dim[2] * p.y.dim[3] * p.y.dim[1] * p.w.dim[1] * p.w.dim[2] * p.w.dim[3];
    if (split_ok && macs >= kSplitFormMinMacs) automatic = DFGPU_CONV_UMMA_F32X3;
    const bool cluster_ok = conv_f32_cluster_supported(p);
    // One launch beats three where the output tiles fit one wave, or all output channels fit one tile (with several tiles
    // along K every one of them splits the same X rows again: the three-launch form splits them once).
    const int64_t pixel_tiles = (p.y.dim[0] * p.y.dim[2] * p.y.dim[3] + 127) / 128, channel_tiles = (p.y.dim[1] + 63) / 64;
    const bool one_launch_pays = automatic != DFGPU_CONV_UMMA_F32X3 || pixel_tiles * channel_tiles <= 148 || channel_tiles == 1;
    if (automatic != DFGPU_CONV_UMMA_BF16 && cluster_ok && one_launch_pays && p.w.dim[1] * p.w.dim[2] * p.w.dim[3] >= kClusterFormMinDepth)
        automatic = DFGPU_CONV_UMMA_F32X3_CLUSTER;   // (also what a bf16 or f16 convolution outside the bf16 tcgen05 kernel's shapes takes: stride, dilation, odd channel counts)
    kernel = p.kernel == DFGPU_CONV_AUTO ? automatic : p.kernel;
    if (kernel == DFGPU_CONV_UMMA_F32X3 && !split_ok)
        return fail(kUnsupported, "CONV_FPROP: the split-operand tcgen05 form needs packed channels-last f32 X, W and Y, C and K multiples of 64, stride 1, dilation 1");
    if (kernel == DFGPU_CONV_UMMA_F32X3_CLUSTER && !cluster_ok)
        return fail(kUnsupported, "CONV_FPROP: the one-launch tcgen05 form needs FLOAT, HALF or BFLOAT16 X, W and Y and at most 64 reduction units (64 channels x one tap) per CTA");
    if (kernel != DFGPU_CONV_UMMA_BF16 && (p.x.dtype == DFGPU_BF16X2 || p.y.dtype == DFGPU_BF16X2))
        return fail(kUnsupported, "CONV_FPROP: split bf16 pair tensors are read and written by the tcgen05 kernel only");
    if (kernel == DFGPU_CONV_IGEMM_FFMA && a.groups != 1)
        return fail(kUnsupported, "CONV_FPROP: the implicit-GEMM kernel needs groups == 1");
    if (kernel == DFGPU_CONV_UMMA_BF16 && !conv_umma_supported(p))
        return fail(kUnsupported, "CONV_FPROP: the tcgen05 kernel needs bf16 NHWC/KRSC, C and K multiples of 64, stride 1, dilation 1");
    if (kernel < DFGPU_CONV_DIRECT || kernel > DFGPU_CONV_UMMA_F32X3_CLUSTER)
        return fail(kInvalidArgument, "CONV_FPROP: unknown kernel id %d", kernel);
    return kOk;
}

}  // namespace
}  // namespace dfgpu

using namespace dfgpu;

extern "C" int dfgpu_query_conv_fprop(const dfgpu_conv_params* p, dfgpu_plan_info* info) {
    if (!p || !info) return fail(kInvalidArgument, "CONV_FPROP: null params");
    ConvArgs a;
    dfgpu_conv_params copy = *p;
    int saved = copy.epilogue_count;
    copy.epilogue_count = 0;  // pointers are not available at query time
    int status = build_args(copy, nullptr, a);
    if (status) return status;
    copy.epilogue_count = saved;
    int kernel;
    status = choose_kernel(copy, a, kernel);
    if (status) return status;
    info->kernel = kernel;
    info->launches = 1;
    info->scratch_bytes = 0;
    if (kernel == DFGPU_CONV_UMMA_F32X3) {
        SplitForm split;
        f32_split_form(copy, split);
        info->launches = 3;
        info->scratch_bytes = split.scratch_bytes;
    }
    return kOk;
}

extern "C" int dfgpu_conv_fprop(const dfgpu_conv_params* p, void* const* tensors, void* scratch, void* stream_handle) {
    if (!p || !tensors) return fail(kInvalidArgument, "CONV_FPROP: null params");
    if (!tensors[0] || !tensors[1] || !tensors[2]) return fail(kInvalidArgument, "CONV_FPROP: null tensor pointer");
    ConvArgs a;
    int status = build_args(*p, tensors, a);
    if (status) return status;
    int kernel;
    status = choose_kernel(*p, a, kernel);
    if (status) return status;
    cudaStream_t stream = as_stream(stream_handle);
    if (kernel == DFGPU_CONV_UMMA_BF16) return launch_conv_umma(*p, tensors, stream);
    if (kernel == DFGPU_CONV_UMMA_F32X3_CLUSTER) return launch_conv_f32_cluster(*p, a, tensors, stream);  // (any f32 pointer: 4-byte alignment is enough)
    int64_t m_total = p->y.dim[0] * p->y.dim[2] * p->y.dim[3];
    if (kernel == DFGPU_CONV_UMMA_F32X3) {
        SplitForm split;
        if (!f32_split_form(*p, split) || !nhwc_f32_fast_form(*p, tensors))
            return fail(kInvalidArgument, "CONV_FPROP: the split-operand tcgen05 form needs 16-byte aligned X and W");
        if (!scratch || (reinterpret_cast<uintptr_t>(scratch) & 15u) != 0)
            return fail(kInvalidArgument, "CONV_FPROP: the split-operand tcgen05 form needs its 16-byte aligned scratch (dfgpu_query_conv_fprop gives the size)");
        uint8_t* base = static_cast<uint8_t*>(scratch);
        uint16_t* xs = reinterpret_cast<uint16_t*>(base + split.xs_offset);
        uint16_t* ws = reinterpret_cast<uint16_t*>(base + split.ws_offset);
        int* flags = reinterpret_cast<int*>(base + split.flags_offset);
        const float* xf = static_cast<const float*>(tensors[0]);
        const float* wf = static_cast<const float*>(tensors[1]);
        const int64_t C = p->x.dim[1];
        const SplitOperand x_pieces{xf, xs, split.x_quads, C / 4, C, kSplitPieces * C, C}, w_pieces{wf, ws, split.w_quads, C / 4, C, kSplitPieces * C, C};
        status = launch_split6(x_pieces, w_pieces, flags, stream);
        if (status) return status;
        void* bf16_tensors[5] = {xs, ws, tensors[2], tensors[3], tensors[4]};
        ConvKSplit k_split = split.k_split;
        k_split.partial = reinterpret_cast<float*>(base + split.partial_offset);
        status = launch_conv_umma(split.bf16, bf16_tensors, stream, &k_split);
        if (status) return status;
        const float* partial = k_split.splits > 1 ? k_split.partial : nullptr;
        unsigned grid_n = static_cast<unsigned>((p->y.dim[1] + 63) / 64);
        if ((m_total + 63) / 64 * grid_n < 2 * sm_count()) {
            dim3 grid(static_cast<unsigned>((m_total + 31) / 32), grid_n);
            conv_nhwc_f32_kernel<32><<<grid, 256, 0, stream>>>(xf, wf, tensors[2], a, static_cast<int>(m_total), flags, split.flag_count, partial, k_split.splits);
        } else {
            dim3 grid(static_cast<unsigned>((m_total + 63) / 64), grid_n);
            conv_nhwc_f32_kernel<64><<<grid, 256, 0, stream>>>(xf, wf, tensors[2], a, static_cast<int>(m_total), flags, split.flag_count, partial, k_split.splits);
        }
        return check_launch("CONV_FPROP");
    }
    if (kernel == DFGPU_CONV_DIRECT) {
        int64_t total = element_count(p->y);
        conv_direct_kernel<<<static_cast<unsigned>((total + 127) / 128), 128, 0, stream>>>(tensors[0], tensors[1], tensors[2], a, total);
    } else {
        int64_t k_total = p->x.dim[1] * p->w.dim[2] * p->w.dim[3];
        bool channels_last = p->x.stride[1] == 1;
        unsigned grid_n = static_cast<unsigned>((p->y.dim[1] + 63) / 64);
        int64_t tiles64 = (m_total + 63) / 64 * grid_n;
        bool small = tiles64 < 2 * sm_count();
        if (nhwc_f32_fast_form(*p, tensors)) {
            const float* xf = static_cast<const float*>(tensors[0]);
            const float* wf = static_cast<const float*>(tensors[1]);
            if (small) {
                dim3 grid(static_cast<unsigned>((m_total + 31) / 32), grid_n);
                conv_nhwc_f32_kernel<32><<<grid, 256, 0, stream>>>(xf, wf, tensors[2], a, static_cast<int>(m_total), nullptr, 0, nullptr, 0);
            } else {
                dim3 grid(static_cast<unsigned>((m_total + 63) / 64), grid_n);
                conv_nhwc_f32_kernel<64><<<grid, 256, 0, stream>>>(xf, wf, tensors[2], a, static_cast<int>(m_total), nullptr, 0, nullptr, 0);
            }
        } else if (small) {
            dim3 grid(static_cast<unsigned>((m_total + 31) / 32), grid_n);
            if (channels_last) conv_igemm_ffma_kernel<32, true><<<grid, 256, 0, stream>>>(tensors[0], tensors[1], tensors[2], a, m_total, k_total);
            else conv_igemm_ffma_kernel<32, false><<<grid, 256, 0, stream>>>(tensors[0], tensors[1], tensors[2], a, m_total, k_total);
        } else {
            dim3 grid(static_cast<unsigned>((m_total + 63) / 64), grid_n);
            if (channels_last) conv_igemm_ffma_kernel<64, true><<<grid, 256, 0, stream>>>(tensors[0], tensors[1], tensors[2], a, m_total, k_total);
            else conv_igemm_ffma_kernel<64, false><<<grid, 256, 0, stream>>>(tensors[0], tensors[1], tensors[2], a, m_total, k_total);
        }
    }
    return check_launch("CONV_FPROP");
}

// ---- two convolutions in one launch -------------------------------------------------------------

namespace {
int check_pair(const dfgpu_conv_pair_params& p, void* const* tensors) {
    dfgpu::ConvArgs a;
    void* first_tensors[5] = {tensors ? tensors[0] : nullptr, tensors ? tensors[1] : nullptr, nullptr, tensors ? tensors[4] : nullptr, tensors ? tensors[5] : nullptr};
    void* second_tensors[5] = {nullptr, tensors ? tensors[2] : nullptr, tensors ? tensors[3] : nullptr, tensors ? tensors[6] : nullptr, tensors ? tensors[7] : nullptr};
    dfgpu_conv_params first = p.first, second = p.second;
    if (!tensors) first.epilogue_count = second.epilogue_count = 0;  // operand pointers are not available at query time
    int status = dfgpu::build_args(first, tensors ? first_tensors : nullptr, a);
    if (status) return status;
    status = dfgpu::build_args(second, tensors ? second_tensors : nullptr, a);
    if (status) return status;
    if (p.first.kernel != DFGPU_CONV_PAIR_AUTO && p.first.kernel != DFGPU_CONV_PAIR_UMMA) return fail(kInvalidArgument, "CONV_FPROP pair: unknown kernel id %d", p.first.kernel);
    if (!dfgpu::conv_pair_umma_supported(p.first, p.second))
        return fail(kUnsupported, "CONV_FPROP pair: needs a wide bf16 filter with 64 output channels and per-channel steps, then a 1 x 1 filter with 128 or 256 output channels");
    return kOk;
}
}  // namespace

extern "C" int dfgpu_query_conv_fprop_pair(const dfgpu_conv_pair_params* p, dfgpu_plan_info* info) {
    if (!p || !info) return fail(kInvalidArgument, "CONV_FPROP pair: null params");
    int status = check_pair(*p, nullptr);
    if (status) return status;
    info->kernel = DFGPU_CONV_PAIR_UMMA;
    info->launches = 1;
    info->scratch_bytes = 0;
    return kOk;
}

extern "C" int dfgpu_conv_fprop_pair(const dfgpu_conv_pair_params* p, void* const* tensors, void* scratch, void* stream_handle) {
    (void)scratch;
    if (!p || !tensors) return fail(kInvalidArgument, "CONV_FPROP pair: null params");
    for (int i = 0; i < 4; ++i)
        if (!tensors[i]) return fail(kInvalidArgument, "CONV_FPROP pair: null tensor pointer");
    int status = check_pair(*p, tensors);
    if (status) return status;
    return dfgpu::launch_conv_pair_umma(p->first, p->second, tensors, as_stream(stream_handle));
}

// f32 operands of a contraction as six-piece bf16 copies for the bf16 tensor cores.
//
// x = xh + xm + xl and w = wh + wm + wl with bf16 pieces (the leading 8 significant bits, the next 8, the last 8; every
// subtraction that forms them is exact), so x * w = xh*wh + xh*wm + xm*wh + xh*wl + xl*wh + xm*wm up to 2^-24 relative:
// a bf16 contraction over six times the depth, the first operand laid out as [xh | xh | xm | xh | xl | xm] and the
// second as [wh | wm | wh | wl | wh | wm], accumulated in f32 by the tensor cores. (Two pieces and three products stop at
// 2^-16, which fails the reference's acceptance rule 1e-4 + 1e-3 |ref| where |ref| is small.)
// A product with an infinite or NaN factor does not survive the split (inf * 0 where the other factor's lower pieces
// are zero), so every CTA of the split kernel also records whether it saw such a value; the caller launches its
// CUDA-core kernel behind the tensor-core one, which redoes the contraction when any CTA did.
#include "common.cuh"
#include "umma.cuh"

namespace dfgpu {
namespace {

// The three bf16 pieces of v; false (and everything in the first piece) when v is infinite or NaN.
__device__ __forceinline__ bool split_f32(float v, uint32_t (&piece)[3]) {
    const uint32_t bits = __float_as_uint(v);
    if ((bits & 0x7f800000u) == 0x7f800000u) {
        piece[0] = bits >> 16 | ((bits & 0xffffu) != 0u ? 0x40u : 0u);  // (a NaN stays a NaN whatever its low bits were)
        piece[1] = piece[2] = 0u;
        return false;
    }
    uint32_t hi = f32_to_bf16_bits(v);
    if ((hi & 0x7f80u) == 0x7f80u) hi = (hi & 0x8000u) | 0x7f7fu;  // rounded past the largest bf16: keep it finite
    const float rest = v - __uint_as_float(hi << 16);
    const uint32_t mid = f32_to_bf16_bits(rest);
    piece[0] = hi;
    piece[1] = mid;
    piece[2] = f32_to_bf16_bits(rest - __uint_as_float(mid << 16));
    return true;
}

__global__ void __launch_bounds__(256)
split6_f32_kernel(SplitOperand first, SplitOperand second, int* __restrict__ flags) {
    bool finite = true;
    float4 v[4];
    bool live[4], in_second[4];
    int64_t quad[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // all four loads in flight before the first is used
        quad[i] = static_cast<int64_t>(blockIdx.x) * kSplitQuadsPerCta + i * 256 + threadIdx.x;
        in_second[i] = quad[i] >= first.quads;
        if (in_second[i]) quad[i] -= first.quads;
        const bool s = in_second[i];
        const int64_t row_quads = s ? second.row_quads : first.row_quads;
        live[i] = quad[i] < (s ? second.quads : first.quads);
        if (live[i]) {
            const int64_t row = quad[i] / row_quads, column = (quad[i] - row * row_quads) * 4;
            v[i] = __ldg(reinterpret_cast<const float4*>((s ? second.source : first.source) + row * (s ? second.source_ld : first.source_ld) + column));
        } else {
            v[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (!live[i]) continue;
        uint32_t p0[3], p1[3], p2[3], p3[3];
        finite = split_f32(v[i].x, p0) && finite;
        finite = split_f32(v[i].y, p1) && finite;
        finite = split_f32(v[i].z, p2) && finite;
        finite = split_f32(v[i].w, p3) && finite;
        uint2 piece[3];
#pragma unroll
        for (int j = 0; j < 3; ++j) piece[j] = make_uint2(p0[j] | (p1[j] << 16), p2[j] | (p3[j] << 16));
        const bool s = in_second[i];
        const int64_t row_quads = s ? second.row_quads : first.row_quads;
        const int64_t row = quad[i] / row_quads, column = (quad[i] - row * row_quads) * 4;
        uint16_t* out = (s ? second.pieces : first.pieces) + row * (s ? second.row_stride : first.row_stride) + column;
        const int64_t piece_stride = s ? second.piece_stride : first.piece_stride;
        // first operand: h h m h l m; second operand: h m h l h m
        const int order_first[kSplitPieces] = {0, 0, 1, 0, 2, 1}, order_second[kSplitPieces] = {0, 1, 0, 2, 0, 1};
#pragma unroll
        for (int j = 0; j < kSplitPieces; ++j) *reinterpret_cast<uint2*>(out + j * piece_stride) = s ? piece[order_second[j]] : piece[order_first[j]];
    }
    const int any = __syncthreads_or(finite ? 0 : 1);
    if (threadIdx.x == 0) flags[blockIdx.x] = any;
}

}  // namespace

int split_flag_count(const SplitOperand& first, const SplitOperand& second) {
    return static_cast<int>((first.quads + second.quads + kSplitQuadsPerCta - 1) / kSplitQuadsPerCta);
}

int launch_split6(const SplitOperand& first, const SplitOperand& second, int* flags, cudaStream_t stream) {
    split6_f32_kernel<<<split_flag_count(first, second), 256, 0, stream>>>(first, second, flags);
    return check_launch("f32 operand split");
}

}  // namespace dfgpu

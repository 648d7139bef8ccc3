// Entry points of the tcgen05 (UMMA) kernels, used by the per-op launchers.
#pragma once

#include "common.cuh"

namespace dfgpu {

// What launch_conv_umma() does with a convolution, worked out from the descriptors alone (a query has no pointers).
struct ConvForm {
    int64_t N, C, H, W, K, P, Q, R, S;
    bool split_in, split_out;   // DFGPU_BF16X2 activations / output
    bool pointwise;             // 1 x 1, no padding: plain GEMM rows
    int bn;
    int rows_per_tile;          // output rows of one image per tile (non-pointwise, one slot per tap)
    bool persistent;            // the persistent kernel (TMA-store epilogue) takes it
    bool halo;                  // ... in the halo form
    int halo_rows;
};
bool conv_umma_form(const dfgpu_conv_params& p, ConvForm& form);

// bf16 NHWC/KRSC convolution as an implicit GEMM on tcgen05 (1x1 and 3x3, stride 1).
bool conv_umma_supported(const dfgpu_conv_params& p);
// K split of the one-tile-per-CTA form, for convolutions with fewer tiles than SMs: `splits` CTAs per tile each take
// k_blocks_per_split 64-deep K slices and store raw f32 partial sums (no epilogue) at partial + z * N*P*Q*K floats; the
// caller adds them in order and applies the epilogue. conv_umma_k_split() proposes a split (splits == 1: none).
constexpr int kMaxKSplits = 8;
struct ConvKSplit {
    int splits;
    int k_blocks_per_split;
    float* partial;
};
ConvKSplit conv_umma_k_split(const dfgpu_conv_params& p);
int launch_conv_umma(const dfgpu_conv_params& p, void* const* tensors, cudaStream_t stream, const ConvKSplit* k_split = nullptr);

// f32 NHWC/KRSC convolution on the bf16 tensor cores in one launch (made for fewer output tiles than SMs): a thread-block
// cluster per output tile, the operands split into bf16 pieces on their way into shared memory (umma_conv_f32.cu).
struct ConvArgs;
bool conv_f32_cluster_supported(const dfgpu_conv_params& p);
int launch_conv_f32_cluster(const dfgpu_conv_params& p, const ConvArgs& a, void* const* tensors, cudaStream_t stream);
int conv_f32_device_status(int* status);
// The same kernel for an unbatched f32 MATMUL (the 1 x 1 convolution of M pixels; B with N or K contiguous).
bool matmul_f32_cluster_supported(const dfgpu_matmul_params& p);
int launch_matmul_f32_cluster(const dfgpu_matmul_params& p, void* const* tensors, cudaStream_t stream);
constexpr int64_t kClusterFormMinDepth = 128;  // AUTO takes the one-launch form from this reduction depth (C R S, or K) on: the CUDA-core kernels walk the depth 16 at a time at ~0.8 us a step, the cluster launch costs 7-9 us whatever the depth

// A wide-filter convolution and the 1 x 1 convolution that consumes it, in one persistent kernel (the intermediate
// stays on the SM). tensors: {X, W first, W second, Y, first.extra0, first.extra1, second.extra0, second.extra1}.
bool conv_pair_umma_supported(const dfgpu_conv_params& first, const dfgpu_conv_params& second);
int launch_conv_pair_umma(const dfgpu_conv_params& first, const dfgpu_conv_params& second, void* const* tensors, cudaStream_t stream);
int conv_pair_device_status(int* status);

// ---- f32 operands as six-piece bf16 copies (split_f32.cu) -------------------------------------------------
// `quads` float4 groups of `source` (rows of row_quads float4, source_ld floats apart) become bf16 pieces at
// pieces + row * row_stride + j * piece_stride + column, j = 0..5 in the operand's piece order. A K-contiguous operand
// [rows, K] becomes [rows, 6K] with row_stride = 6K and piece_stride = K; an N-contiguous operand [K, N] becomes
// [6K, N] with row_stride = N and piece_stride = K * N. One flag per CTA (split_flag_count of them): 1 when the CTA saw
// an infinity or a NaN.
constexpr int kSplitQuadsPerCta = 1024;  // 256 threads x 4 float4
constexpr int kSplitPieces = 6;           // bf16 values per f32 value
constexpr int64_t kSplitFormMinMacs = int64_t{1} << 24;  // AUTO takes the split-operand form from this many multiply-adds on; below, one CUDA-core launch is quicker than three
struct SplitOperand {
    const float* source;
    uint16_t* pieces;
    int64_t quads, row_quads, source_ld, row_stride, piece_stride;
};
int split_flag_count(const SplitOperand& first, const SplitOperand& second);
int launch_split6(const SplitOperand& first, const SplitOperand& second, int* flags, cudaStream_t stream);

// MATMUL on tcgen05: kernel is DFGPU_MATMUL_UMMA_BF16 or DFGPU_MATMUL_UMMA_MXF8.
bool matmul_umma_supported(const dfgpu_matmul_params& p, int kernel);
int launch_matmul_umma(const dfgpu_matmul_params& p, void* const* tensors, int kernel, cudaStream_t stream);

// MATMUL on MXFP8 codes + E8M0 block scales (tcgen05 block-scaled kind), no dequantize pass.
bool matmul_mxf8_supported(const dfgpu_matmul_params& p);
int launch_matmul_mxf8(const dfgpu_matmul_params& p, void* const* tensors, cudaStream_t stream);
// MATMUL_FP8 on the same kernel: unit block scales, the three scalars and Amax_C applied in the epilogue.
bool matmul_fp8_umma_supported(const dfgpu_matmul_fp8_params& p);
int launch_matmul_fp8_umma(const dfgpu_matmul_fp8_params& p, void* const* tensors, cudaStream_t stream);
int mxf8_device_status(int* status);

// SDPA forward on tcgen05 (bf16, head dim 128, contiguous K/V).
bool sdpa_umma_supported(const dfgpu_sdpa_params& p);
int launch_sdpa_umma(const dfgpu_sdpa_params& p, void* const* tensors, void* scratch, cudaStream_t stream);
int sdpa_umma_device_status(int* status);  // reads and clears that unit's status word

// Paged-KV decode on TMA + tcgen05 (bf16, head dim 128, Sq = 1); partials go to `scratch`, the
// CUDA-core merge kernel in sdpa.cu finishes the job.
bool decode_umma_supported(const dfgpu_sdpa_params& p);
int decode_umma_chunks(const dfgpu_sdpa_params& p);
int64_t decode_umma_scratch_bytes(const dfgpu_sdpa_params& p);
int launch_decode_umma(const dfgpu_sdpa_params& p, void* const* tensors, void* scratch, const int* prefix_ok, cudaStream_t stream);  // prefix_ok: the validation result of compact page tables (null without them)
int sdpa_device_status(int* status);  // (sdpa.cu: compact page table validation)
int decode_umma_device_status(int* status);

}  // namespace dfgpu

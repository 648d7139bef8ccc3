// Kernel arguments and the fused epilogue shared by the CONV_FPROP kernels.
#pragma once

#include "common.cuh"

namespace dfgpu {

struct ConvArgs {
    View x, w, y;
    View extra[2];
    const void* extra_data[2];
    Epilogue epilogue;
    int32_t pad_h, pad_w, stride_h, stride_w, dilation_h, dilation_w;
    int32_t pad_d, stride_d, dilation_d;   // the depth axis of a rank-5 convolution (0, 1, 1 otherwise)
    int32_t reverse;
    int32_t groups;
    int64_t c_per_group, k_per_group;
};

// (n, k, p, q): the output element; d: its depth in a rank-5 convolution, whose operands align with [N, K, D, P, Q].
__device__ __forceinline__ float apply_epilogue(float value, const ConvArgs& a, int64_t n, int64_t k, int64_t p, int64_t q, int64_t d = 0) {
    for (int step = 0; step < a.epilogue.count; ++step) {
        if (a.epilogue.op[step] == DFGPU_EPI_ADD) {
            const View& t = a.extra[a.epilogue.operand[step]];
            const bool volume = a.y.rank == 5;
            int64_t index[5] = {n, k, volume ? d : p, volume ? p : q, q};
            int shift = (volume ? 5 : 4) - t.rank;
            int64_t offset = 0;
            for (int i = 0; i < t.rank; ++i) offset += (t.dim[i] == 1 ? 0 : index[i + shift]) * t.stride[i];
            value = __fadd_rn(value, load_as_f32(a.extra_data[a.epilogue.operand[step]], t.dtype, offset));
        } else {
            value = relu_forward(value, a.epilogue.lower[step], a.epilogue.upper[step], a.epilogue.slope[step]);
        }
    }
    return value;
}

}  // namespace dfgpu

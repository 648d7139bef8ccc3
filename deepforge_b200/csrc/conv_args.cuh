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
    int32_t reverse;
    int32_t groups;
    int64_t c_per_group, k_per_group;
};

__device__ __forceinline__ float apply_epilogue(float value, const ConvArgs& a, int64_t n, int64_t k, int64_t p, int64_t q) {
    for (int step = 0; step < a.epilogue.count; ++step) {
        if (a.epilogue.op[step] == DFGPU_EPI_ADD) {
            const View& t = a.extra[a.epilogue.operand[step]];
            int64_t index[4] = {n, k, p, q};
            int shift = 4 - t.rank;
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

// Error reporting and small host utilities shared by every launcher.
#include "common.cuh"

#include <cstring>

namespace dfgpu {

namespace {
thread_local char g_error[512] = "";
}

int fail(int code, const char* format, ...) {
    va_list arguments;
    va_start(arguments, format);
    vsnprintf(g_error, sizeof(g_error), format, arguments);
    va_end(arguments);
    return code;
}

int check_launch(const char* what) {
    cudaError_t error = cudaGetLastError();
    if (error != cudaSuccess) return fail(kExecutionFailed, "%s: kernel launch failed: %s", what, cudaGetErrorString(error));
    return kOk;
}

int sm_count() {
    static thread_local int cached_device = -1;
    static thread_local int cached_count = 148;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 148;
    if (device != cached_device) {
        int count = 0;
        if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && count > 0) {
            cached_count = count;
            cached_device = device;
        }
    }
    return cached_count;
}

// Epilogue operands must broadcast onto the output with trailing-axis alignment
// (the POINTWISE rule, lib/Compiler/FoundationalGraph.cpp:2552-2567).
int validate_epilogue(int count, const dfgpu_epilogue_step* steps, const dfgpu_tensor* extra,
                      void* const* extra_pointers, const dfgpu_tensor& out, const char* what) {
    if (count < 0 || count > DFGPU_MAX_EPILOGUE) return fail(kInvalidArgument, "%s: epilogue has %d steps (max %d)", what, count, DFGPU_MAX_EPILOGUE);
    for (int i = 0; i < count; ++i) {
        if (steps[i].op == DFGPU_EPI_RELU) continue;
        if (steps[i].op != DFGPU_EPI_ADD) return fail(kUnsupported, "%s: epilogue step %d has unknown op %d", what, i, steps[i].op);
        int operand = steps[i].operand;
        if (operand < 0 || operand > 1) return fail(kInvalidArgument, "%s: epilogue operand index %d out of range", what, operand);
        const dfgpu_tensor& t = extra[operand];
        if (!valid_tensor(t) || t.rank > out.rank) return fail(kInvalidShape, "%s: epilogue operand %d has no usable descriptor", what, operand);
        if (t.dtype != DFGPU_F32 && t.dtype != DFGPU_BF16 && t.dtype != DFGPU_F16)
            return fail(kUnsupported, "%s: epilogue operand %d has an unsupported type", what, operand);
        int shift = out.rank - t.rank;
        for (int axis = 0; axis < t.rank; ++axis)
            if (t.dim[axis] != 1 && t.dim[axis] != out.dim[axis + shift])
                return fail(kInvalidShape, "%s: epilogue operand %d does not broadcast onto the output", what, operand);
        if (!extra_pointers || !extra_pointers[operand]) return fail(kInvalidArgument, "%s: epilogue operand %d pointer is null", what, operand);
    }
    return kOk;
}

}  // namespace dfgpu

extern "C" const char* dfgpu_last_error(void) { return dfgpu::g_error; }
// Bumped whenever a params struct, a pointer list or an enumeration changes.
// 2: dfgpu_sdpa_params gained bias and alibi_mask. 3: it gained sink and block_mask (14 pointers); DFGPU_BF16X2.
// 4: dfgpu_conv_fprop_pair, dfgpu_block_scale_quantize_pair. 5: dfgpu_sdpa_params gained page_offsets_k / page_offsets_v
// (16 pointers), DFGPU_I64, DFGPU_CONV_UMMA_F32X3, DFGPU_MATMUL_UMMA_F32X3 in place of the two-SM MXFP8 id.
// 6: DFGPU_CONV_UMMA_F32X3_CLUSTER, DFGPU_MATMUL_UMMA_F32X3_CLUSTER. 7: dfgpu_conv_params gained the depth attributes (rank 5).
// 8: dfgpu_sdpa_params gained dropout (21 pointers). 9: DFGPU_FP4, DFGPU_I4.
// 10: dfgpu_pointwise_params gained in2, elu_alpha, softplus_beta, swish_beta, axis (every POINTWISE mode; 4 pointers).
// 11: dfgpu_constants (graph-owned pass-by-value scalars).
extern "C" int dfgpu_abi_version(void) { return 11; }

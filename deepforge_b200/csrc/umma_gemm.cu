#include "umma.cuh"
namespace dfgpu {
bool conv_umma_supported(const dfgpu_conv_params&) { return false; }
int launch_conv_umma(const dfgpu_conv_params&, void* const*, cudaStream_t) { return fail(kUnsupported, "not built"); }
bool matmul_umma_supported(const dfgpu_matmul_params&, int) { return false; }
int launch_matmul_umma(const dfgpu_matmul_params&, void* const*, int, cudaStream_t) { return fail(kUnsupported, "not built"); }
bool sdpa_umma_supported(const dfgpu_sdpa_params&) { return false; }
int launch_sdpa_umma(const dfgpu_sdpa_params&, void* const*, void*, cudaStream_t) { return fail(kUnsupported, "not built"); }
}

// Result of the GPU kernel-selection lowering: an ordered list of launches through the
// dfgpu C ABI, with every tensor slot bound either to a variant-pack UID or to an
// offset inside the caller's workspace. This takes the place of the reference's
// LLVM/x86 object emission for the hot-path tags.
#pragma once

#include "dfgpu.h"

#include <cstdint>
#include <string>
#include <variant>
#include <vector>

namespace deepforge::compiler {

enum class KernelOp : std::uint8_t { kBlockScaleQuantize, kBlockScaleDequantize, kPointwise, kConvFprop, kMatmul, kSdpaForward, kMatmulFp8, kConvFpropPair, kBlockScaleQuantizePair, kConstants };

struct TensorBinding {
    enum class Kind : std::uint8_t { kAbsent, kArgument, kWorkspace } kind = Kind::kAbsent;
    std::int64_t uid = 0;            // kArgument: variant-pack UID; kWorkspace: the virtual tensor's UID
    std::uint64_t offset = 0;        // kWorkspace: byte offset into the workspace (a virtual tensor, or a graph-owned constant)
};

using KernelParams = std::variant<dfgpu_bsq_params, dfgpu_bsd_params, dfgpu_pointwise_params, dfgpu_conv_params,
                                  dfgpu_matmul_params, dfgpu_sdpa_params, dfgpu_matmul_fp8_params, dfgpu_conv_pair_params, dfgpu_bsq_pair_params,
                                  dfgpu_constants_params>;

struct KernelStep {
    KernelOp op = KernelOp::kPointwise;
    std::string label;                     // "conv1+bias_add+relu" style: the fused node names
    std::vector<std::size_t> nodes;        // indices of the graph nodes this launch covers
    KernelParams params;
    std::vector<TensorBinding> tensors;    // in the port order of the dfgpu entry point
    TensorBinding scratch;                 // kernel scratch inside the workspace, if any
    std::int32_t kernel = 0;               // kernel id the library resolved for these params
    std::int32_t launches = 1;
};

struct KernelPlan {
    std::vector<KernelStep> steps;
    [[nodiscard]] std::string to_text() const;  // one line per launch (the --dump-plan view)
};

}  // namespace deepforge::compiler

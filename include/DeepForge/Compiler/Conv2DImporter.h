// Metadata of the single-node CONV_FPROP path. Same struct names and fields as the reference's
// include/DeepForge/Compiler/Conv2DImporter.h:17-41 (its MLIR import functions have no counterpart here: the
// convolution is lowered to a kernel launch, not to Linalg IR).
#pragma once

#include "DeepForge/Compiler/GraphMetadata.h"

#include <array>
#include <cstdint>
#include <string>

namespace deepforge::compiler {

struct Conv2DImportOptions {
    std::string function_name = "deepforge_conv2d";
};

// For a graph that is one f32 CONV_FPROP on packed NHWC / KRSC tensors (the reference's MVP path,
// lib/MLIR/Conv2DImporter.cpp:332-370): the three UIDs, the PHYSICAL shapes (N, H, W, C / K, R, S, C), the input
// shape after padding and the convolution attributes; `arguments` then holds exactly X, W, Y in that order and under
// those names, FLOAT, rank 4 with packed strides, alignment 4, read / read / write. For every other graph the
// convolution fields stay zero and `arguments` is the generic table.
struct Conv2DCompileMetadata : GraphCompileMetadata {
    std::int64_t x_uid = 0, w_uid = 0, y_uid = 0;
    std::array<std::int64_t, 4> x_shape{}, w_shape{}, y_shape{}, padded_x_shape{};
    std::array<std::int64_t, 2> pre_padding{}, post_padding{}, stride{}, dilation{};
    bool operator==(Conv2DCompileMetadata const&) const = default;
};

// The checks the reference's runtime applies to a conv-adapter executable (lib/Runtime/Executable.cpp:735-768):
// exactly three rank-4 FLOAT arguments named X, W, Y bound to x_uid / w_uid / y_uid with read / read / write access and
// the shapes above, and no dynamic-shape or override metadata.
[[nodiscard]] import::Status validate_conv2d_adapter_metadata(Conv2DCompileMetadata const& metadata);

}  // namespace deepforge::compiler

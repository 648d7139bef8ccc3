// Argument table of a compiled graph: one entry per non-virtual tensor, ascending UID (X, W, Y for the single-node
// convolution adapter). Type and field names are those of the reference's include/DeepForge/Compiler/GraphMetadata.h
// so that callers and artifacts read the same way; the override and ragged fields exist for source compatibility and
// always hold their "none" values here (shape overrides and ragged storage are not executable on this backend).
#pragma once

#include "DeepForge/Import/SerializedGraph.h"
#include "DeepForge/Import/Status.h"

#include <cstdint>
#include <string>
#include <vector>

namespace deepforge::compiler {

// Which argument-table convention a compilation follows. The numeric values are the reference's; the kernel plan
// itself travels in artifacts under adapter kind 2 (see Artifact.h).
enum class InvocationAdapterKind : std::uint32_t { kConv2DRankedMemref = 0, kGenericRankedMemrefPointerTable = 1 };
enum class TensorAccess : std::uint8_t { kRead, kWrite, kReadWrite };
enum class ShapeOverridePolicy : std::uint8_t { kNone = 0, kPointwiseExact, kMatmul, kSdpaForward, kReshape, kReduction, kTranspose, kConcatenate, kBlockScaleMatmul };
enum class TensorStoragePolicy : std::uint8_t { kStrided = 0, kRaggedBatchPrefix };

struct TensorArgumentMetadata {
    std::int64_t uid = 0;
    std::string name;
    import::DataType data_type = import::DataType::kFloat32;
    std::vector<std::int64_t> dimensions;
    std::vector<std::int64_t> strides;
    std::uint64_t size_bytes = 0;  // storage span
    std::uint64_t alignment = 1;   // clamp(element bytes, 1, 8); 16 (scales: 4) where a TMA-fed kernel reads or writes the argument
    TensorAccess access = TensorAccess::kRead;
    TensorStoragePolicy storage_policy = TensorStoragePolicy::kStrided;  // always strided here
    std::int64_t ragged_offset_uid = 0, ragged_sequence_uid = 0, ragged_sequence_divisor = 1;
    bool operator==(TensorArgumentMetadata const&) const = default;
};

struct GraphCompileMetadata {
    std::string function_name;
    std::vector<TensorArgumentMetadata> arguments;
    bool dynamic_shape_enabled = false, override_shape_enabled = false;  // always false here
    ShapeOverridePolicy override_policy = ShapeOverridePolicy::kNone;
    std::vector<std::int64_t> override_role_uids, override_axis_map;     // always empty here
    bool operator==(GraphCompileMetadata const&) const = default;
};

// 1..4096 arguments, unique UIDs, non-empty NUL-free names, rank 1..64 with equal stride
// rank, power-of-two alignment <= 4096, size_bytes equal to the recomputed storage span; strided storage without
// ragged references, no override metadata (lib/Runtime/GraphMetadata.cpp:317-690 of the reference).
[[nodiscard]] import::Status validate_graph_compile_metadata(GraphCompileMetadata const& metadata);

}  // namespace deepforge::compiler

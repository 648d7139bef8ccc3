// In-memory model of a cudnn-frontend v1.24.0 serialized Graph, restricted to what the
// GPU hot path executes: CONV_FPROP, POINTWISE, MATMUL, SDPA, BLOCK_SCALE_QUANTIZE and
// BLOCK_SCALE_DEQUANTIZE. Other tags parse into kUnsupportedNode.
#pragma once

#include <cstdint>
#include <map>
#include <optional>
#include <string>
#include <string_view>
#include <variant>
#include <vector>

namespace deepforge::import {

enum class DataType : std::uint8_t {
    kFloat32,
    kFloat16,
    kBFloat16,
    kFp8E4M3,
    kFp8E5M2,
    kFp8E8M0,
    kInt32,
    kInt64,
    kInt8,
    kUint8,
    kBoolean,
    kFloat64,
    kFp4E2M1,
    kInt4,
};

// Serialized spellings ("FLOAT", "HALF", "BFLOAT16", "FP8_E4M3", ...).
[[nodiscard]] std::optional<DataType> data_type_from_name(std::string_view name) noexcept;
[[nodiscard]] std::string_view data_type_name(DataType type) noexcept;
[[nodiscard]] std::uint32_t data_type_storage_bits(DataType type) noexcept;

enum class OperationTag : std::uint8_t {
    kConvFprop,
    kPointwise,
    kMatmul,
    kSdpa,
    kBlockScaleQuantize,
    kBlockScaleDequantize,
    kMatmulFp8,
};
[[nodiscard]] std::string_view operation_tag_name(OperationTag tag) noexcept;

// The Frontend's scalar variant for a graph-owned constant (reference: include/DeepForge/Import/SerializedGraph.h:104-123).
// The kind's number is the variant index the serializer writes.
enum class PassByValueKind : std::uint8_t { kInt64 = 0, kInt32 = 1, kFloat16 = 2, kFloat32 = 3, kFloat64 = 4, kBFloat16 = 5 };

struct PassByValueScalar {
    // FLOAT: the f32 bit pattern (uint32). HALF / DOUBLE / BFLOAT16: the bits of the JSON number as a double (uint64),
    // narrowed to the tensor's type where the constant is materialised.
    using Storage = std::variant<std::int64_t, std::int32_t, std::uint32_t, std::uint64_t>;
    PassByValueKind kind = PassByValueKind::kFloat32;
    Storage value = std::uint32_t{0};

    bool operator==(PassByValueScalar const&) const = default;
};

struct TensorDesc {
    std::int64_t uid = 0;
    std::string name;
    DataType data_type = DataType::kFloat32;
    std::vector<std::int64_t> dim;
    std::vector<std::int64_t> stride;
    bool is_virtual = false;
    // is_pass_by_value without a payload: a one-element argument the caller passes like any other tensor. With a
    // payload: a constant the graph owns, absent from the argument table (a pointer the caller passes for it is ignored).
    bool is_pass_by_value = false;
    std::optional<PassByValueScalar> pass_by_value;
    std::string reordering_type = "NONE";
    // Ragged batch-prefix storage (reference: include/DeepForge/Import/SerializedGraph.h:136-137): entry (b, ...) of the
    // tensor lies at offsets[b] + the inner strides. Executable here for SDPA page tables only (compact page tables).
    std::optional<std::int64_t> ragged_offset_uid;
    std::optional<std::string> ragged_offset_name;

    bool operator==(TensorDesc const&) const = default;
};

// null | bool | integer | real | string | integer array | real array
using AttributeValue = std::variant<std::monostate, bool, std::int64_t, double, std::string,
                                    std::vector<std::int64_t>, std::vector<double>>;

struct OperationDesc {
    OperationTag tag = OperationTag::kPointwise;
    std::string name;
    std::map<std::string, std::int64_t> inputs;   // port -> tensor UID
    std::map<std::string, std::int64_t> outputs;  // port -> tensor UID
    std::map<std::string, AttributeValue> attributes;

    bool operator==(OperationDesc const&) const = default;
};

struct GraphContext {
    std::optional<std::string> name;
    std::optional<DataType> compute_data_type;
    std::optional<DataType> intermediate_data_type;
    std::optional<DataType> io_data_type;
    std::int64_t sm_count = -1;
    std::optional<bool> is_dynamic_shape_enabled;
    std::optional<bool> is_override_shape_enabled;

    bool operator==(GraphContext const&) const = default;
};

struct SerializedGraph {
    GraphContext context;
    std::uint64_t graph_uid = 0;
    std::string cudnn_backend_version;
    std::map<std::int64_t, TensorDesc> tensors;
    std::vector<OperationDesc> nodes;

    [[nodiscard]] std::size_t tensor_count() const noexcept { return tensors.size(); }
    // The graph's only node when it is one stride-1, dilation-1, cross-correlation f32
    // CONV_FPROP (the reference's optimised single-node path), else nullptr.
    [[nodiscard]] OperationDesc const* single_conv_fprop() const noexcept;

    bool operator==(SerializedGraph const&) const = default;
};

// Bytes spanned by a tensor's strided storage (max element offset + 1, times the element
// size; sub-byte types are rejected upstream). False on overflow.
[[nodiscard]] bool tensor_storage_bytes(TensorDesc const& tensor, std::uint64_t& bytes) noexcept;

}  // namespace deepforge::import

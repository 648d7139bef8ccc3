// Strict importer for the serialized Graph subset the GPU hot path executes.
//
// Protocol rules follow the reference importer (lib/Import/SerializedGraphImporter.cpp):
// json_version "1.0", cudnn_frontend_version 12400, the seven context fields, the
// twelve tensor fields, per-tag required attributes (lib/Import/Schema.cpp), integer
// UID references, no execution metadata the backend cannot honour, producers before
// consumers. Unknown fields are errors, not ignored.
#include "DeepForge/Import/SerializedGraphImporter.h"

#include <nlohmann/json.hpp>

#include <algorithm>
#include <array>
#include <bit>
#include <charconv>
#include <fstream>
#include <limits>
#include <set>

namespace deepforge::import {
namespace {

using Json = nlohmann::json;

Status fail(ErrorCode code, std::string_view subject, std::string_view detail) { return Status::failure(code, subject, detail); }

std::string join(std::string_view parent, std::string_view child) {
    std::string path(parent);
    if (!path.empty()) path += '.';
    path += child;
    return path;
}

struct TypeName {
    std::string_view name;
    DataType type;
    std::uint32_t bits;
};
constexpr std::array<TypeName, 14> kTypes{{
    {"FLOAT", DataType::kFloat32, 32},     {"HALF", DataType::kFloat16, 16},      {"BFLOAT16", DataType::kBFloat16, 16},
    {"FP8_E4M3", DataType::kFp8E4M3, 8},   {"FP8_E5M2", DataType::kFp8E5M2, 8},   {"FP8_E8M0", DataType::kFp8E8M0, 8},
    {"INT32", DataType::kInt32, 32},       {"INT64", DataType::kInt64, 64},       {"INT8", DataType::kInt8, 8},
    {"UINT8", DataType::kUint8, 8},        {"BOOLEAN", DataType::kBoolean, 8},    {"DOUBLE", DataType::kFloat64, 64},
    {"FP4_E2M1", DataType::kFp4E2M1, 4},   {"INT4", DataType::kInt4, 4},
}};

struct TagSchema {
    OperationTag tag;
    std::string_view name;
    std::vector<std::string_view> required;
    std::vector<std::string_view> optional;
    std::vector<std::string_view> inputs;
    std::vector<std::string_view> outputs;
};

// Attribute and port names per tag, as the pinned Frontend serializer emits them.
std::vector<TagSchema> const& schemas() {
    static const std::vector<TagSchema> table{
        {OperationTag::kBlockScaleDequantize, "BLOCK_SCALE_DEQUANTIZE", {"compute_data_type", "block_size", "is_negative_scale"}, {}, {"X", "scale"}, {"Y"}},
        {OperationTag::kBlockScaleQuantize, "BLOCK_SCALE_QUANTIZE", {"compute_data_type", "block_size", "axis"}, {}, {"X"}, {"Y", "scale"}},
        {OperationTag::kConvFprop, "CONV_FPROP", {"compute_data_type", "pre_padding", "post_padding", "stride", "dilation", "math_mode"}, {}, {"X", "W"}, {"Y"}},
        {OperationTag::kMatmul, "MATMUL", {"compute_data_type", "padding_value"}, {}, {"A", "B", "M_override", "N_override", "K_override"}, {"C"}},
        {OperationTag::kMatmulFp8, "MATMUL_FP8", {"compute_data_type"}, {},
         {"A", "B", "Descale_A", "Descale_B", "M_override", "N_override", "K_override", "Scale_C"}, {"C", "Amax_C"}},
        {OperationTag::kPointwise, "POINTWISE",
         {"compute_data_type", "mode", "axis", "relu_lower_clip", "relu_upper_clip", "relu_lower_clip_slope", "swish_beta", "elu_alpha", "softplus_beta"},
         {}, {"IN_0", "IN_1", "IN_2"}, {"OUT_0"}},
        {OperationTag::kSdpa, "SDPA",
         {"generate_stats", "alibi_mask", "padding_mask", "dropout_probability", "attn_scale_value", "max_seq_len_kv", "mma_core_mode", "left_bound",
          "right_bound", "diagonal_alignment", "implementation", "is_mxfp8", "unfuse_fma"},
         {"rescale_threshold", "compute_data_type"},
         {"Q", "K", "V", "Attn_scale", "Bias", "SEQ_LEN_Q", "SEQ_LEN_KV", "Seed", "Offset", "Dropout_mask", "Dropout_scale", "Page_table_K",
          "Page_table_V", "Block_mask", "Descale_Q", "Descale_K", "Descale_V", "Descale_S", "Scale_S", "Scale_O", "SINK_TOKEN"},
         {"O", "Stats", "Max", "Sum_exp", "RNG_DUMP", "Amax_S", "Amax_O"}},
    };
    return table;
}

// Tags the Frontend can serialize but this backend does not execute.
constexpr std::array<std::string_view, 32> kOtherTags{{
    "ADA_LAYER_NORM", "ADA_LAYER_NORM_BPROP", "BATCHNORM", "BATCHNORM_INFERENCE", "BN_FINALIZE", "CONCATENATE", "CONV_DGRAD", "CONV_WGRAD",
    "DBN", "DBN_WEIGHT", "DIAGONAL_BAND_MASK", "DLN", "DIN", "DRMS_NORM", "GEN_STATS", "INSTANCE_NORM", "LAYER_NORM",
    "MOE_GROUPED_MATMUL", "MOE_GROUPED_MATMUL_BWD", "PAGED_CACHE_LOAD", "REDUCTION", "RESAMPLE", "RESHAPE", "RMS_NORM", "RNG", "ROPE",
    "ROPE_BWD", "SDPA_BWD", "SDPA_FP8", "SDPA_FP8_BWD", "SLICE", "TRANSPOSE",
}};

bool read_int(Json const& value, std::int64_t& out) {
    if (value.is_number_unsigned()) {
        auto raw = value.get<std::uint64_t>();
        if (raw > static_cast<std::uint64_t>(std::numeric_limits<std::int64_t>::max())) return false;
        out = static_cast<std::int64_t>(raw);
        return true;
    }
    if (value.is_number_integer()) {
        out = value.get<std::int64_t>();
        return true;
    }
    return false;
}

Status read_data_type(Json const& object, std::string const& path, char const* field, bool nullable, std::optional<DataType>& out) {
    auto it = object.find(field);
    if (it == object.end()) return fail(ErrorCode::kMissingField, join(path, field), "required field is missing");
    if (it->is_null() && nullable) {
        out.reset();
        return Status::ok();
    }
    if (!it->is_string()) return fail(ErrorCode::kInvalidFieldType, join(path, field), "expected a data type name");
    auto type = data_type_from_name(it->get<std::string>());
    if (!type) {
        if (it->get<std::string>() == "NOT_SET" && nullable) {
            out.reset();
            return Status::ok();
        }
        return fail(ErrorCode::kUnsupportedDataType, join(path, field), "unknown data type name");
    }
    out = type;
    return Status::ok();
}

Status parse_context(Json const& root, GraphContext& context) {
    auto it = root.find("context");
    if (it == root.end()) return fail(ErrorCode::kMissingField, "context", "required field is missing");
    if (!it->is_object()) return fail(ErrorCode::kInvalidFieldType, "context", "expected object");
    constexpr std::array<std::string_view, 7> fields{{"name", "compute_data_type", "intermediate_data_type", "io_data_type", "sm_count",
                                                       "is_dynamic_shape_enabled", "is_override_shape_enabled"}};
    for (auto name : fields)
        if (!it->contains(std::string(name))) return fail(ErrorCode::kMissingField, join("context", name), "serialized context field is missing");
    for (auto field = it->begin(); field != it->end(); ++field)
        if (std::find(fields.begin(), fields.end(), field.key()) == fields.end())
            return fail(ErrorCode::kInvalidValue, join("context", field.key()), "field is not emitted by the pinned context serializer");
    auto const& name = (*it)["name"];
    if (name.is_string()) {
        context.name = name.get<std::string>();
        if (context.name->find('\0') != std::string::npos) return fail(ErrorCode::kInvalidValue, "context.name", "name contains NUL");
    } else if (!name.is_null()) {
        return fail(ErrorCode::kInvalidFieldType, "context.name", "expected string or null");
    }
    for (auto [field, target] : {std::pair{"compute_data_type", &context.compute_data_type},
                                 std::pair{"intermediate_data_type", &context.intermediate_data_type},
                                 std::pair{"io_data_type", &context.io_data_type}}) {
        auto status = read_data_type(*it, "context", field, true, *target);
        if (status.is_bad()) return status;
    }
    if (!read_int((*it)["sm_count"], context.sm_count)) return fail(ErrorCode::kInvalidFieldType, "context.sm_count", "expected integer");
    for (auto [field, target] : {std::pair{"is_dynamic_shape_enabled", &context.is_dynamic_shape_enabled},
                                 std::pair{"is_override_shape_enabled", &context.is_override_shape_enabled}}) {
        auto const& value = (*it)[field];
        if (value.is_boolean()) *target = value.get<bool>();
        else if (value.is_null()) target->reset();
        else return fail(ErrorCode::kInvalidFieldType, join("context", field), "expected boolean or null");
    }
    return Status::ok();
}

Status read_int_array(Json const& value, std::string const& path, std::vector<std::int64_t>& out) {
    if (!value.is_array()) return fail(ErrorCode::kInvalidFieldType, path, "expected integer array");
    out.clear();
    for (auto const& item : value) {
        std::int64_t element = 0;
        if (!read_int(item, element)) return fail(ErrorCode::kInvalidFieldType, path, "expected integer array");
        out.push_back(element);
    }
    return Status::ok();
}

std::optional<PassByValueKind> pass_by_value_kind(DataType type) {
    switch (type) {
        case DataType::kInt64: return PassByValueKind::kInt64;
        case DataType::kInt32: return PassByValueKind::kInt32;
        case DataType::kFloat16: return PassByValueKind::kFloat16;
        case DataType::kFloat32: return PassByValueKind::kFloat32;
        case DataType::kFloat64: return PassByValueKind::kFloat64;
        case DataType::kBFloat16: return PassByValueKind::kBFloat16;
        default: return std::nullopt;
    }
}

// {"index": variant index, "value": ...} (lib/Import/SerializedGraphImporter.cpp:190-268): the index must be the one of
// the tensor's data type; INT64 / INT32 values are integers, FLOAT is its bit pattern as 8 hexadecimal digits, HALF /
// DOUBLE / BFLOAT16 are JSON numbers.
Status parse_pass_by_value(Json const& value, DataType tensor_type, std::string const& path, PassByValueScalar& out) {
    if (!value.is_object()) return fail(ErrorCode::kInvalidFieldType, path, "expected Frontend scalar variant object");
    if (value.size() != 2 || !value.contains("index") || !value.contains("value"))
        return fail(ErrorCode::kInvalidValue, path, "Frontend scalar variant requires only index and value");
    std::int64_t index = 0;
    if (!read_int(value["index"], index)) return fail(ErrorCode::kInvalidFieldType, join(path, "index"), "expected integer");
    if (index < 0 || index > 5) return fail(ErrorCode::kInvalidValue, join(path, "index"), "Frontend scalar variant index must be in [0, 5]");
    auto const expected = pass_by_value_kind(tensor_type);
    if (!expected || static_cast<std::int64_t>(*expected) != index)
        return fail(ErrorCode::kInvalidValue, join(path, "index"), "Frontend scalar variant type does not match tensor data_type");
    out.kind = *expected;
    auto const& scalar = value["value"];
    switch (*expected) {
        case PassByValueKind::kInt64: {
            std::int64_t integer = 0;
            if (!read_int(scalar, integer)) return fail(ErrorCode::kInvalidFieldType, join(path, "value"), "expected integer");
            out.value = integer;
            return Status::ok();
        }
        case PassByValueKind::kInt32: {
            std::int64_t integer = 0;
            if (!read_int(scalar, integer)) return fail(ErrorCode::kInvalidFieldType, join(path, "value"), "expected integer");
            if (integer < std::numeric_limits<std::int32_t>::min() || integer > std::numeric_limits<std::int32_t>::max())
                return fail(ErrorCode::kInvalidValue, join(path, "value"), "Frontend INT32 scalar is out of range");
            out.value = static_cast<std::int32_t>(integer);
            return Status::ok();
        }
        case PassByValueKind::kFloat32: {
            if (!scalar.is_string()) return fail(ErrorCode::kInvalidFieldType, join(path, "value"), "Frontend FLOAT scalar requires an 8-digit hexadecimal bit pattern");
            auto const text = scalar.get<std::string>();
            std::uint32_t bits = 0;
            auto const parsed = std::from_chars(text.data(), text.data() + text.size(), bits, 16);
            if (text.size() != 8 || parsed.ec != std::errc{} || parsed.ptr != text.data() + text.size())
                return fail(ErrorCode::kInvalidValue, join(path, "value"), "Frontend FLOAT scalar requires exactly 8 hexadecimal digits");
            out.value = bits;
            return Status::ok();
        }
        default:
            if (!scalar.is_number()) return fail(ErrorCode::kInvalidFieldType, join(path, "value"), "Frontend floating scalar requires a numeric value");
            out.value = std::bit_cast<std::uint64_t>(scalar.get<double>());
            return Status::ok();
    }
}

// The root map "pass_by_values" repeats every embedded payload under its tensor's UID
// (lib/Import/SerializedGraphImporter.cpp:860-925): both sides must hold the same scalars.
Status validate_pass_by_values(Json const& root, SerializedGraph const& graph) {
    auto const values = root.find("pass_by_values");
    if (values == root.end()) {
        for (auto const& [uid, tensor] : graph.tensors)
            if (tensor.pass_by_value) return fail(ErrorCode::kMissingField, "pass_by_values", "embedded scalar payload requires the Frontend root map");
        return Status::ok();
    }
    if (!values->is_object()) return fail(ErrorCode::kInvalidFieldType, "pass_by_values", "expected object keyed by tensor UID");
    std::set<std::int64_t> seen;
    for (auto it = values->begin(); it != values->end(); ++it) {
        auto const path = join("pass_by_values", it.key());
        std::int64_t uid = 0;
        auto const& key = it.key();
        auto const parsed = std::from_chars(key.data(), key.data() + key.size(), uid);
        if (key.empty() || parsed.ec != std::errc{} || parsed.ptr != key.data() + key.size() || std::to_string(uid) != key)
            return fail(ErrorCode::kInvalidValue, path, "root scalar key must be a canonical decimal int64 UID");
        auto const tensor = graph.tensors.find(uid);
        if (tensor == graph.tensors.end()) return fail(ErrorCode::kMissingUid, path, "root scalar UID has no tensor descriptor");
        if (!tensor->second.pass_by_value) return fail(ErrorCode::kInvalidValue, path, "root scalar UID has no matching tensor payload");
        PassByValueScalar scalar;
        auto status = parse_pass_by_value(it.value(), tensor->second.data_type, path, scalar);
        if (status.is_bad()) return status;
        if (scalar != *tensor->second.pass_by_value) return fail(ErrorCode::kInvalidValue, path, "root and tensor scalar payloads differ");
        seen.insert(uid);
    }
    for (auto const& [uid, tensor] : graph.tensors)
        if (tensor.pass_by_value && !seen.count(uid))
            return fail(ErrorCode::kMissingField, join("pass_by_values", std::to_string(uid)), "tensor scalar payload has no matching root entry");
    return Status::ok();
}

Status parse_tensor(Json const& value, std::string const& path, TensorDesc& tensor) {
    if (!value.is_object()) return fail(ErrorCode::kInvalidFieldType, path, "expected tensor object");
    constexpr std::array<std::string_view, 12> fields{{"name", "data_type", "dim", "stride", "is_virtual", "pass_by_value", "is_pass_by_value",
                                                        "reordering_type", "uid", "uid_assigned", "ragged_offset_uid", "ragged_offset_name"}};
    for (auto it = value.begin(); it != value.end(); ++it)
        if (std::find(fields.begin(), fields.end(), it.key()) == fields.end())
            return fail(ErrorCode::kInvalidValue, join(path, it.key()), "field is not emitted by the pinned tensor serializer");
    for (auto required : {"name", "data_type", "dim", "stride", "is_virtual", "pass_by_value", "is_pass_by_value", "reordering_type", "uid", "uid_assigned"})
        if (!value.contains(required)) return fail(ErrorCode::kMissingField, join(path, required), "required field is missing");
    if (!value["name"].is_string()) return fail(ErrorCode::kInvalidFieldType, join(path, "name"), "expected string");
    tensor.name = value["name"].get<std::string>();
    if (tensor.name.empty() || tensor.name.find('\0') != std::string::npos)
        return fail(ErrorCode::kInvalidValue, join(path, "name"), "tensor name must be non-empty and NUL-free");
    std::optional<DataType> type;
    auto status = read_data_type(value, path, "data_type", false, type);
    if (status.is_bad()) return status;
    tensor.data_type = *type;
    status = read_int_array(value["dim"], join(path, "dim"), tensor.dim);
    if (status.is_bad()) return status;
    status = read_int_array(value["stride"], join(path, "stride"), tensor.stride);
    if (status.is_bad()) return status;
    // lib/Import/SerializedGraphImporter.cpp: ranks 1..64 parse (the kernels execute up to 8, which the lowering checks)
    if (tensor.dim.empty() || tensor.dim.size() > 64) return fail(ErrorCode::kInvalidValue, join(path, "dim"), "tensor rank must be between 1 and 64");
    if (tensor.dim.size() != tensor.stride.size()) return fail(ErrorCode::kInvalidValue, join(path, "stride"), "dimension and stride ranks must match");
    std::uint64_t count = 1;
    for (std::size_t axis = 0; axis < tensor.dim.size(); ++axis) {
        if (tensor.dim[axis] <= 0) return fail(ErrorCode::kInvalidShape, join(path, "dim"), "extents must be positive");
        if (tensor.stride[axis] <= 0) return fail(ErrorCode::kInvalidLayout, join(path, "stride"), "strides must be positive");
        if (count > static_cast<std::uint64_t>(std::numeric_limits<std::int64_t>::max()) / static_cast<std::uint64_t>(tensor.dim[axis]))
            return fail(ErrorCode::kDimensionOverflow, join(path, "dim"), "element count overflows int64");
        count *= static_cast<std::uint64_t>(tensor.dim[axis]);
    }
    std::uint64_t bytes = 0;
    if (!tensor_storage_bytes(tensor, bytes)) return fail(ErrorCode::kDimensionOverflow, path, "storage span overflows int64");
    for (auto [field, target] : {std::pair{"is_virtual", &tensor.is_virtual}, std::pair{"is_pass_by_value", &tensor.is_pass_by_value}}) {
        if (!value[field].is_boolean()) return fail(ErrorCode::kInvalidFieldType, join(path, field), "expected boolean");
        *target = value[field].get<bool>();
    }
    if (!value["reordering_type"].is_string()) return fail(ErrorCode::kInvalidFieldType, join(path, "reordering_type"), "expected string");
    tensor.reordering_type = value["reordering_type"].get<std::string>();
    if (tensor.reordering_type != "NONE" && tensor.reordering_type != "F8_128x4" && tensor.reordering_type != "INT8x32" && tensor.reordering_type != "F16x16")
        return fail(ErrorCode::kInvalidValue, join(path, "reordering_type"), "unknown reordering type");
    if (!read_int(value["uid"], tensor.uid)) return fail(ErrorCode::kInvalidFieldType, join(path, "uid"), "expected integer");
    if (!value["uid_assigned"].is_boolean()) return fail(ErrorCode::kInvalidFieldType, join(path, "uid_assigned"), "expected boolean");
    if (!value["uid_assigned"].get<bool>()) return fail(ErrorCode::kMissingUid, join(path, "uid_assigned"), "tensor has no assigned UID");
    if (!value["pass_by_value"].is_null()) {
        PassByValueScalar payload;
        auto payload_status = parse_pass_by_value(value["pass_by_value"], tensor.data_type, join(path, "pass_by_value"), payload);
        if (payload_status.is_bad()) return payload_status;
        tensor.pass_by_value = payload;
    }
    if (tensor.pass_by_value && !tensor.is_pass_by_value)
        return fail(ErrorCode::kInvalidValue, join(path, "is_pass_by_value"), "scalar payload requires is_pass_by_value=true");
    // lib/Import/SerializedGraphImporter.cpp:687-711: both or neither
    if (auto it = value.find("ragged_offset_uid"); it != value.end() && !it->is_null()) {
        std::int64_t offsets = 0;
        if (!read_int(*it, offsets)) return fail(ErrorCode::kInvalidFieldType, join(path, "ragged_offset_uid"), "expected integer");
        tensor.ragged_offset_uid = offsets;
    }
    if (auto it = value.find("ragged_offset_name"); it != value.end() && !it->is_null()) {
        if (!it->is_string()) return fail(ErrorCode::kInvalidFieldType, join(path, "ragged_offset_name"), "expected string");
        tensor.ragged_offset_name = it->get<std::string>();
    }
    if (tensor.ragged_offset_uid.has_value() != tensor.ragged_offset_name.has_value())
        return fail(ErrorCode::kInvalidValue, path, "ragged offset UID and name must appear together");
    return Status::ok();
}

Status to_attribute(Json const& value, std::string const& path, AttributeValue& out) {
    std::int64_t integer = 0;
    if (value.is_null()) out = std::monostate{};
    else if (value.is_boolean()) out = value.get<bool>();
    else if (read_int(value, integer)) out = integer;
    else if (value.is_number()) out = value.get<double>();
    else if (value.is_string()) out = value.get<std::string>();
    else if (value.is_array()) {
        bool all_int = true;
        for (auto const& item : value) {
            if (!item.is_number()) return fail(ErrorCode::kInvalidFieldType, path, "arrays must hold numbers");
            std::int64_t unused = 0;
            all_int = all_int && read_int(item, unused);
        }
        if (all_int) {
            std::vector<std::int64_t> items;
            for (auto const& item : value) {
                read_int(item, integer);
                items.push_back(integer);
            }
            out = std::move(items);
        } else {
            std::vector<double> items;
            for (auto const& item : value) items.push_back(item.get<double>());
            out = std::move(items);
        }
    } else {
        return fail(ErrorCode::kInvalidFieldType, path, "attribute must be null, boolean, number, string or numeric array");
    }
    return Status::ok();
}

Status parse_ports(Json const& node, std::string const& path, char const* field, std::vector<std::string_view> const& allowed,
                   std::map<std::int64_t, TensorDesc> const& tensors, std::map<std::string, std::int64_t>& out) {
    auto it = node.find(field);
    if (it == node.end()) return fail(ErrorCode::kMissingField, join(path, field), "required field is missing");
    if (!it->is_object()) return fail(ErrorCode::kInvalidFieldType, join(path, field), "expected object");
    for (auto port = it->begin(); port != it->end(); ++port) {
        if (std::find(allowed.begin(), allowed.end(), port.key()) == allowed.end())
            return fail(ErrorCode::kInvalidValue, join(join(path, field), port.key()), "unknown port for this operation");
        if (port->is_null()) continue;
        std::int64_t uid = 0;
        if (port->is_string()) return fail(ErrorCode::kMissingUid, join(join(path, field), port.key()), "name references are not accepted; use an integer UID");
        if (!read_int(port.value(), uid)) return fail(ErrorCode::kInvalidFieldType, join(join(path, field), port.key()), "tensor references must be integer UIDs");
        if (!tensors.count(uid)) return fail(ErrorCode::kMissingUid, join(join(path, field), port.key()), "tensor reference is unresolved");
        out[port.key()] = uid;
    }
    return Status::ok();
}

constexpr std::array<std::string_view, 50> kPointwiseModes{{
    "ADD", "MUL", "SQRT", "MAX", "MIN", "RELU_FWD", "TANH_FWD", "SIGMOID_FWD", "ELU_FWD", "GELU_FWD", "SOFTPLUS_FWD", "SWISH_FWD", "RELU_BWD",
    "TANH_BWD", "SIGMOID_BWD", "ELU_BWD", "GELU_BWD", "SOFTPLUS_BWD", "SWISH_BWD", "ERF", "IDENTITY", "GELU_APPROX_TANH_BWD",
    "GELU_APPROX_TANH_FWD", "GEN_INDEX", "BINARY_SELECT", "EXP", "LOG", "NEG", "MOD", "POW", "ABS", "CEIL", "COS", "FLOOR", "RSQRT", "SIN",
    "LOGICAL_NOT", "TAN", "SUB", "ADD_SQUARE", "DIV", "CMP_EQ", "CMP_NEQ", "CMP_GT", "CMP_GE", "CMP_LT", "CMP_LE", "LOGICAL_AND", "LOGICAL_OR",
    "RECIPROCAL"}};

// Inputs a POINTWISE mode reads (lib/Import/Schema.cpp:353-377); 0 for a name outside the list.
std::size_t pointwise_input_count(std::string_view mode) {
    if (std::find(kPointwiseModes.begin(), kPointwiseModes.end(), mode) == kPointwiseModes.end()) return 0;
    if (mode == "BINARY_SELECT") return 3;
    constexpr std::array<std::string_view, 17> binary{{"ADD", "MUL", "DIV", "ADD_SQUARE", "SUB", "CMP_EQ", "CMP_NEQ", "CMP_GT", "CMP_GE", "CMP_LT", "CMP_LE",
                                                       "LOGICAL_AND", "LOGICAL_OR", "MIN", "MAX", "MOD", "POW"}};
    bool const backward = mode.size() > 4 && mode.substr(mode.size() - 4) == "_BWD";
    return backward || std::find(binary.begin(), binary.end(), mode) != binary.end() ? 2 : 1;
}

bool fits_int32(Json const& value) {
    std::int64_t integer = 0;
    return read_int(value, integer) && integer >= std::numeric_limits<std::int32_t>::min() && integer <= std::numeric_limits<std::int32_t>::max();
}

// The value type every attribute of the executable tags must have (lib/Import/SerializedGraphImporter.cpp:1096-1192).
bool attribute_value_is_valid(Json const& value, OperationTag tag, std::string_view name) {
    auto one_of = [&](std::initializer_list<std::string_view> allowed, bool nullable) {
        if (value.is_null()) return nullable;
        if (!value.is_string()) return false;
        auto const text = value.get<std::string>();
        return std::find(allowed.begin(), allowed.end(), std::string_view(text)) != allowed.end();
    };
    auto integer = [](Json const& item) { return item.is_number_integer() || item.is_number_unsigned(); };
    if (name == "compute_data_type" || name == "mma_core_mode") return value.is_null() || (value.is_string() && data_type_from_name(value.get<std::string>()).has_value());
    if (name == "mode") {
        if (tag != OperationTag::kPointwise) return one_of({"NONE", "GATHER", "SCATTER"}, false);
        return value.is_string() && pointwise_input_count(value.get<std::string>()) != 0;
    }
    if (name == "math_mode") return one_of({"CONVOLUTION", "CROSS_CORRELATION"}, false);
    if (name == "diagonal_alignment") return one_of({"TOP_LEFT", "BOTTOM_RIGHT"}, false);
    if (name == "implementation") return one_of({"AUTO", "COMPOSITE", "UNIFIED"}, false);
    if (name == "pre_padding" || name == "post_padding" || name == "stride" || name == "dilation")
        return value.is_array() && std::all_of(value.begin(), value.end(), integer);
    if (name == "block_size") {
        if (tag == OperationTag::kBlockScaleDequantize) return value.is_array() && std::all_of(value.begin(), value.end(), fits_int32);
        return value.is_null() || fits_int32(value);
    }
    if (name == "is_negative_scale" || name == "alibi_mask" || name == "padding_mask" || name == "is_deterministic_algorithm" || name == "is_mxfp8" ||
        name == "unfuse_fma" || name == "is_deterministic")
        return value.is_boolean();
    if (name == "generate_stats" || name == "generate_index") return value.is_null() || value.is_boolean();
    if (name == "max_seq_len_kv") return value.is_null() || fits_int32(value);
    if (name == "axis" || name == "seed" || name == "left_bound" || name == "right_bound" || name == "max_total_seq_len_q" || name == "max_total_seq_len_kv")
        return value.is_null() || integer(value);
    if (name == "padding_value" || name == "relu_lower_clip" || name == "relu_upper_clip" || name == "relu_lower_clip_slope" || name == "swish_beta" ||
        name == "elu_alpha" || name == "softplus_beta" || name == "dropout_probability" || name == "attn_scale_value" || name == "rescale_threshold")
        return value.is_null() || value.is_number();
    return true;  // an attribute the reference's table does not constrain
}

Status parse_node(Json const& node, std::string const& path, std::map<std::int64_t, TensorDesc> const& tensors, OperationDesc& operation) {
    if (!node.is_object()) return fail(ErrorCode::kInvalidFieldType, path, "expected node object");
    auto tag_it = node.find("tag");
    if (tag_it == node.end()) return fail(ErrorCode::kMissingField, join(path, "tag"), "required field is missing");
    if (!tag_it->is_string()) return fail(ErrorCode::kInvalidFieldType, join(path, "tag"), "expected string");
    auto const tag = tag_it->get<std::string>();
    TagSchema const* schema = nullptr;
    for (auto const& candidate : schemas())
        if (candidate.name == tag) schema = &candidate;
    if (!schema) {
        bool known = std::find(kOtherTags.begin(), kOtherTags.end(), tag) != kOtherTags.end();
        return fail(ErrorCode::kUnsupportedNode, join(path, "tag"),
                    known ? "operation tag '" + tag + "' is outside the GPU hot path" : "unknown operation tag '" + tag + "'");
    }
    operation.tag = schema->tag;
    auto name_it = node.find("name");
    if (name_it == node.end()) return fail(ErrorCode::kMissingField, join(path, "name"), "required field is missing");
    if (!name_it->is_string()) return fail(ErrorCode::kInvalidFieldType, join(path, "name"), "expected string");
    operation.name = name_it->get<std::string>();
    if (operation.name.empty() || operation.name.find('\0') != std::string::npos) return fail(ErrorCode::kInvalidValue, join(path, "name"), "node name is empty or contains NUL");
    auto status = parse_ports(node, path, "inputs", schema->inputs, tensors, operation.inputs);
    if (status.is_bad()) return status;
    status = parse_ports(node, path, "outputs", schema->outputs, tensors, operation.outputs);
    if (status.is_bad()) return status;
    for (auto required : schema->required)
        if (!node.contains(std::string(required))) return fail(ErrorCode::kMissingField, join(path, required), "required attribute is missing");
    for (auto it = node.begin(); it != node.end(); ++it) {
        auto const& key = it.key();
        if (key == "tag" || key == "name" || key == "inputs" || key == "outputs") continue;
        bool known = std::find(schema->required.begin(), schema->required.end(), key) != schema->required.end() ||
                     std::find(schema->optional.begin(), schema->optional.end(), key) != schema->optional.end();
        if (!known) return fail(ErrorCode::kInvalidValue, join(path, key), "unknown attribute for this operation");
        if (!attribute_value_is_valid(it.value(), schema->tag, key))
            return fail(ErrorCode::kInvalidFieldType, join(path, key), "attribute has a value outside the pinned schema");
        AttributeValue attribute;
        status = to_attribute(it.value(), join(path, key), attribute);
        if (status.is_bad()) return status;
        operation.attributes[key] = std::move(attribute);
    }
    if (operation.outputs.empty()) return fail(ErrorCode::kInvalidValue, join(path, "outputs"), "operation must expose at least one serialized output");
    if (schema->tag == OperationTag::kPointwise) {  // lib/Import/SerializedGraphImporter.cpp:1325-1342
        auto const expected = pointwise_input_count(node["mode"].get<std::string>());
        if (operation.inputs.size() != expected || operation.outputs.size() != 1 || !operation.outputs.count("OUT_0"))
            return fail(ErrorCode::kInvalidValue, path, "pointwise ports do not match mode arity");
        for (std::size_t index = 0; index < expected; ++index)
            if (!operation.inputs.count("IN_" + std::to_string(index)))
                return fail(ErrorCode::kInvalidValue, join(path, "inputs"), "pointwise inputs must be contiguous from IN_0");
    }
    return Status::ok();
}

Status expect_empty(Json const& root, char const* field) {
    auto it = root.find(field);
    if (it == root.end()) return Status::ok();
    bool empty = (it->is_object() || it->is_array()) ? it->empty() : it->is_null();
    if (!empty) return fail(ErrorCode::kUnsupportedExecutionMetadata, field, "must be empty for this backend");
    return Status::ok();
}

Status validate_document(Json const& root, SerializedGraph& graph) {
    if (!root.is_object()) return fail(ErrorCode::kInvalidFieldType, "document", "expected a JSON object");
    // Unknown top-level fields are tolerated, as the reference importer tolerates them; every nested
    // object (context, tensors, nodes) is closed.
    for (auto required : {"json_version", "cudnn_backend_version", "cudnn_frontend_version", "graph_uid", "nodes", "tensors"})
        if (!root.contains(required)) return fail(ErrorCode::kMissingField, required, "required field is missing");
    if (!root["json_version"].is_string()) return fail(ErrorCode::kInvalidFieldType, "json_version", "expected string");
    if (root["json_version"].get<std::string>() != "1.0") return fail(ErrorCode::kSchemaVersionMismatch, "json_version", "version 1.0 is required");
    if (!root["cudnn_backend_version"].is_string()) return fail(ErrorCode::kInvalidFieldType, "cudnn_backend_version", "expected string");
    graph.cudnn_backend_version = root["cudnn_backend_version"].get<std::string>();
    std::int64_t frontend = 0;
    if (!read_int(root["cudnn_frontend_version"], frontend)) return fail(ErrorCode::kInvalidFieldType, "cudnn_frontend_version", "expected integer");
    if (frontend != kPinnedFrontendVersion) return fail(ErrorCode::kFrontendVersionMismatch, "cudnn_frontend_version", "cuDNN Frontend v1.24.0 (12400) is required");
    if (!root["graph_uid"].is_number_unsigned() && !root["graph_uid"].is_number_integer()) return fail(ErrorCode::kInvalidFieldType, "graph_uid", "expected unsigned integer");
    if (!root["graph_uid"].is_number_unsigned() && root["graph_uid"].get<std::int64_t>() < 0) return fail(ErrorCode::kInvalidValue, "graph_uid", "expected a non-negative integer");
    graph.graph_uid = root["graph_uid"].get<std::uint64_t>();
    auto status = parse_context(root, graph.context);
    if (status.is_bad()) return status;

    auto const& tensors = root["tensors"];
    if (!tensors.is_object()) return fail(ErrorCode::kInvalidFieldType, "tensors", "expected object");
    std::set<std::string> names;
    for (auto it = tensors.begin(); it != tensors.end(); ++it) {
        TensorDesc tensor;
        auto const path = join("tensors", it.key());
        // a tensor without an assigned UID is keyed by its name (and is then refused below: execution needs UIDs)
        if (it.value().is_object() && it.value().contains("uid_assigned") && it.value()["uid_assigned"].is_boolean() && !it.value()["uid_assigned"].get<bool>() &&
            it.value().contains("name") && it.value()["name"].is_string() && it.value()["name"].get<std::string>() != it.key())
            return fail(ErrorCode::kInvalidValue, path, "name-keyed tensor requires a map key matching tensor.name");
        status = parse_tensor(it.value(), path, tensor);
        if (status.is_bad()) return status;
        if (it.key() != std::to_string(tensor.uid)) return fail(ErrorCode::kInvalidValue, path, "UID-assigned tensor requires a matching decimal map key");
        if (!graph.tensors.emplace(tensor.uid, std::move(tensor)).second) return fail(ErrorCode::kDuplicateUid, path, "tensor UID is used twice");
    }
    status = validate_pass_by_values(root, graph);
    if (status.is_bad()) return status;

    auto const& nodes = root["nodes"];
    if (!nodes.is_array()) return fail(ErrorCode::kInvalidFieldType, "nodes", "expected array");
    if (nodes.empty()) return fail(ErrorCode::kInvalidValue, "nodes", "graph has no nodes");
    std::map<std::int64_t, std::size_t> producer;
    std::set<std::int64_t> used;
    for (std::size_t index = 0; index < nodes.size(); ++index) {
        OperationDesc operation;
        auto const path = "nodes[" + std::to_string(index) + "]";
        status = parse_node(nodes[index], path, graph.tensors, operation);
        if (status.is_bad()) return status;
        for (auto const& [port, uid] : operation.inputs) {
            auto const& tensor = graph.tensors.at(uid);
            if (tensor.is_virtual && !producer.count(uid))
                return fail(ErrorCode::kInvalidValue, join(join(path, "inputs"), port), "virtual tensor is consumed before any node produces it");
            used.insert(uid);
        }
        for (auto const& [port, uid] : operation.outputs) {
            if (!producer.emplace(uid, index).second)
                return fail(ErrorCode::kInvalidValue, join(join(path, "outputs"), port), "tensor is produced by more than one node");
            used.insert(uid);
        }
        graph.nodes.push_back(std::move(operation));
    }
    // a ragged tensor's offsets are reached through the tensor that names them, not through a port
    for (auto const& [uid, tensor] : graph.tensors)
        if (tensor.ragged_offset_uid && used.count(uid)) used.insert(*tensor.ragged_offset_uid);
    for (auto const& [uid, tensor] : graph.tensors)
        if (!used.count(uid) && tensor.is_virtual)  // (an external tensor, or an embedded scalar, that no node reads is legal)
            return fail(ErrorCode::kInvalidValue, "tensors." + std::to_string(uid), "virtual tensor is not referenced by any node");

    for (auto field : {"workspace_modifications", "variant_pack_replacements"}) {
        status = expect_empty(root, field);
        if (status.is_bad()) return status;
    }
    // The single-node convolution graph is pinned harder than a DAG, as in the reference: no dynamic
    // shapes, no shape overrides, no Frontend-owned workspace.
    const bool single_conv = graph.nodes.size() == 1 && graph.nodes.front().tag == OperationTag::kConvFprop;
    if (single_conv && graph.tensors.size() != 3) return fail(ErrorCode::kInvalidValue, "tensors", "the single-node convolution graph holds exactly its X, W and Y tensors");
    if (single_conv)  // lib/Import/SerializedGraphImporter.cpp:1667-1672
        for (auto const& [uid, tensor] : graph.tensors)
            if (tensor.is_pass_by_value)
                return fail(ErrorCode::kUnsupportedExecutionMetadata, "tensors." + std::to_string(uid) + ".is_pass_by_value", "the single-node convolution graph does not accept pass-by-value tensors");
    if (single_conv && graph.context.is_dynamic_shape_enabled.value_or(false))
        return fail(ErrorCode::kUnsupportedExecutionMetadata, "context.is_dynamic_shape_enabled", "the single-node convolution graph has static shapes");
    if (single_conv && graph.context.is_override_shape_enabled.value_or(false))
        return fail(ErrorCode::kUnsupportedExecutionMetadata, "context.is_override_shape_enabled", "the single-node convolution graph takes no shape overrides");
    if (single_conv) {  // the Frontend's execution metadata is pinned for the single-node graph only
        for (auto const& [uid, tensor] : graph.tensors) {
            if (tensor.data_type != DataType::kFloat32 && tensor.data_type != DataType::kFloat16 && tensor.data_type != DataType::kBFloat16)
                return fail(ErrorCode::kUnsupportedDataType, "tensors." + std::to_string(uid) + ".data_type", "the single-node convolution graph takes FLOAT, HALF or BFLOAT16 tensors");
            if (tensor.dim.size() < 3 || tensor.dim.size() > 5)  // (the reference's single-node path takes rank 4 only; ranks 3 and 5 run here as well)
                return fail(ErrorCode::kInvalidShape, "tensors." + std::to_string(uid), "the single-node convolution graph requires rank-3 to rank-5 tensors");
            if (tensor.reordering_type != "NONE")
                return fail(ErrorCode::kInvalidLayout, "tensors." + std::to_string(uid) + ".reordering_type", "the single-node convolution graph requires NONE reordering");
        }
        if (auto it = root.find("fe_workspace_size"); it != root.end()) {
            std::int64_t size = 0;
            if (!read_int(*it, size)) return fail(ErrorCode::kInvalidFieldType, "fe_workspace_size", "expected integer");
            if (size != 0) return fail(ErrorCode::kUnsupportedExecutionMetadata, "fe_workspace_size", "a Frontend-owned workspace is not supported");
        }
        if (auto it = root.find("variant_pack_uids"); it != root.end()) {
            std::vector<std::int64_t> listed;
            status = read_int_array(*it, "variant_pack_uids", listed);
            if (status.is_bad()) return status;
            std::set<std::int64_t> expected;
            for (auto const& [uid, tensor] : graph.tensors)
                if (!tensor.is_virtual) expected.insert(uid);
            if (std::set<std::int64_t>(listed.begin(), listed.end()) != expected || listed.size() != expected.size())
                return fail(ErrorCode::kUnsupportedExecutionMetadata, "variant_pack_uids", "does not list exactly the non-virtual tensors");
        }
    }
    return Status::ok();
}

Status decode_json(std::span<std::uint8_t const> bytes, Json& document) {
    document = Json::parse(bytes.begin(), bytes.end(), nullptr, false, false);
    if (document.is_discarded()) return fail(ErrorCode::kParseError, "json", "document is not valid JSON");
    return Status::ok();
}

Status decode_ubjson(std::span<std::uint8_t const> bytes, Json& document) {
    document = Json::from_ubjson(bytes.begin(), bytes.end(), true, false);
    if (document.is_discarded()) return fail(ErrorCode::kParseError, "ubjson", "document is not valid UBJSON");
    // canonical form only: the bytes must be exactly what the default encoder emits
    std::vector<std::uint8_t> canonical = Json::to_ubjson(document);
    if (canonical.size() != bytes.size() || !std::equal(canonical.begin(), canonical.end(), bytes.begin()))
        return fail(ErrorCode::kParseError, "ubjson", "document is not in canonical UBJSON encoding");
    return Status::ok();
}

}  // namespace

std::optional<DataType> data_type_from_name(std::string_view name) noexcept {
    for (auto const& entry : kTypes)
        if (entry.name == name) return entry.type;
    return std::nullopt;
}

std::string_view data_type_name(DataType type) noexcept {
    for (auto const& entry : kTypes)
        if (entry.type == type) return entry.name;
    return "NOT_SET";
}

std::uint32_t data_type_storage_bits(DataType type) noexcept {
    for (auto const& entry : kTypes)
        if (entry.type == type) return entry.bits;
    return 0;
}

std::string_view operation_tag_name(OperationTag tag) noexcept {
    for (auto const& schema : schemas())
        if (schema.tag == tag) return schema.name;
    return "UNKNOWN";
}

bool tensor_storage_bytes(TensorDesc const& tensor, std::uint64_t& bytes) noexcept {
    std::uint64_t span = 0;  // max element offset
    constexpr std::uint64_t limit = static_cast<std::uint64_t>(std::numeric_limits<std::int64_t>::max());
    for (std::size_t axis = 0; axis < tensor.dim.size(); ++axis) {
        if (tensor.dim[axis] <= 0 || tensor.stride[axis] < 0) return false;
        auto extent = static_cast<std::uint64_t>(tensor.dim[axis] - 1);
        auto stride = static_cast<std::uint64_t>(tensor.stride[axis]);
        if (extent != 0 && stride > limit / extent) return false;
        if (span > limit - extent * stride) return false;
        span += extent * stride;
    }
    if (tensor.reordering_type == "F8_128x4") {
        // the reordered layout occupies the full dim product
        std::uint64_t count = 1;
        for (auto d : tensor.dim) count *= static_cast<std::uint64_t>(d);
        span = count - 1;
    }
    std::uint64_t bits = data_type_storage_bits(tensor.data_type);
    if (bits == 0) return false;
    std::uint64_t elements = span + 1;
    if (elements > limit / 8) return false;
    bytes = (elements * bits + 7) / 8;
    return true;
}

OperationDesc const* SerializedGraph::single_conv_fprop() const noexcept {
    if (nodes.size() != 1 || nodes.front().tag != OperationTag::kConvFprop) return nullptr;
    auto const& node = nodes.front();
    auto ones = [&](char const* key) {
        auto it = node.attributes.find(key);
        if (it == node.attributes.end()) return false;
        auto const* values = std::get_if<std::vector<std::int64_t>>(&it->second);
        return values && std::all_of(values->begin(), values->end(), [](std::int64_t v) { return v == 1; });
    };
    auto mode = node.attributes.find("math_mode");
    bool cross = mode != node.attributes.end() && std::get_if<std::string>(&mode->second) && std::get<std::string>(mode->second) == "CROSS_CORRELATION";
    for (auto const& [uid, tensor] : tensors)
        if (tensor.data_type != DataType::kFloat32 || tensor.dim.size() != 4) return nullptr;
    return ones("stride") && ones("dilation") && cross ? &node : nullptr;
}

Status SerializedGraphImporter::parse(std::span<std::uint8_t const> bytes, InputFormat format, SerializedGraph& output) const {
    if (bytes.empty()) return fail(ErrorCode::kInvalidArgument, "input", "serialized Graph is empty");
    if (bytes.size() > kMaximumSerializedGraphBytes) return fail(ErrorCode::kInvalidArgument, "input", "serialized Graph exceeds the 16 MiB input limit");
    if (format != InputFormat::kAuto && format != InputFormat::kJson && format != InputFormat::kUbjson)
        return fail(ErrorCode::kInvalidArgument, "format", "unknown input format");
    Status json_status = Status::ok();
    if (format != InputFormat::kUbjson) {
        Json document;
        json_status = decode_json(bytes, document);
        if (json_status.is_good()) {
            SerializedGraph candidate;
            auto status = validate_document(document, candidate);
            if (status.is_good()) output = std::move(candidate);
            return status;
        }
        if (format == InputFormat::kJson) return json_status;
    }
    Json document;
    auto ubjson_status = decode_ubjson(bytes, document);
    if (ubjson_status.is_bad()) {
        if (format == InputFormat::kUbjson) return ubjson_status;
        return fail(ErrorCode::kParseError, "auto", "neither JSON nor UBJSON decoded (JSON: " + json_status.message() + "; UBJSON: " + ubjson_status.message() + ")");
    }
    SerializedGraph candidate;
    auto status = validate_document(document, candidate);
    if (status.is_good()) output = std::move(candidate);
    return status;
}

Status SerializedGraphImporter::parse_file(std::filesystem::path const& path, InputFormat format, SerializedGraph& output) const {
    std::ifstream stream(path, std::ios::binary);
    if (!stream) return fail(ErrorCode::kIoError, path.string(), "cannot open file");
    std::vector<std::uint8_t> bytes((std::istreambuf_iterator<char>(stream)), std::istreambuf_iterator<char>());
    if (stream.bad()) return fail(ErrorCode::kIoError, path.string(), "read failed");
    return parse(std::span<std::uint8_t const>(bytes), format, output);
}

}  // namespace deepforge::import

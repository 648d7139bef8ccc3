// Thin C face over the REFERENCE importer (compiled from the reference's own sources where they
// lie, never copied): lets the tests feed the same documents to both importers and compare
// accept/reject and error codes. Test infrastructure only; built into oracle/_ref/.
#include "DeepForge/Import/SerializedGraphImporter.h"

#include <cstdint>
#include <cstring>
#include <span>

extern "C" __attribute__((visibility("default"))) int ref_parse(const std::uint8_t* bytes, std::size_t size, int format, std::int64_t* tensors,
                                                                 std::int64_t* nodes, char* message, std::size_t capacity) {
    deepforge::import::SerializedGraph graph;
    deepforge::import::SerializedGraphImporter importer;
    auto chosen = format == 1 ? deepforge::import::InputFormat::kJson
                              : (format == 2 ? deepforge::import::InputFormat::kUbjson : deepforge::import::InputFormat::kAuto);
    auto status = importer.parse(std::span<std::uint8_t const>(bytes, size), chosen, graph);
    if (status.is_good()) {
        if (tensors) *tensors = static_cast<std::int64_t>(graph.tensor_count());
        if (nodes) *nodes = static_cast<std::int64_t>(graph.nodes.size());
    }
    if (message && capacity) {
        std::strncpy(message, status.message().c_str(), capacity - 1);
        message[capacity - 1] = '\0';
    }
    return static_cast<int>(status.code());
}

// ---- canonical text of the parsed model ------------------------------------------------------------
// The same lines df_dump_graph() of the new host library writes for its own model, produced here from the
// REFERENCE's SerializedGraph, so that the two importers can be compared field by field (context, every tensor,
// every node with its ports and attributes), not only by error code.
#include "DeepForge/Import/Capability.h"

#include <cstdio>
#include <string>
#include <type_traits>

namespace {
using namespace deepforge::import;

std::string real_text(double value) {
    char text[40];
    std::snprintf(text, sizeof(text), "%.17g", value);
    return text;
}

std::string value_text(SerializedValue const& value) {
    return std::visit([](auto const& v) -> std::string {
        using T = std::decay_t<decltype(v)>;
        if constexpr (std::is_same_v<T, std::nullptr_t>) return "null";
        else if constexpr (std::is_same_v<T, bool>) return v ? "true" : "false";
        else if constexpr (std::is_same_v<T, std::int64_t> || std::is_same_v<T, std::uint64_t>) return std::to_string(v);
        else if constexpr (std::is_same_v<T, double>) return real_text(v);
        else if constexpr (std::is_same_v<T, std::string>) return "\"" + v + "\"";
        else if constexpr (std::is_same_v<T, SerializedValue::Array>) {
            std::string out = "[";
            for (std::size_t i = 0; i < v.size(); ++i) out += (i ? "," : "") + value_text(v[i]);
            return out + "]";
        } else {
            std::string out = "{";
            bool first = true;
            for (auto const& [key, item] : v) {
                out += (first ? "" : ",") + key + ":" + value_text(item);
                first = false;
            }
            return out + "}";
        }
    }, value.value);
}

std::string list_text(std::vector<std::int64_t> const& values) {
    std::string out = "[";
    for (std::size_t i = 0; i < values.size(); ++i) out += (i ? "," : "") + std::to_string(values[i]);
    return out + "]";
}

template <class Pair>
std::string pair_text(Pair const& values) { return "[" + std::to_string(values[0]) + "," + std::to_string(values[1]) + "]"; }

std::string reference_text(TensorReference const& reference) {
    if (auto const* uid = std::get_if<std::int64_t>(&reference)) return std::to_string(*uid);
    return "\"" + std::get<std::string>(reference) + "\"";
}

std::string dump(SerializedGraph const& graph) {
    std::string out;
    auto type_or_null = [](std::optional<DataType> const& t) { return t ? std::string(data_type_name(*t)) : std::string("null"); };
    auto flag_or_null = [](std::optional<bool> const& f) { return f ? std::string(*f ? "true" : "false") : std::string("null"); };
    out += "context name=" + (graph.context.name ? "\"" + *graph.context.name + "\"" : std::string("null")) + " compute=" + type_or_null(graph.context.compute_data_type) +
           " intermediate=" + type_or_null(graph.context.intermediate_data_type) + " io=" + type_or_null(graph.context.io_data_type) +
           " sm_count=" + (graph.context.sm_count ? std::to_string(*graph.context.sm_count) : std::string("null")) + " dynamic=" + flag_or_null(graph.context.is_dynamic_shape_enabled) +
           " override=" + flag_or_null(graph.context.is_override_shape_enabled) + "\n";
    out += "graph uid=" + std::to_string(graph.graph_uid) + " backend=\"" + graph.cudnn_backend_version + "\"\n";
    for (auto const& [uid, t] : graph.tensors)
        out += "tensor " + std::to_string(uid) + " name=\"" + t.name + "\" type=" + std::string(data_type_name(t.data_type)) + " dim=" + list_text(t.dim) + " stride=" + list_text(t.stride) +
               " virtual=" + (t.is_virtual ? "1" : "0") + " by_value=" + (t.is_pass_by_value ? "1" : "0") + " reorder=" + t.reordering_type + "\n";
    for (auto const& [name, t] : graph.named_tensors) out += "named_tensor \"" + name + "\"\n";
    for (std::size_t i = 0; i < graph.nodes.size(); ++i) {
        auto const& node = graph.nodes[i];
        out += "node " + std::to_string(i) + " tag=" + std::string(operation_tag_name(node.tag)) + " name=\"" + node.name + "\"\n";
        if (auto const* conv = std::get_if<ConvFpropDesc>(&node.attributes)) {
            out += "  conv compute=\"" + std::string(data_type_name(conv->compute_data_type)) + "\" x=" + std::to_string(conv->x_uid) + " w=" + std::to_string(conv->w_uid) +
                   " y=" + std::to_string(conv->y_uid) + " pre=" + pair_text(conv->pre_padding) + " post=" + pair_text(conv->post_padding) + " stride=" + pair_text(conv->stride) +
                   " dilation=" + pair_text(conv->dilation) + "\n";
        } else if (auto const* generic = std::get_if<GenericOperationDesc>(&node.attributes)) {
            for (auto const& [port, reference] : generic->inputs) out += "  in " + port + "=" + reference_text(reference) + "\n";
            for (auto const& [port, references] : generic->input_lists) {
                out += "  in_list " + port + "=[";
                for (std::size_t k = 0; k < references.size(); ++k) out += (k ? "," : "") + reference_text(references[k]);
                out += "]\n";
            }
            for (auto const& [port, reference] : generic->outputs) out += "  out " + port + "=" + reference_text(reference) + "\n";
            for (auto const& [key, value] : generic->attributes) out += "  attr " + key + "=" + value_text(value) + "\n";
        }
    }
    return out;
}
}  // namespace

extern "C" __attribute__((visibility("default"))) int ref_dump(const std::uint8_t* bytes, std::size_t size, int format, char* buffer, std::size_t capacity, std::size_t* length) {
    deepforge::import::SerializedGraph graph;
    deepforge::import::SerializedGraphImporter importer;
    auto chosen = format == 1 ? deepforge::import::InputFormat::kJson
                              : (format == 2 ? deepforge::import::InputFormat::kUbjson : deepforge::import::InputFormat::kAuto);
    auto status = importer.parse(std::span<std::uint8_t const>(bytes, size), chosen, graph);
    if (status.is_bad()) return static_cast<int>(status.code());
    auto const text = dump(graph);
    if (length) *length = text.size();
    if (buffer && capacity) std::memcpy(buffer, text.data(), text.size() < capacity ? text.size() : capacity);
    return 0;
}

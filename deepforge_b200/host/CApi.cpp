// Flat C API (include/deepforge_b200.h) over the C++ host side.
#include "deepforge_b200.h"

#include "DeepForge/Compiler/Artifact.h"
#include "DeepForge/Compiler/Codegen.h"

#include <algorithm>
#include <cstring>
#include <span>

using namespace deepforge;

struct df_executable {
    compiler::CompilationResult result;
};

namespace {
thread_local std::string g_error;

int report(import::Status const& status) {
    if (status.is_bad()) g_error = status.message();
    return static_cast<int>(status.code());
}

import::InputFormat to_format(int format) {
    return format == DF_FORMAT_JSON ? import::InputFormat::kJson : format == DF_FORMAT_UBJSON ? import::InputFormat::kUbjson : import::InputFormat::kAuto;
}
}  // namespace

extern "C" const char* df_last_error(void) { return g_error.c_str(); }

extern "C" int df_parse(const uint8_t* document, size_t size, int format, int64_t* tensor_count, int64_t* node_count) {
    import::SerializedGraph graph;
    import::SerializedGraphImporter importer;
    auto status = importer.parse(std::span<const uint8_t>(document, size), to_format(format), graph);
    if (status.is_good()) {
        if (tensor_count) *tensor_count = static_cast<int64_t>(graph.tensor_count());
        if (node_count) *node_count = static_cast<int64_t>(graph.nodes.size());
    }
    return report(status);
}

namespace {
// Canonical text of a parsed graph. A convolution node the reference's importer turns into its ConvFpropDesc
// (lib/Import/SerializedGraphImporter.cpp:1437-1461: FLOAT compute, ports X, W, Y by UID, two-element integer
// padding / stride / dilation, cross-correlation) is written through the fields that description keeps; every other
// node with all its ports and attributes.
std::string real_text(double value) {
    char text[40];
    std::snprintf(text, sizeof(text), "%.17g", value);
    return text;
}
std::string attribute_text(import::AttributeValue const& value) {
    return std::visit([](auto const& v) -> std::string {
        using T = std::decay_t<decltype(v)>;
        if constexpr (std::is_same_v<T, std::monostate>) return "null";
        else if constexpr (std::is_same_v<T, bool>) return v ? "true" : "false";
        else if constexpr (std::is_same_v<T, std::int64_t>) return std::to_string(v);
        else if constexpr (std::is_same_v<T, double>) return real_text(v);
        else if constexpr (std::is_same_v<T, std::string>) return "\"" + v + "\"";
        else {
            std::string out = "[";
            for (std::size_t i = 0; i < v.size(); ++i) {
                if (i) out += ",";
                if constexpr (std::is_same_v<T, std::vector<std::int64_t>>) out += std::to_string(v[i]);
                else out += real_text(v[i]);
            }
            return out + "]";
        }
    }, value);
}
std::string list_text(std::vector<std::int64_t> const& values) {
    std::string out = "[";
    for (std::size_t i = 0; i < values.size(); ++i) out += (i ? "," : "") + std::to_string(values[i]);
    return out + "]";
}
std::string dump_graph(import::SerializedGraph const& graph) {
    std::string out;
    auto type_or_null = [](std::optional<import::DataType> const& t) { return t ? std::string(import::data_type_name(*t)) : std::string("null"); };
    auto flag_or_null = [](std::optional<bool> const& f) { return f ? std::string(*f ? "true" : "false") : std::string("null"); };
    out += "context name=" + (graph.context.name ? "\"" + *graph.context.name + "\"" : std::string("null")) + " compute=" + type_or_null(graph.context.compute_data_type) +
           " intermediate=" + type_or_null(graph.context.intermediate_data_type) + " io=" + type_or_null(graph.context.io_data_type) +
           " sm_count=" + std::to_string(graph.context.sm_count) + " dynamic=" + flag_or_null(graph.context.is_dynamic_shape_enabled) +
           " override=" + flag_or_null(graph.context.is_override_shape_enabled) + "\n";
    out += "graph uid=" + std::to_string(graph.graph_uid) + " backend=\"" + graph.cudnn_backend_version + "\"\n";
    for (auto const& [uid, t] : graph.tensors)
        out += "tensor " + std::to_string(uid) + " name=\"" + t.name + "\" type=" + std::string(import::data_type_name(t.data_type)) + " dim=" + list_text(t.dim) +
               " stride=" + list_text(t.stride) + " virtual=" + (t.is_virtual ? "1" : "0") + " by_value=" + (t.is_pass_by_value ? "1" : "0") + " reorder=" + t.reordering_type + "\n";
    auto described_as_conv = [](import::OperationDesc const& node) {
        if (node.tag != import::OperationTag::kConvFprop || node.inputs.size() != 2 || node.outputs.size() != 1) return false;
        if (!node.inputs.count("X") || !node.inputs.count("W") || !node.outputs.count("Y")) return false;
        auto find = [&](char const* key) -> import::AttributeValue const* {
            auto it = node.attributes.find(key);
            return it == node.attributes.end() ? nullptr : &it->second;
        };
        auto const* compute = find("compute_data_type");
        auto const* mode = find("math_mode");
        if (!compute || !std::holds_alternative<std::string>(*compute) || std::get<std::string>(*compute) != "FLOAT") return false;
        if (!mode || !std::holds_alternative<std::string>(*mode) || std::get<std::string>(*mode) != "CROSS_CORRELATION") return false;
        for (auto key : {"pre_padding", "post_padding", "stride", "dilation"}) {
            auto const* value = find(key);
            if (!value || !std::holds_alternative<std::vector<std::int64_t>>(*value) || std::get<std::vector<std::int64_t>>(*value).size() != 2) return false;
        }
        return true;
    };
    for (std::size_t i = 0; i < graph.nodes.size(); ++i) {
        auto const& node = graph.nodes[i];
        out += "node " + std::to_string(i) + " tag=" + std::string(import::operation_tag_name(node.tag)) + " name=\"" + node.name + "\"\n";
        if (described_as_conv(node)) {
            auto text = [&](char const* key) {
                auto it = node.attributes.find(key);
                return it == node.attributes.end() ? std::string("?") : attribute_text(it->second);
            };
            out += "  conv compute=" + text("compute_data_type") + " x=" + std::to_string(node.inputs.at("X")) + " w=" + std::to_string(node.inputs.at("W")) +
                   " y=" + std::to_string(node.outputs.at("Y")) + " pre=" + text("pre_padding") + " post=" + text("post_padding") + " stride=" + text("stride") +
                   " dilation=" + text("dilation") + "\n";
            continue;
        }
        for (auto const& [port, uid] : node.inputs) out += "  in " + port + "=" + std::to_string(uid) + "\n";
        for (auto const& [port, uid] : node.outputs) out += "  out " + port + "=" + std::to_string(uid) + "\n";
        for (auto const& [key, value] : node.attributes) out += "  attr " + key + "=" + attribute_text(value) + "\n";
    }
    return out;
}
}  // namespace

extern "C" int df_dump_graph(const uint8_t* document, size_t size, int format, char* buffer, size_t capacity, size_t* length) {
    import::SerializedGraph graph;
    import::SerializedGraphImporter importer;
    auto status = importer.parse(std::span<const uint8_t>(document, size), to_format(format), graph);
    if (status.is_bad()) return report(status);
    auto const text = dump_graph(graph);
    if (length) *length = text.size();
    if (buffer && capacity) std::memcpy(buffer, text.data(), std::min(capacity, text.size()));
    return 0;
}

extern "C" int df_compile(const uint8_t* document, size_t size, int format, uint32_t options, df_executable** out) {
    if (!out) return report(import::Status::failure(import::ErrorCode::kInvalidArgument, "out", "null output pointer"));
    *out = nullptr;
    import::SerializedGraph graph;
    import::SerializedGraphImporter importer;
    auto status = importer.parse(std::span<const uint8_t>(document, size), to_format(format), graph);
    if (status.is_bad()) return report(status);
    compiler::CompileOptions compile_options;
    compile_options.fuse = !(options & DF_OPTION_NO_FUSION);
    compile_options.narrow_virtual_tensors = !(options & DF_OPTION_NO_NARROWING);
    compile_options.disable_tensor_cores = (options & DF_OPTION_NO_TENSOR_CORES) != 0;
    compile_options.bf16_virtual_tensors = (options & DF_OPTION_BF16_INTERMEDIATES) != 0;
    compile_options.fuse_convolution_pairs = !(options & DF_OPTION_NO_CONV_PAIRS);
    auto holder = std::make_unique<df_executable>();
    status = compiler::compile_graph(graph, compile_options, holder->result);
    if (status.is_bad()) return report(status);
    *out = holder.release();
    return 0;
}

extern "C" void df_destroy(df_executable* executable) { delete executable; }

extern "C" int64_t df_workspace_size(const df_executable* executable) { return executable->result.executable->get_workspace_size(); }
extern "C" int64_t df_launch_count(const df_executable* executable) { return executable->result.executable->launch_count(); }

extern "C" size_t df_plan_text(const df_executable* executable, char* buffer, size_t capacity) {
    auto text = executable->result.executable->plan_text();
    if (buffer && capacity) {
        size_t n = std::min(capacity - 1, text.size());
        std::memcpy(buffer, text.data(), n);
        buffer[n] = '\0';
    }
    return text.size();
}

extern "C" int64_t df_argument_count(const df_executable* executable) { return static_cast<int64_t>(executable->result.metadata.arguments.size()); }

extern "C" int df_argument_info(const df_executable* executable, int64_t index, int64_t* uid, uint64_t* size_bytes, uint64_t* alignment, int32_t* access) {
    auto const& arguments = executable->result.metadata.arguments;
    if (index < 0 || index >= static_cast<int64_t>(arguments.size()))
        return report(import::Status::failure(import::ErrorCode::kInvalidArgument, "index", "argument index out of range"));
    auto const& argument = arguments[static_cast<size_t>(index)];
    if (uid) *uid = argument.uid;
    if (size_bytes) *size_bytes = argument.size_bytes;
    if (alignment) *alignment = argument.alignment;
    if (access) *access = static_cast<int32_t>(argument.access);
    return 0;
}

extern "C" size_t df_argument_name(const df_executable* executable, int64_t index, char* buffer, size_t capacity) {
    auto const& arguments = executable->result.metadata.arguments;
    if (index < 0 || index >= static_cast<int64_t>(arguments.size())) return 0;
    auto const& name = arguments[static_cast<size_t>(index)].name;
    if (buffer && capacity) {
        size_t n = std::min(capacity - 1, name.size());
        std::memcpy(buffer, name.data(), n);
        buffer[n] = '\0';
    }
    return name.size();
}

extern "C" int df_conv2d_metadata(const df_executable* executable, int32_t* adapter_kind, int64_t* values) {
    auto const& m = executable->result.metadata;
    if (adapter_kind) *adapter_kind = static_cast<int32_t>(executable->result.adapter_kind);
    if (values) {
        int64_t* out = values;
        *out++ = m.x_uid;
        *out++ = m.w_uid;
        *out++ = m.y_uid;
        for (auto const* shape : {&m.x_shape, &m.w_shape, &m.y_shape, &m.padded_x_shape}) out = std::copy(shape->begin(), shape->end(), out);
        for (auto const* pair : {&m.pre_padding, &m.post_padding, &m.stride, &m.dilation}) out = std::copy(pair->begin(), pair->end(), out);
    }
    return 0;
}

extern "C" void df_set_stream(df_executable* executable, void* stream) { executable->result.executable->set_stream(stream); }

extern "C" int df_execute(const df_executable* executable, void* handle, const int64_t* uids, void* const* pointers, size_t count, void* workspace) {
    runtime::VariantPack pack;
    pack.reserve(count);
    for (size_t i = 0; i < count; ++i) pack[uids[i]] = pointers[i];
    return report(executable->result.executable->execute(handle, pack, workspace));
}

extern "C" int df_execute_on(const df_executable* executable, void* stream, const int64_t* uids, void* const* pointers, size_t count, void* workspace) {
    runtime::VariantPack pack;
    pack.reserve(count);
    for (size_t i = 0; i < count; ++i) pack[uids[i]] = pointers[i];
    return report(executable->result.executable->execute_on(stream, pack, workspace));
}

extern "C" int64_t df_step_count(const df_executable* executable) { return static_cast<int64_t>(executable->result.plan.steps.size()); }

extern "C" int df_step_info(const df_executable* executable, int64_t step, char* label, size_t label_capacity, int32_t* op, int32_t* kernel,
                            int32_t* launches, uint64_t* bound_bytes) {
    auto const& steps = executable->result.plan.steps;
    if (step < 0 || step >= static_cast<int64_t>(steps.size()))
        return report(import::Status::failure(import::ErrorCode::kInvalidArgument, "step", "step index out of range"));
    auto const& s = steps[static_cast<size_t>(step)];
    if (label && label_capacity) {
        size_t n = std::min(label_capacity - 1, s.label.size());
        std::memcpy(label, s.label.data(), n);
        label[n] = '\0';
    }
    if (op) *op = static_cast<int32_t>(s.op);
    if (kernel) *kernel = s.kernel;
    if (launches) *launches = s.launches;
    if (bound_bytes) {
        // bytes of every tensor bound to this launch, each counted once
        uint64_t total = 0;
        std::vector<std::pair<int, int64_t>> seen;
        for (auto const& binding : s.tensors) {
            if (binding.kind == compiler::TensorBinding::Kind::kAbsent) continue;
            std::pair<int, int64_t> key{static_cast<int>(binding.kind), binding.uid};
            if (std::find(seen.begin(), seen.end(), key) != seen.end()) continue;
            seen.push_back(key);
            if (binding.kind == compiler::TensorBinding::Kind::kArgument) {
                for (auto const& argument : executable->result.metadata.arguments)
                    if (argument.uid == binding.uid) total += argument.size_bytes;
            } else {
                for (auto const& allocation : executable->result.workspace.allocations)
                    if (allocation.offset == binding.offset && allocation.name.rfind("scratch.", 0) != 0) { total += allocation.size_bytes; break; }
            }
        }
        *bound_bytes = total;
    }
    return 0;
}

extern "C" int df_execute_steps(const df_executable* executable, int64_t first, int64_t last, const int64_t* uids, void* const* pointers,
                                size_t count, void* workspace) {
    runtime::VariantPack pack;
    pack.reserve(count);
    for (size_t i = 0; i < count; ++i) pack[uids[i]] = pointers[i];
    return report(executable->result.executable->execute_steps(first, last, pack, workspace));
}

extern "C" int df_serialize_artifact(const df_executable* executable, uint8_t* buffer, size_t capacity, size_t* size) {
    std::vector<std::uint8_t> bytes;
    auto status = compiler::serialize_artifact(executable->result, bytes);
    if (status.is_bad()) return report(status);
    if (size) *size = bytes.size();
    if (buffer && capacity) std::memcpy(buffer, bytes.data(), std::min(capacity, bytes.size()));
    return 0;
}

extern "C" int df_write_artifact(const df_executable* executable, const char* path) {
    if (!path) return report(import::Status::failure(import::ErrorCode::kInvalidArgument, "path", "null path"));
    return report(compiler::write_artifact(path, executable->result));
}

namespace {
int adopt(import::Status status, std::unique_ptr<df_executable> holder, compiler::ArtifactInfo& info, df_executable** out) {
    if (status.is_bad()) return report(status);
    holder->result.metadata = std::move(info.metadata);
    holder->result.adapter_kind = info.invocation;
    holder->result.workspace = std::move(info.workspace);
    holder->result.plan = std::move(info.plan);
    holder->result.target_triple = info.target_triple;
    *out = holder.release();
    return 0;
}
}  // namespace

extern "C" int df_load_artifact(const uint8_t* bytes, size_t size, df_executable** out) {
    if (!out || !bytes) return report(import::Status::failure(import::ErrorCode::kInvalidArgument, "out", "null pointer"));
    *out = nullptr;
    auto holder = std::make_unique<df_executable>();
    compiler::ArtifactInfo info;
    auto status = compiler::load_artifact_executable(std::span<const uint8_t>(bytes, size), holder->result.executable, &info);
    return adopt(status, std::move(holder), info, out);
}

extern "C" int df_load_artifact_file(const char* path, df_executable** out) {
    if (!out || !path) return report(import::Status::failure(import::ErrorCode::kInvalidArgument, "out", "null pointer"));
    *out = nullptr;
    auto holder = std::make_unique<df_executable>();
    compiler::ArtifactInfo info;
    auto status = compiler::load_artifact_executable(std::filesystem::path(path), holder->result.executable, &info);
    return adopt(status, std::move(holder), info, out);
}

extern "C" int df_plan_workspace(size_t count, const char* const* names, const uint64_t* sizes, const uint64_t* alignments, const uint64_t* live_starts,
                                 const uint64_t* live_ends, uint64_t* offsets, int64_t* placement_order, uint64_t* total_bytes) {
    std::vector<compiler::WorkspaceRequest> requests(count);
    for (size_t i = 0; i < count; ++i) requests[i] = {names[i], sizes[i], alignments[i], live_starts[i], live_ends[i]};
    compiler::WorkspacePlan plan;
    auto status = compiler::plan_workspace(requests, plan);
    if (status.is_bad()) return report(status);
    for (size_t order = 0; order < plan.allocations.size(); ++order)
        for (size_t i = 0; i < count; ++i)
            if (plan.allocations[order].name == names[i]) {
                offsets[i] = plan.allocations[order].offset;
                if (placement_order) placement_order[i] = static_cast<int64_t>(order);
            }
    if (total_bytes) *total_bytes = plan.size_bytes;
    return 0;
}

// Artifact container: writer, bounds-checked reader and loader (see include/DeepForge/Compiler/Artifact.h).
// Field order of the common part follows the reference's format 12 (docs/artifact-format.en.md:55-123).
#include "DeepForge/Compiler/Artifact.h"

#include "Internal.h"

#include <atomic>
#include <bit>
#include <cstring>
#include <fstream>
#include <map>
#include <set>
#include <variant>
#include <system_error>
#include <unistd.h>

namespace deepforge::compiler {
namespace {

using import::ErrorCode;
using import::Status;

constexpr std::uint8_t kMagic[8] = {'D', 'F', 'O', 'B', 'J', '\r', '\n', 0x1a};
constexpr std::uint32_t kEndianMarker = 0x01020304u;
constexpr char kBackendVersion[] = "deepforge_b200 1";
constexpr char kFrontendVersion[] = "1.24.0";
constexpr char kTarget[] = "sm_100a";
constexpr std::uint64_t kMaxBytes = 1ull << 30;

Status bad(std::string_view detail) { return Status::failure(ErrorCode::kParseError, "artifact", detail); }
Status invalid(std::string_view subject, std::string_view detail) { return Status::failure(ErrorCode::kInvalidValue, subject, detail); }

std::uint64_t fnv1a(std::uint8_t const* data, std::size_t size) {
    std::uint64_t hash = 0xcbf29ce484222325ull;
    for (std::size_t i = 0; i < size; ++i) {
        hash ^= data[i];
        hash *= 0x100000001b3ull;
    }
    return hash;
}

struct Writer {
    std::vector<std::uint8_t> bytes;
    void raw(void const* data, std::size_t size) {
        auto const* p = static_cast<std::uint8_t const*>(data);
        bytes.insert(bytes.end(), p, p + size);
    }
    void u32(std::uint32_t v) {
        for (int i = 0; i < 4; ++i) bytes.push_back(static_cast<std::uint8_t>(v >> (8 * i)));
    }
    void u64(std::uint64_t v) {
        for (int i = 0; i < 8; ++i) bytes.push_back(static_cast<std::uint8_t>(v >> (8 * i)));
    }
    void i64(std::int64_t v) { u64(static_cast<std::uint64_t>(v)); }
    void f64(double v) { u64(std::bit_cast<std::uint64_t>(v)); }
    void string(std::string_view v) {
        u32(static_cast<std::uint32_t>(v.size()));
        raw(v.data(), v.size());
    }
};

// Every read checks the remaining length; after a failed read all further reads fail too.
struct Reader {
    std::uint8_t const* data;
    std::size_t size;
    std::size_t at = 0;
    bool ok = true;
    bool need(std::size_t count) {
        if (!ok || count > size - at) ok = false;
        return ok;
    }
    std::uint32_t u32() {
        if (!need(4)) return 0;
        std::uint32_t v = 0;
        for (int i = 0; i < 4; ++i) v |= static_cast<std::uint32_t>(data[at + i]) << (8 * i);
        at += 4;
        return v;
    }
    std::uint64_t u64() {
        if (!need(8)) return 0;
        std::uint64_t v = 0;
        for (int i = 0; i < 8; ++i) v |= static_cast<std::uint64_t>(data[at + i]) << (8 * i);
        at += 8;
        return v;
    }
    std::int64_t i64() { return static_cast<std::int64_t>(u64()); }
    double f64() { return std::bit_cast<double>(u64()); }
    std::string string() {
        std::uint32_t count = u32();
        if (!need(count)) return {};
        std::string v(reinterpret_cast<char const*>(data + at), count);
        at += count;
        return v;
    }
    void raw(void* out, std::size_t count) {
        if (!need(count)) return;
        std::memcpy(out, data + at, count);
        at += count;
    }
};

template <class T>
constexpr std::uint32_t params_size() { return static_cast<std::uint32_t>(sizeof(T)); }

std::uint32_t params_size_of(KernelOp op) {
    switch (op) {
        case KernelOp::kBlockScaleQuantize: return params_size<dfgpu_bsq_params>();
        case KernelOp::kBlockScaleDequantize: return params_size<dfgpu_bsd_params>();
        case KernelOp::kPointwise: return params_size<dfgpu_pointwise_params>();
        case KernelOp::kConvFprop: return params_size<dfgpu_conv_params>();
        case KernelOp::kMatmul: return params_size<dfgpu_matmul_params>();
        case KernelOp::kSdpaForward: return params_size<dfgpu_sdpa_params>();
        case KernelOp::kMatmulFp8: return params_size<dfgpu_matmul_fp8_params>();
        case KernelOp::kConvFpropPair: return params_size<dfgpu_conv_pair_params>();
        case KernelOp::kBlockScaleQuantizePair: return params_size<dfgpu_bsq_pair_params>();
        case KernelOp::kConstants: return params_size<dfgpu_constants_params>();
    }
    return 0;
}

// Number of tensor slots of each dfgpu entry point (the constants launch: one per constant).
std::size_t tensor_slots(KernelStep const& step) {
    switch (step.op) {
        case KernelOp::kConstants: {
            auto const count = std::get<dfgpu_constants_params>(step.params).count;
            return count > 0 ? static_cast<std::size_t>(count) : 0;
        }
        case KernelOp::kBlockScaleQuantize: return 3;
        case KernelOp::kBlockScaleDequantize: return 3;
        case KernelOp::kPointwise: return 4;
        case KernelOp::kConvFprop: return 5;
        case KernelOp::kMatmul: return 7;
        case KernelOp::kSdpaForward: return 21;
        case KernelOp::kMatmulFp8: return 7;
        case KernelOp::kConvFpropPair: return 8;
        case KernelOp::kBlockScaleQuantizePair: return 6;
    }
    return 0;
}

constexpr std::uint32_t kLastOp = static_cast<std::uint32_t>(KernelOp::kConstants);

void write_binding(Writer& w, TensorBinding const& binding) {
    w.u32(static_cast<std::uint32_t>(binding.kind));
    w.i64(binding.uid);
    w.u64(binding.offset);
}

void write_plan(Writer& w, KernelPlan const& plan) {
    w.u32(static_cast<std::uint32_t>(dfgpu_abi_version()));
    w.u32(static_cast<std::uint32_t>(plan.steps.size()));
    for (auto const& step : plan.steps) {
        w.u32(static_cast<std::uint32_t>(step.op));
        w.string(step.label);
        w.u32(static_cast<std::uint32_t>(step.nodes.size()));
        for (auto node : step.nodes) w.u64(node);
        w.u32(static_cast<std::uint32_t>(step.kernel));
        w.u32(static_cast<std::uint32_t>(step.launches));
        std::visit([&](auto const& params) {
            w.u32(static_cast<std::uint32_t>(sizeof(params)));
            w.raw(&params, sizeof(params));  // POD with explicit reserved fields: no implicit padding
        }, step.params);
        w.u32(static_cast<std::uint32_t>(step.tensors.size()));
        for (auto const& binding : step.tensors) write_binding(w, binding);
        write_binding(w, step.scratch);
    }
}

bool power_of_two(std::uint64_t v) { return v != 0 && (v & (v - 1)) == 0; }

Status check_workspace(WorkspacePlan const& workspace) {
    if (!power_of_two(workspace.alignment) || workspace.alignment > 4096) return invalid("workspace", "alignment must be a power of two up to 4096");
    std::uint64_t top = 0;
    for (auto const& allocation : workspace.allocations) {
        if (!power_of_two(allocation.alignment) || allocation.offset % allocation.alignment != 0) return invalid("workspace", "allocation '" + allocation.name + "' is misaligned");
        if (allocation.size_bytes > kMaxBytes * 256 || allocation.offset > kMaxBytes * 256) return invalid("workspace", "allocation '" + allocation.name + "' is out of range");
        if (allocation.live_start > allocation.live_end) return invalid("workspace", "allocation '" + allocation.name + "' ends before it starts");
        top = std::max(top, allocation.offset + allocation.size_bytes);
    }
    // exactly the 64-byte aligned high-water mark of the plan, as the reference's artifact validator requires
    if (workspace.size_bytes != (top + 63) / 64 * 64) return invalid("workspace", "size is not the aligned high-water mark of its allocations");
    return Status::ok();
}

bool tensor_in_range(dfgpu_tensor const& t) { return t.rank >= 0 && t.rank <= DFGPU_MAX_RANK && t.dtype >= 0 && t.dtype <= DFGPU_BF16X2; }

bool params_in_range(KernelParams const& params) {
    return std::visit([](auto const& p) {
        using T = std::decay_t<decltype(p)>;
        if constexpr (std::is_same_v<T, dfgpu_bsq_params>) return tensor_in_range(p.x) && tensor_in_range(p.y) && tensor_in_range(p.scale);
        else if constexpr (std::is_same_v<T, dfgpu_bsd_params>) return tensor_in_range(p.x) && tensor_in_range(p.y) && tensor_in_range(p.scale);
        else if constexpr (std::is_same_v<T, dfgpu_constants_params>) {
            if (p.count < 1 || p.count > DFGPU_MAX_CONSTANTS) return false;
            for (int i = 0; i < p.count; ++i)
                if (p.bytes[i] != 2 && p.bytes[i] != 4 && p.bytes[i] != 8) return false;
            return true;
        }
        else if constexpr (std::is_same_v<T, dfgpu_pointwise_params>) return tensor_in_range(p.in0) && tensor_in_range(p.in1) && tensor_in_range(p.out) && tensor_in_range(p.in2);
        else if constexpr (std::is_same_v<T, dfgpu_conv_params>)
            return tensor_in_range(p.x) && tensor_in_range(p.w) && tensor_in_range(p.y) && tensor_in_range(p.extra[0]) && tensor_in_range(p.extra[1]) &&
                   p.epilogue_count >= 0 && p.epilogue_count <= DFGPU_MAX_EPILOGUE;
        else if constexpr (std::is_same_v<T, dfgpu_bsq_pair_params>)
            return tensor_in_range(p.first.x) && tensor_in_range(p.first.y) && tensor_in_range(p.first.scale) && tensor_in_range(p.second.x) && tensor_in_range(p.second.y) &&
                   tensor_in_range(p.second.scale);
        else if constexpr (std::is_same_v<T, dfgpu_conv_pair_params>) {
            for (auto const* c : {&p.first, &p.second})
                if (!(tensor_in_range(c->x) && tensor_in_range(c->w) && tensor_in_range(c->y) && tensor_in_range(c->extra[0]) && tensor_in_range(c->extra[1]) &&
                      c->epilogue_count >= 0 && c->epilogue_count <= DFGPU_MAX_EPILOGUE)) return false;
            return true;
        }
        else if constexpr (std::is_same_v<T, dfgpu_matmul_params>)
            return tensor_in_range(p.a) && tensor_in_range(p.b) && tensor_in_range(p.c) && tensor_in_range(p.a_scale) && tensor_in_range(p.b_scale) &&
                   tensor_in_range(p.extra[0]) && tensor_in_range(p.extra[1]) && p.epilogue_count >= 0 && p.epilogue_count <= DFGPU_MAX_EPILOGUE;
        else if constexpr (std::is_same_v<T, dfgpu_sdpa_params>)
            return tensor_in_range(p.q) && tensor_in_range(p.k) && tensor_in_range(p.v) && tensor_in_range(p.o) && tensor_in_range(p.stats) &&
                   tensor_in_range(p.max) && tensor_in_range(p.sum_exp) && tensor_in_range(p.seq_q) && tensor_in_range(p.seq_kv) &&
                   tensor_in_range(p.page_table_k) && tensor_in_range(p.page_table_v) && tensor_in_range(p.bias) && tensor_in_range(p.sink) && tensor_in_range(p.block_mask);
        else return tensor_in_range(p.a) && tensor_in_range(p.b) && tensor_in_range(p.c);
    }, params);
}

template <class T>
KernelParams read_params(Reader& r) {
    T params{};
    r.raw(&params, sizeof(T));
    return params;
}

bool read_binding(Reader& r, TensorBinding& binding) {
    std::uint32_t kind = r.u32();
    binding.uid = r.i64();
    binding.offset = r.u64();
    if (!r.ok || kind > static_cast<std::uint32_t>(TensorBinding::Kind::kWorkspace)) return false;
    binding.kind = static_cast<TensorBinding::Kind>(kind);
    return true;
}

Status read_plan(Reader& r, ArtifactInfo& info) {
    info.kernel_abi_version = static_cast<std::int32_t>(r.u32());
    std::uint32_t count = r.u32();
    if (!r.ok || count == 0 || count > 65536) return bad("kernel plan: launch count out of range");
    for (std::uint32_t s = 0; s < count; ++s) {
        KernelStep step;
        std::uint32_t op = r.u32();
        if (!r.ok || op > kLastOp) return bad("kernel plan: unknown entry point");
        step.op = static_cast<KernelOp>(op);
        step.label = r.string();
        std::uint32_t nodes = r.u32();
        if (!r.ok || nodes > 4096 || !r.need(static_cast<std::size_t>(nodes) * 8)) return bad("kernel plan: node list out of range");
        for (std::uint32_t n = 0; n < nodes; ++n) step.nodes.push_back(static_cast<std::size_t>(r.u64()));
        step.kernel = static_cast<std::int32_t>(r.u32());
        step.launches = static_cast<std::int32_t>(r.u32());
        std::uint32_t size = r.u32();
        if (!r.ok || size != params_size_of(step.op)) return bad("kernel plan: params block has the wrong size for its entry point");
        switch (step.op) {
            case KernelOp::kBlockScaleQuantize: step.params = read_params<dfgpu_bsq_params>(r); break;
            case KernelOp::kBlockScaleDequantize: step.params = read_params<dfgpu_bsd_params>(r); break;
            case KernelOp::kPointwise: step.params = read_params<dfgpu_pointwise_params>(r); break;
            case KernelOp::kConvFprop: step.params = read_params<dfgpu_conv_params>(r); break;
            case KernelOp::kMatmul: step.params = read_params<dfgpu_matmul_params>(r); break;
            case KernelOp::kSdpaForward: step.params = read_params<dfgpu_sdpa_params>(r); break;
            case KernelOp::kMatmulFp8: step.params = read_params<dfgpu_matmul_fp8_params>(r); break;
            case KernelOp::kConvFpropPair: step.params = read_params<dfgpu_conv_pair_params>(r); break;
            case KernelOp::kBlockScaleQuantizePair: step.params = read_params<dfgpu_bsq_pair_params>(r); break;
            case KernelOp::kConstants: step.params = read_params<dfgpu_constants_params>(r); break;
        }
        if (!r.ok || !params_in_range(step.params)) return bad("kernel plan: tensor descriptor out of range");
        if (step.kernel < 0 || step.launches < 1 || step.launches > 16) return bad("kernel plan: kernel id or launch count out of range");
        std::uint32_t tensors = r.u32();
        if (!r.ok || tensors != tensor_slots(step)) return bad("kernel plan: wrong number of tensor bindings for the entry point");
        step.tensors.resize(tensors);
        for (auto& binding : step.tensors)
            if (!read_binding(r, binding)) return bad("kernel plan: tensor binding out of range");
        if (!read_binding(r, step.scratch) || step.scratch.kind == TensorBinding::Kind::kArgument) return bad("kernel plan: scratch binding out of range");
        info.plan.steps.push_back(std::move(step));
    }
    return Status::ok();
}

std::uint64_t element_bytes(int dtype) {
    switch (dtype) {
        case DFGPU_F32: case DFGPU_I32: case DFGPU_BF16X2: return 4;
        case DFGPU_I64: return 8;
        case DFGPU_F16: case DFGPU_BF16: return 2;
        default: return 1;
    }
}

// Bytes from the tensor's base to the end of its last element, the import::tensor_storage_bytes rule applied to a
// kernel descriptor. False on a negative extent or stride, or when the span does not fit.
bool descriptor_span(dfgpu_tensor const& t, std::uint64_t& bytes) {
    constexpr std::uint64_t limit = std::uint64_t{1} << 56;
    std::uint64_t last = 0, count = 1;
    for (int axis = 0; axis < t.rank; ++axis) {
        if (t.dim[axis] <= 0 || t.stride[axis] < 0) return false;
        auto const extent = static_cast<std::uint64_t>(t.dim[axis]), stride = static_cast<std::uint64_t>(t.stride[axis]);
        if (extent > limit || stride > limit || (extent > 1 && stride > limit / (extent - 1))) return false;
        last += (extent - 1) * stride;
        if (last > limit || count > limit / extent) return false;
        count *= extent;
    }
    auto const elements = t.reorder == DFGPU_REORDER_F8_128x4 ? count : last + 1;
    bytes = t.dtype == DFGPU_FP4 || t.dtype == DFGPU_I4 ? (elements + 1) / 2 : elements * element_bytes(t.dtype);   // (two four-bit codes per byte)
    return true;
}

// The descriptor the launch applies to tensor slot `slot`, or null for a slot that carries one FLOAT value
// (MATMUL_FP8's Amax_C and scales).
dfgpu_tensor const* slot_descriptor(KernelStep const& step, std::size_t slot) {
    return std::visit([slot](auto const& p) -> dfgpu_tensor const* {
        using T = std::decay_t<decltype(p)>;
        if constexpr (std::is_same_v<T, dfgpu_bsq_params>) { dfgpu_tensor const* t[] = {&p.x, &p.y, &p.scale}; return slot < 3 ? t[slot] : nullptr; }
        else if constexpr (std::is_same_v<T, dfgpu_bsd_params>) { dfgpu_tensor const* t[] = {&p.x, &p.scale, &p.y}; return slot < 3 ? t[slot] : nullptr; }
        else if constexpr (std::is_same_v<T, dfgpu_constants_params>) return nullptr;
        else if constexpr (std::is_same_v<T, dfgpu_pointwise_params>) { dfgpu_tensor const* t[] = {&p.in0, &p.in1, &p.out, &p.in2}; return slot < 4 ? t[slot] : nullptr; }
        else if constexpr (std::is_same_v<T, dfgpu_conv_params>) { dfgpu_tensor const* t[] = {&p.x, &p.w, &p.y, &p.extra[0], &p.extra[1]}; return slot < 5 ? t[slot] : nullptr; }
        else if constexpr (std::is_same_v<T, dfgpu_matmul_params>) { dfgpu_tensor const* t[] = {&p.a, &p.b, &p.c, &p.a_scale, &p.b_scale, &p.extra[0], &p.extra[1]}; return slot < 7 ? t[slot] : nullptr; }
        else if constexpr (std::is_same_v<T, dfgpu_bsq_pair_params>) {
            dfgpu_tensor const* t[] = {&p.first.x, &p.first.y, &p.first.scale, &p.second.x, &p.second.y, &p.second.scale};
            return slot < 6 ? t[slot] : nullptr;
        }
        else if constexpr (std::is_same_v<T, dfgpu_conv_pair_params>) {
            dfgpu_tensor const* t[] = {&p.first.x, &p.first.w, &p.second.w, &p.second.y, &p.first.extra[0], &p.first.extra[1], &p.second.extra[0], &p.second.extra[1]};
            return slot < 8 ? t[slot] : nullptr;
        }
        else if constexpr (std::is_same_v<T, dfgpu_sdpa_params>) {
            dfgpu_tensor const* t[] = {&p.q, &p.k, &p.v, &p.o, &p.stats, &p.max, &p.sum_exp, &p.seq_q, &p.seq_kv, &p.page_table_k, &p.page_table_v, &p.bias, &p.sink, &p.block_mask,
                                       &p.page_offsets_k, &p.page_offsets_v, &p.dropout_mask, &p.dropout_scale, &p.seed, &p.offset, &p.rng_dump};
            return slot < 21 ? t[slot] : nullptr;
        } else { dfgpu_tensor const* t[] = {&p.a, &p.b, &p.c}; return slot < 3 ? t[slot] : nullptr; }
    }, step.params);
}

// Bindings must name an argument of the table or lie inside the workspace, and what the launch will read or write
// through a binding (the storage span of the descriptor in its params block) must fit the argument's size_bytes or
// the rest of the workspace: a stale or edited artifact must fail here, not write past the caller's buffers.
Status check_bindings(ArtifactInfo const& info) {
    std::map<std::int64_t, std::uint64_t> argument_bytes;
    for (auto const& argument : info.metadata.arguments) argument_bytes[argument.uid] = argument.size_bytes;
    for (auto const& step : info.plan.steps) {
        for (std::size_t slot = 0; slot < step.tensors.size(); ++slot) {
            auto const& binding = step.tensors[slot];
            if (binding.kind == TensorBinding::Kind::kAbsent) continue;
            std::uint64_t span = step.op == KernelOp::kConstants ? 8 : 4;
            if (auto const* descriptor = slot_descriptor(step, slot)) {
                if (descriptor->rank == 0) return bad("kernel plan: '" + step.label + "' binds a tensor its params block marks absent");
                if (!descriptor_span(*descriptor, span)) return bad("kernel plan: '" + step.label + "' has a tensor descriptor without a storage span");
            }
            if (binding.kind == TensorBinding::Kind::kArgument) {
                auto it = argument_bytes.find(binding.uid);
                if (it == argument_bytes.end()) return bad("kernel plan: '" + step.label + "' binds a tensor that is neither an argument nor inside the workspace");
                if (span > it->second) return bad("kernel plan: '" + step.label + "' reads or writes past the end of argument " + std::to_string(binding.uid));
            } else {
                if (binding.offset >= info.workspace.size_bytes || binding.offset % 16 != 0)
                    return bad("kernel plan: '" + step.label + "' binds a tensor that is neither an argument nor inside the workspace");
                if (span > info.workspace.size_bytes - binding.offset) return bad("kernel plan: '" + step.label + "' reads or writes past the end of the workspace");
            }
        }
        if (step.scratch.kind == TensorBinding::Kind::kWorkspace && (step.scratch.offset >= info.workspace.size_bytes || step.scratch.offset % 16 != 0))
            return bad("kernel plan: '" + step.label + "' has its scratch outside the workspace");
    }
    return Status::ok();
}

// The single-node convolution form is recognisable from the table (exactly X, W, Y, rank-4 FLOAT, one CONV_FPROP
// launch): rebuild the fields compile_graph derived, so that a loaded artifact describes itself like a compiled one.
void restore_conv_metadata(ArtifactInfo& info) {
    auto const& arguments = info.metadata.arguments;
    if (arguments.size() != 3 || info.plan.steps.size() != 1 || info.plan.steps[0].op != KernelOp::kConvFprop) return;
    if (arguments[0].name != "X" || arguments[1].name != "W" || arguments[2].name != "Y") return;
    for (auto const& argument : arguments)
        if (argument.data_type != import::DataType::kFloat32 || argument.dimensions.size() != 4) return;
    auto const& params = std::get<dfgpu_conv_params>(info.plan.steps[0].params);
    auto& m = info.metadata;
    m.x_uid = arguments[0].uid;
    m.w_uid = arguments[1].uid;
    m.y_uid = arguments[2].uid;
    std::copy(arguments[0].dimensions.begin(), arguments[0].dimensions.end(), m.x_shape.begin());
    std::copy(arguments[1].dimensions.begin(), arguments[1].dimensions.end(), m.w_shape.begin());
    std::copy(arguments[2].dimensions.begin(), arguments[2].dimensions.end(), m.y_shape.begin());
    m.padded_x_shape = m.x_shape;
    m.padded_x_shape[1] += params.pre_pad[0] + params.post_pad[0];
    m.padded_x_shape[2] += params.pre_pad[1] + params.post_pad[1];
    for (int i = 0; i < 2; ++i) {
        m.pre_padding[i] = params.pre_pad[i];
        m.post_padding[i] = params.post_pad[i];
        m.stride[i] = params.stride[i];
        m.dilation[i] = params.dilation[i];
    }
    if (validate_conv2d_adapter_metadata(m).is_good()) info.invocation = InvocationAdapterKind::kConv2DRankedMemref;
}

std::atomic<std::uint64_t> g_publish_sequence{0};

Status read_file(std::filesystem::path const& path, std::vector<std::uint8_t>& bytes) {
    std::ifstream file(path, std::ios::binary | std::ios::ate);
    if (!file) return Status::failure(ErrorCode::kIoError, path.string(), "cannot open the artifact");
    auto const size = file.tellg();
    if (size < 0 || static_cast<std::uint64_t>(size) > kMaxBytes) return Status::failure(ErrorCode::kIoError, path.string(), "artifact size out of range");
    bytes.resize(static_cast<std::size_t>(size));
    file.seekg(0);
    if (!bytes.empty() && !file.read(reinterpret_cast<char*>(bytes.data()), size)) return Status::failure(ErrorCode::kIoError, path.string(), "short read");
    return Status::ok();
}

}  // namespace

Status serialize_artifact(CompilationResult const& compilation, std::vector<std::uint8_t>& output) {
    if (compilation.metadata.arguments.empty()) return invalid("arguments", "an artifact needs a non-empty argument table");
    auto status = validate_graph_compile_metadata(compilation.metadata);
    if (status.is_bad()) return Status::failure(ErrorCode::kInvalidValue, "arguments", status.message());
    if ((status = check_workspace(compilation.workspace)).is_bad()) return status;
    if (compilation.plan.steps.empty()) return invalid("plan", "an artifact needs at least one launch");
    for (auto const& step : compilation.plan.steps)
        if (step.tensors.size() != tensor_slots(step)) return invalid("plan", "launch '" + step.label + "' has the wrong number of tensor bindings");

    Writer w;
    w.raw(kMagic, sizeof(kMagic));
    w.u32(kArtifactFormatVersion);
    w.u32(kEndianMarker);
    w.string(kBackendVersion);
    w.string("");  // llvm_version: none
    w.string(kFrontendVersion);
    w.string(compilation.target_triple);
    w.string(compilation.metadata.function_name);
    w.u32(0);  // dynamic_shape_enabled
    w.u32(0);  // override_shape_enabled
    w.u32(0);  // shape_override_policy: none
    w.u32(0);  // override_role_count
    w.u32(0);  // override_axis_count
    w.u32(static_cast<std::uint32_t>(compilation.metadata.arguments.size()));
    for (auto const& argument : compilation.metadata.arguments) {
        w.i64(argument.uid);
        w.string(argument.name);
        w.u32(static_cast<std::uint32_t>(argument.data_type));
        w.u32(static_cast<std::uint32_t>(argument.access));
        w.u32(static_cast<std::uint32_t>(argument.storage_policy));  // strided, or the ragged batch prefix of a compact page table
        w.i64(argument.ragged_offset_uid);
        w.i64(argument.ragged_sequence_uid);
        w.i64(argument.ragged_sequence_divisor);
        w.u64(argument.alignment);
        w.u64(argument.size_bytes);
        w.u32(static_cast<std::uint32_t>(argument.dimensions.size()));
        for (auto extent : argument.dimensions) w.i64(extent);
        for (auto stride : argument.strides) w.i64(stride);
    }
    w.u32(static_cast<std::uint32_t>(ArtifactAdapterKind::kGpuKernelPlan));
    Writer plan;
    write_plan(plan, compilation.plan);
    w.u64(plan.bytes.size());
    w.raw(plan.bytes.data(), plan.bytes.size());
    w.u64(compilation.workspace.size_bytes);
    w.u64(compilation.workspace.alignment);
    w.u32(static_cast<std::uint32_t>(compilation.workspace.allocations.size()));
    for (auto const& allocation : compilation.workspace.allocations) {
        w.string(allocation.name);
        w.u64(allocation.offset);
        w.u64(allocation.size_bytes);
        w.u64(allocation.alignment);
        w.u64(allocation.live_start);
        w.u64(allocation.live_end);
    }
    w.f64(kDefaultAbsoluteTolerance);
    w.f64(kDefaultRelativeTolerance);
    w.u32(0);  // variant_count: the code is in the kernel library
    w.u64(fnv1a(w.bytes.data(), w.bytes.size()));
    output = std::move(w.bytes);
    return Status::ok();
}

Status parse_artifact(std::span<std::uint8_t const> input, ArtifactInfo& output) {
    if (input.size() < sizeof(kMagic) + 8 + 8) return bad("shorter than the fixed header and checksum");
    if (input.size() > kMaxBytes) return bad("larger than 1 GiB");
    if (std::memcmp(input.data(), kMagic, sizeof(kMagic)) != 0) return bad("magic bytes do not match");
    Reader r{input.data(), input.size() - 8};  // everything before the checksum
    r.at = sizeof(kMagic);
    ArtifactInfo info;
    info.format_version = r.u32();
    if (r.u32() != kEndianMarker) return bad("endian marker does not match");
    if (info.format_version >= 1 && info.format_version <= kReferenceArtifactFormatVersion)
        return bad("format " + std::to_string(info.format_version) + " holds x86 objects; this backend loads format " + std::to_string(kArtifactFormatVersion));
    if (info.format_version != kArtifactFormatVersion) return bad("unknown format version " + std::to_string(info.format_version));
    {
        Reader tail{input.data(), input.size()};
        tail.at = input.size() - 8;
        if (tail.u64() != fnv1a(input.data(), input.size() - 8)) return bad("checksum does not match");
    }
    info.deepforge_version = r.string();
    info.llvm_version = r.string();
    info.frontend_version = r.string();
    info.target_triple = r.string();
    info.metadata.function_name = r.string();
    std::uint32_t dynamic_shape = r.u32(), override_shape = r.u32(), policy = r.u32(), roles = r.u32(), axes = r.u32();
    if (!r.ok) return bad("truncated header");
    if (dynamic_shape > 1 || override_shape > 1) return bad("a boolean flag holds neither 0 nor 1");
    if (dynamic_shape || override_shape || policy != 0 || roles != 0 || axes != 0) return bad("shape-override metadata is not executable on this backend");
    std::uint32_t arguments = r.u32();
    if (!r.ok || arguments == 0 || arguments > 4096) return bad("argument count out of range");
    for (std::uint32_t i = 0; i < arguments; ++i) {
        TensorArgumentMetadata argument;
        argument.uid = r.i64();
        argument.name = r.string();
        std::uint32_t data_type = r.u32(), access = r.u32(), storage_policy = r.u32();
        std::int64_t ragged_offset = r.i64(), ragged_sequence = r.i64(), divisor = r.i64();
        argument.alignment = r.u64();
        argument.size_bytes = r.u64();
        std::uint32_t rank = r.u32();
        if (!r.ok) return bad("truncated argument table");
        if (data_type > static_cast<std::uint32_t>(import::DataType::kInt4)) return bad("argument '" + argument.name + "': unknown data type");
        if (access > static_cast<std::uint32_t>(TensorAccess::kReadWrite)) return bad("argument '" + argument.name + "': unknown access");
        if (storage_policy > static_cast<std::uint32_t>(TensorStoragePolicy::kRaggedBatchPrefix)) return bad("argument '" + argument.name + "': unknown storage policy");
        if (storage_policy == 0 && (ragged_offset != 0 || ragged_sequence != 0 || divisor != 1)) return bad("argument '" + argument.name + "': a strided argument carries no ragged references");
        if (storage_policy != 0 && divisor < 1) return bad("argument '" + argument.name + "': ragged sequence divisor must be positive");
        argument.storage_policy = static_cast<TensorStoragePolicy>(storage_policy);
        argument.ragged_offset_uid = ragged_offset;
        argument.ragged_sequence_uid = ragged_sequence;
        argument.ragged_sequence_divisor = divisor;
        if (rank < 1 || rank > 64 || !r.need(static_cast<std::size_t>(rank) * 16)) return bad("argument '" + argument.name + "': rank out of range");
        argument.data_type = static_cast<import::DataType>(data_type);
        argument.access = static_cast<TensorAccess>(access);
        for (std::uint32_t axis = 0; axis < rank; ++axis) argument.dimensions.push_back(r.i64());
        for (std::uint32_t axis = 0; axis < rank; ++axis) argument.strides.push_back(r.i64());
        info.metadata.arguments.push_back(std::move(argument));
    }
    if (auto status = validate_graph_compile_metadata(info.metadata); status.is_bad()) return bad("argument table: " + status.message());
    std::uint32_t adapter = r.u32();
    std::uint64_t adapter_size = r.u64();
    if (!r.ok) return bad("truncated adapter header");
    if (adapter != static_cast<std::uint32_t>(ArtifactAdapterKind::kGpuKernelPlan)) return bad("adapter kind " + std::to_string(adapter) + " is a CPU invocation adapter");
    if (!r.need(adapter_size)) return bad("adapter section runs past the end");
    {
        Reader plan{input.data() + r.at, static_cast<std::size_t>(adapter_size)};
        if (auto status = read_plan(plan, info); status.is_bad()) return status;
        if (!plan.ok || plan.at != plan.size) return bad("kernel plan does not fill its section");
        r.at += static_cast<std::size_t>(adapter_size);
    }
    info.adapter_kind = ArtifactAdapterKind::kGpuKernelPlan;
    info.workspace.size_bytes = r.u64();
    info.workspace.alignment = r.u64();
    std::uint32_t allocations = r.u32();
    if (!r.ok || allocations > 65536) return bad("workspace allocation count out of range");
    for (std::uint32_t i = 0; i < allocations; ++i) {
        WorkspaceAllocation allocation;
        allocation.name = r.string();
        allocation.offset = r.u64();
        allocation.size_bytes = r.u64();
        allocation.alignment = r.u64();
        allocation.live_start = r.u64();
        allocation.live_end = r.u64();
        if (!r.ok) return bad("truncated workspace plan");
        info.workspace.allocations.push_back(std::move(allocation));
    }
    if (auto status = check_workspace(info.workspace); status.is_bad()) return bad("workspace plan: " + status.message());
    info.absolute_tolerance = r.f64();
    info.relative_tolerance = r.f64();
    std::uint32_t variants = r.u32();
    if (!r.ok) return bad("truncated tail");
    if (variants != 0) return bad("a kernel-plan artifact carries no code variants");
    if (r.at != r.size) return bad("bytes between the last field and the checksum");
    if (auto status = check_bindings(info); status.is_bad()) return status;
    restore_conv_metadata(info);
    output = std::move(info);
    return Status::ok();
}

Status write_artifact(std::filesystem::path const& path, CompilationResult const& compilation) {
    std::vector<std::uint8_t> bytes;
    auto status = serialize_artifact(compilation, bytes);
    if (status.is_bad()) return status;
    auto temporary = path;
    temporary += ".tmp." + std::to_string(static_cast<long long>(::getpid())) + "." + std::to_string(g_publish_sequence.fetch_add(1));
    {
        std::ofstream file(temporary, std::ios::binary | std::ios::trunc);
        if (!file) return Status::failure(ErrorCode::kIoError, temporary.string(), "cannot create the temporary file");
        file.write(reinterpret_cast<char const*>(bytes.data()), static_cast<std::streamsize>(bytes.size()));
        file.flush();
        if (!file) {
            std::error_code ignored;
            std::filesystem::remove(temporary, ignored);
            return Status::failure(ErrorCode::kIoError, temporary.string(), "short write");
        }
    }
    std::error_code error;
    std::filesystem::rename(temporary, path, error);
    if (error) {
        std::error_code ignored;
        std::filesystem::remove(temporary, ignored);
        return Status::failure(ErrorCode::kIoError, path.string(), "cannot publish the artifact: " + error.message());
    }
    return Status::ok();
}

Status read_artifact(std::filesystem::path const& path, ArtifactInfo& output) {
    std::vector<std::uint8_t> bytes;
    auto status = read_file(path, bytes);
    if (status.is_bad()) return status;
    return parse_artifact(bytes, output);
}

Status load_artifact_executable(std::span<std::uint8_t const> input, std::unique_ptr<runtime::Executable>& output, ArtifactInfo* info) {
    ArtifactInfo parsed;
    auto status = parse_artifact(input, parsed);
    if (status.is_bad()) return status;
    if (parsed.kernel_abi_version != dfgpu_abi_version())
        return Status::failure(ErrorCode::kInvalidValue, "artifact", "built against kernel ABI " + std::to_string(parsed.kernel_abi_version) + ", this library is ABI " +
                                                                         std::to_string(dfgpu_abi_version()) + ": recompile the graph");
    for (auto const& step : parsed.plan.steps) {
        KernelStep probe = step;
        std::int64_t scratch = 0;
        if ((status = query_kernel_step(probe, scratch)).is_bad())
            return Status::failure(ErrorCode::kInvalidValue, "artifact", "the kernel library rejects launch '" + step.label + "': " + status.message());
        if (probe.kernel != step.kernel || probe.launches != step.launches)
            return Status::failure(ErrorCode::kInvalidValue, "artifact", "launch '" + step.label + "' resolves to another kernel in this library: recompile the graph");
        if (scratch > 0) {
            if (step.scratch.kind != TensorBinding::Kind::kWorkspace || step.scratch.offset + static_cast<std::uint64_t>(scratch) > parsed.workspace.size_bytes)
                return Status::failure(ErrorCode::kInvalidValue, "artifact", "launch '" + step.label + "' needs " + std::to_string(scratch) + " bytes of scratch that the workspace plan does not hold");
        }
    }
    output = runtime::ExecutableFactory::create(parsed.metadata, parsed.workspace, parsed.plan);
    if (info) *info = std::move(parsed);
    return Status::ok();
}

Status load_artifact_executable(std::filesystem::path const& path, std::unique_ptr<runtime::Executable>& output, ArtifactInfo* info) {
    std::vector<std::uint8_t> bytes;
    auto status = read_file(path, bytes);
    if (status.is_bad()) return status;
    return load_artifact_executable(bytes, output, info);
}

}  // namespace deepforge::compiler

// compile_graph: graph analysis, GPU kernel selection and workspace planning.
//
// Takes the place of the reference's compile_graph (lib/Compiler/Compiler.cpp:367) for
// the hot-path tags: where the reference builds an MLIR module and emits x86 objects,
// this lowers each node (or fused group of nodes) to one launch through the dfgpu C
// ABI. The analysis keeps the reference's contract (lib/Compiler/FoundationalGraph.cpp
// :1705-2136): argument table in ascending UID order, alignment = clamp(element bytes,
// 1, 8), size_bytes = storage span, one workspace request per materialised virtual
// tensor with lifetime [producer, last consumer].
#include "DeepForge/Compiler/Codegen.h"

#include "Internal.h"

#include <algorithm>
#include <array>
#include <bit>
#include <cfloat>
#include <cmath>
#include <map>
#include <optional>
#include <set>
#include <sstream>

namespace deepforge::compiler {
namespace {

using import::AttributeValue;
using import::DataType;
using import::ErrorCode;
using import::OperationDesc;
using import::OperationTag;
using import::SerializedGraph;
using import::Status;
using import::TensorDesc;

Status fail(ErrorCode code, std::string_view subject, std::string_view detail) { return Status::failure(code, subject, detail); }

// ---- attribute access ------------------------------------------------------------------

AttributeValue const* attribute(OperationDesc const& node, char const* key) {
    auto it = node.attributes.find(key);
    return it == node.attributes.end() ? nullptr : &it->second;
}
bool is_null(OperationDesc const& node, char const* key) {
    auto const* value = attribute(node, key);
    return value == nullptr || std::holds_alternative<std::monostate>(*value);
}
std::optional<std::int64_t> get_int(OperationDesc const& node, char const* key) {
    auto const* value = attribute(node, key);
    if (value && std::holds_alternative<std::int64_t>(*value)) return std::get<std::int64_t>(*value);
    return std::nullopt;
}
std::optional<double> get_number(OperationDesc const& node, char const* key) {
    auto const* value = attribute(node, key);
    if (!value) return std::nullopt;
    if (std::holds_alternative<std::int64_t>(*value)) return static_cast<double>(std::get<std::int64_t>(*value));
    if (std::holds_alternative<double>(*value)) return std::get<double>(*value);
    return std::nullopt;
}
std::optional<bool> get_bool(OperationDesc const& node, char const* key) {
    auto const* value = attribute(node, key);
    if (value && std::holds_alternative<bool>(*value)) return std::get<bool>(*value);
    return std::nullopt;
}
std::optional<std::string> get_string(OperationDesc const& node, char const* key) {
    auto const* value = attribute(node, key);
    if (value && std::holds_alternative<std::string>(*value)) return std::get<std::string>(*value);
    return std::nullopt;
}
std::optional<std::vector<std::int64_t>> get_int_array(OperationDesc const& node, char const* key) {
    auto const* value = attribute(node, key);
    if (value && std::holds_alternative<std::vector<std::int64_t>>(*value)) return std::get<std::vector<std::int64_t>>(*value);
    return std::nullopt;
}

std::optional<std::int64_t> port(std::map<std::string, std::int64_t> const& ports, char const* name) {
    auto it = ports.find(name);
    if (it == ports.end()) return std::nullopt;
    return it->second;
}

// ---- tensors -----------------------------------------------------------------------------

std::optional<int> to_dfgpu_dtype(DataType type) {
    switch (type) {
        case DataType::kFloat32: return DFGPU_F32;
        case DataType::kFloat16: return DFGPU_F16;
        case DataType::kBFloat16: return DFGPU_BF16;
        case DataType::kFp8E4M3: return DFGPU_E4M3;
        case DataType::kFp8E8M0: return DFGPU_E8M0;
        case DataType::kInt32: return DFGPU_I32;
        case DataType::kFp8E5M2: return DFGPU_E5M2;
        case DataType::kUint8: return DFGPU_U8;
        case DataType::kInt64: return DFGPU_I64;
        case DataType::kFp4E2M1: return DFGPU_FP4;
        case DataType::kInt4: return DFGPU_I4;
        default: return std::nullopt;
    }
}

struct Lowering {
    SerializedGraph const& graph;
    CompileOptions const& options;
    std::map<std::int64_t, int> producer;                       // uid -> node index
    std::map<std::int64_t, std::vector<std::size_t>> consumers;  // uid -> node indices
    std::map<std::int64_t, int> storage_override;                // virtual uid -> dfgpu dtype
    std::vector<int> absorbed_into;                              // node -> anchor node, or -1
    KernelPlan plan;

    explicit Lowering(SerializedGraph const& g, CompileOptions const& o) : graph(g), options(o), absorbed_into(g.nodes.size(), -1) {}

    TensorDesc const& tensor(std::int64_t uid) const { return graph.tensors.at(uid); }

    // FP8_E5M2 is executable as a MATMUL_FP8 operand or output and as the codes of BLOCK_SCALE_QUANTIZE / DEQUANTIZE,
    // UINT8 as the SDPA block mask only.
    // allow_special: the port takes the types only some ports execute (FP8_E5M2, UINT8, INT64) and ragged storage
    Status describe(std::int64_t uid, dfgpu_tensor& out, std::string const& where, bool allow_special = false) const {
        auto const& t = tensor(uid);
        auto dtype = to_dfgpu_dtype(t.data_type);
        if (dtype && (*dtype == DFGPU_E5M2 || *dtype == DFGPU_U8 || *dtype == DFGPU_I64 || *dtype == DFGPU_FP4 || *dtype == DFGPU_I4) && !allow_special) dtype.reset();
        if (t.ragged_offset_uid && !allow_special)
            return fail(ErrorCode::kUnsupportedOperation, where, "tensor '" + t.name + "' uses ragged storage, which this backend executes for SDPA page tables only");
        if (t.reordering_type != "NONE" && t.reordering_type != "F8_128x4")
            return fail(ErrorCode::kUnsupportedOperation, where, "tensor '" + t.name + "' uses reordering " + t.reordering_type + ", which this backend does not execute");
        if (!dtype) return fail(ErrorCode::kUnsupportedDataType, where, "tensor '" + t.name + "' has data type " + std::string(import::data_type_name(t.data_type)) + ", which this backend does not execute");
        if (t.dim.size() > DFGPU_MAX_RANK) return fail(ErrorCode::kInvalidShape, where, "tensor rank above 8");
        out = dfgpu_tensor{};
        auto narrowed = storage_override.find(uid);
        out.dtype = narrowed != storage_override.end() ? narrowed->second : *dtype;
        out.rank = static_cast<std::int32_t>(t.dim.size());
        out.reorder = t.reordering_type == "F8_128x4" ? DFGPU_REORDER_F8_128x4 : DFGPU_REORDER_NONE;
        for (std::size_t i = 0; i < t.dim.size(); ++i) {
            out.dim[i] = t.dim[i];
            out.stride[i] = t.stride[i];
        }
        return Status::ok();
    }

    TensorBinding bind(std::int64_t uid) const {
        TensorBinding binding;
        // a virtual tensor and a graph-owned constant both live in the workspace; everything else is the caller's
        binding.kind = tensor(uid).is_virtual || tensor(uid).pass_by_value ? TensorBinding::Kind::kWorkspace : TensorBinding::Kind::kArgument;
        binding.uid = uid;
        return binding;
    }

    bool single_consumer(std::int64_t uid, std::size_t& node) const {
        auto it = consumers.find(uid);
        if (it == consumers.end() || it->second.size() != 1) return false;
        node = it->second.front();
        return true;
    }

    // Is `uid` ready before node `anchor` runs (a graph input, or written by an earlier node)?
    bool available_before(std::int64_t uid, std::size_t anchor) const {
        auto it = producer.find(uid);
        return it == producer.end() || static_cast<std::size_t>(it->second) < anchor;
    }
};

std::string node_path(std::size_t index, OperationDesc const& node) {
    return "nodes[" + std::to_string(index) + "] " + std::string(import::operation_tag_name(node.tag)) + " '" + node.name + "'";
}

Status require_float_compute(OperationDesc const& node, std::string const& where) {
    auto compute = get_string(node, "compute_data_type");
    if (!compute || *compute != "FLOAT") return fail(ErrorCode::kUnsupportedOperation, where, "compute_data_type must be FLOAT");
    return Status::ok();
}

// The reference's mode names (lib/Import/Schema.cpp:301-316) in the order of DFGPU_PW_*.
constexpr std::array<std::string_view, DFGPU_PW_MODE_COUNT> kPointwiseModeNames{{
    "ADD", "RELU_FWD", "IDENTITY", "MUL", "SUB", "DIV", "ADD_SQUARE", "MIN", "MAX", "MOD", "POW", "SQRT", "RSQRT", "EXP",
    "LOG", "NEG", "ABS", "CEIL", "FLOOR", "COS", "SIN", "TAN", "ERF", "RECIPROCAL", "GEN_INDEX", "LOGICAL_NOT",
    "LOGICAL_AND", "LOGICAL_OR", "BINARY_SELECT", "CMP_EQ", "CMP_NEQ", "CMP_GT", "CMP_GE", "CMP_LT", "CMP_LE", "RELU_BWD",
    "TANH_FWD", "TANH_BWD", "SIGMOID_FWD", "SIGMOID_BWD", "ELU_FWD", "ELU_BWD", "SOFTPLUS_FWD", "SOFTPLUS_BWD",
    "SWISH_FWD", "SWISH_BWD", "GELU_FWD", "GELU_BWD", "GELU_APPROX_TANH_FWD", "GELU_APPROX_TANH_BWD"}};

// POINTWISE node -> mode and scalar attributes (validate_pointwise, lib/Compiler/FoundationalGraph.cpp:721-775: every
// numeric attribute null or a finite f32, lower clip <= upper clip, softplus beta > 0, GEN_INDEX with an axis).
Status pointwise_mode(OperationDesc const& node, std::string const& where, dfgpu_pointwise_params& params) {
    auto name = get_string(node, "mode");
    if (!name) return fail(ErrorCode::kInvalidValue, where, "mode must be a string");
    auto found = std::find(kPointwiseModeNames.begin(), kPointwiseModeNames.end(), std::string_view(*name));
    if (found == kPointwiseModeNames.end()) return fail(ErrorCode::kInvalidValue, where, "pointwise mode " + *name + " is not a mode of the schema");
    params.mode = static_cast<std::int32_t>(found - kPointwiseModeNames.begin());
    struct Attribute { char const* key; float* target; double fallback; };
    Attribute const attributes[] = {{"relu_lower_clip", &params.relu_lower, 0.0}, {"relu_upper_clip", &params.relu_upper, static_cast<double>(FLT_MAX)},
                                    {"relu_lower_clip_slope", &params.relu_slope, 0.0}, {"elu_alpha", &params.elu_alpha, 1.0},
                                    {"softplus_beta", &params.softplus_beta, 1.0}, {"swish_beta", &params.swish_beta, 1.0}};
    for (auto const& attribute : attributes) {
        auto value = get_number(node, attribute.key);
        if (!value && !is_null(node, attribute.key)) return fail(ErrorCode::kInvalidValue, where, std::string(attribute.key) + " must be a number or null");
        if (value && (!std::isfinite(*value) || std::fabs(*value) > static_cast<double>(FLT_MAX)))
            return fail(ErrorCode::kInvalidValue, where, std::string(attribute.key) + " must fit a finite f32");
        *attribute.target = static_cast<float>(value.value_or(attribute.fallback));
    }
    if (get_number(node, "relu_lower_clip") && get_number(node, "relu_upper_clip") && *get_number(node, "relu_lower_clip") > *get_number(node, "relu_upper_clip"))
        return fail(ErrorCode::kInvalidValue, where, "ReLU lower clip exceeds upper clip");
    if (auto beta = get_number(node, "softplus_beta"); beta && *beta <= 0.0) return fail(ErrorCode::kInvalidValue, where, "softplus beta must be positive");
    auto axis = get_int(node, "axis");
    if (!axis && !is_null(node, "axis")) return fail(ErrorCode::kInvalidValue, where, "axis must be an integer or null");
    params.axis = static_cast<std::int32_t>(axis.value_or(0));
    if (params.mode == DFGPU_PW_GEN_INDEX && !axis) return fail(ErrorCode::kInvalidValue, where, "GEN_INDEX requires an axis in the output rank");
    return Status::ok();
}

bool broadcasts_onto(TensorDesc const& small, TensorDesc const& big) {
    if (small.dim.size() > big.dim.size()) return false;
    std::size_t shift = big.dim.size() - small.dim.size();
    for (std::size_t i = 0; i < small.dim.size(); ++i)
        if (small.dim[i] != 1 && small.dim[i] != big.dim[i + shift]) return false;
    return true;
}

// Walk the chain of single-consumer POINTWISE nodes hanging off `value` and absorb ADD /
// RELU_FWD steps into the contraction at `anchor`. Returns the UID finally written.
Status absorb_epilogue(Lowering& low, std::size_t anchor, std::int64_t value, dfgpu_epilogue_step* steps, std::int32_t& count,
                       dfgpu_tensor* extra, std::vector<std::int64_t>& extra_uids, std::vector<std::size_t>& nodes, std::string& label,
                       std::int64_t& final_uid) {
    final_uid = value;
    count = 0;
    if (!low.options.fuse) return Status::ok();
    for (;;) {
        auto const& current = low.tensor(final_uid);
        std::size_t next = 0;
        if (!current.is_virtual || !low.single_consumer(final_uid, next) || count >= DFGPU_MAX_EPILOGUE) break;
        auto const& node = low.graph.nodes[next];
        if (node.tag != OperationTag::kPointwise || low.absorbed_into[next] >= 0) break;
        dfgpu_pointwise_params described_mode{};
        if (pointwise_mode(node, "", described_mode).is_bad()) break;
        int const mode = described_mode.mode;
        float const lower = described_mode.relu_lower, upper = described_mode.relu_upper, slope = described_mode.relu_slope;
        auto in0 = port(node.inputs, "IN_0"), in1 = port(node.inputs, "IN_1"), out = port(node.outputs, "OUT_0");
        if (!in0 || !out || port(node.inputs, "IN_2")) break;
        auto const& out_tensor = low.tensor(*out);
        if (out_tensor.dim != current.dim) break;
        dfgpu_epilogue_step step{};
        if (mode == DFGPU_PW_RELU_FWD) {
            if (*in0 != final_uid || in1) break;
            step.op = DFGPU_EPI_RELU;
            step.relu_lower = lower;
            step.relu_upper = upper;
            step.relu_slope = slope;
        } else if (mode == DFGPU_PW_ADD) {
            if (!in1 || (*in0 != final_uid && *in1 != final_uid) || *in0 == *in1) break;
            std::int64_t other = *in0 == final_uid ? *in1 : *in0;
            if (extra_uids.size() >= 2 || !low.available_before(other, anchor) || !broadcasts_onto(low.tensor(other), out_tensor)) break;
            auto other_type = low.tensor(other).data_type;
            if (other_type != DataType::kFloat32 && other_type != DataType::kBFloat16 && other_type != DataType::kFloat16) break;
            dfgpu_tensor described;
            if (low.describe(other, described, "").is_bad()) break;
            step.op = DFGPU_EPI_ADD;
            step.operand = static_cast<std::int32_t>(extra_uids.size());
            extra[extra_uids.size()] = described;
            extra_uids.push_back(other);
        } else {
            break;
        }
        steps[count++] = step;
        low.absorbed_into[next] = static_cast<int>(anchor);
        nodes.push_back(next);
        label += "+" + node.name;
        final_uid = *out;
    }
    return Status::ok();
}

Status lower_conv(Lowering& low, std::size_t index) {
    auto const& node = low.graph.nodes[index];
    auto const where = node_path(index, node);
    auto status = require_float_compute(node, where);
    if (status.is_bad()) return status;
    auto x = port(node.inputs, "X"), w = port(node.inputs, "W"), y = port(node.outputs, "Y");
    if (!x || !w || !y || node.inputs.size() != 2 || node.outputs.size() != 1)
        return fail(ErrorCode::kInvalidValue, where, "convolution ports are incomplete");
    auto mode = get_string(node, "math_mode");
    if (!mode || (*mode != "CROSS_CORRELATION" && *mode != "CONVOLUTION")) return fail(ErrorCode::kInvalidValue, where, "math_mode must be CROSS_CORRELATION or CONVOLUTION");
    auto pre = get_int_array(node, "pre_padding"), post = get_int_array(node, "post_padding"), stride = get_int_array(node, "stride"),
         dilation = get_int_array(node, "dilation");
    if (!pre || !post || !stride || !dilation) return fail(ErrorCode::kInvalidValue, where, "padding, stride and dilation must be integer arrays");
    auto const rank = low.tensor(*x).dim.size();
    if (rank < 3 || rank > 5 || low.tensor(*w).dim.size() != rank || low.tensor(*y).dim.size() != rank || pre->size() != rank - 2 ||
        post->size() != rank - 2 || stride->size() != rank - 2 || dilation->size() != rank - 2)
        return fail(ErrorCode::kInvalidShape, where, "convolution requires matching rank 3-5 tensors and spatial attributes");
    // A 1-D (rank-3) convolution runs as the 2-D one over images of a single row: a unit axis goes in before the last
    // axis of every tensor, and the attributes of that axis are the neutral ones.
    auto as_single_row = [](dfgpu_tensor& t) {
        if (t.rank < 2 || t.rank >= DFGPU_MAX_RANK) return;
        t.dim[t.rank] = t.dim[t.rank - 1];
        t.stride[t.rank] = t.stride[t.rank - 1];
        t.dim[t.rank - 1] = 1;
        t.stride[t.rank - 1] = t.dim[t.rank] * t.stride[t.rank];   // (never multiplied by anything but 0)
        ++t.rank;
    };

    KernelStep step;
    step.op = KernelOp::kConvFprop;
    step.label = node.name;
    step.nodes = {index};
    dfgpu_conv_params params{};
    params.stride[0] = params.dilation[0] = 1;   // (rank 3: the single row)
    params.depth_stride = params.depth_dilation = 1;
    for (std::size_t i = 0; i < rank - 2; ++i) {
        if (rank == 5 && i == 0) {   // the depth axis of a 3-D convolution has attributes of its own
            params.depth_pre_pad = (*pre)[0];
            params.depth_post_pad = (*post)[0];
            params.depth_stride = (*stride)[0];
            params.depth_dilation = (*dilation)[0];
            continue;
        }
        std::size_t const axis = rank == 3 ? 1 : i - (rank - 4);
        params.pre_pad[axis] = (*pre)[i];
        params.post_pad[axis] = (*post)[i];
        params.stride[axis] = (*stride)[i];
        params.dilation[axis] = (*dilation)[i];
    }
    params.reverse_filter = *mode == "CONVOLUTION";
    std::vector<std::int64_t> extras;
    std::int64_t final_uid = *y;
    status = absorb_epilogue(low, index, *y, params.epilogue, params.epilogue_count, params.extra, extras, step.nodes, step.label, final_uid);
    if (status.is_bad()) return status;
    if ((status = low.describe(*x, params.x, where)).is_bad()) return status;
    if ((status = low.describe(*w, params.w, where)).is_bad()) return status;
    if ((status = low.describe(final_uid, params.y, where)).is_bad()) return status;
    if (low.tensor(final_uid).dim != low.tensor(*y).dim) return fail(ErrorCode::kInvalidShape, where, "fused output shape differs from the convolution output");
    if (rank == 3) {
        as_single_row(params.x);
        as_single_row(params.w);
        as_single_row(params.y);
        for (int i = 0; i < 2; ++i) as_single_row(params.extra[i]);   // (operands of fewer axes stay aligned with the last one)
    }
    if (low.options.disable_tensor_cores && rank != 5) params.kernel = low.tensor(*x).dim[1] == low.tensor(*w).dim[1] ? DFGPU_CONV_IGEMM_FFMA : DFGPU_CONV_DIRECT;   // (3-D: one kernel only)
    step.tensors = {low.bind(*x), low.bind(*w), low.bind(final_uid), TensorBinding{}, TensorBinding{}};
    for (std::size_t i = 0; i < extras.size(); ++i) step.tensors[3 + i] = low.bind(extras[i]);
    // Filter and ADD operands that no node of the graph writes, behind another convolution of the same plan: the
    // kernel may fetch them while the previous kernel is still draining (see dfgpu_conv_params::reserved).
    bool static_operands = !low.plan.steps.empty() && low.plan.steps.back().op == KernelOp::kConvFprop && low.producer.find(*w) == low.producer.end();
    for (auto uid : extras) static_operands = static_operands && low.producer.find(uid) == low.producer.end();
    if (static_operands) params.reserved |= 2;
    step.params = params;
    low.plan.steps.push_back(std::move(step));
    return Status::ok();
}

// Would the tcgen05 bf16 kernel cover this MATMUL if its floating operands were bf16? Then
// dequantize nodes in front of it are kept as separate launches whose outputs are stored as
// bf16 (exact: an E4M3 code times a power of two has four significant bits), instead of being
// folded into the CUDA-core matmul's operand loads.
bool matmul_fits_tensor_cores(Lowering const& low, OperationDesc const& node) {
    if (low.options.disable_tensor_cores || !low.options.narrow_virtual_tensors) return false;
    auto a = port(node.inputs, "A"), b = port(node.inputs, "B"), c = port(node.outputs, "C");
    if (!a || !b || !c) return false;
    dfgpu_matmul_params trial{};
    if (low.describe(*a, trial.a, "").is_bad() || low.describe(*b, trial.b, "").is_bad() || low.describe(*c, trial.c, "").is_bad()) return false;
    auto floating = [](int t) { return t == DFGPU_F32 || t == DFGPU_BF16; };
    if (!floating(trial.a.dtype) || !floating(trial.b.dtype)) return false;
    if (trial.a.dtype == DFGPU_F32 && !low.tensor(*a).is_virtual) return false;  // a real f32 input cannot be narrowed
    if (trial.b.dtype == DFGPU_F32 && !low.tensor(*b).is_virtual) return false;
    trial.a.dtype = trial.b.dtype = DFGPU_BF16;
    if (trial.c.dtype == DFGPU_F32 && low.tensor(*c).is_virtual) trial.c.dtype = DFGPU_BF16;
    trial.kernel = DFGPU_MATMUL_UMMA_BF16;
    dfgpu_plan_info info{};
    return dfgpu_query_matmul(&trial, &info) == 0;
}

// BLOCK_SCALE_DEQUANTIZE feeding only this MATMUL operand: describes the codes and scales the matmul
// would read directly (no policy here).
bool describe_dequantize(Lowering const& low, std::size_t matmul_index, std::int64_t operand_uid, dfgpu_tensor& operand, dfgpu_tensor& scale,
                         std::int64_t* block, std::int64_t& codes_uid, std::int64_t& scale_uid, std::size_t& dequant_index) {
    auto const& t = low.tensor(operand_uid);
    auto producer = low.producer.find(operand_uid);
    std::size_t only = 0;
    if (!t.is_virtual || producer == low.producer.end() || !low.single_consumer(operand_uid, only) || only != matmul_index) return false;
    auto const& node = low.graph.nodes[producer->second];
    if (node.tag != OperationTag::kBlockScaleDequantize) return false;
    auto x = port(node.inputs, "X"), s = port(node.inputs, "scale");
    auto blocks = get_int_array(node, "block_size");
    if (!x || !s || !blocks || blocks->empty() || blocks->size() > 2) return false;
    auto const& codes = low.tensor(*x);
    auto const& scales = low.tensor(*s);
    if (codes.data_type != DataType::kFp8E4M3 || scales.data_type != DataType::kFp8E8M0 || scales.reordering_type != "NONE") return false;
    if (codes.dim != t.dim || scales.dim.size() != t.dim.size() || t.dim.size() < 2) return false;
    if (low.describe(*x, operand, "").is_bad() || low.describe(*s, scale, "").is_bad()) return false;
    block[0] = blocks->size() == 2 ? (*blocks)[0] : 1;
    block[1] = blocks->back();
    if (block[0] <= 0 || block[1] <= 0) return false;
    codes_uid = *x;
    scale_uid = *s;
    dequant_index = static_cast<std::size_t>(producer->second);
    return true;
}

// Both operands are MXFP8 (E4M3 codes, one E8M0 scale per 32 elements along K) and the shape fits the
// block-scaled tensor-core kernel: the matmul then reads codes and scales itself and neither dequantize
// runs (no bf16 copies of A and B are written or read).
bool matmul_fits_mxf8(Lowering const& low, std::size_t matmul_index) {
    if (low.options.disable_tensor_cores || !low.options.fuse) return false;
    auto const& node = low.graph.nodes[matmul_index];
    auto a = port(node.inputs, "A"), b = port(node.inputs, "B"), c = port(node.outputs, "C");
    if (!a || !b || !c) return false;
    dfgpu_matmul_params trial{};
    std::int64_t codes = 0, scales = 0;
    std::size_t dequant = 0;
    if (!describe_dequantize(low, matmul_index, *a, trial.a, trial.a_scale, trial.a_block, codes, scales, dequant)) return false;
    if (!describe_dequantize(low, matmul_index, *b, trial.b, trial.b_scale, trial.b_block, codes, scales, dequant)) return false;
    if (low.describe(*c, trial.c, "").is_bad()) return false;
    trial.kernel = DFGPU_MATMUL_UMMA_MXF8;
    dfgpu_plan_info info{};
    return dfgpu_query_matmul(&trial, &info) == 0;
}

// Policy: read through the dequantize when the block-scaled tensor-core kernel takes both operands, or
// when no tensor-core kernel fits at all (the CUDA-core matmul decodes on the fly); when only the bf16
// tensor-core kernel fits, the dequantize stays a launch of its own and stores bf16 (exact for E4M3 x 2^k).
bool try_absorb_dequantize(Lowering& low, std::size_t matmul_index, std::int64_t operand_uid, dfgpu_tensor& operand, dfgpu_tensor& scale,
                           std::int64_t* block, std::int64_t& codes_uid, std::int64_t& scale_uid, std::size_t& dequant_index) {
    if (!low.options.fuse) return false;
    if (!matmul_fits_mxf8(low, matmul_index) && matmul_fits_tensor_cores(low, low.graph.nodes[matmul_index])) return false;
    return describe_dequantize(low, matmul_index, operand_uid, operand, scale, block, codes_uid, scale_uid, dequant_index);
}

Status lower_matmul(Lowering& low, std::size_t index) {
    auto const& node = low.graph.nodes[index];
    auto const where = node_path(index, node);
    auto status = require_float_compute(node, where);
    if (status.is_bad()) return status;
    auto a = port(node.inputs, "A"), b = port(node.inputs, "B"), c = port(node.outputs, "C");
    if (!a || !b || !c) return fail(ErrorCode::kInvalidValue, where, "matmul ports are incomplete");
    for (auto name : {"M_override", "N_override", "K_override"})
        if (port(node.inputs, name)) return fail(ErrorCode::kUnsupportedOperation, where, "extent override tensors are not executable on this backend");
    KernelStep step;
    step.op = KernelOp::kMatmul;
    step.label = node.name;
    step.nodes = {index};
    dfgpu_matmul_params params{};
    std::int64_t a_uid = *a, b_uid = *b, a_scale_uid = 0, b_scale_uid = 0;
    bool a_fused = false, b_fused = false;
    std::size_t dequant = 0;
    if (try_absorb_dequantize(low, index, *a, params.a, params.a_scale, params.a_block, a_uid, a_scale_uid, dequant)) {
        a_fused = true;
        low.absorbed_into[dequant] = static_cast<int>(index);
        step.nodes.push_back(dequant);
        step.label = low.graph.nodes[dequant].name + "+" + step.label;
    } else if ((status = low.describe(*a, params.a, where)).is_bad()) {
        return status;
    }
    if (try_absorb_dequantize(low, index, *b, params.b, params.b_scale, params.b_block, b_uid, b_scale_uid, dequant)) {
        b_fused = true;
        low.absorbed_into[dequant] = static_cast<int>(index);
        step.nodes.push_back(dequant);
        step.label = low.graph.nodes[dequant].name + "+" + step.label;
    } else if ((status = low.describe(*b, params.b, where)).is_bad()) {
        return status;
    }
    std::vector<std::int64_t> extras;
    std::int64_t final_uid = *c;
    status = absorb_epilogue(low, index, *c, params.epilogue, params.epilogue_count, params.extra, extras, step.nodes, step.label, final_uid);
    if (status.is_bad()) return status;
    if ((status = low.describe(final_uid, params.c, where)).is_bad()) return status;
    if (low.options.disable_tensor_cores) params.kernel = DFGPU_MATMUL_FFMA;
    step.tensors = {low.bind(a_uid), low.bind(b_uid), low.bind(final_uid), TensorBinding{}, TensorBinding{}, TensorBinding{}, TensorBinding{}};
    if (a_fused) step.tensors[3] = low.bind(a_scale_uid);
    if (b_fused) step.tensors[4] = low.bind(b_scale_uid);
    for (std::size_t i = 0; i < extras.size(); ++i) step.tensors[5 + i] = low.bind(extras[i]);
    step.params = params;
    low.plan.steps.push_back(std::move(step));
    return Status::ok();
}

// MATMUL_FP8 (reference checks: lib/Compiler/SpecializedGraph.cpp:409-496): A, B, two descales, Scale_C in; C and
// Amax_C out; the scales and Amax_C hold one FLOAT element each.
Status lower_matmul_fp8(Lowering& low, std::size_t index) {
    auto const& node = low.graph.nodes[index];
    auto const where = node_path(index, node);
    auto status = require_float_compute(node, where);
    if (status.is_bad()) return status;
    for (auto name : {"M_override", "N_override", "K_override"})
        if (port(node.inputs, name)) return fail(ErrorCode::kUnsupportedOperation, where, "extent override tensors are not executable on this backend");
    if (node.inputs.size() != 5 || node.outputs.size() != 2)
        return fail(ErrorCode::kInvalidValue, where, "MATMUL_FP8 requires A, B, two descales, Scale_C, C, and Amax_C");
    auto a = port(node.inputs, "A"), b = port(node.inputs, "B"), c = port(node.outputs, "C"), amax = port(node.outputs, "Amax_C");
    auto descale_a = port(node.inputs, "Descale_A"), descale_b = port(node.inputs, "Descale_B"), scale_c = port(node.inputs, "Scale_C");
    if (!a || !b || !c || !amax || !descale_a || !descale_b || !scale_c)
        return fail(ErrorCode::kInvalidValue, where, "MATMUL_FP8 requires A, B, two descales, Scale_C, C, and Amax_C");
    auto one_float = [&](std::int64_t uid, char const* name, char const* message) -> Status {
        auto const& t = low.tensor(uid);
        if (t.data_type != DataType::kFloat32) return fail(ErrorCode::kUnsupportedDataType, where + "." + name, "expected FLOAT");
        std::int64_t count = 1;
        for (auto extent : t.dim) count *= extent;
        if (count != 1) return fail(ErrorCode::kInvalidShape, where + "." + name, message);
        return Status::ok();
    };
    if ((status = one_float(*amax, "Amax_C", "Amax_C must contain one FLOAT element")).is_bad()) return status;
    for (auto [uid, name] : {std::pair{*descale_a, "Descale_A"}, std::pair{*descale_b, "Descale_B"}, std::pair{*scale_c, "Scale_C"}})
        if ((status = one_float(uid, name, "scale tensors must contain one FLOAT element")).is_bad()) return status;
    auto typed = [&](std::int64_t uid, char const* name, std::initializer_list<DataType> allowed) -> Status {
        auto const type = low.tensor(uid).data_type;
        if (std::find(allowed.begin(), allowed.end(), type) != allowed.end()) return Status::ok();
        return fail(ErrorCode::kUnsupportedDataType, where + "." + name, std::string(import::data_type_name(type)) + " is not supported on this port");
    };
    if ((status = typed(*a, "A", {DataType::kFp8E4M3, DataType::kFp8E5M2})).is_bad()) return status;
    if ((status = typed(*b, "B", {DataType::kFp8E4M3, DataType::kFp8E5M2})).is_bad()) return status;
    if ((status = typed(*c, "C", {DataType::kFp8E4M3, DataType::kFp8E5M2, DataType::kFloat32, DataType::kFloat16, DataType::kBFloat16})).is_bad()) return status;
    dfgpu_matmul_fp8_params params{};
    if ((status = low.describe(*a, params.a, where, true)).is_bad()) return status;
    if ((status = low.describe(*b, params.b, where, true)).is_bad()) return status;
    if ((status = low.describe(*c, params.c, where, true)).is_bad()) return status;
    auto const& ta = low.tensor(*a);
    auto const& tb = low.tensor(*b);
    auto const& tc = low.tensor(*c);
    if (ta.dim.size() < 2 || ta.dim.size() != tb.dim.size() || tc.dim.size() != ta.dim.size())
        return fail(ErrorCode::kInvalidShape, where, "A, B, and C must have equal rank of at least two");
    auto const rank = ta.dim.size();
    if (ta.dim[rank - 1] != tb.dim[rank - 2] || tc.dim[rank - 2] != ta.dim[rank - 2] || tc.dim[rank - 1] != tb.dim[rank - 1])
        return fail(ErrorCode::kInvalidShape, where, "matrix M, N, and K dimensions are inconsistent");
    for (std::size_t axis = 0; axis + 2 < rank; ++axis)
        if ((ta.dim[axis] != 1 && ta.dim[axis] != tc.dim[axis]) || (tb.dim[axis] != 1 && tb.dim[axis] != tc.dim[axis]))
            return fail(ErrorCode::kInvalidShape, where, "batch dimensions are not broadcast-compatible");
    if (low.options.disable_tensor_cores) params.kernel = DFGPU_MATMUL_FP8_SCALAR;
    KernelStep step;
    step.op = KernelOp::kMatmulFp8;
    step.label = node.name;
    step.nodes = {index};
    step.tensors = {low.bind(*a), low.bind(*b), low.bind(*c), low.bind(*amax), low.bind(*descale_a), low.bind(*descale_b), low.bind(*scale_c)};
    step.params = params;
    low.plan.steps.push_back(std::move(step));
    return Status::ok();
}

Status lower_pointwise(Lowering& low, std::size_t index) {
    auto const& node = low.graph.nodes[index];
    auto const where = node_path(index, node);
    auto status = require_float_compute(node, where);
    if (status.is_bad()) return status;
    dfgpu_pointwise_params params{};
    if ((status = pointwise_mode(node, where, params)).is_bad()) return status;
    auto in0 = port(node.inputs, "IN_0"), in1 = port(node.inputs, "IN_1"), in2 = port(node.inputs, "IN_2"), out = port(node.outputs, "OUT_0");
    int const inputs = dfgpu_pointwise_input_count(params.mode);
    if (!in0 || !out || (inputs >= 2) != in1.has_value() || (inputs >= 3) != in2.has_value() || static_cast<int>(node.inputs.size()) != inputs)
        return fail(ErrorCode::kInvalidValue, where, "pointwise input count does not match the mode");
    if ((status = low.describe(*in0, params.in0, where)).is_bad()) return status;
    if (in1 && (status = low.describe(*in1, params.in1, where)).is_bad()) return status;
    if (in2 && (status = low.describe(*in2, params.in2, where)).is_bad()) return status;
    if ((status = low.describe(*out, params.out, where)).is_bad()) return status;
    if (params.mode == DFGPU_PW_GEN_INDEX && (params.axis < 0 || params.axis >= params.out.rank))
        return fail(ErrorCode::kInvalidValue, where, "GEN_INDEX requires an axis in the output rank");
    KernelStep step;
    step.op = KernelOp::kPointwise;
    step.label = node.name;
    step.nodes = {index};
    step.tensors = {low.bind(*in0), in1 ? low.bind(*in1) : TensorBinding{}, low.bind(*out), in2 ? low.bind(*in2) : TensorBinding{}};
    step.params = params;
    low.plan.steps.push_back(std::move(step));
    return Status::ok();
}

Status lower_quantize(Lowering& low, std::size_t index) {
    auto const& node = low.graph.nodes[index];
    auto const where = node_path(index, node);
    auto status = require_float_compute(node, where);
    if (status.is_bad()) return status;
    auto x = port(node.inputs, "X"), y = port(node.outputs, "Y"), scale = port(node.outputs, "scale");
    if (!x || !y || !scale) return fail(ErrorCode::kInvalidValue, where, "block-scale quantize ports are incomplete");
    auto block = get_int(node, "block_size");
    if (!block || *block <= 0) return fail(ErrorCode::kInvalidValue, where, "block_size must be a positive integer");
    dfgpu_bsq_params params{};
    params.block_size = *block;
    auto axis = get_int(node, "axis");
    if (!axis && !is_null(node, "axis")) return fail(ErrorCode::kInvalidValue, where, "axis must be an integer or null");
    params.axis = axis ? static_cast<std::int32_t>(*axis) : -1;
    if (axis && (*axis < 0 || *axis >= static_cast<std::int64_t>(low.tensor(*x).dim.size()))) return fail(ErrorCode::kInvalidValue, where, "axis is out of range");
    if ((status = low.describe(*x, params.x, where)).is_bad()) return status;
    // (E5M2 and packed FP4 codes: the general kernel)
    if ((status = low.describe(*y, params.y, where, low.tensor(*y).data_type == DataType::kFp8E5M2 || low.tensor(*y).data_type == DataType::kFp4E2M1)).is_bad()) return status;
    if ((status = low.describe(*scale, params.scale, where)).is_bad()) return status;
    KernelStep step;
    step.op = KernelOp::kBlockScaleQuantize;
    step.label = node.name;
    step.nodes = {index};
    step.tensors = {low.bind(*x), low.bind(*y), low.bind(*scale)};
    step.params = params;
    low.plan.steps.push_back(std::move(step));
    return Status::ok();
}

Status lower_dequantize(Lowering& low, std::size_t index) {
    auto const& node = low.graph.nodes[index];
    auto const where = node_path(index, node);
    auto status = require_float_compute(node, where);
    if (status.is_bad()) return status;
    auto x = port(node.inputs, "X"), scale = port(node.inputs, "scale"), y = port(node.outputs, "Y");
    if (!x || !y || !scale) return fail(ErrorCode::kInvalidValue, where, "block-scale dequantize ports are incomplete");
    auto blocks = get_int_array(node, "block_size");
    if (!blocks || blocks->empty() || blocks->size() > DFGPU_MAX_RANK) return fail(ErrorCode::kInvalidValue, where, "block_size must be a non-empty integer array");
    if (!get_bool(node, "is_negative_scale")) return fail(ErrorCode::kInvalidValue, where, "is_negative_scale must be a boolean");
    dfgpu_bsd_params params{};
    params.block_count = static_cast<std::int32_t>(blocks->size());
    for (std::size_t i = 0; i < blocks->size(); ++i) params.block[i] = (*blocks)[i];
    auto const code_type = low.tensor(*x).data_type;
    if ((status = low.describe(*x, params.x, where, code_type == DataType::kFp8E5M2 || code_type == DataType::kFp4E2M1 || code_type == DataType::kInt4)).is_bad()) return status;
    if ((status = low.describe(*scale, params.scale, where)).is_bad()) return status;
    if ((status = low.describe(*y, params.y, where)).is_bad()) return status;
    KernelStep step;
    step.op = KernelOp::kBlockScaleDequantize;
    step.label = node.name;
    step.nodes = {index};
    step.tensors = {low.bind(*x), low.bind(*scale), low.bind(*y)};
    step.params = params;
    low.plan.steps.push_back(std::move(step));
    return Status::ok();
}

Status lower_sdpa(Lowering& low, std::size_t index) {
    auto const& node = low.graph.nodes[index];
    auto const where = node_path(index, node);
    for (auto name : {"Attn_scale", "Dropout_scale_inv", "Descale_Q", "Descale_K", "Descale_V", "Descale_S", "Scale_S", "Scale_O"})
        if (port(node.inputs, name)) return fail(ErrorCode::kUnsupportedOperation, where, std::string("input port ") + name + " is outside the GPU hot path");
    for (auto name : {"Amax_S", "Amax_O"})
        if (port(node.outputs, name)) return fail(ErrorCode::kUnsupportedOperation, where, std::string("output port ") + name + " is outside the GPU hot path");
    auto q = port(node.inputs, "Q"), k = port(node.inputs, "K"), v = port(node.inputs, "V"), o = port(node.outputs, "O");
    if (!q || !k || !v || !o) return fail(ErrorCode::kInvalidValue, where, "SDPA ports are incomplete");
    auto alibi = get_bool(node, "alibi_mask");
    if (!alibi) return fail(ErrorCode::kInvalidValue, where, "alibi_mask must be a boolean");
    auto bias = port(node.inputs, "Bias");
    // Dropout (lib/Compiler/SequenceGraph.cpp:418-500): a probability with Seed and Offset, or the caller's mask and scale; never both.
    auto probability = get_number(node, "dropout_probability");
    if (!probability && !is_null(node, "dropout_probability")) return fail(ErrorCode::kInvalidValue, where + ".dropout_probability", "expected a number or null");
    if (probability && (!std::isfinite(*probability) || *probability < 0.0 || *probability >= 1.0))
        return fail(ErrorCode::kInvalidValue, where + ".dropout_probability", "probability must be finite and in [0, 1)");
    auto dropout_mask = port(node.inputs, "Dropout_mask"), dropout_scale = port(node.inputs, "Dropout_scale");
    auto seed = port(node.inputs, "Seed"), offset = port(node.inputs, "Offset"), rng_dump = port(node.outputs, "RNG_DUMP");
    if (probability && dropout_mask) return fail(ErrorCode::kInvalidValue, where, "internal and custom dropout cannot be combined");
    if (probability) {
        if (!seed || !offset) return fail(ErrorCode::kInvalidValue, where, "probability dropout requires Seed and Offset");
        if (dropout_scale) return fail(ErrorCode::kInvalidValue, where, "Dropout_scale is implicit for probability dropout");
    } else if (dropout_mask) {
        if (!dropout_scale) return fail(ErrorCode::kInvalidValue, where, "custom dropout requires Dropout_scale");
        if (seed || offset) return fail(ErrorCode::kInvalidValue, where, "custom dropout does not accept Seed or Offset");
        if (rng_dump) return fail(ErrorCode::kInvalidValue, where + ".RNG_DUMP", "RNG_DUMP requires probability dropout");
    } else if (seed || offset || dropout_scale || rng_dump) {
        return fail(ErrorCode::kInvalidValue, where, "Seed, Offset, Dropout_scale and RNG_DUMP require a configured dropout mode");
    }
    if (get_bool(node, "is_mxfp8").value_or(true)) return fail(ErrorCode::kUnsupportedOperation, where, "is_mxfp8 must be false");
    auto padding = get_bool(node, "padding_mask"), stats_flag = get_bool(node, "generate_stats");
    if (!padding || !stats_flag) return fail(ErrorCode::kInvalidValue, where, "padding_mask and generate_stats must be booleans");
    auto stats = port(node.outputs, "Stats"), max = port(node.outputs, "Max"), sum_exp = port(node.outputs, "Sum_exp");
    if (*stats_flag != stats.has_value()) return fail(ErrorCode::kInvalidValue, where, "generate_stats must be set exactly when the Stats output is present");
    auto alignment = get_string(node, "diagonal_alignment");
    if (!alignment || (*alignment != "TOP_LEFT" && *alignment != "BOTTOM_RIGHT")) return fail(ErrorCode::kInvalidValue, where, "diagonal_alignment must be TOP_LEFT or BOTTOM_RIGHT");

    dfgpu_sdpa_params params{};
    Status status = Status::ok();
    if ((status = low.describe(*q, params.q, where)).is_bad()) return status;
    if ((status = low.describe(*k, params.k, where)).is_bad()) return status;
    if ((status = low.describe(*v, params.v, where)).is_bad()) return status;
    if ((status = low.describe(*o, params.o, where)).is_bad()) return status;
    if (stats && (status = low.describe(*stats, params.stats, where)).is_bad()) return status;
    if (max && (status = low.describe(*max, params.max, where)).is_bad()) return status;
    if (sum_exp && (status = low.describe(*sum_exp, params.sum_exp, where)).is_bad()) return status;
    auto seq_q = port(node.inputs, "SEQ_LEN_Q"), seq_kv = port(node.inputs, "SEQ_LEN_KV");
    auto table_k = port(node.inputs, "Page_table_K"), table_v = port(node.inputs, "Page_table_V");
    if (*padding != (seq_q.has_value() && seq_kv.has_value()) || seq_q.has_value() != seq_kv.has_value())
        return fail(ErrorCode::kInvalidValue, where, "padding_mask requires both SEQ_LEN_Q and SEQ_LEN_KV, and only then");
    if ((table_k || table_v) && !*padding) return fail(ErrorCode::kInvalidValue, where, "paged K/V requires padding_mask with sequence lengths");
    if (seq_q && (status = low.describe(*seq_q, params.seq_q, where)).is_bad()) return status;
    if (seq_kv && (status = low.describe(*seq_kv, params.seq_kv, where)).is_bad()) return status;
    if (table_k && (status = low.describe(*table_k, params.page_table_k, where, true)).is_bad()) return status;
    if (table_v && (status = low.describe(*table_v, params.page_table_v, where, true)).is_bad()) return status;
    // compact page tables (lib/Compiler/SequenceGraph.cpp:741-773, :1811-1864): the table's entry names the INT32 / INT64
    // tensor [B+1,1,1,1] of per-batch element offsets into its storage
    std::optional<std::int64_t> offsets_k, offsets_v;
    for (int which = 0; which < 2; ++which) {
        auto const& table = which ? table_v : table_k;
        if (!table) continue;
        auto const& t = low.tensor(*table);
        if (t.data_type != DataType::kInt32) return fail(ErrorCode::kUnsupportedDataType, where, "page tables are INT32");
        if (!t.ragged_offset_uid) continue;
        auto const port_name = where + (which ? ".Page_table_V" : ".Page_table_K");
        if (t.is_virtual) return fail(ErrorCode::kInvalidValue, port_name, "ragged attention data must be an external tensor");
        auto found = low.graph.tensors.find(*t.ragged_offset_uid);
        if (found == low.graph.tensors.end()) return fail(ErrorCode::kMissingUid, port_name, "ragged offset tensor is unresolved");
        auto const& offsets = found->second;
        if (offsets.dim != std::vector<std::int64_t>{t.dim[0] + 1, 1, 1, 1}) return fail(ErrorCode::kInvalidShape, port_name, "ragged offset must have dimensions [B+1,1,1,1]");
        if ((offsets.data_type != DataType::kInt32 && offsets.data_type != DataType::kInt64) || offsets.is_virtual || offsets.reordering_type != "NONE" || offsets.ragged_offset_uid)
            return fail(ErrorCode::kUnsupportedOperation, port_name, "ragged offsets must be an external plain INT32 or INT64 tensor");
        if ((status = low.describe(*t.ragged_offset_uid, which ? params.page_offsets_v : params.page_offsets_k, where, true)).is_bad()) return status;
        (which ? offsets_v : offsets_k) = *t.ragged_offset_uid;
    }
    if (params.q.rank != 4 || params.k.rank != 4 || params.v.rank != 4) return fail(ErrorCode::kInvalidShape, where, "Q, K and V must have rank 4");
    params.attn_scale = static_cast<float>(get_number(node, "attn_scale_value").value_or(1.0));
    params.padding_mask = *padding;
    if (auto bound = get_int(node, "left_bound")) {
        params.has_left_bound = 1;
        params.left_bound = *bound;
    } else if (!is_null(node, "left_bound")) {
        return fail(ErrorCode::kInvalidValue, where, "left_bound must be an integer or null");
    }
    if (auto bound = get_int(node, "right_bound")) {
        params.has_right_bound = 1;
        params.right_bound = *bound;
    } else if (!is_null(node, "right_bound")) {
        return fail(ErrorCode::kInvalidValue, where, "right_bound must be an integer or null");
    }
    params.bottom_right = *alignment == "BOTTOM_RIGHT";
    // logical key/value length: max_seq_len_kv when given, else the container/table capacity
    auto max_len = get_int(node, "max_seq_len_kv");
    std::int64_t capacity_k = table_k ? params.page_table_k.dim[2] * params.k.dim[2] : params.k.dim[2];
    std::int64_t capacity_v = table_v ? params.page_table_v.dim[2] * params.v.dim[2] : params.v.dim[2];
    params.s_kv = max_len ? *max_len : std::min(capacity_k, capacity_v);
    if (bias) {
        // reference checks: lib/Compiler/SequenceGraph.cpp:692-697 (rank 4; the key length of a both-paged graph without
        // max_seq_len_kv comes from the bias), :879-883 (broadcast onto [B, Hq, Sq, Skv])
        if ((status = low.describe(*bias, params.bias, where)).is_bad()) return status;
        if (params.bias.rank != 4) return fail(ErrorCode::kInvalidShape, where + ".Bias", "Bias must have rank 4");
        if (!max_len && table_k && table_v) params.s_kv = params.bias.dim[3];
    }
    if (params.s_kv <= 0 || params.s_kv > capacity_k || params.s_kv > capacity_v)
        return fail(ErrorCode::kInvalidShape, where, "key/value capacity is below the logical sequence length");
    if (bias) {
        const std::int64_t scores[4] = {params.q.dim[0], params.q.dim[1], params.q.dim[2], params.s_kv};
        for (int axis = 0; axis < 4; ++axis)
            if (params.bias.dim[axis] != 1 && params.bias.dim[axis] != scores[axis])
                return fail(ErrorCode::kInvalidShape, where + ".Bias", "bias is not broadcast-compatible with attention scores");
    }
    params.alibi_mask = *alibi;
    auto block_mask = port(node.inputs, "Block_mask");
    if (block_mask) {
        // lib/Compiler/SequenceGraph.cpp:854-877: an external plain UINT8 tensor, one bit per 128 x 128 score tile
        if ((status = low.describe(*block_mask, params.block_mask, where, true)).is_bad()) return status;
        auto const& t = low.tensor(*block_mask);
        if (t.data_type != DataType::kUint8) return fail(ErrorCode::kUnsupportedDataType, where + ".Block_mask", std::string(import::data_type_name(t.data_type)) + " is not supported on this port");
        const std::int64_t query_tiles = (params.q.dim[2] - 1) / 128 + 1, key_tiles = (params.s_kv - 1) / 128 + 1;
        if (t.dim != std::vector<std::int64_t>{params.q.dim[0], params.q.dim[1], query_tiles, (key_tiles + 7) / 8})
            return fail(ErrorCode::kInvalidShape, where + ".Block_mask", "block mask must have dimensions [B,Hq,ceil(Sq/128),ceil(ceil(Skv/128)/8)]");
        if (t.is_virtual || t.is_pass_by_value || t.reordering_type != "NONE") return fail(ErrorCode::kUnsupportedOperation, where + ".Block_mask", "block mask must be an external plain UINT8 tensor");
    }
    auto sink = port(node.inputs, "SINK_TOKEN");
    if (sink) {
        // lib/Compiler/SequenceGraph.cpp:561-577: an external plain FLOAT tensor [1, Hq, 1, 1]
        if ((status = low.describe(*sink, params.sink, where)).is_bad()) return status;
        auto const& t = low.tensor(*sink);
        if (t.dim != std::vector<std::int64_t>{1, params.q.dim[1], 1, 1}) return fail(ErrorCode::kInvalidShape, where + ".SINK_TOKEN", "sink token must have dimensions [1,Hq,1,1]");
        if (t.is_virtual || t.is_pass_by_value || t.reordering_type != "NONE" || t.data_type != DataType::kFloat32)  // lib/Compiler/SequenceGraph.cpp:570-576
            return fail(ErrorCode::kUnsupportedOperation, where + ".SINK_TOKEN", "sink token must be an external plain FLOAT tensor");
    }
    auto one_element = [](TensorDesc const& t) {
        for (auto extent : t.dim)
            if (extent != 1) return false;
        return !t.dim.empty();
    };
    if (probability) {
        params.dropout_kind = 1;
        params.dropout_probability = *probability;
        if ((status = low.describe(*seed, params.seed, where, true)).is_bad()) return status;
        if ((status = low.describe(*offset, params.offset, where, true)).is_bad()) return status;
        for (auto const* t : {&low.tensor(*seed), &low.tensor(*offset)})
            if (t->data_type != DataType::kInt64 || !one_element(*t)) return fail(ErrorCode::kInvalidShape, where, "Seed and Offset must be INT64 scalars");
        if (rng_dump) {
            if ((status = low.describe(*rng_dump, params.rng_dump, where)).is_bad()) return status;
            if (low.tensor(*rng_dump).data_type != DataType::kFloat32) return fail(ErrorCode::kUnsupportedDataType, where + ".RNG_DUMP", "RNG_DUMP must be FLOAT");
        }
    } else if (dropout_mask) {
        params.dropout_kind = 2;
        if ((status = low.describe(*dropout_mask, params.dropout_mask, where)).is_bad()) return status;
        if ((status = low.describe(*dropout_scale, params.dropout_scale, where)).is_bad()) return status;
        if (low.tensor(*dropout_mask).data_type != DataType::kFloat32 || low.tensor(*dropout_scale).data_type != DataType::kFloat32)
            return fail(ErrorCode::kUnsupportedDataType, where, "Dropout_mask and Dropout_scale must be FLOAT");
        if (!one_element(low.tensor(*dropout_scale))) return fail(ErrorCode::kInvalidShape, where + ".Dropout_scale", "Dropout_scale must be a scalar");
    }
    // lib/Compiler/SequenceGraph.cpp:951-955
    if (params.bottom_right && params.has_right_bound && (bias || *alibi || params.dropout_kind != 0))
        return fail(ErrorCode::kUnsupportedOperation, where, "cuDNN bottom-right causal masking does not combine with bias, ALiBi, or dropout");
    KernelStep step;
    step.op = KernelOp::kSdpaForward;
    step.label = node.name;
    step.nodes = {index};
    auto optional_binding = [&](std::optional<std::int64_t> uid) { return uid ? low.bind(*uid) : TensorBinding{}; };
    step.tensors = {low.bind(*q), low.bind(*k), low.bind(*v), low.bind(*o), optional_binding(stats), optional_binding(max), optional_binding(sum_exp),
                    optional_binding(seq_q), optional_binding(seq_kv), optional_binding(table_k), optional_binding(table_v), optional_binding(bias), optional_binding(sink), optional_binding(block_mask),
                    optional_binding(offsets_k), optional_binding(offsets_v), optional_binding(dropout_mask), optional_binding(dropout_scale), optional_binding(seed),
                    optional_binding(offset), optional_binding(rng_dump)};
    step.params = params;
    low.plan.steps.push_back(std::move(step));
    return Status::ok();
}

bool is_contraction(KernelOp op) { return op == KernelOp::kConvFprop || op == KernelOp::kMatmul; }

dfgpu_tensor* step_output(KernelStep& step) {
    if (auto* conv = std::get_if<dfgpu_conv_params>(&step.params)) return &conv->y;
    if (auto* matmul = std::get_if<dfgpu_matmul_params>(&step.params)) return &matmul->c;
    return nullptr;
}

// A virtual f32 tensor written by a bf16 contraction and read only by contractions is
// stored as bf16: the consuming tensor-core kernel would round it to bf16 anyway, and
// the narrower store halves the traffic of the intermediate.
void narrow_virtual_tensors(Lowering& low) {
    if (!low.options.narrow_virtual_tensors || low.options.disable_tensor_cores) return;
    std::map<std::int64_t, std::vector<std::size_t>> readers;
    std::map<std::int64_t, std::size_t> writer;
    for (std::size_t s = 0; s < low.plan.steps.size(); ++s) {
        auto const& step = low.plan.steps[s];
        for (std::size_t slot = 0; slot < step.tensors.size(); ++slot) {
            auto const& binding = step.tensors[slot];
            if (binding.kind != TensorBinding::Kind::kWorkspace) continue;
            bool is_output = is_contraction(step.op) ? slot == 2 : false;
            if (step.op == KernelOp::kPointwise) is_output = slot == 2;
            if (step.op == KernelOp::kBlockScaleQuantize) is_output = slot >= 1;
            if (step.op == KernelOp::kBlockScaleDequantize) is_output = slot == 2;
            if (step.op == KernelOp::kSdpaForward) is_output = (slot >= 3 && slot <= 6) || slot == 20;
            if (is_output) writer[binding.uid] = s;
            else readers[binding.uid].push_back(s);
        }
    }
    // pass 1: dequantize outputs (exactly representable in bf16) that only feed contractions which
    // would then run on the tensor cores; pass 2: contraction outputs with bf16 inputs.
    for (int pass = 0; pass < 2; ++pass)
    for (auto const& [uid, step_index] : writer) {
        auto& step = low.plan.steps[step_index];
        if (low.tensor(uid).data_type != DataType::kFloat32 || low.storage_override.count(uid)) continue;
        bool only_contractions = !readers[uid].empty();
        for (auto reader : readers[uid]) only_contractions = only_contractions && is_contraction(low.plan.steps[reader].op);
        if (!only_contractions) continue;
        if (pass == 0) {
            auto* dequantize = std::get_if<dfgpu_bsd_params>(&step.params);
            if (!dequantize || dequantize->x.dtype != DFGPU_E4M3 || dequantize->scale.dtype != DFGPU_E8M0) continue;
            bool wanted = true;
            for (auto reader : readers[uid]) {
                auto const& consumer = low.plan.steps[reader];
                wanted = wanted && consumer.op == KernelOp::kMatmul && matmul_fits_tensor_cores(low, low.graph.nodes[consumer.nodes.front()]);
            }
            if (!wanted) continue;
            dequantize->y.dtype = DFGPU_BF16;
        } else {
            if (!low.options.bf16_virtual_tensors) continue;  // lossy: only on request
            if (!is_contraction(step.op)) continue;
            bool bf16_inputs = false;
            if (auto* conv = std::get_if<dfgpu_conv_params>(&step.params)) bf16_inputs = conv->x.dtype == DFGPU_BF16 && conv->w.dtype == DFGPU_BF16;
            if (auto* matmul = std::get_if<dfgpu_matmul_params>(&step.params)) bf16_inputs = matmul->a.dtype == DFGPU_BF16 && matmul->b.dtype == DFGPU_BF16;
            if (!bf16_inputs) continue;
            step_output(step)->dtype = DFGPU_BF16;
        }
        low.storage_override[uid] = DFGPU_BF16;
        for (auto reader : readers[uid]) {
            auto& consumer = low.plan.steps[reader];
            for (std::size_t slot = 0; slot < consumer.tensors.size(); ++slot) {
                if (consumer.tensors[slot].kind != TensorBinding::Kind::kWorkspace || consumer.tensors[slot].uid != uid) continue;
                if (auto* conv = std::get_if<dfgpu_conv_params>(&consumer.params)) {
                    if (slot == 0) conv->x.dtype = DFGPU_BF16;
                    if (slot == 1) conv->w.dtype = DFGPU_BF16;
                    if (slot >= 3) conv->extra[slot - 3].dtype = DFGPU_BF16;
                }
                if (auto* matmul = std::get_if<dfgpu_matmul_params>(&consumer.params)) {
                    if (slot == 0) matmul->a.dtype = DFGPU_BF16;
                    if (slot == 1) matmul->b.dtype = DFGPU_BF16;
                    if (slot >= 5) matmul->extra[slot - 5].dtype = DFGPU_BF16;
                }
            }
        }
    }
}

// FLOAT virtual tensors between bf16 tcgen05 convolutions -> DFGPU_BF16X2 (hi, lo) pairs. A tensor qualifies when
// a convolution writes it and only convolutions read it, as their X; the set is then trimmed until the kernel
// library resolves every touched launch to the tcgen05 kernel with those types (a launch that cannot take a
// split tensor drops the tensors around it back to FLOAT).
void split_virtual_tensors(Lowering& low) {
    if (!low.options.narrow_virtual_tensors || low.options.disable_tensor_cores || low.options.bf16_virtual_tensors) return;
    std::map<std::int64_t, std::size_t> writer;
    std::map<std::int64_t, std::vector<std::size_t>> readers;
    std::set<std::int64_t> disqualified;
    for (std::size_t s = 0; s < low.plan.steps.size(); ++s) {
        auto const& step = low.plan.steps[s];
        for (std::size_t slot = 0; slot < step.tensors.size(); ++slot) {
            auto const& binding = step.tensors[slot];
            if (binding.kind != TensorBinding::Kind::kWorkspace) continue;
            if (step.op != KernelOp::kConvFprop || (slot != 0 && slot != 2)) disqualified.insert(binding.uid);
            else if (slot == 2) writer[binding.uid] = s;
            else readers[binding.uid].push_back(s);
        }
    }
    std::set<std::int64_t> chosen;
    for (auto const& [uid, s] : writer)
        if (!disqualified.count(uid) && !readers[uid].empty() && low.tensor(uid).data_type == DataType::kFloat32 && !low.storage_override.count(uid)) chosen.insert(uid);
    auto resolves = [&](std::size_t s) {
        auto const& step = low.plan.steps[s];
        dfgpu_conv_params trial = std::get<dfgpu_conv_params>(step.params);
        if (step.tensors[0].kind == TensorBinding::Kind::kWorkspace && chosen.count(step.tensors[0].uid)) trial.x.dtype = DFGPU_BF16X2;
        if (step.tensors[2].kind == TensorBinding::Kind::kWorkspace && chosen.count(step.tensors[2].uid)) trial.y.dtype = DFGPU_BF16X2;
        dfgpu_plan_info info{};
        return dfgpu_query_conv_fprop(&trial, &info) == 0 && info.kernel == DFGPU_CONV_UMMA_BF16;
    };
    for (bool changed = true; changed && !chosen.empty();) {
        changed = false;
        for (auto uid : std::vector<std::int64_t>(chosen.begin(), chosen.end())) {
            bool ok = resolves(writer[uid]);
            for (auto reader : readers[uid]) ok = ok && resolves(reader);
            if (!ok) {
                chosen.erase(uid);
                changed = true;
            }
        }
    }
    for (auto uid : chosen) {
        low.storage_override[uid] = DFGPU_BF16X2;
        std::get<dfgpu_conv_params>(low.plan.steps[writer[uid]].params).y.dtype = DFGPU_BF16X2;
        for (auto reader : readers[uid]) std::get<dfgpu_conv_params>(low.plan.steps[reader].params).x.dtype = DFGPU_BF16X2;
    }
}

// A convolution whose only reader is the 1 x 1 convolution launched right after it becomes one launch with it when
// the kernel library has a fused kernel for the pair: the tensor between them then needs no workspace at all (it is
// handed over inside the SM). Runs after the storage types are settled, so the pair is offered to the library with
// the types the two launches would have used.
void fuse_convolution_pairs(Lowering& low) {
    if (!low.options.fuse || !low.options.fuse_convolution_pairs || low.options.disable_tensor_cores) return;
    auto uses = [&](std::int64_t uid) {
        int count = 0;
        for (auto const& step : low.plan.steps)
            for (auto const& binding : step.tensors) count += binding.kind == TensorBinding::Kind::kWorkspace && binding.uid == uid;
        return count;
    };
    for (std::size_t s = 0; s + 1 < low.plan.steps.size(); ++s) {
        auto& first = low.plan.steps[s];
        auto& second = low.plan.steps[s + 1];
        if (first.op != KernelOp::kConvFprop || second.op != KernelOp::kConvFprop) continue;
        auto const& between = first.tensors[2];
        if (between.kind != TensorBinding::Kind::kWorkspace || second.tensors[0].kind != TensorBinding::Kind::kWorkspace || second.tensors[0].uid != between.uid) continue;
        if (uses(between.uid) != 2) continue;  // written here, read there, nowhere else
        dfgpu_conv_pair_params pair{};
        pair.first = std::get<dfgpu_conv_params>(first.params);
        pair.second = std::get<dfgpu_conv_params>(second.params);
        dfgpu_plan_info info{};
        if (dfgpu_query_conv_fprop_pair(&pair, &info) != 0) continue;
        KernelStep fused;
        fused.op = KernelOp::kConvFpropPair;
        fused.label = first.label + ">" + second.label;
        fused.nodes = first.nodes;
        fused.nodes.insert(fused.nodes.end(), second.nodes.begin(), second.nodes.end());
        fused.tensors = {first.tensors[0], first.tensors[1], second.tensors[1], second.tensors[2], first.tensors[3], first.tensors[4], second.tensors[3], second.tensors[4]};
        fused.params = pair;
        low.plan.steps[s] = std::move(fused);
        low.plan.steps.erase(low.plan.steps.begin() + static_cast<std::ptrdiff_t>(s) + 1);
    }
}

// Two BLOCK_SCALE_QUANTIZE launches next to each other that do not touch each other's tensors become one launch
// when the kernel library takes the pair (both in a bf16 fast form): these launches are ~10 us each, a third of it
// ramp and tail, which one grid pays once.
void fuse_quantize_pairs(Lowering& low) {
    if (!low.options.fuse) return;
    for (std::size_t s = 0; s + 1 < low.plan.steps.size(); ++s) {
        auto& first = low.plan.steps[s];
        auto& second = low.plan.steps[s + 1];
        if (first.op != KernelOp::kBlockScaleQuantize || second.op != KernelOp::kBlockScaleQuantize) continue;
        bool independent = true;
        for (auto const& a : first.tensors)
            for (auto const& b : second.tensors)
                independent = independent && !(a.kind == b.kind && a.kind != TensorBinding::Kind::kAbsent && a.uid == b.uid);
        if (!independent) continue;
        dfgpu_bsq_pair_params pair{};
        pair.first = std::get<dfgpu_bsq_params>(first.params);
        pair.second = std::get<dfgpu_bsq_params>(second.params);
        dfgpu_plan_info info{};
        if (dfgpu_query_block_scale_quantize_pair(&pair, &info) != 0) continue;
        KernelStep fused;
        fused.op = KernelOp::kBlockScaleQuantizePair;
        fused.label = first.label + "|" + second.label;
        fused.nodes = first.nodes;
        fused.nodes.insert(fused.nodes.end(), second.nodes.begin(), second.nodes.end());
        fused.tensors = {first.tensors[0], first.tensors[1], first.tensors[2], second.tensors[0], second.tensors[1], second.tensors[2]};
        fused.params = pair;
        low.plan.steps[s] = std::move(fused);
        low.plan.steps.erase(low.plan.steps.begin() + static_cast<std::ptrdiff_t>(s) + 1);
    }
}

// Fills the conv-adapter metadata when the graph is the reference's single-node case; false otherwise (the generic
// table stands).
bool single_conv_metadata(SerializedGraph const& graph, CompileOptions const& options, Conv2DCompileMetadata& metadata) {
    auto const* node = graph.single_conv_fprop();
    if (!node || graph.tensors.size() != 3) return false;
    auto x = port(node->inputs, "X"), w = port(node->inputs, "W"), y = port(node->outputs, "Y");
    auto pre = get_int_array(*node, "pre_padding"), post = get_int_array(*node, "post_padding"), stride = get_int_array(*node, "stride"),
         dilation = get_int_array(*node, "dilation");
    if (!x || !w || !y || !pre || !post || !stride || !dilation || pre->size() != 2 || post->size() != 2 || stride->size() != 2 || dilation->size() != 2) return false;
    auto packed_channels_last = [](TensorDesc const& t) {
        return t.dim.size() == 4 && !t.is_virtual && t.stride[1] == 1 && t.stride[3] == t.dim[1] && t.stride[2] == t.dim[3] * t.dim[1] &&
               t.stride[0] == t.dim[2] * t.dim[3] * t.dim[1];
    };
    auto const &tx = graph.tensors.at(*x), &tw = graph.tensors.at(*w), &ty = graph.tensors.at(*y);
    if (!packed_channels_last(tx) || !packed_channels_last(tw) || !packed_channels_last(ty)) return false;  // e.g. the NCHW-strided extension
    auto physical = [](TensorDesc const& t) { return std::array<std::int64_t, 4>{t.dim[0], t.dim[2], t.dim[3], t.dim[1]}; };
    metadata.function_name = options.importer.function_name;
    metadata.x_uid = *x;
    metadata.w_uid = *w;
    metadata.y_uid = *y;
    metadata.x_shape = physical(tx);
    metadata.w_shape = physical(tw);
    metadata.y_shape = physical(ty);
    metadata.padded_x_shape = metadata.x_shape;
    metadata.padded_x_shape[1] += (*pre)[0] + (*post)[0];
    metadata.padded_x_shape[2] += (*pre)[1] + (*post)[1];
    for (int i = 0; i < 2; ++i) {
        metadata.pre_padding[i] = (*pre)[i];
        metadata.post_padding[i] = (*post)[i];
        metadata.stride[i] = (*stride)[i];
        metadata.dilation[i] = (*dilation)[i];
    }
    metadata.arguments.clear();
    auto append = [&](std::int64_t uid, char const* name, std::array<std::int64_t, 4> const& shape, TensorAccess access) {
        TensorArgumentMetadata argument;
        argument.uid = uid;
        argument.name = name;
        argument.data_type = DataType::kFloat32;
        argument.dimensions.assign(shape.begin(), shape.end());
        argument.strides = {shape[1] * shape[2] * shape[3], shape[2] * shape[3], shape[3], 1};
        argument.size_bytes = static_cast<std::uint64_t>(shape[0] * shape[1] * shape[2] * shape[3]) * 4;
        argument.alignment = alignof(float);
        argument.access = access;
        metadata.arguments.push_back(std::move(argument));
    };
    append(*x, "X", metadata.x_shape, TensorAccess::kRead);
    append(*w, "W", metadata.w_shape, TensorAccess::kRead);
    append(*y, "Y", metadata.y_shape, TensorAccess::kWrite);
    return true;
}

// A correctly rounded double -> binary16 / bfloat16 (round to nearest even), as the reference narrows an embedded
// HALF / BFLOAT16 scalar from the JSON number (FloatAttr::get(type, double), lib/Compiler/FoundationalGraph.cpp:2193-2200).
std::uint16_t narrow_double(double value, int exponent_bits, int mantissa_bits) {
    auto const bits = std::bit_cast<std::uint64_t>(value);
    auto const sign = static_cast<std::uint16_t>((bits >> 63) << (exponent_bits + mantissa_bits));
    auto const exponent_mask = static_cast<std::uint16_t>(((1u << exponent_bits) - 1u) << mantissa_bits);
    if (std::isnan(value)) return static_cast<std::uint16_t>(sign | exponent_mask | (1u << (mantissa_bits - 1)));
    double const magnitude = std::fabs(value);
    int const bias = (1 << (exponent_bits - 1)) - 1;
    if (std::isinf(value)) return static_cast<std::uint16_t>(sign | exponent_mask);
    if (magnitude == 0.0) return sign;
    int exponent = 0;
    (void)std::frexp(magnitude, &exponent);          // magnitude = f * 2^exponent, f in [0.5, 1)
    int unbiased = std::max(exponent - 1, 1 - bias);  // subnormals share the smallest normal exponent
    // magnitude / 2^(unbiased - mantissa_bits) is exact in double for every finite input; nearbyint rounds to even
    double const scaled = std::nearbyint(std::ldexp(magnitude, mantissa_bits - unbiased));
    auto mantissa = static_cast<std::uint64_t>(scaled);  // in [0, 2^(mantissa_bits + 1)]
    std::uint64_t encoded = 0;
    if (mantissa < (1ull << mantissa_bits)) encoded = mantissa;  // subnormal (or zero after rounding)
    else encoded = (static_cast<std::uint64_t>(unbiased + bias - 1) << mantissa_bits) + mantissa;  // a carry into 2^(m+1) bumps the exponent by itself
    if (encoded >= exponent_mask) encoded = exponent_mask;  // overflow rounds to infinity
    return static_cast<std::uint16_t>(sign | encoded);
}

// The stored bits of an embedded scalar, as its tensor's data type holds the value (pass_by_value_initializer,
// lib/Compiler/FoundationalGraph.cpp:2165-2214).
void constant_bits(TensorDesc const& tensor, std::uint64_t& bits, std::int32_t& bytes) {
    auto const& scalar = *tensor.pass_by_value;
    switch (scalar.kind) {
        case import::PassByValueKind::kInt64: bits = static_cast<std::uint64_t>(std::get<std::int64_t>(scalar.value)); bytes = 8; break;
        case import::PassByValueKind::kInt32: bits = static_cast<std::uint32_t>(std::get<std::int32_t>(scalar.value)); bytes = 4; break;
        case import::PassByValueKind::kFloat32: bits = std::get<std::uint32_t>(scalar.value); bytes = 4; break;
        case import::PassByValueKind::kFloat64: bits = std::get<std::uint64_t>(scalar.value); bytes = 8; break;
        case import::PassByValueKind::kFloat16: bits = narrow_double(std::bit_cast<double>(std::get<std::uint64_t>(scalar.value)), 5, 10); bytes = 2; break;
        case import::PassByValueKind::kBFloat16: bits = narrow_double(std::bit_cast<double>(std::get<std::uint64_t>(scalar.value)), 8, 7); bytes = 2; break;
    }
}

// Graph-owned constants that some launch reads are written into their workspace slots by launches at the head of the
// plan (DFGPU_MAX_CONSTANTS each): their lifetime then runs from the first step to their last reader.
void materialise_constants(Lowering& low) {
    std::set<std::int64_t> wanted;
    for (auto const& step : low.plan.steps)
        for (auto const& binding : step.tensors)
            if (binding.kind == TensorBinding::Kind::kWorkspace && low.tensor(binding.uid).pass_by_value) wanted.insert(binding.uid);
    std::vector<KernelStep> head;
    KernelStep fill;
    auto flush = [&] {
        if (fill.tensors.empty()) return;
        fill.op = KernelOp::kConstants;
        fill.label = "constants";
        head.push_back(std::move(fill));
        fill = KernelStep{};
    };
    dfgpu_constants_params params{};
    for (auto uid : wanted) {
        constant_bits(low.tensor(uid), params.bits[params.count], params.bytes[params.count]);
        ++params.count;
        fill.tensors.push_back(low.bind(uid));
        fill.params = params;
        if (params.count == DFGPU_MAX_CONSTANTS) {
            flush();
            params = dfgpu_constants_params{};
        }
    }
    flush();
    low.plan.steps.insert(low.plan.steps.begin(), std::make_move_iterator(head.begin()), std::make_move_iterator(head.end()));
}

// Alignment the resolved kernel's launcher demands of the pointer in tensor slot `slot` (0: no demand of its own).
// The TMA-fed kernels read and write 16-byte units and have no narrower fallback (the block-scale launchers do).
std::uint64_t kernel_alignment(KernelStep const& step, std::size_t slot) {
    switch (step.op) {
        case KernelOp::kConvFprop: return step.kernel == DFGPU_CONV_UMMA_BF16 || step.kernel == DFGPU_CONV_UMMA_F32X3 ? 16 : 0;  // (the one-launch f32 form takes any pointer: see dfgpu_conv_fprop)
        case KernelOp::kMatmul:
            if (step.kernel != DFGPU_MATMUL_UMMA_BF16 && step.kernel != DFGPU_MATMUL_UMMA_MXF8 && step.kernel != DFGPU_MATMUL_UMMA_F32X3) return 0;
            return slot == 3 || slot == 4 ? 4 : 16;  // the scale tensors are gathered with 4-byte loads
        case KernelOp::kSdpaForward:
            if (step.kernel == DFGPU_SDPA_UMMA) return slot <= 3 ? 16 : 0;
            if (step.kernel == DFGPU_SDPA_PAGED_DECODE_UMMA || step.kernel == DFGPU_SDPA_PAGED_DECODE) return slot <= 2 ? 16 : 0;
            return 0;
        case KernelOp::kMatmulFp8: return step.kernel == DFGPU_MATMUL_FP8_UMMA && slot <= 2 ? 16 : 0;
        case KernelOp::kConvFpropPair: return 16;
        case KernelOp::kBlockScaleQuantizePair: return slot % 3 == 0 ? 16 : 8;
        case KernelOp::kBlockScaleQuantize:   // packed FP4 codes are written a nibble at a time through their aligned word
            return slot == 1 && std::get<dfgpu_bsq_params>(step.params).y.dtype == DFGPU_FP4 ? 4 : 0;
        default: return 0;
    }
}

}  // namespace

Status query_kernel_step(KernelStep& step, std::int64_t& scratch_bytes) {
    dfgpu_plan_info info{};
    int code = 0;
    switch (step.op) {
        case KernelOp::kBlockScaleQuantize: code = dfgpu_query_block_scale_quantize(&std::get<dfgpu_bsq_params>(step.params), &info); break;
        case KernelOp::kBlockScaleDequantize: code = dfgpu_query_block_scale_dequantize(&std::get<dfgpu_bsd_params>(step.params), &info); break;
        case KernelOp::kPointwise: code = dfgpu_query_pointwise(&std::get<dfgpu_pointwise_params>(step.params), &info); break;
        case KernelOp::kConvFprop: code = dfgpu_query_conv_fprop(&std::get<dfgpu_conv_params>(step.params), &info); break;
        case KernelOp::kMatmul: code = dfgpu_query_matmul(&std::get<dfgpu_matmul_params>(step.params), &info); break;
        case KernelOp::kSdpaForward: code = dfgpu_query_sdpa_forward(&std::get<dfgpu_sdpa_params>(step.params), &info); break;
        case KernelOp::kMatmulFp8: code = dfgpu_query_matmul_fp8(&std::get<dfgpu_matmul_fp8_params>(step.params), &info); break;
        case KernelOp::kConvFpropPair: code = dfgpu_query_conv_fprop_pair(&std::get<dfgpu_conv_pair_params>(step.params), &info); break;
        case KernelOp::kBlockScaleQuantizePair: code = dfgpu_query_block_scale_quantize_pair(&std::get<dfgpu_bsq_pair_params>(step.params), &info); break;
        case KernelOp::kConstants: code = dfgpu_query_constants(&std::get<dfgpu_constants_params>(step.params), &info); break;
    }
    if (code != 0) return Status::failure(static_cast<ErrorCode>(code), step.label, dfgpu_last_error());
    step.kernel = info.kernel;
    step.launches = info.launches;
    scratch_bytes = info.scratch_bytes;
    return Status::ok();
}


char const* kernel_op_name(KernelOp op) {
    switch (op) {
        case KernelOp::kBlockScaleQuantize: return "block_scale_quantize";
        case KernelOp::kBlockScaleDequantize: return "block_scale_dequantize";
        case KernelOp::kPointwise: return "pointwise";
        case KernelOp::kConvFprop: return "conv_fprop";
        case KernelOp::kMatmul: return "matmul";
        case KernelOp::kSdpaForward: return "sdpa_forward";
        case KernelOp::kMatmulFp8: return "matmul_fp8";
        case KernelOp::kConvFpropPair: return "conv_fprop_pair";
        case KernelOp::kBlockScaleQuantizePair: return "block_scale_quantize_pair";
        case KernelOp::kConstants: return "constants";
    }
    return "?";
}

std::string KernelPlan::to_text() const {
    std::ostringstream out;
    for (std::size_t i = 0; i < steps.size(); ++i) {
        auto const& step = steps[i];
        out << i << ": " << kernel_op_name(step.op) << " kernel=" << step.kernel << " launches=" << step.launches << " [" << step.label << "]";
        for (auto const& binding : step.tensors) {
            if (binding.kind == TensorBinding::Kind::kAbsent) out << " -";
            else if (binding.kind == TensorBinding::Kind::kArgument) out << " uid" << binding.uid;
            else out << " ws+" << binding.offset << "(uid" << binding.uid << ")";
        }
        if (step.scratch.kind == TensorBinding::Kind::kWorkspace) out << " scratch=ws+" << step.scratch.offset;
        out << "\n";
    }
    return out.str();
}

Status compile_graph(SerializedGraph const& graph, CompileOptions const& options, CompilationResult& output) {
    if (graph.nodes.empty()) return fail(ErrorCode::kInvalidValue, "graph", "graph has no nodes");
    if (graph.context.is_override_shape_enabled.value_or(false))
        return fail(ErrorCode::kUnsupportedOperation, "context.is_override_shape_enabled", "shape overrides are not executable on this backend");
    Lowering low(graph, options);
    for (std::size_t index = 0; index < graph.nodes.size(); ++index) {
        for (auto const& [name, uid] : graph.nodes[index].inputs) {
            if (!graph.tensors.count(uid)) return fail(ErrorCode::kMissingUid, node_path(index, graph.nodes[index]), "tensor reference is unresolved");
            low.consumers[uid].push_back(index);
        }
        for (auto const& [name, uid] : graph.nodes[index].outputs) {
            if (!graph.tensors.count(uid)) return fail(ErrorCode::kMissingUid, node_path(index, graph.nodes[index]), "tensor reference is unresolved");
            if (low.producer.count(uid)) return fail(ErrorCode::kInvalidValue, node_path(index, graph.nodes[index]), "tensor is produced twice");
            for (auto const& [input_name, input_uid] : graph.nodes[index].inputs)  // lib/Compiler/FoundationalGraph.cpp:1897-1906
                if (input_uid == uid) return fail(ErrorCode::kUnsupportedOperation, node_path(index, graph.nodes[index]), "in-place reuse of a tensor UID by one operation is unsupported");
            low.producer[uid] = static_cast<int>(index);
        }
    }
    for (auto const& [uid, tensor] : graph.tensors)
        if (tensor.is_virtual && !low.producer.count(uid)) return fail(ErrorCode::kInvalidValue, "tensors." + std::to_string(uid), "virtual tensor has no producer");
    // pass-by-value scalars (validate_tensor, lib/Compiler/FoundationalGraph.cpp:411-490; input-only, :1870-1876)
    for (auto const& [uid, tensor] : graph.tensors) {
        if (!tensor.is_pass_by_value) continue;
        auto const path = "tensors." + std::to_string(uid);
        switch (tensor.data_type) {
            case DataType::kInt64: case DataType::kInt32: case DataType::kFloat16: case DataType::kFloat32: case DataType::kFloat64: case DataType::kBFloat16: break;
            default: return fail(ErrorCode::kUnsupportedDataType, path, "runtime pass-by-value scalar type is outside the cuDNN Frontend scalar set");
        }
        if (tensor.is_virtual || tensor.ragged_offset_uid || tensor.ragged_offset_name || tensor.reordering_type != "NONE")
            return fail(ErrorCode::kUnsupportedOperation, path, "pass-by-value requires an external plain tensor");
        if (!std::all_of(tensor.dim.begin(), tensor.dim.end(), [](std::int64_t extent) { return extent == 1; }))
            return fail(ErrorCode::kUnsupportedOperation, path, "pass-by-value requires every dimension to equal one");
        if (low.producer.count(uid)) return fail(ErrorCode::kUnsupportedOperation, path, "pass-by-value tensors are input-only");
    }

    // dequantize nodes that a later MATMUL will absorb must not be emitted on their own:
    // decide that first, by lowering MATMULs' operand fusion lazily in node order.
    std::vector<std::size_t> order;
    for (std::size_t index = 0; index < graph.nodes.size(); ++index) order.push_back(index);
    // First pass: find absorbable dequantize producers.
    if (options.fuse) {
        for (std::size_t index = 0; index < graph.nodes.size(); ++index) {
            if (graph.nodes[index].tag != OperationTag::kMatmul) continue;
            for (auto name : {"A", "B"}) {
                auto uid = port(graph.nodes[index].inputs, name);
                if (!uid) continue;
                dfgpu_tensor operand{}, scale{};
                std::int64_t block[2] = {1, 1}, codes = 0, scales = 0;
                std::size_t dequant = 0;
                if (try_absorb_dequantize(low, index, *uid, operand, scale, block, codes, scales, dequant)) low.absorbed_into[dequant] = static_cast<int>(index);
            }
        }
    }
    for (std::size_t index : order) {
        if (low.absorbed_into[index] >= 0) continue;
        Status status = Status::ok();
        switch (graph.nodes[index].tag) {
            case OperationTag::kConvFprop: status = lower_conv(low, index); break;
            case OperationTag::kMatmul: status = lower_matmul(low, index); break;
            case OperationTag::kPointwise: status = lower_pointwise(low, index); break;
            case OperationTag::kBlockScaleQuantize: status = lower_quantize(low, index); break;
            case OperationTag::kBlockScaleDequantize: status = lower_dequantize(low, index); break;
            case OperationTag::kSdpa: status = lower_sdpa(low, index); break;
            case OperationTag::kMatmulFp8: status = lower_matmul_fp8(low, index); break;
        }
        if (status.is_bad()) return status;
    }
    narrow_virtual_tensors(low);
    split_virtual_tensors(low);
    fuse_convolution_pairs(low);
    fuse_quantize_pairs(low);
    materialise_constants(low);

    // argument table: ascending UID, non-virtual tensors only
    Conv2DCompileMetadata metadata;
    metadata.function_name = options.foundational_function_name;
    for (auto const& [uid, tensor] : graph.tensors) {
        if (tensor.is_virtual || tensor.pass_by_value) continue;  // a graph-owned constant is no argument: a pointer passed for it is ignored
        TensorArgumentMetadata argument;
        argument.uid = uid;
        argument.name = tensor.name;
        argument.data_type = tensor.data_type;
        argument.dimensions = tensor.dim;
        argument.strides = tensor.stride;
        if (!import::tensor_storage_bytes(tensor, argument.size_bytes)) return fail(ErrorCode::kDimensionOverflow, tensor.name, "storage span overflows int64");
        std::uint64_t element_bytes = std::max<std::uint64_t>(1, import::data_type_storage_bits(tensor.data_type) / 8);
        argument.alignment = std::clamp<std::uint64_t>(element_bytes, 1, 8);
        bool read = low.consumers.count(uid) != 0, written = low.producer.count(uid) != 0;
        argument.access = read && written ? TensorAccess::kReadWrite : (written ? TensorAccess::kWrite : TensorAccess::kRead);
        metadata.arguments.push_back(std::move(argument));
    }
    // compact page tables: ragged batch-prefix storage, bounded by B * inner span (lib/Compiler/FoundationalGraph.cpp:2070-2095)
    for (auto const& step : low.plan.steps) {
        if (step.op != KernelOp::kSdpaForward) continue;
        auto const& params = std::get<dfgpu_sdpa_params>(step.params);
        for (int which = 0; which < 2; ++which) {
            auto const& offsets = step.tensors[14 + which];
            if (offsets.kind == TensorBinding::Kind::kAbsent) continue;
            auto const table_uid = step.tensors[9 + which].uid;
            for (auto& argument : metadata.arguments) {
                if (argument.uid != table_uid) continue;
                argument.storage_policy = TensorStoragePolicy::kRaggedBatchPrefix;
                argument.ragged_offset_uid = offsets.uid;
                argument.ragged_sequence_uid = step.tensors[8].uid;
                argument.ragged_sequence_divisor = which ? params.v.dim[2] : params.k.dim[2];
                std::uint64_t inner = 1;
                for (std::size_t axis = 1; axis < argument.dimensions.size(); ++axis) inner += static_cast<std::uint64_t>(argument.dimensions[axis] - 1) * static_cast<std::uint64_t>(argument.strides[axis]);
                argument.size_bytes = static_cast<std::uint64_t>(argument.dimensions[0]) * inner * 4;
            }
        }
    }
    Status status = Status::ok();
    // The reference's single-node path (one f32 CONV_FPROP on packed NHWC / KRSC tensors) carries its own metadata
    // and argument convention (lib/MLIR/Conv2DImporter.cpp:332-370): X, W, Y by those names, physical shapes.
    bool const conv_adapter = single_conv_metadata(graph, options, metadata);

    // kernel queries + workspace requests (lifetimes in plan-step indices)
    std::vector<WorkspaceRequest> requests;
    std::map<std::int64_t, std::pair<std::size_t, std::size_t>> lifetime;
    for (std::size_t s = 0; s < low.plan.steps.size(); ++s) {
        auto& step = low.plan.steps[s];
        std::int64_t scratch = 0;
        if ((status = query_kernel_step(step, scratch)).is_bad()) return status;
        for (auto const& binding : step.tensors) {
            if (binding.kind != TensorBinding::Kind::kWorkspace) continue;
            auto it = lifetime.find(binding.uid);
            if (it == lifetime.end()) lifetime[binding.uid] = {s, s};
            else it->second.second = s;
        }
        if (scratch > 0) {
            requests.push_back({"scratch." + std::to_string(s), static_cast<std::uint64_t>(scratch), kWorkspaceAlignment, s, s});
            step.scratch.kind = TensorBinding::Kind::kWorkspace;
        }
        // The reference's rule is alignment = clamp(element bytes, 1, 8); the TMA-fed kernels need 16, and saying so in
        // the argument table makes execute() refuse a misaligned pack up front (DFE_INVALID_VARIANT_PACK) instead of
        // part-way through the plan.
        for (std::size_t slot = 0; slot < step.tensors.size(); ++slot)
            if (step.tensors[slot].kind == TensorBinding::Kind::kArgument)
                for (auto& argument : metadata.arguments)
                    if (argument.uid == step.tensors[slot].uid) argument.alignment = std::max(argument.alignment, kernel_alignment(step, slot));
    }
    if ((status = validate_graph_compile_metadata(metadata)).is_bad()) return status;
    for (auto const& [uid, range] : lifetime) {
        auto tensor = graph.tensors.at(uid);
        auto narrowed = low.storage_override.find(uid);
        if (narrowed != low.storage_override.end() && narrowed->second == DFGPU_BF16) tensor.data_type = DataType::kBFloat16;  // a (hi, lo) pair keeps FLOAT's 4 bytes
        std::uint64_t bytes = 0;
        if (!import::tensor_storage_bytes(tensor, bytes)) return fail(ErrorCode::kDimensionOverflow, tensor.name, "storage span overflows int64");
        requests.push_back({tensor.name, bytes, kWorkspaceAlignment, range.first, range.second});
    }
    WorkspacePlan workspace;
    if ((status = plan_workspace(requests, workspace)).is_bad()) return status;
    std::map<std::string, std::uint64_t> offsets;
    for (auto const& allocation : workspace.allocations) offsets[allocation.name] = allocation.offset;
    for (std::size_t s = 0; s < low.plan.steps.size(); ++s) {
        auto& step = low.plan.steps[s];
        for (auto& binding : step.tensors)
            if (binding.kind == TensorBinding::Kind::kWorkspace) binding.offset = offsets.at(graph.tensors.at(binding.uid).name);
        if (step.scratch.kind == TensorBinding::Kind::kWorkspace) step.scratch.offset = offsets.at("scratch." + std::to_string(s));
    }

    if (conv_adapter && (status = validate_conv2d_adapter_metadata(metadata)).is_bad()) return status;
    output.adapter_kind = conv_adapter ? InvocationAdapterKind::kConv2DRankedMemref : InvocationAdapterKind::kGenericRankedMemrefPointerTable;
    output.metadata = metadata;
    output.workspace = workspace;
    output.plan = low.plan;
    output.target_triple = "sm_100a";
    output.variants = {};
    output.variants[0].variant = runtime::CpuVariant::kScalar;
    output.variants[0].symbol = metadata.function_name;
    output.variants[0].required_features = "sm_100a";
    output.variants[0].schedule = "kernel-plan";
    output.variants[1].variant = runtime::CpuVariant::kAvx2;
    output.variants[2].variant = runtime::CpuVariant::kAvx512;
    output.executable = runtime::ExecutableFactory::create(metadata, workspace, low.plan);
    return Status::ok();
}

Status compile_file(std::filesystem::path const& path, CompileOptions const& options, CompilationResult& output) {
    import::SerializedGraph graph;
    import::SerializedGraphImporter importer;
    auto status = importer.parse_file(path, options.input_format, graph);
    if (status.is_bad()) return status;
    return compile_graph(graph, options, output);
}

Status validate_conv2d_adapter_metadata(Conv2DCompileMetadata const& metadata) {
    if (metadata.arguments.size() != 3) return fail(ErrorCode::kInvalidValue, "metadata.arguments", "Conv adapter requires a function name and three arguments");
    if (metadata.dynamic_shape_enabled || metadata.override_shape_enabled || metadata.override_policy != ShapeOverridePolicy::kNone)
        return fail(ErrorCode::kInvalidValue, "metadata.override", "Conv adapter does not support dynamic or override metadata");
    for (auto const& argument : metadata.arguments)
        if (argument.data_type != DataType::kFloat32 || argument.dimensions.size() != 4)
            return fail(ErrorCode::kInvalidValue, "metadata.arguments", "Conv adapter requires rank-4 FLOAT arguments");
    auto const &x = metadata.arguments[0], &w = metadata.arguments[1], &y = metadata.arguments[2];
    auto same = [](TensorArgumentMetadata const& argument, std::array<std::int64_t, 4> const& shape) {
        return std::equal(argument.dimensions.begin(), argument.dimensions.end(), shape.begin());
    };
    bool const matches = x.uid == metadata.x_uid && w.uid == metadata.w_uid && y.uid == metadata.y_uid && x.name == "X" && w.name == "W" && y.name == "Y" &&
                         x.access == TensorAccess::kRead && w.access == TensorAccess::kRead && y.access == TensorAccess::kWrite &&
                         same(x, metadata.x_shape) && same(w, metadata.w_shape) && same(y, metadata.y_shape);
    if (!matches) return fail(ErrorCode::kInvalidValue, "metadata.arguments", "argument table does not match the Conv adapter");
    return Status::ok();
}

Status validate_graph_compile_metadata(GraphCompileMetadata const& metadata) {
    if (metadata.arguments.empty() || metadata.arguments.size() > 4096) return fail(ErrorCode::kInvalidValue, "metadata", "argument count must be between 1 and 4096");
    // no override or dynamic-shape metadata on this backend (override_shape_enabled == (policy != none) in the reference)
    if (metadata.dynamic_shape_enabled || metadata.override_shape_enabled || metadata.override_policy != ShapeOverridePolicy::kNone ||
        !metadata.override_role_uids.empty() || !metadata.override_axis_map.empty())
        return fail(ErrorCode::kInvalidValue, "metadata.override", "shape-override metadata is not executable on this backend");
    for (auto const& argument : metadata.arguments) {
        if (argument.storage_policy == TensorStoragePolicy::kStrided) {
            if (argument.ragged_offset_uid != 0 || argument.ragged_sequence_uid != 0 || argument.ragged_sequence_divisor != 1)
                return fail(ErrorCode::kInvalidValue, argument.name, "a strided argument carries no ragged references and divisor 1");
            continue;
        }
        // ragged batch prefix (compact page tables): an INT32 [B,1,P,1] table whose offsets and sequence lengths are arguments too
        auto is_argument = [&](std::int64_t uid) { return std::any_of(metadata.arguments.begin(), metadata.arguments.end(), [&](auto const& other) { return other.uid == uid && other.uid != argument.uid; }); };
        if (argument.storage_policy != TensorStoragePolicy::kRaggedBatchPrefix || argument.data_type != import::DataType::kInt32 || argument.dimensions.size() != 4 ||
            !is_argument(argument.ragged_offset_uid) || !is_argument(argument.ragged_sequence_uid) || argument.ragged_sequence_divisor < 1)
            return fail(ErrorCode::kInvalidValue, argument.name, "ragged metadata references are unresolved");
    }
    std::set<std::int64_t> uids;
    for (auto const& argument : metadata.arguments) {
        if (!uids.insert(argument.uid).second) return fail(ErrorCode::kDuplicateUid, argument.name, "argument UID is used twice");
        if (argument.name.empty() || argument.name.find('\0') != std::string::npos) return fail(ErrorCode::kInvalidValue, "metadata", "argument names must be non-empty and NUL-free");
        if (argument.dimensions.empty() || argument.dimensions.size() > 64 || argument.dimensions.size() != argument.strides.size())
            return fail(ErrorCode::kInvalidShape, argument.name, "rank must be between 1 and 64 with matching strides");
        if (argument.alignment == 0 || (argument.alignment & (argument.alignment - 1)) != 0 || argument.alignment > 4096)
            return fail(ErrorCode::kInvalidValue, argument.name, "alignment must be a power of two no greater than 4096");
        // size_bytes is the storage span of the strided view, or the full extent product for a reordered (F8_128x4) tensor
        import::TensorDesc view;
        view.data_type = argument.data_type;
        view.dim = argument.dimensions;
        view.stride = argument.strides;
        view.reordering_type = "NONE";
        std::uint64_t strided = 0, reordered = 0;
        if (!import::tensor_storage_bytes(view, strided)) return fail(ErrorCode::kInvalidShape, argument.name, "extents, strides or data type do not give a storage span");
        view.reordering_type = "F8_128x4";
        (void)import::tensor_storage_bytes(view, reordered);
        std::uint64_t ragged = 0;
        if (argument.storage_policy == TensorStoragePolicy::kRaggedBatchPrefix) {
            std::uint64_t inner = 1;
            for (std::size_t axis = 1; axis < argument.dimensions.size(); ++axis) inner += static_cast<std::uint64_t>(argument.dimensions[axis] - 1) * static_cast<std::uint64_t>(argument.strides[axis]);
            ragged = static_cast<std::uint64_t>(argument.dimensions[0]) * inner * std::max<std::uint64_t>(1, import::data_type_storage_bits(argument.data_type) / 8);
            if (argument.size_bytes != ragged) return fail(ErrorCode::kInvalidValue, argument.name, "size_bytes is not the ragged storage bound of the tensor");
            continue;
        }
        if (argument.size_bytes != strided && argument.size_bytes != reordered)
            return fail(ErrorCode::kInvalidValue, argument.name, "size_bytes is not the storage span of the tensor");
    }
    return Status::ok();
}

}  // namespace deepforge::compiler

// Runtime: variant-pack validation, then the kernel plan's launches through the dfgpu ABI.
//
// Validation order and error codes follow the reference's execute_variant
// (lib/Runtime/Executable.cpp:1023-1223): every argument UID present, non-null and
// aligned; no two argument byte ranges overlap when either is written; workspace
// non-null (when needed), 64-byte aligned and disjoint from every argument. All of these
// are DFE_INVALID_VARIANT_PACK. Extra UIDs in the pack and the handle are ignored.
// Pointers are device pointers: they are compared and offset, never dereferenced here.
#include "Internal.h"

#include <mutex>

namespace deepforge::runtime {

using compiler::KernelOp;
using compiler::KernelStep;
using compiler::TensorAccess;
using compiler::TensorBinding;
using import::ErrorCode;
using import::Status;

struct Executable::Impl {
    compiler::GraphCompileMetadata metadata;
    compiler::WorkspacePlan workspace;
    compiler::KernelPlan plan;
    void* stream = nullptr;
    std::int64_t launches = 0;
    mutable std::mutex mutex;
};

std::string_view cpu_variant_name(CpuVariant variant) noexcept {
    switch (variant) {
        case CpuVariant::kScalar: return "scalar";
        case CpuVariant::kAvx2: return "avx2";
        case CpuVariant::kAvx512: return "avx512";
    }
    return "unknown";
}

Executable::Executable(std::unique_ptr<Impl> impl) : impl_(std::move(impl)) {}
Executable::~Executable() = default;
Executable::Executable(Executable&&) noexcept = default;
Executable& Executable::operator=(Executable&&) noexcept = default;

std::unique_ptr<Executable> ExecutableFactory::create(compiler::GraphCompileMetadata metadata, compiler::WorkspacePlan workspace,
                                                      compiler::KernelPlan plan) {
    auto impl = std::make_unique<Executable::Impl>();
    impl->metadata = std::move(metadata);
    impl->workspace = std::move(workspace);
    impl->plan = std::move(plan);
    for (auto const& step : impl->plan.steps) impl->launches += step.launches;
    return std::unique_ptr<Executable>(new Executable(std::move(impl)));
}

std::int64_t Executable::get_workspace_size() const noexcept { return static_cast<std::int64_t>(impl_->workspace.size_bytes); }

Status Executable::get_workspace_size(std::int64_t& workspace_size) const {
    workspace_size = get_workspace_size();
    return Status::ok();
}

namespace {
Status reject_overrides(OverrideUids const& uids, OverrideShapes const& shapes, OverrideStrides const& strides) {
    if (uids.empty() && shapes.empty() && strides.empty()) return Status::ok();
    return Status::failure(ErrorCode::kInvalidVariantPack, "override", "the graph was compiled without shape overrides");
}
}  // namespace

Status Executable::get_workspace_size(FrontendHandle, std::int64_t& workspace_size, OverrideUids const& uids, OverrideShapes const& shapes,
                                      OverrideStrides const& strides) const {
    auto status = reject_overrides(uids, shapes, strides);
    if (status.is_bad()) return status;
    return get_workspace_size(workspace_size);
}

std::int64_t Executable::get_workspace_size(FrontendHandle, OverrideUids const& uids, OverrideShapes const& shapes, OverrideStrides const& strides) const {
    return reject_overrides(uids, shapes, strides).is_good() ? get_workspace_size() : -1;
}

bool Executable::supports_variant(CpuVariant variant) const noexcept { return variant == CpuVariant::kScalar; }
CpuVariant Executable::selected_variant() const noexcept { return CpuVariant::kScalar; }
void Executable::set_stream(void* stream) noexcept {
    std::lock_guard<std::mutex> lock(impl_->mutex);
    impl_->stream = stream;
}

Status Executable::execute_on(void* stream, VariantPack& pack, void* workspace) const {
    return run_steps(0, static_cast<std::int64_t>(impl_->plan.steps.size()), pack, workspace, stream, true);
}
std::int64_t Executable::launch_count() const noexcept { return impl_->launches; }
std::string Executable::plan_text() const { return impl_->plan.to_text(); }

Status Executable::execute(FrontendHandle handle, VariantPack& pack, void* workspace) const {
    return execute_variant(CpuVariant::kScalar, handle, pack, workspace);
}

Status Executable::execute(FrontendHandle handle, VariantPack& pack, void* workspace, OverrideUids const& uids, OverrideShapes const& shapes,
                           OverrideStrides const& strides) const {
    return execute_variant(CpuVariant::kScalar, handle, pack, workspace, uids, shapes, strides);
}

Status Executable::execute_variant(CpuVariant variant, FrontendHandle handle, VariantPack& pack, void* workspace, OverrideUids const& uids,
                                   OverrideShapes const& shapes, OverrideStrides const& strides) const {
    auto status = reject_overrides(uids, shapes, strides);
    if (status.is_bad()) return status;
    return execute_variant(variant, handle, pack, workspace);
}

Status Executable::execute_variant(CpuVariant variant, FrontendHandle, VariantPack& pack, void* workspace) const {
    if (!supports_variant(variant))
        return Status::failure(ErrorCode::kUnsupportedCpuFeature, cpu_variant_name(variant), "this executable carries one sm_100a kernel plan; use the scalar variant name");
    return execute_steps(0, static_cast<std::int64_t>(impl_->plan.steps.size()), pack, workspace);
}

Status Executable::execute_steps(std::int64_t first, std::int64_t last, VariantPack& pack, void* workspace) const {
    return run_steps(first, last, pack, workspace, nullptr, false);
}

Status Executable::run_steps(std::int64_t first, std::int64_t last, VariantPack& pack, void* workspace, void* call_stream, bool own_stream) const {
    auto const& impl = *impl_;
    if (first < 0 || last > static_cast<std::int64_t>(impl.plan.steps.size()) || first > last)
        return Status::failure(ErrorCode::kInvalidArgument, "steps", "step range is outside the kernel plan");

    struct Range {
        std::uintptr_t begin, end;
        bool written;
        std::string const* name;
    };
    std::vector<Range> ranges;
    ranges.reserve(impl.metadata.arguments.size());
    for (auto const& argument : impl.metadata.arguments) {
        auto it = pack.find(argument.uid);
        if (it == pack.end()) return Status::failure(ErrorCode::kInvalidVariantPack, argument.name, "UID " + std::to_string(argument.uid) + " is missing from the variant pack");
        if (it->second == nullptr) return Status::failure(ErrorCode::kInvalidVariantPack, argument.name, "pointer is null");
        auto address = reinterpret_cast<std::uintptr_t>(it->second);
        if (address % argument.alignment != 0) return Status::failure(ErrorCode::kInvalidVariantPack, argument.name, "pointer is not aligned to " + std::to_string(argument.alignment) + " bytes");
        ranges.push_back({address, address + argument.size_bytes, argument.access != TensorAccess::kRead, &argument.name});
    }
    for (std::size_t i = 0; i < ranges.size(); ++i)
        for (std::size_t j = i + 1; j < ranges.size(); ++j)
            if ((ranges[i].written || ranges[j].written) && ranges[i].begin < ranges[j].end && ranges[j].begin < ranges[i].end)
                return Status::failure(ErrorCode::kInvalidVariantPack, *ranges[i].name, "storage overlaps '" + *ranges[j].name + "' and at least one of them is written");
    auto const workspace_bytes = impl.workspace.size_bytes;
    if (workspace_bytes != 0) {
        if (workspace == nullptr) return Status::failure(ErrorCode::kInvalidVariantPack, "workspace", "pointer is null but " + std::to_string(workspace_bytes) + " bytes are required");
        auto address = reinterpret_cast<std::uintptr_t>(workspace);
        if (address % compiler::kWorkspaceAlignment != 0) return Status::failure(ErrorCode::kInvalidVariantPack, "workspace", "pointer is not aligned to 64 bytes");
        for (auto const& range : ranges)
            if (address < range.end && range.begin < address + workspace_bytes)
                return Status::failure(ErrorCode::kInvalidVariantPack, "workspace", "storage overlaps '" + *range.name + "'");
    }

    // The plan is immutable and the launchers keep no state between calls, so a call with its own stream needs no
    // lock; calls on the shared stream take it, so that the launches of one plan stay together on that stream.
    std::unique_lock<std::mutex> lock(impl.mutex, std::defer_lock);
    void* stream = call_stream;
    if (!own_stream) {
        lock.lock();
        stream = impl.stream;
    }
    auto resolve = [&](TensorBinding const& binding) -> void* {
        switch (binding.kind) {
            case TensorBinding::Kind::kArgument: return pack.at(binding.uid);
            case TensorBinding::Kind::kWorkspace: return static_cast<char*>(workspace) + binding.offset;
            default: return nullptr;
        }
    };
    std::vector<void*> pointers;
    for (std::int64_t index = first; index < last; ++index) {
        auto const& step = impl.plan.steps[static_cast<std::size_t>(index)];
        pointers.clear();
        for (auto const& binding : step.tensors) pointers.push_back(resolve(binding));
        void* scratch = resolve(step.scratch);
        int code = 0;
        switch (step.op) {
            case KernelOp::kBlockScaleQuantize: code = dfgpu_block_scale_quantize(&std::get<dfgpu_bsq_params>(step.params), pointers.data(), scratch, stream); break;
            case KernelOp::kBlockScaleDequantize: code = dfgpu_block_scale_dequantize(&std::get<dfgpu_bsd_params>(step.params), pointers.data(), scratch, stream); break;
            case KernelOp::kConstants: code = dfgpu_constants(&std::get<dfgpu_constants_params>(step.params), pointers.data(), scratch, stream); break;
            case KernelOp::kPointwise: code = dfgpu_pointwise(&std::get<dfgpu_pointwise_params>(step.params), pointers.data(), scratch, stream); break;
            case KernelOp::kConvFprop: {
                // bit 1 of `reserved` (set by the lowering) promises that the kernel launched just before this one is the
                // plan's previous step; that does not hold for the first launch of a call
                dfgpu_conv_params params = std::get<dfgpu_conv_params>(step.params);
                if (index == first) params.reserved &= ~2;
                code = dfgpu_conv_fprop(&params, pointers.data(), scratch, stream);
                break;
            }
            case KernelOp::kMatmul: code = dfgpu_matmul(&std::get<dfgpu_matmul_params>(step.params), pointers.data(), scratch, stream); break;
            case KernelOp::kSdpaForward: code = dfgpu_sdpa_forward(&std::get<dfgpu_sdpa_params>(step.params), pointers.data(), scratch, stream); break;
            case KernelOp::kMatmulFp8: code = dfgpu_matmul_fp8(&std::get<dfgpu_matmul_fp8_params>(step.params), pointers.data(), scratch, stream); break;
            case KernelOp::kBlockScaleQuantizePair: code = dfgpu_block_scale_quantize_pair(&std::get<dfgpu_bsq_pair_params>(step.params), pointers.data(), scratch, stream); break;
            case KernelOp::kConvFpropPair: {
                dfgpu_conv_pair_params params = std::get<dfgpu_conv_pair_params>(step.params);
                if (index == first) params.first.reserved &= ~2;  // see kConvFprop above
                code = dfgpu_conv_fprop_pair(&params, pointers.data(), scratch, stream);
                break;
            }
        }
        if (code != 0) {
            auto mapped = code == 19 ? ErrorCode::kGraphExecutionFailed : static_cast<ErrorCode>(code);
            return Status::failure(mapped, step.label, dfgpu_last_error());
        }
    }
    return Status::ok();
}

}  // namespace deepforge::runtime

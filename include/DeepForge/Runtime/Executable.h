// The drop-in boundary: Frontend-shaped execute(handle, UID -> pointer map, workspace).
// Member signatures are those of the reference's include/DeepForge/Runtime/Executable.h
// :45-114 (and of cudnn-frontend v1.24.0's UID overloads); the pointers in the map and
// the workspace are DEVICE pointers here. No CUDA or compiler headers are included.
#pragma once

#include "DeepForge/Import/Status.h"

#include <cstdint>
#include <memory>
#include <string>
#include <string_view>
#include <unordered_map>
#include <vector>

namespace deepforge::runtime {

struct ExecutableFactory;

using FrontendHandle = void*;
using VariantPack = std::unordered_map<std::int64_t, void*>;
using OverrideUids = std::vector<std::int64_t>;
using OverrideShapes = std::vector<std::vector<std::int64_t>>;
using OverrideStrides = std::vector<std::vector<std::int64_t>>;

// Kept for source compatibility with callers that name a variant: there is one
// compiled variant (the sm_100a kernel plan) and every name maps to it.
enum class CpuVariant : std::uint8_t { kScalar = 0, kAvx2, kAvx512 };
[[nodiscard]] std::string_view cpu_variant_name(CpuVariant variant) noexcept;

class Executable final {
public:
    ~Executable();
    Executable(Executable&&) noexcept;
    Executable& operator=(Executable&&) noexcept;
    Executable(Executable const&) = delete;
    Executable& operator=(Executable const&) = delete;

    [[nodiscard]] import::Status get_workspace_size(std::int64_t& workspace_size) const;
    [[nodiscard]] import::Status get_workspace_size(FrontendHandle handle, std::int64_t& workspace_size,
                                                    OverrideUids const& override_uids,
                                                    OverrideShapes const& override_shapes,
                                                    OverrideStrides const& override_strides) const;
    [[nodiscard]] std::int64_t get_workspace_size() const noexcept;
    [[nodiscard]] std::int64_t get_workspace_size(FrontendHandle handle, OverrideUids const& override_uids,
                                                  OverrideShapes const& override_shapes,
                                                  OverrideStrides const& override_strides) const;

    // The handle is accepted for Frontend source compatibility and never inspected.
    // Launches are asynchronous on the stream set with set_stream(); the call returns
    // once every kernel of the plan is enqueued.
    [[nodiscard]] import::Status execute(FrontendHandle handle, VariantPack& uid_to_device_ptr, void* workspace) const;
    [[nodiscard]] import::Status execute(FrontendHandle handle, VariantPack& uid_to_device_ptr, void* workspace,
                                         OverrideUids const& override_uids, OverrideShapes const& override_shapes,
                                         OverrideStrides const& override_strides) const;
    [[nodiscard]] import::Status execute_variant(CpuVariant variant, FrontendHandle handle,
                                                 VariantPack& uid_to_device_ptr, void* workspace) const;
    [[nodiscard]] import::Status execute_variant(CpuVariant variant, FrontendHandle handle,
                                                 VariantPack& uid_to_device_ptr, void* workspace,
                                                 OverrideUids const& override_uids,
                                                 OverrideShapes const& override_shapes,
                                                 OverrideStrides const& override_strides) const;

    [[nodiscard]] bool supports_variant(CpuVariant variant) const noexcept;
    [[nodiscard]] CpuVariant selected_variant() const noexcept;

    // GPU-side additions (not in the reference): the CUDA stream launches go to (a
    // cudaStream_t, null = legacy default stream), the number of kernel launches one
    // execute() makes, and a text dump of the kernel plan.
    // Threading: concurrent execute() calls on one Executable are legal with distinct
    // workspaces and outputs, as in the reference (which serialises them with a mutex,
    // lib/Runtime/Executable.cpp:1154). Calls that share the stream of set_stream() are
    // enqueued one whole plan after the other (a lock is held while a call enqueues);
    // execute_on() takes the stream per call and holds no lock, so calls on different
    // streams also overlap on the device. set_stream() takes the same lock.
    void set_stream(void* stream) noexcept;
    [[nodiscard]] import::Status execute_on(void* stream, VariantPack& uid_to_device_ptr, void* workspace) const;
    [[nodiscard]] std::int64_t launch_count() const noexcept;
    [[nodiscard]] std::string plan_text() const;
    // Runs plan steps [first, last) only, after the same validation as execute().
    [[nodiscard]] import::Status execute_steps(std::int64_t first, std::int64_t last, VariantPack& uid_to_device_ptr, void* workspace) const;

private:
    import::Status run_steps(std::int64_t first, std::int64_t last, VariantPack& pack, void* workspace, void* stream, bool own_stream) const;

public:

private:
    struct Impl;
    explicit Executable(std::unique_ptr<Impl> impl);
    friend struct ExecutableFactory;
    std::unique_ptr<Impl> impl_;
};

}  // namespace deepforge::runtime

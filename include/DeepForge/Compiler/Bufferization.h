// Static workspace planning for statically sized temporaries (virtual tensors and kernel
// scratch). Same request/plan types and placement rule as the reference's planner
// (include/DeepForge/Compiler/Bufferization.h:16-55, lib/Transforms/WorkspacePlanner.cpp).
#pragma once

#include "DeepForge/Import/Status.h"

#include <cstdint>
#include <span>
#include <string>
#include <vector>

namespace deepforge::compiler {

inline constexpr std::uint64_t kWorkspaceAlignment = 64;

struct WorkspaceRequest {
    std::string name;
    std::uint64_t size_bytes = 0;
    std::uint64_t alignment = kWorkspaceAlignment;
    std::uint64_t live_start = 0;
    std::uint64_t live_end = 0;
};

struct WorkspaceAllocation {
    std::string name;
    std::uint64_t offset = 0;
    std::uint64_t size_bytes = 0;
    std::uint64_t alignment = kWorkspaceAlignment;
    std::uint64_t live_start = 0;
    std::uint64_t live_end = 0;
    bool operator==(WorkspaceAllocation const&) const = default;
};

struct WorkspacePlan {
    std::uint64_t size_bytes = 0;
    std::uint64_t alignment = kWorkspaceAlignment;
    std::vector<WorkspaceAllocation> allocations;  // in placement order
    bool operator==(WorkspacePlan const&) const = default;
};

// Requests are placed in (live_start, live_end, name) order, each at the lowest aligned
// offset that does not collide with an already placed request whose lifetime overlaps.
// The total is rounded up to 64 bytes. `output` is untouched on failure.
[[nodiscard]] import::Status plan_workspace(std::span<WorkspaceRequest const> requests, WorkspacePlan& output);

}  // namespace deepforge::compiler

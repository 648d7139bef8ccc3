// Static first-fit workspace planner with lifetime sharing.
//
// Placement rule (the reference's lib/Transforms/WorkspacePlanner.cpp:71-182): visit
// requests ordered by (live_start, live_end, name); put each at the lowest offset,
// aligned to its alignment, whose byte range is disjoint from every already placed
// request with an overlapping [live_start, live_end]; bump past the furthest
// conflicting end and retry. Total = 64-byte rounded high watermark, must fit int64.
#include "DeepForge/Compiler/Bufferization.h"

#include <algorithm>
#include <limits>
#include <numeric>
#include <set>

namespace deepforge::compiler {
namespace {

using import::ErrorCode;
using import::Status;

constexpr std::uint64_t kMax = std::numeric_limits<std::uint64_t>::max();

bool round_up(std::uint64_t value, std::uint64_t alignment, std::uint64_t& out) {
    std::uint64_t remainder = value % alignment;
    if (remainder == 0) {
        out = value;
        return true;
    }
    std::uint64_t pad = alignment - remainder;
    if (value > kMax - pad) return false;
    out = value + pad;
    return true;
}

}  // namespace

Status plan_workspace(std::span<WorkspaceRequest const> requests, WorkspacePlan& output) {
    std::set<std::string_view> seen;
    for (auto const& r : requests) {
        if (r.name.empty()) return Status::failure(ErrorCode::kInvalidArgument, "workspace.request", "allocation name must not be empty");
        if (!seen.insert(r.name).second) return Status::failure(ErrorCode::kInvalidValue, "workspace.request", "allocation names must be unique");
        if (r.size_bytes == 0) return Status::failure(ErrorCode::kInvalidArgument, r.name, "allocation size must be positive");
        bool power_of_two = r.alignment != 0 && (r.alignment & (r.alignment - 1)) == 0;
        if (!power_of_two || r.alignment > kWorkspaceAlignment)
            return Status::failure(ErrorCode::kInvalidArgument, r.name, "alignment must be a power of two no greater than 64");
        if (r.live_start > r.live_end) return Status::failure(ErrorCode::kInvalidArgument, r.name, "lifetime start must not exceed lifetime end");
    }

    std::vector<std::size_t> order(requests.size());
    std::iota(order.begin(), order.end(), std::size_t{0});
    std::stable_sort(order.begin(), order.end(), [&](std::size_t a, std::size_t b) {
        auto const& x = requests[a];
        auto const& y = requests[b];
        return std::tie(x.live_start, x.live_end, x.name) < std::tie(y.live_start, y.live_end, y.name);
    });

    WorkspacePlan plan;
    std::uint64_t watermark = 0;
    for (std::size_t index : order) {
        auto const& r = requests[index];
        std::uint64_t offset = 0;
        for (;;) {
            if (!round_up(offset, r.alignment, offset)) return Status::failure(ErrorCode::kDimensionOverflow, r.name, "workspace offset alignment overflows uint64");
            if (offset > kMax - r.size_bytes) return Status::failure(ErrorCode::kDimensionOverflow, r.name, "workspace allocation range overflows uint64");
            std::uint64_t end = offset + r.size_bytes;
            std::uint64_t bump = 0;
            for (auto const& placed : plan.allocations) {
                bool alive_together = placed.live_start <= r.live_end && r.live_start <= placed.live_end;
                if (!alive_together) continue;
                std::uint64_t placed_end = placed.offset + placed.size_bytes;
                if (offset < placed_end && placed.offset < end) bump = std::max(bump, placed_end);
            }
            if (bump == 0) {
                plan.allocations.push_back({r.name, offset, r.size_bytes, r.alignment, r.live_start, r.live_end});
                watermark = std::max(watermark, end);
                break;
            }
            offset = bump;
        }
    }
    if (watermark != 0 && !round_up(watermark, kWorkspaceAlignment, plan.size_bytes))
        return Status::failure(ErrorCode::kDimensionOverflow, "workspace", "total workspace size overflows uint64");
    if (plan.size_bytes > static_cast<std::uint64_t>(std::numeric_limits<std::int64_t>::max()))
        return Status::failure(ErrorCode::kDimensionOverflow, "workspace", "total workspace size does not fit int64");
    output = std::move(plan);
    return Status::ok();
}

}  // namespace deepforge::compiler

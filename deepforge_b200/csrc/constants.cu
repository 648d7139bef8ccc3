// Graph-owned constants: the embedded pass-by-value scalars of a graph, written into their workspace slots by one
// launch at the head of the plan. The reference keeps them as private globals of the compiled module
// (lib/Compiler/FoundationalGraph.cpp:2216-2250); here they live in the caller's workspace like every other
// intermediate, so that the Executable owns no device memory and a captured CUDA graph replays them.
#include "common.cuh"

namespace dfgpu {
namespace {

struct ConstantTargets {
    void* pointer[DFGPU_MAX_CONSTANTS];
};

__global__ void constants_kernel(dfgpu_constants_params p, ConstantTargets targets) {
    const int i = threadIdx.x;
    if (i >= p.count) return;
    void* target = targets.pointer[i];
    const unsigned long long bits = p.bits[i];
    switch (p.bytes[i]) {
        case 2: *static_cast<uint16_t*>(target) = static_cast<uint16_t>(bits); break;
        case 4: *static_cast<uint32_t*>(target) = static_cast<uint32_t>(bits); break;
        default: *static_cast<unsigned long long*>(target) = bits; break;
    }
}

int validate(const dfgpu_constants_params& p) {
    if (p.count < 1 || p.count > DFGPU_MAX_CONSTANTS) return fail(kInvalidValue, "CONSTANTS: count %d is outside 1..%d", p.count, DFGPU_MAX_CONSTANTS);
    for (int i = 0; i < p.count; ++i)
        if (p.bytes[i] != 2 && p.bytes[i] != 4 && p.bytes[i] != 8) return fail(kInvalidValue, "CONSTANTS: constant %d has %d bytes (2, 4 or 8)", i, p.bytes[i]);
    return kOk;
}

}  // namespace
}  // namespace dfgpu

using namespace dfgpu;

extern "C" int dfgpu_query_constants(const dfgpu_constants_params* p, dfgpu_plan_info* info) {
    if (!p || !info) return fail(kInvalidArgument, "CONSTANTS: null params");
    int status = validate(*p);
    if (status) return status;
    info->kernel = 1;
    info->launches = 1;
    info->scratch_bytes = 0;
    return kOk;
}

extern "C" int dfgpu_constants(const dfgpu_constants_params* p, void* const* tensors, void* scratch, void* stream_handle) {
    (void)scratch;
    if (!p || !tensors) return fail(kInvalidArgument, "CONSTANTS: null params");
    int status = validate(*p);
    if (status) return status;
    ConstantTargets targets{};
    for (int i = 0; i < p->count; ++i) {
        if (!tensors[i] || (reinterpret_cast<uintptr_t>(tensors[i]) % static_cast<uintptr_t>(p->bytes[i])) != 0)
            return fail(kInvalidArgument, "CONSTANTS: destination %d is null or not aligned to its %d bytes", i, p->bytes[i]);
        targets.pointer[i] = tensors[i];
    }
    constants_kernel<<<1, 32, 0, as_stream(stream_handle)>>>(*p, targets);
    return check_launch("CONSTANTS");
}

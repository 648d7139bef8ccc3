// Schedule policy names of the reference's direct-convolution code generator (include/DeepForge/Compiler/Schedule.h
// :11-24), kept so that callers which set CompileOptions::schedule_policy still compile. Kernel selection on this
// backend is done by the kernel library (dfgpu_query_*), not by a CPU cost model: the value is accepted and ignored.
#pragma once

#include <cstdint>

namespace deepforge::compiler {

enum class Conv2DSchedulePolicy : std::uint8_t { kBaseline = 0, kAuto = 1 };

}  // namespace deepforge::compiler

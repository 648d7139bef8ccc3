// Declarations shared between the compiler front and the runtime inside the host library.
#pragma once

#include "DeepForge/Compiler/Bufferization.h"
#include "DeepForge/Compiler/GraphMetadata.h"
#include "DeepForge/Compiler/KernelPlan.h"
#include "DeepForge/Runtime/Executable.h"

#include <memory>

namespace deepforge::compiler {
char const* kernel_op_name(KernelOp op);
// Asks the kernel library about one launch: fills step.kernel / step.launches and reports its scratch need.
import::Status query_kernel_step(KernelStep& step, std::int64_t& scratch_bytes);
}

namespace deepforge::runtime {

// The only way to build an Executable (its constructor is private, as in the reference).
struct ExecutableFactory {
    static std::unique_ptr<Executable> create(compiler::GraphCompileMetadata metadata, compiler::WorkspacePlan workspace,
                                              compiler::KernelPlan plan);
};

}  // namespace deepforge::runtime

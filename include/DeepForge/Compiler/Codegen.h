// compile_graph / compile_file: serialized graph -> validated metadata, workspace plan,
// kernel plan and an Executable. Same entry points as the reference's
// include/DeepForge/Compiler/Codegen.h:52-60; the result carries a kernel plan where
// the reference carries three x86 objects.
#pragma once

#include "DeepForge/Compiler/Bufferization.h"
#include "DeepForge/Compiler/GraphMetadata.h"
#include "DeepForge/Compiler/KernelPlan.h"
#include "DeepForge/Import/SerializedGraphImporter.h"
#include "DeepForge/Runtime/Executable.h"

#include <filesystem>
#include <memory>
#include <string>

namespace deepforge::compiler {

struct CompileOptions {
    std::string foundational_function_name = "deepforge_graph";
    import::InputFormat input_format = import::InputFormat::kAuto;
    // Fuse POINTWISE consumers into contraction epilogues and BLOCK_SCALE_DEQUANTIZE
    // producers into MATMUL operand loads.
    bool fuse = true;
    // Re-type FLOAT virtual tensors that only tensor-core contractions read, without giving up the FLOAT
    // semantics of the graph: a dequantize output becomes bf16 (exact: an E4M3 code times a power of two),
    // a tensor between two bf16 tcgen05 convolutions becomes a (hi, lo) bf16 pair per element (DFGPU_BF16X2:
    // 4 bytes like FLOAT, the value kept to 2^-17 relative, both halves multiplied by the bf16 filter).
    bool narrow_virtual_tensors = true;
    // Lossy and off by default: store such tensors as one bf16 instead (half the intermediate traffic; every
    // narrowed tensor adds a rounding of up to 2^-9 relative to what its readers see, so a chain of
    // contractions can leave the bf16 gate against the all-FLOAT evaluation of the graph).
    bool bf16_virtual_tensors = false;
    // Force the CUDA-core kernels (used by tests to cross-check the tcgen05 paths).
    bool disable_tensor_cores = false;
};

struct CompilationResult {
    std::unique_ptr<runtime::Executable> executable;
    GraphCompileMetadata metadata;
    WorkspacePlan workspace;
    KernelPlan plan;
    std::string target = "sm_100a";
};

[[nodiscard]] import::Status compile_graph(import::SerializedGraph const& graph, CompileOptions const& options, CompilationResult& output);
[[nodiscard]] import::Status compile_file(std::filesystem::path const& path, CompileOptions const& options, CompilationResult& output);

}  // namespace deepforge::compiler

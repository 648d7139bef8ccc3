// compile_graph / compile_file: serialized graph -> validated metadata, workspace plan,
// kernel plan and an Executable. Same entry points as the reference's
// include/DeepForge/Compiler/Codegen.h:52-60; the result carries a kernel plan where
// the reference carries three x86 objects.
#pragma once

#include "DeepForge/Compiler/Bufferization.h"
#include "DeepForge/Compiler/Conv2DImporter.h"
#include "DeepForge/Compiler/GraphMetadata.h"
#include "DeepForge/Compiler/KernelPlan.h"
#include "DeepForge/Compiler/Schedule.h"
#include "DeepForge/Import/SerializedGraphImporter.h"
#include "DeepForge/Runtime/Executable.h"

#include <array>
#include <filesystem>
#include <memory>
#include <string>
#include <vector>

namespace deepforge::compiler {

struct CompileOptions {
    // The reference's fields (include/DeepForge/Compiler/Codegen.h:17-26). The x86 emission switches are accepted
    // and have no effect: there is no object code, LLVM IR or MLIR to emit, capture or schedule here.
    Conv2DImportOptions importer;
    std::string foundational_function_name = "deepforge_graph";
    import::InputFormat input_format = import::InputFormat::kAuto;
    bool build_avx_variants = true;
    bool emit_object = true;
    bool emit_llvm_ir = true;
    bool capture_mlir = false;
    Conv2DSchedulePolicy schedule_policy = Conv2DSchedulePolicy::kAuto;
    // ---- this backend's own switches ----
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
    // Hand a convolution and the 1 x 1 convolution that alone reads it to the fused two-convolution kernel when the
    // kernel library has one for the pair (needs `fuse`).
    bool fuse_convolution_pairs = true;
    // Force the CUDA-core kernels (used by tests to cross-check the tcgen05 paths).
    bool disable_tensor_cores = false;
};

// One entry per variant name of the reference (scalar, AVX2, AVX-512). There is one compiled form, the kernel plan:
// the scalar entry names it ("kernel-plan" as schedule, "sm_100a" as required features), the other two stay empty, and
// no entry carries code (mlir, llvm_ir and object are always empty).
struct VariantCode {
    runtime::CpuVariant variant = runtime::CpuVariant::kScalar;
    std::string symbol, required_features, schedule, mlir, llvm_ir;
    std::vector<std::uint8_t> object;
};

struct CompilationResult {
    std::unique_ptr<runtime::Executable> executable;
    InvocationAdapterKind adapter_kind = InvocationAdapterKind::kGenericRankedMemrefPointerTable;
    Conv2DCompileMetadata metadata;
    WorkspacePlan workspace;
    std::string target_triple = "sm_100a";
    std::string imported_mlir, bufferized_mlir;  // always empty
    std::array<VariantCode, 3> variants;
    KernelPlan plan;                             // what this backend compiles to
};

[[nodiscard]] import::Status compile_graph(import::SerializedGraph const& graph, CompileOptions const& options, CompilationResult& output);
[[nodiscard]] import::Status compile_file(std::filesystem::path const& path, CompileOptions const& options, CompilationResult& output);

}  // namespace deepforge::compiler

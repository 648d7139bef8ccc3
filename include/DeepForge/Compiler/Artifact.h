// Compiled-graph artifacts (".dfo"): an Executable written to bytes and loaded back without
// recompiling. Same entry points as the reference (include/DeepForge/Compiler/Artifact.h:45-69) and
// the same container as its format 12 (docs/artifact-format.en.md:55-123): magic, version, endian
// marker, version strings, override flags, the argument table, a length-delimited adapter section,
// the workspace plan, tolerances, the variant list and an FNV-1a 64 checksum over every preceding
// byte. Format 13 adds adapter kind 2, whose payload is the kernel plan (one record per launch:
// the dfgpu entry point, its POD params, tensor bindings and scratch); its variant list is empty,
// since the code lives in the kernel library, not in the artifact. Formats 1..12 hold x86 objects
// and are rejected here.
#pragma once

#include "DeepForge/Compiler/Codegen.h"

#include <cstdint>
#include <filesystem>
#include <memory>
#include <span>
#include <string>
#include <vector>

namespace deepforge::compiler {

inline constexpr std::uint32_t kReferenceArtifactFormatVersion = 12;  // the last format of the CPU reference
inline constexpr std::uint32_t kArtifactFormatVersion = 13;
inline constexpr double kDefaultAbsoluteTolerance = 1.0e-4;
inline constexpr double kDefaultRelativeTolerance = 1.0e-3;

enum class ArtifactAdapterKind : std::uint32_t { kConv2DRankedMemref = 0, kGenericPointerTable = 1, kGpuKernelPlan = 2 };

struct ArtifactInfo {
    std::uint32_t format_version = 0;
    ArtifactAdapterKind adapter_kind = ArtifactAdapterKind::kGpuKernelPlan;
    std::string deepforge_version;
    std::string llvm_version;      // empty: no LLVM in this backend
    std::string frontend_version;
    std::string target_triple;     // "sm_100a"
    std::int32_t kernel_abi_version = 0;
    // The convolution fields are filled when the artifact holds the single-node CONV_FPROP form (arguments X, W, Y):
    // UIDs and shapes from the argument table, padding / stride / dilation from the launch's params block.
    InvocationAdapterKind invocation = InvocationAdapterKind::kGenericRankedMemrefPointerTable;
    Conv2DCompileMetadata metadata;
    WorkspacePlan workspace;
    KernelPlan plan;
    double absolute_tolerance = kDefaultAbsoluteTolerance;
    double relative_tolerance = kDefaultRelativeTolerance;
};

// `output` is replaced on success and untouched on failure. The same compilation always gives the same bytes.
[[nodiscard]] import::Status serialize_artifact(CompilationResult const& compilation, std::vector<std::uint8_t>& output);

// Bounds, version, checksum and every field's range are checked before `output` is modified.
[[nodiscard]] import::Status parse_artifact(std::span<std::uint8_t const> input, ArtifactInfo& output);

// Writes <path>.tmp.<pid>.<sequence> beside the destination and publishes it with rename.
[[nodiscard]] import::Status write_artifact(std::filesystem::path const& path, CompilationResult const& compilation);
[[nodiscard]] import::Status read_artifact(std::filesystem::path const& path, ArtifactInfo& output);

// Parses, then asks the kernel library whether it still accepts every launch's params and resolves them to the
// kernel the plan recorded, and builds the Executable.
[[nodiscard]] import::Status load_artifact_executable(std::span<std::uint8_t const> input, std::unique_ptr<runtime::Executable>& output,
                                                      ArtifactInfo* info = nullptr);
[[nodiscard]] import::Status load_artifact_executable(std::filesystem::path const& path, std::unique_ptr<runtime::Executable>& output,
                                                      ArtifactInfo* info = nullptr);

}  // namespace deepforge::compiler

// Strict importer for cudnn-frontend v1.24.0 serialized Graphs (JSON text or canonical
// UBJSON). Same call shape as the reference's SerializedGraphImporter
// (include/DeepForge/Import/SerializedGraphImporter.h:22-41): the output graph is
// written only when the whole document validates.
#pragma once

#include "DeepForge/Import/SerializedGraph.h"
#include "DeepForge/Import/Status.h"

#include <cstddef>
#include <cstdint>
#include <filesystem>
#include <span>

namespace deepforge::import {

inline constexpr std::size_t kMaximumSerializedGraphBytes = 16u * 1024u * 1024u;
inline constexpr std::int64_t kPinnedFrontendVersion = 12400;

enum class InputFormat : std::uint8_t { kAuto, kJson, kUbjson };

class SerializedGraphImporter {
public:
    [[nodiscard]] Status parse(std::span<std::uint8_t const> bytes, InputFormat format, SerializedGraph& output) const;
    [[nodiscard]] Status parse_file(std::filesystem::path const& path, InputFormat format, SerializedGraph& output) const;
};

}  // namespace deepforge::import

// Thin C face over the REFERENCE importer (compiled from the reference's own sources where they
// lie, never copied): lets the tests feed the same documents to both importers and compare
// accept/reject and error codes. Test infrastructure only; built into oracle/_ref/.
#include "DeepForge/Import/SerializedGraphImporter.h"

#include <cstdint>
#include <cstring>
#include <span>

extern "C" __attribute__((visibility("default"))) int ref_parse(const std::uint8_t* bytes, std::size_t size, int format, std::int64_t* tensors,
                                                                 std::int64_t* nodes, char* message, std::size_t capacity) {
    deepforge::import::SerializedGraph graph;
    deepforge::import::SerializedGraphImporter importer;
    auto chosen = format == 1 ? deepforge::import::InputFormat::kJson
                              : (format == 2 ? deepforge::import::InputFormat::kUbjson : deepforge::import::InputFormat::kAuto);
    auto status = importer.parse(std::span<std::uint8_t const>(bytes, size), chosen, graph);
    if (status.is_good()) {
        if (tensors) *tensors = static_cast<std::int64_t>(graph.tensor_count());
        if (nodes) *nodes = static_cast<std::int64_t>(graph.nodes.size());
    }
    if (message && capacity) {
        std::strncpy(message, status.message().c_str(), capacity - 1);
        message[capacity - 1] = '\0';
    }
    return static_cast<int>(status.code());
}

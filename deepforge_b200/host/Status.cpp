#include "DeepForge/Import/Status.h"

namespace deepforge::import {

std::string_view error_code_name(ErrorCode code) noexcept {
    switch (code) {
        case ErrorCode::kOk: return "DFE_OK";
        case ErrorCode::kInvalidArgument: return "DFE_INVALID_ARGUMENT";
        case ErrorCode::kIoError: return "DFE_IO_ERROR";
        case ErrorCode::kParseError: return "DFE_PARSE_ERROR";
        case ErrorCode::kSchemaVersionMismatch: return "DFE_SCHEMA_VERSION_MISMATCH";
        case ErrorCode::kFrontendVersionMismatch: return "DFE_FRONTEND_VERSION_MISMATCH";
        case ErrorCode::kMissingField: return "DFE_MISSING_FIELD";
        case ErrorCode::kInvalidFieldType: return "DFE_INVALID_FIELD_TYPE";
        case ErrorCode::kInvalidValue: return "DFE_INVALID_VALUE";
        case ErrorCode::kUnsupportedNode: return "DFE_UNSUPPORTED_NODE";
        case ErrorCode::kUnsupportedDataType: return "DFE_UNSUPPORTED_DATA_TYPE";
        case ErrorCode::kUnsupportedExecutionMetadata: return "DFE_UNSUPPORTED_EXECUTION_METADATA";
        case ErrorCode::kDuplicateUid: return "DFE_DUPLICATE_UID";
        case ErrorCode::kMissingUid: return "DFE_MISSING_UID";
        case ErrorCode::kInvalidLayout: return "DFE_INVALID_LAYOUT";
        case ErrorCode::kInvalidShape: return "DFE_INVALID_SHAPE";
        case ErrorCode::kDimensionOverflow: return "DFE_DIMENSION_OVERFLOW";
        case ErrorCode::kInvalidVariantPack: return "DFE_INVALID_VARIANT_PACK";
        case ErrorCode::kUnsupportedCpuFeature: return "DFE_UNSUPPORTED_CPU_FEATURE";
        case ErrorCode::kGraphExecutionFailed: return "DFE_GRAPH_EXECUTION_FAILED";
        case ErrorCode::kUnsupportedOperation: return "DFE_UNSUPPORTED_OPERATION";
    }
    return "DFE_UNKNOWN";
}

Status Status::failure(ErrorCode code, std::string_view subject, std::string_view detail) {
    std::string message(error_code_name(code));
    message += ": ";
    message += subject;
    if (!detail.empty()) {
        message += ": ";
        message += detail;
    }
    return Status(code, std::move(message));
}

}  // namespace deepforge::import

/*
 * Flat C API over the C++ host side (importer -> compile_graph -> Executable), for
 * callers that bind through an FFI (ctypes, cgo, JNI) instead of including the C++
 * headers. Each function stands for one call of the reference's C++ interface:
 *   df_compile        SerializedGraphImporter::parse + compiler::compile_graph
 *                     (include/DeepForge/Import/SerializedGraphImporter.h:22-41,
 *                      include/DeepForge/Compiler/Codegen.h:52-60)
 *   df_execute        runtime::Executable::execute (include/DeepForge/Runtime/Executable.h:75-78)
 *   df_workspace_size runtime::Executable::get_workspace_size (Executable.h:64)
 * Return values are DeepForge Status codes (0 = DFE_OK); the message of the last
 * failure on the calling thread is available from df_last_error().
 */
#ifndef DEEPFORGE_B200_H
#define DEEPFORGE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct df_executable df_executable;

enum { DF_FORMAT_AUTO = 0, DF_FORMAT_JSON = 1, DF_FORMAT_UBJSON = 2 };
/* DF_OPTION_BF16_INTERMEDIATES: lossy, see CompileOptions::bf16_virtual_tensors. DF_OPTION_NO_CONV_PAIRS: every
   convolution is its own launch (CompileOptions::fuse_convolution_pairs = false). */
enum { DF_OPTION_NO_FUSION = 1, DF_OPTION_NO_NARROWING = 2, DF_OPTION_NO_TENSOR_CORES = 4, DF_OPTION_BF16_INTERMEDIATES = 8, DF_OPTION_NO_CONV_PAIRS = 16 };

const char* df_last_error(void);

/* Parse only: validates a serialized graph and reports the tensor and node counts. */
int df_parse(const uint8_t* document, size_t size, int format, int64_t* tensor_count, int64_t* node_count);

/* Parse, then write the canonical model as text (one line per context field, tensor, node, port and attribute, in a
   fixed order): what SerializedGraph::operator== compares, in a form two importers can be diffed by. Copies up to
   `capacity` bytes and always reports the full length in *length. */
int df_dump_graph(const uint8_t* document, size_t size, int format, char* buffer, size_t capacity, size_t* length);

int df_compile(const uint8_t* document, size_t size, int format, uint32_t options, df_executable** out);
void df_destroy(df_executable* executable);

int64_t df_workspace_size(const df_executable* executable);
int64_t df_launch_count(const df_executable* executable);
/* Copies the kernel plan dump (one line per launch) into buffer; returns the full length. */
size_t df_plan_text(const df_executable* executable, char* buffer, size_t capacity);

/* Argument table (ascending UID). access: 0 read, 1 write, 2 read-write. */
int64_t df_argument_count(const df_executable* executable);
int df_argument_info(const df_executable* executable, int64_t index, int64_t* uid, uint64_t* size_bytes,
                     uint64_t* alignment, int32_t* access);

/* Name of argument `index` ("X", "W", "Y" for the single-node convolution form, the tensor's name otherwise);
   returns the full length. */
size_t df_argument_name(const df_executable* executable, int64_t index, char* buffer, size_t capacity);
/* Metadata of the single-node CONV_FPROP form (Conv2DCompileMetadata, include/DeepForge/Compiler/Conv2DImporter.h
   :24-37 of the reference). *adapter_kind: 0 = that form (arguments X, W, Y), 1 = the generic table. values[27] =
   x_uid, w_uid, y_uid, x_shape[4], w_shape[4], y_shape[4], padded_x_shape[4] (physical N, H, W, C order),
   pre_padding[2], post_padding[2], stride[2], dilation[2]; all zero under the generic table. */
int df_conv2d_metadata(const df_executable* executable, int32_t* adapter_kind, int64_t* values);

/* stream: a cudaStream_t (NULL = legacy default stream). */
void df_set_stream(df_executable* executable, void* stream);

/* uids[i] -> pointers[i] is the variant pack; pointers and workspace are device pointers. */
int df_execute(const df_executable* executable, void* handle, const int64_t* uids, void* const* pointers, size_t count,
               void* workspace);

/* df_execute with the launches on `stream` (a cudaStream_t) for this call only: calls on different streams with
   different workspaces and outputs may run concurrently from different threads (Executable::execute_on). */
int df_execute_on(const df_executable* executable, void* stream, const int64_t* uids, void* const* pointers, size_t count,
                  void* workspace);

/* Kernel plan introspection and partial execution (used for per-kernel timing): the plan has
   df_step_count() launches groups; df_execute_steps runs steps [first, last) only. */
int64_t df_step_count(const df_executable* executable);
int df_step_info(const df_executable* executable, int64_t step, char* label, size_t label_capacity, int32_t* op, int32_t* kernel,
                 int32_t* launches, uint64_t* bound_bytes);
int df_execute_steps(const df_executable* executable, int64_t first, int64_t last, const int64_t* uids, void* const* pointers,
                     size_t count, void* workspace);

/* Artifacts (compiler::serialize_artifact / write_artifact / load_artifact_executable,
   include/DeepForge/Compiler/Artifact.h:45-69 of the reference): a compiled executable as bytes or as a file
   published by rename, and back without recompiling. df_serialize_artifact copies up to `capacity` bytes and
   always reports the full size. */
int df_serialize_artifact(const df_executable* executable, uint8_t* buffer, size_t capacity, size_t* size);
int df_write_artifact(const df_executable* executable, const char* path);
int df_load_artifact(const uint8_t* bytes, size_t size, df_executable** out);
int df_load_artifact_file(const char* path, df_executable** out);

/* Workspace planner on its own: sizes/alignments/live ranges in, offsets + total out. */
int df_plan_workspace(size_t count, const char* const* names, const uint64_t* sizes, const uint64_t* alignments,
                      const uint64_t* live_starts, const uint64_t* live_ends, uint64_t* offsets, int64_t* placement_order,
                      uint64_t* total_bytes);

#ifdef __cplusplus
}
#endif
#endif

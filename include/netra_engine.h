/* Netra engine runtime C ABI, re-backed for NVIDIA B200 (sm_100a).
 *
 * Same exported names, struct layouts, status values and call order as the reference's
 * runtime/gfx950/engine/netra_engine.h:12-108; the differences are:
 *   - hipStream_t -> cudaStream_t (both opaque pointers);
 *   - NETRA_STATUS_CUDA is an alias of value 7 (NETRA_STATUS_HIP in the reference);
 *   - the engine manifest names target "sm_100a", wave_size 32, required_cuda{minimum},
 *     and each kernel operation names an engine-relative "cubin/..." file;
 *   - a third argument kind, "tensor_map" (a TMA descriptor built by the runtime from a bound or
 *     workspace pointer and compile-time shape fields), next to "pointer" and "u32_constant".
 */
#pragma once

#include <cuda_runtime_api.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct netra_engine netra_engine_t;

/* runtime/gfx950/engine/netra_engine.h:14-25 */
typedef enum netra_status {
  NETRA_STATUS_OK = 0,
  NETRA_STATUS_INVALID_ARGUMENT = 1,
  NETRA_STATUS_IO = 2,
  NETRA_STATUS_MANIFEST = 3,
  NETRA_STATUS_UNSUPPORTED_TARGET = 4,
  NETRA_STATUS_UNSUPPORTED_PROFILE = 5,
  NETRA_STATUS_BINDING = 6,
  NETRA_STATUS_HIP = 7,
  NETRA_STATUS_CUDA = 7,
  NETRA_STATUS_BUSY = 8,
  NETRA_STATUS_FALLBACK_REQUIRED = 9
} netra_status_t;

/* runtime/gfx950/engine/netra_engine.h:27-31 */
typedef struct netra_engine_options {
  uint32_t struct_size;
  int32_t device_id;
  uint32_t enable_graph_capture;
} netra_engine_options_t;

/* runtime/gfx950/engine/netra_engine.h:33-45 */
typedef struct netra_profile_info {
  uint32_t struct_size;
  uint32_t profile_id;
  uint32_t min_m;
  uint32_t max_m;
  uint32_t min_batch;
  uint32_t max_batch;
  uint64_t min_sequence;
  uint64_t max_sequence;
  uint32_t tensor_parallel;
  uint64_t workspace_bytes;
  uint32_t requires_fallback;
} netra_profile_info_t;

/* runtime/gfx950/engine/netra_engine.h:47-52 */
typedef struct netra_launch_shape {
  uint32_t m;
  uint32_t batch;
  uint64_t sequence;
  uint32_t tensor_parallel;
} netra_launch_shape_t;

/* runtime/gfx950/engine/netra_engine.h:54-58 */
typedef struct netra_pointer_binding {
  uint32_t argument_index;
  uint32_t reserved;
  void* pointer;
} netra_pointer_binding_t;

/* runtime/gfx950/engine/netra_engine.h:60-62.  Loads engine.json, checks target / runtime
 * version, allocates the static workspace, loads the cubins and resolves every kernel symbol. */
netra_status_t netra_engine_create(const char* engine_directory, const netra_engine_options_t* options,
                                   netra_engine_t** output);
/* runtime/gfx950/engine/netra_engine.h:63 */
size_t netra_engine_profile_count(const netra_engine_t* engine);
/* runtime/gfx950/engine/netra_engine.h:64-66 */
netra_status_t netra_engine_query_profile(const netra_engine_t* engine, uint32_t profile_id,
                                          netra_profile_info_t* output);
/* runtime/gfx950/engine/netra_engine.h:70-72.  Control plane; not thread-safe with launch. */
netra_status_t netra_engine_bind(netra_engine_t* engine, uint32_t profile_id, uint32_t operation_index,
                                 uint32_t argument_index, void* pointer);
/* runtime/gfx950/engine/netra_engine.h:76.  Ends the binding phase; records become immutable. */
netra_status_t netra_engine_finalize_bindings(netra_engine_t* engine);
/* runtime/gfx950/engine/netra_engine.h:80-82.  Captures the profile's launches into a CUDA graph. */
netra_status_t netra_engine_prepare_profile(netra_engine_t* engine, uint32_t profile_id, cudaStream_t stream);
/* runtime/gfx950/engine/netra_engine.h:84-87 */
netra_status_t netra_engine_launch(netra_engine_t* engine, uint32_t profile_id, const netra_launch_shape_t* shape,
                                   cudaStream_t caller_stream);
/* runtime/gfx950/engine/netra_engine.h:91-93 */
netra_status_t netra_engine_launch_operation(netra_engine_t* engine, uint32_t profile_id, uint32_t operation_index,
                                             const netra_launch_shape_t* shape, cudaStream_t caller_stream);
/* runtime/gfx950/engine/netra_engine.h:98-102.  Pointers live in caller-local launch storage. */
netra_status_t netra_engine_launch_operation_bound(netra_engine_t* engine, uint32_t profile_id,
                                                   uint32_t operation_index, const netra_launch_shape_t* shape,
                                                   const netra_pointer_binding_t* bindings, uint32_t binding_count,
                                                   cudaStream_t caller_stream);
/* runtime/gfx950/engine/netra_engine.h:103 */
const char* netra_engine_last_error(const netra_engine_t* engine);
/* runtime/gfx950/engine/netra_engine.h:108.  BUSY while a launch call is inside the API. */
netra_status_t netra_engine_destroy(netra_engine_t* engine);

/* No counterpart in the reference: parses and checks <engine_directory>/engine.json exactly as
 * netra_engine_create does, without touching a device (manifest checks on machines with no GPU,
 * host-side failure tests).  Writes a message into error (if non-null) on failure. */
netra_status_t netra_engine_check_manifest(const char* engine_directory, char* error, size_t error_bytes);
/* No counterpart in the reference: address of the engine-owned static workspace (for callers that
 * read intermediate results, e.g. parity harnesses).  NULL if the engine has no workspace. */
void* netra_engine_workspace(const netra_engine_t* engine);

#ifdef __cplusplus
}
#endif

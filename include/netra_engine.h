/* Netra engine runtime C ABI, re-backed for NVIDIA B200 (sm_100a).
 *
 * Binary-compatible with the reference's runtime/gfx950/engine/netra_engine.h:12-108: the same exported
 * names, the same struct layouts and status values, the same call order.  Differences:
 *   - hipStream_t -> cudaStream_t (both opaque pointers);
 *   - NETRA_STATUS_CUDA is an alias of value 7 (NETRA_STATUS_HIP in the reference);
 *   - the engine manifest names target "sm_100a", wave_size 32, required_cuda{minimum},
 *     and each kernel operation names an engine-relative "cubin/..." file;
 *   - a third argument kind, "tensor_map" (a TMA descriptor built by the runtime from a bound or
 *     workspace pointer and compile-time shape fields), next to "pointer" and "u32_constant";
 *   - an optional launch field "registers_per_thread" that the loaded code object must report.
 *
 * Life cycle: create -> query_profile* -> bind* -> finalize_bindings -> [prepare_profile] ->
 * launch* -> destroy.  bind / finalize / prepare are control-plane calls that the caller serialises;
 * launch calls may run concurrently once the bindings are final.
 */
#pragma once

#include <cuda_runtime_api.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status values (reference lines 14-25); every entry point returns one of them ---------------- */
typedef enum netra_status {
  NETRA_STATUS_OK = 0,                  /* success */
  NETRA_STATUS_INVALID_ARGUMENT = 1,    /* null pointer, wrong struct_size, index out of range, call out of order */
  NETRA_STATUS_IO = 2,                  /* a file of the engine directory could not be read */
  NETRA_STATUS_MANIFEST = 3,            /* engine.json is malformed or inconsistent */
  NETRA_STATUS_UNSUPPORTED_TARGET = 4,  /* not an sm_100a device, or the driver is older than required_cuda */
  NETRA_STATUS_UNSUPPORTED_PROFILE = 5, /* the launch shape lies outside the profile's guards */
  NETRA_STATUS_BINDING = 6,             /* a binding slot is missing, null or bound twice differently */
  NETRA_STATUS_HIP = 7,                 /* name kept for source compatibility with reference callers */
  NETRA_STATUS_CUDA = 7,                /* a CUDA runtime or driver call failed (see last_error) */
  NETRA_STATUS_BUSY = 8,                /* destroy while a launch call is inside the API */
  NETRA_STATUS_FALLBACK_REQUIRED = 9    /* the profile contains an operation without a fixed kernel */
} netra_status_t;

/* ---- plain-data records; struct_size is sizeof() as seen by the caller ------------------------------ */
typedef struct netra_engine netra_engine_t;   /* opaque */

typedef struct netra_engine_options {   /* reference lines 27-31 */
  uint32_t struct_size;
  int32_t device_id;                    /* CUDA device ordinal the engine lives on */
  uint32_t enable_graph_capture;        /* 0: prepare_profile is a no-op and launches are direct */
} netra_engine_options_t;

typedef struct netra_profile_info {     /* reference lines 33-45; guards are inclusive ranges */
  uint32_t struct_size;
  uint32_t profile_id;
  uint32_t min_m;
  uint32_t max_m;
  uint32_t min_batch;
  uint32_t max_batch;
  uint64_t min_sequence;
  uint64_t max_sequence;
  uint32_t tensor_parallel;             /* 0 = decided by the deployment */
  uint64_t workspace_bytes;             /* engine-owned static workspace of this profile */
  uint32_t requires_fallback;           /* 1: launch returns NETRA_STATUS_FALLBACK_REQUIRED */
} netra_profile_info_t;

typedef struct netra_launch_shape {     /* reference lines 47-52; checked against the guards at every launch */
  uint32_t m;
  uint32_t batch;
  uint64_t sequence;
  uint32_t tensor_parallel;
} netra_launch_shape_t;

typedef struct netra_pointer_binding {  /* reference lines 54-58; one boundary pointer of a bound launch */
  uint32_t argument_index;
  uint32_t reserved;                    /* must be 0 */
  void* pointer;
} netra_pointer_binding_t;

/* ---- construction and inspection ------------------------------------------------------------------- */
/* Reference lines 60-62.  Reads engine.json, checks target and runtime version, allocates the static
 * workspace, loads the cubins, resolves every kernel symbol and checks its register contract. */
netra_status_t netra_engine_create(const char* engine_directory, const netra_engine_options_t* options,
                                   netra_engine_t** output);
/* No counterpart in the reference, whose create reports every failure as MANIFEST and drops the text with the
 * half-built engine.  Here create returns IO when a file of the directory cannot be read, UNSUPPORTED_TARGET for
 * a device that is not sm_100a or a driver older than required_cuda, CUDA for a failed runtime or driver call,
 * MANIFEST for a malformed or inconsistent engine.json - and this returns the text of the calling thread's most
 * recent failed create ("" after a successful one). */
const char* netra_engine_create_error(void);
/* Reference line 108.  BUSY while a launch call is inside the API; the caller quiesces its streams first. */
netra_status_t netra_engine_destroy(netra_engine_t* engine);
/* Reference line 103.  Message of the most recent failure on this engine. */
const char* netra_engine_last_error(const netra_engine_t* engine);
/* Reference lines 63-66. */
size_t netra_engine_profile_count(const netra_engine_t* engine);
netra_status_t netra_engine_query_profile(const netra_engine_t* engine, uint32_t profile_id,
                                          netra_profile_info_t* output);

/* ---- binding phase (control plane, not thread-safe with launch) -------------------------------------- */
/* Reference lines 70-72.  Slots are the numeric indices of graph_recipe.json. */
netra_status_t netra_engine_bind(netra_engine_t* engine, uint32_t profile_id, uint32_t operation_index,
                                 uint32_t argument_index, void* pointer);
/* Reference line 76.  After this the launch records are immutable. */
netra_status_t netra_engine_finalize_bindings(netra_engine_t* engine);
/* Reference lines 80-82.  Captures the profile's launches into a CUDA graph on `stream`. */
netra_status_t netra_engine_prepare_profile(netra_engine_t* engine, uint32_t profile_id, cudaStream_t stream);

/* ---- launches (enqueue only: no allocation, no synchronisation) ------------------------------------ */
/* Reference lines 84-87: the whole profile (graph replay when prepared, direct launches otherwise). */
netra_status_t netra_engine_launch(netra_engine_t* engine, uint32_t profile_id, const netra_launch_shape_t* shape,
                                   cudaStream_t caller_stream);
/* Reference lines 91-93: one already-selected operation, for callers migrating one boundary at a time. */
netra_status_t netra_engine_launch_operation(netra_engine_t* engine, uint32_t profile_id, uint32_t operation_index,
                                             const netra_launch_shape_t* shape, cudaStream_t caller_stream);
/* Reference lines 98-102: the same with boundary pointers kept in caller-local launch storage, so that
 * concurrent calls cannot mix pointer sets. */
netra_status_t netra_engine_launch_operation_bound(netra_engine_t* engine, uint32_t profile_id,
                                                   uint32_t operation_index, const netra_launch_shape_t* shape,
                                                   const netra_pointer_binding_t* bindings, uint32_t binding_count,
                                                   cudaStream_t caller_stream);

/* ---- additions without a counterpart in the reference ------------------------------------------------ */
/* Parses and checks <engine_directory>/engine.json exactly as netra_engine_create does, without touching
 * a device (manifest checks on machines with no GPU, host-side failure tests).  Writes a message into
 * `error` (if non-null) on failure. */
netra_status_t netra_engine_check_manifest(const char* engine_directory, char* error, size_t error_bytes);
/* Address of the engine-owned static workspace (for callers that read intermediate results, e.g. parity
 * harnesses).  NULL if the engine has no workspace. */
void* netra_engine_workspace(const netra_engine_t* engine);

#ifdef __cplusplus
}
#endif

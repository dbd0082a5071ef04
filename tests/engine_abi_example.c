/* A C caller of the engine runtime ABI (include/netra_engine.h), as a reference-side integrator would write it:
 * the call sequence of the reference's runtime (runtime/gfx950/engine/README.md: create, query_profile, bind,
 * finalize_bindings, prepare_profile, launch, destroy) with cudaStream_t in place of hipStream_t.
 *
 * usage: engine_abi_example ENGINE_DIR SLOTS_FILE M
 *   SLOTS_FILE holds one line per binding slot of ENGINE_DIR/graph_recipe.json ("binding_slots"):
 *     <tensor name> <operation index> <argument index> <bytes>
 *   Every tensor is allocated once (zero-filled) and bound to each of its slots; M is the profile's token count.
 * Prints "ok" and exits 0 when every call returned NETRA_STATUS_OK and the stream drained without error.
 * The block between the two marker comments is quoted in INTEGRATION.md; a test keeps the two identical. */
#include <cuda_runtime_api.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "netra_engine.h"

#define MAX_TENSORS 32

struct tensor {
  char name[64];
  void* device;
};

static void* tensor_pointer(struct tensor* table, int* count, const char* name, size_t bytes) {
  for (int i = 0; i < *count; ++i)
    if (strcmp(table[i].name, name) == 0) return table[i].device;
  if (*count == MAX_TENSORS) return NULL;
  void* p = NULL;
  if (cudaMalloc(&p, bytes) != cudaSuccess || cudaMemset(p, 0, bytes) != cudaSuccess) return NULL;
  snprintf(table[*count].name, sizeof table[*count].name, "%s", name);
  table[*count].device = p;
  ++*count;
  return p;
}

int main(int argc, char** argv) {
  if (argc != 4) {
    fprintf(stderr, "usage: %s ENGINE_DIR SLOTS_FILE M\n", argv[0]);
    return 2;
  }
  const char* engine_dir = argv[1];
  FILE* slots = fopen(argv[2], "r");
  const uint32_t m = (uint32_t)strtoul(argv[3], NULL, 10);
  if (!slots) return 2;
  struct tensor tensors[MAX_TENSORS];
  int tensor_count = 0;
  cudaStream_t stream;
  if (cudaStreamCreate(&stream) != cudaSuccess) return 3;

  /* [integration-snippet-begin] */
  netra_engine_options_t options = {sizeof options, /*device_id=*/0, /*enable_graph_capture=*/1};
  netra_engine_t* engine = NULL;
  netra_status_t st = netra_engine_create(engine_dir, &options, &engine);
  if (st != NETRA_STATUS_OK) {
    fprintf(stderr, "create: status %d: %s\n", (int)st, netra_engine_create_error());
    return 1;
  }
  const uint32_t profile_id = 0;                      /* index into engine.json "profiles" */
  netra_profile_info_t info = {sizeof info};
  st = netra_engine_query_profile(engine, profile_id, &info);
  if (st != NETRA_STATUS_OK || info.requires_fallback || m < info.min_m || m > info.max_m) return 1;

  /* one bind per (operation, argument) slot of graph_recipe.json "binding_slots"; the caller owns every pointer */
  char name[64];
  unsigned operation_index, argument_index;
  unsigned long long bytes;
  while (fscanf(slots, "%63s %u %u %llu", name, &operation_index, &argument_index, &bytes) == 4) {
    void* pointer = tensor_pointer(tensors, &tensor_count, name, (size_t)bytes);
    if (!pointer) return 3;
    st = netra_engine_bind(engine, profile_id, operation_index, argument_index, pointer);
    if (st != NETRA_STATUS_OK) goto fail;
  }
  st = netra_engine_finalize_bindings(engine);         /* the binding table is immutable from here on */
  if (st != NETRA_STATUS_OK) goto fail;
  st = netra_engine_prepare_profile(engine, profile_id, stream);   /* captures the launches into a CUDA graph */
  if (st != NETRA_STATUS_OK) goto fail;

  netra_launch_shape_t shape = {m, /*batch=*/1, /*sequence=*/0, info.tensor_parallel};
  for (int step = 0; step < 3; ++step) {               /* hot loop: enqueue only, on the caller's stream */
    st = netra_engine_launch(engine, profile_id, &shape, stream);
    if (st != NETRA_STATUS_OK) goto fail;
  }
  if (cudaStreamSynchronize(stream) != cudaSuccess) return 3;
  st = netra_engine_destroy(engine);                    /* BUSY while a launch call is still inside the runtime */
  /* [integration-snippet-end] */
  if (st != NETRA_STATUS_OK) return 1;
  for (int i = 0; i < tensor_count; ++i) cudaFree(tensors[i].device);
  fclose(slots);
  cudaStreamDestroy(stream);
  printf("ok\n");
  return 0;

fail:
  fprintf(stderr, "status %d: %s\n", (int)st, netra_engine_last_error(engine));
  return 1;
}

// The reference's 768-row prefill bridge (runtime/gfx950/fp8/moe/moe_prefill_m768_bridge.h:10-23,
// moe_prefill_m768_bridge.hip:60-160) on the sm_100a kernels.  Same exported names and argument list: quantised
// token rows, the expert slabs, and the routing in the sorted-id format its fused producer consumes
// (kernels/gfx950/templates/moe/prefill/fused_splitk2/entry_routing.inc:67-111):
//   sorted_token_ids  [23360] words  token | slot << 24, grouped in blocks of 64 that belong to one expert each,
//                     blocks padded with words whose token is >= 768
//   sorted_expert_ids [365]   the expert of each 64-entry block
//   num_valid_ids     [1]     number of words in use (a multiple of 64)
//   topk_weights      [768, 9] routing weights in slot order (slot 8 = the shared expert, id 256)
// Here a small kernel turns that format back into the nine-slot id table, after which the layer's own stages run:
// stable expert sort, row gather, grouped gate_up, grouped down, slot-ordered combine.  At 768 rows the swap-AB
// GEMMs serve the call and the rows between down and combine are FP32, so partials_f16 and
// route_scale_workspace_f32 are accepted for signature compatibility and left untouched.
// Included by api.cu (uses its helpers and launch_stage()).
#include <mutex>

namespace netra {

constexpr int kM768Rows = 768;
constexpr int kM768SortedCapacity = 365 * 64;

// grid ceil(23360 / 256), block 256.  violations counts entries this path cannot represent: a routed slot (0-7) that
// names the shared expert, or slot 8 naming a routed expert.
extern "C" __global__ void __launch_bounds__(256)
netra_m768_import_sorted_sm100(int32_t* __restrict__ ids9, float* __restrict__ w9, const int32_t* __restrict__ sorted_token_ids,
                               const int32_t* __restrict__ sorted_expert_ids, const int32_t* __restrict__ num_valid_ids,
                               const float* __restrict__ topk_weights, uint32_t* __restrict__ violations) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < kM768Rows * kSlots) w9[i] = topk_weights[i];
  if (i < kM768Rows) ids9[i * kSlots + kTopK] = kRouted;
  const int valid = min(max(num_valid_ids[0], 0), kM768SortedCapacity);
  if (i >= valid) return;
  const uint32_t word = (uint32_t)sorted_token_ids[i];
  const uint32_t token = word & 0xffffffu, slot = word >> 24;
  if (token >= (uint32_t)kM768Rows || slot >= (uint32_t)kSlots) return;     // padding
  const int expert = sorted_expert_ids[i >> 6];
  if (slot < (uint32_t)kTopK) {
    if (expert < 0 || expert >= kRouted) atomicAdd(violations, 1u);
    ids9[token * kSlots + slot] = min(max(expert, 0), kRouted - 1);
  } else if (expert != kRouted) {
    atomicAdd(violations, 1u);
  }
}

}  // namespace netra

namespace {

struct M768State {
  std::mutex mutex;
  bool loaded = false;
  int device = -1;
  void* workspace = nullptr;
  uint64_t workspace_bytes = 0;
  netra_moe_layer* layer = nullptr;
  const void* weights[4] = {nullptr, nullptr, nullptr, nullptr};
};
M768State g_m768;

void m768_drop_layer() {
  if (g_m768.layer) netra_moe_layer_destroy(g_m768.layer);
  g_m768.layer = nullptr;
  for (auto& w : g_m768.weights) w = nullptr;
}

}  // namespace

extern "C" {

// The kernels are linked into the library: the two code-object paths of the reference's load() are ignored (NULL is
// accepted).  load() allocates the bridge's scratch (about 90 MB for 768 rows) on the current device; launch() allocates
// nothing.  Idempotent.
int netra_moe_prefill_m768_load(const char*, const char*) {
  std::lock_guard<std::mutex> lock(g_m768.mutex);
  if (g_m768.loaded) return 0;
  int device = 0;
  if (int rc = current_device_index(&device)) return rc;
  if (int rc = umma_setup()) return rc;
  netra_moe_workspace_layout_t lay;
  lay.struct_size = sizeof lay;
  if (int rc = netra_moe_workspace_layout_query(netra::kM768Rows, &lay)) return rc;
  void* ws = nullptr;
  cudaError_t e = cudaMalloc(&ws, lay.total_bytes);
  if (e != cudaSuccess) return fail_cuda("prefill_m768_load: cudaMalloc(scratch)", e);
  e = cudaMemset(ws, 0, lay.total_bytes);
  if (e != cudaSuccess) { cudaFree(ws); return fail_cuda("prefill_m768_load: cudaMemset(scratch)", e); }
  g_m768.workspace = ws;
  g_m768.workspace_bytes = lay.total_bytes;
  g_m768.device = device;
  g_m768.loaded = true;
  return 0;
}

int netra_moe_prefill_m768_launch(const void* hidden_fp8, const float* hidden_scale_f32, const void* w13_fp8, const float* w13_scale_f32,
                                  const void* w2_fp8, const float* w2_scale_f32, const int32_t* sorted_token_ids_i32,
                                  const float* sorted_weights_f32, const int32_t* sorted_expert_ids_i32,
                                  const int32_t* num_valid_ids_i32, const float* topk_weights_f32, float* route_scale_workspace_f32,
                                  void* partials_f16, void* output_bf16, cudaStream_t stream) {
  if (!g_m768.loaded) return fail("prefill_m768: call netra_moe_prefill_m768_load first");
  if (!hidden_fp8 || !hidden_scale_f32 || !w13_fp8 || !w13_scale_f32 || !w2_fp8 || !w2_scale_f32 || !sorted_token_ids_i32 ||
      !sorted_weights_f32 || !sorted_expert_ids_i32 || !num_valid_ids_i32 || !topk_weights_f32 || !route_scale_workspace_f32 ||
      !partials_f16 || !output_bf16)
    return fail("prefill_m768: launch pointers must be nonnull");
  int device = 0;
  if (int rc = current_device_index(&device)) return rc;
  if (device != g_m768.device) return fail("prefill_m768: the current device is not the one the bridge was loaded on");
  const void* weights[4] = {w13_fp8, w13_scale_f32, w2_fp8, w2_scale_f32};
  if (g_m768.layer == nullptr || memcmp(weights, g_m768.weights, sizeof weights) != 0) {
    // First call with this set of expert slabs: encode their descriptors (host work plus one small memset; make
    // this first call outside stream capture).  Later calls with the same pointers go straight to the launches.
    std::lock_guard<std::mutex> lock(g_m768.mutex);
    m768_drop_layer();
    netra_moe_layer_desc_t d;
    memset(&d, 0, sizeof d);
    d.struct_size = sizeof d;
    d.max_tokens = netra::kM768Rows;
    d.router_weight_bf16 = w13_fp8;      // the router stages are never launched by this bridge; any valid 1 MiB range serves the descriptor
    d.w13_fp8 = w13_fp8;
    d.w13_scale_f32 = w13_scale_f32;
    d.w2_fp8 = w2_fp8;
    d.w2_scale_f32 = w2_scale_f32;
    d.workspace = g_m768.workspace;
    d.workspace_bytes = g_m768.workspace_bytes;
    d.weights_tiled = 0;                 // the checkpoint's row-major slabs [257, 1024, 2048] / [257, 2048, 512]
    d.num_expert_slabs = 0;
    if (int rc = netra_moe_layer_create(&d, &g_m768.layer)) return rc;
    memcpy(g_m768.weights, weights, sizeof weights);
  }
  netra_moe_layer* layer = g_m768.layer;
  const netra_moe_workspace_layout_t& L = layer->lay;
  uint8_t* ws = (uint8_t*)g_m768.workspace;
  const uint32_t rows = netra::kM768Rows, pairs = rows * netra::kTopK;
  netra::netra_m768_import_sorted_sm100<<<(netra::kM768SortedCapacity + 255) / 256, 256, 0, stream>>>(
      (int32_t*)(ws + L.topk_ids), (float*)(ws + L.topk_weights), sorted_token_ids_i32, sorted_expert_ids_i32, num_valid_ids_i32,
      topk_weights_f32, (uint32_t*)(ws + L.status) + 3);
  cudaError_t e = cudaMemcpyAsync(ws + L.a_fp8 + (size_t)pairs * netra::kHidden, hidden_fp8, (size_t)rows * netra::kHidden,
                                  cudaMemcpyDeviceToDevice, stream);
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(ws + L.a_scale + (size_t)pairs * netra::kHiddenBlocks * 4, hidden_scale_f32,
                        (size_t)rows * netra::kHiddenBlocks * 4, cudaMemcpyDeviceToDevice, stream);
  if (e != cudaSuccess) return fail_cuda("prefill_m768: cudaMemcpyAsync(token rows)", e);
  layer->external_topk = true;      // the routing came from the caller: the sort is a launch of its own
  int rc = 0;
  for (uint32_t stage = 2; stage < kStageCount && rc == 0; ++stage) rc = launch_stage(layer, stage, hidden_fp8, nullptr, output_bf16, rows, stream);
  layer->external_topk = false;
  return rc ? rc : check_launch("prefill_m768 launch");
}

// Device status words of the last launches (synchronises): 0 gate_up wait expired, 1 down wait expired, 3 number of
// routing entries the bridge could not represent (see the import kernel).  No counterpart in the reference.
int netra_moe_prefill_m768_status(uint32_t status_out[4]) {
  if (!g_m768.loaded || !status_out) return fail("prefill_m768_status: not loaded or null pointer");
  netra_moe_workspace_layout_t lay;
  lay.struct_size = sizeof lay;
  if (int rc = netra_moe_workspace_layout_query(netra::kM768Rows, &lay)) return rc;
  cudaError_t e = cudaMemcpy(status_out, (uint8_t*)g_m768.workspace + lay.status, 16, cudaMemcpyDeviceToHost);
  return e == cudaSuccess ? 0 : fail_cuda("prefill_m768_status: cudaMemcpy", e);
}

int netra_moe_prefill_m768_unload(void) {
  std::lock_guard<std::mutex> lock(g_m768.mutex);
  m768_drop_layer();
  if (g_m768.workspace) cudaFree(g_m768.workspace);
  g_m768.workspace = nullptr;
  g_m768.loaded = false;
  return 0;
}

const char* netra_moe_prefill_m768_last_error(void) { return g_error; }

}  // extern "C"

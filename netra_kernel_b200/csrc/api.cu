// Host side of the C ABI declared in include/netra_moe.h: argument checks, tensor-map encoding
// and kernel launches.  Launch functions do not allocate, synchronise or read back.
#include <cuda.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <new>

#include "../../include/netra_moe.h"
#include "common.cuh"

// Single translation unit: the kernels are included so that no relocatable device code is needed.
#include "bridge_kernels.cu"
#include "route_kernels.cu"
#include "umma_kernels.cu"
#include "umma_tokmajor.cu"
#include "router_umma.cu"
#include "ep_kernels.cu"
#include "mxfp4_kernels.cu"

using namespace netra;

namespace {

thread_local char g_error[512] = "";

int fail(const char* message) {
  snprintf(g_error, sizeof g_error, "%s", message);
  return -1;
}
int fail_cuda(const char* what, cudaError_t e) {
  snprintf(g_error, sizeof g_error, "%s: %s", what, cudaGetErrorString(e));
  return (int)e;
}
int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : fail_cuda(what, e);
}

uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// 2-D byte tensor [rows, row_bytes], box = 128 bytes x box_rows, 128-byte swizzle.
int encode_u8_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail("cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_error, sizeof g_error, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return -1;
  }
  return 0;
}

// MXFP4 code blocks written by netra_moe_mxfp4_pack_launch: [tile_rows, 128] four-bit elements, 64 bytes per row in
// memory.  The copy engine widens each group of 16 codes (8 bytes) to 16 bytes of shared memory, so 128 x 128
// elements land as the same 16 KiB, 128-byte-swizzled tile an E4M3 box gives; a box is two such blocks.
int encode_fp4_tiles(CUtensorMap* map, const void* base, uint64_t tile_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return fail("cuTensorMapEncodeTiled is not available from the driver");
  if (((uintptr_t)base & 31) != 0) return fail("MXFP4 code blocks must be 32-byte aligned");
  cuuint64_t dims[2] = {128, tile_rows};
  cuuint64_t strides[1] = {64};
  cuuint32_t box[2] = {128, 256};      // two blocks per copy: boxes of 128 four-bit rows do not reach the HBM rate
  cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, const_cast<void*>(base), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_error, sizeof g_error, "cuTensorMapEncodeTiled (MXFP4 tiles) failed with CUresult %d", (int)r);
    return -1;
  }
  return 0;
}

// Per-device set-up of the tensor-core kernels: the opt-in to more than 48 KiB of dynamic shared memory is a
// per-device function attribute, so a process that drives several GPUs runs this once for each of them.
constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
bool g_umma_ready[kMaxDevices] = {};
bool g_tokmajor_ok[kMaxDevices] = {};   // the token-major kernels were built with the register allocation they assume

int current_device_index(int* device) {
  cudaError_t e = cudaGetDevice(device);
  if (e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  if (*device < 0 || *device >= kMaxDevices) return fail("device index out of range (0..63)");
  return 0;
}

int umma_setup() {
  int device = 0;
  if (int rc = current_device_index(&device)) return rc;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_umma_ready[device]) return 0;
  int major = 0;
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (major != 10) return fail("this library targets sm_100a (compute capability 10.x)");
  cudaError_t e = cudaFuncSetAttribute(netra_moe_gate_up_umma_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       gate_up_smem_bytes());
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(gate_up)", e);
  e = cudaFuncSetAttribute(netra_moe_down_umma_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, down_smem_bytes());
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(down)", e);
  e = cudaFuncSetAttribute(netra_moe_gate_up_umma_gather_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, gate_up_smem_bytes());
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(gate_up_gather)", e);
  e = cudaFuncSetAttribute(netra_moe_gate_up_down_umma_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, gate_up_down_smem_bytes());
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(gate_up_down)", e);
  e = cudaFuncSetAttribute(netra_moe_gate_up_mxfp4_umma_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, gate_up_mxfp4_smem_bytes());
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(gate_up_mxfp4)", e);
  e = cudaFuncSetAttribute(netra_moe_down_mxfp4_umma_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, down_mxfp4_smem_bytes());
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(down_mxfp4)", e);
  e = cudaFuncSetAttribute(netra_moe_gate_up_mxfp4_tokmajor_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, gate_up_mxfp4_tokmajor_smem_bytes());
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(gate_up_mxfp4_tokmajor)", e);
  e = cudaFuncSetAttribute(netra_moe_down_mxfp4_tokmajor_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, down_mxfp4_tokmajor_smem_bytes());
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(down_mxfp4_tokmajor)", e);
  e = cudaFuncSetAttribute(netra_moe_gate_up_tokmajor_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, gate_up_tokmajor_smem_bytes());
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(gate_up_tokmajor)", e);
  e = cudaFuncSetAttribute(netra_moe_down_tokmajor_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, down_tokmajor_smem_bytes());
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(down_tokmajor)", e);
  e = cudaFuncSetAttribute(netra_moe_gate_up_tokmajor_gather_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, gate_up_tokmajor_smem_bytes());
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(gate_up_tokmajor_gather)", e);
  e = cudaFuncSetAttribute(netra_moe_down_tokmajor_f16_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, down_tokmajor_f16_smem_bytes());
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(down_tokmajor_f16)", e);
  e = cudaFuncSetAttribute(netra_router_logits_f32_umma_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, router_umma_smem_bytes());
  if (e != cudaSuccess) return fail_cuda("cudaFuncSetAttribute(router_umma)", e);
  {
    // the register re-balancing inside these kernels is only deadlock-free for the launch allocation it was written for
    cudaFuncAttributes a0, a1, a2, a3, a4, a5;
    e = cudaFuncGetAttributes(&a0, netra_moe_gate_up_tokmajor_sm100);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a1, netra_moe_down_tokmajor_sm100);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a2, netra_moe_down_tokmajor_f16_sm100);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a3, netra_moe_gate_up_tokmajor_gather_sm100);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a4, netra_moe_gate_up_mxfp4_tokmajor_sm100);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a5, netra_moe_down_mxfp4_tokmajor_sm100);
    if (e != cudaSuccess) return fail_cuda("cudaFuncGetAttributes(tokmajor)", e);
    g_tokmajor_ok[device] = a0.numRegs == kTmRegsLaunch && a1.numRegs == kTmRegsLaunch && a2.numRegs == kTmRegsLaunch &&
                            a3.numRegs == kTmRegsLaunch && a4.numRegs == kTmRegsLaunch && a5.numRegs == kTmRegsLaunch;
  }
  g_umma_ready[device] = true;
  return 0;
}

// The token-major GEMMs pay off once an expert's rows fill a good part of a 128-row tile: from an average
// of 32 rows per routed expert (1,024 tokens on one GPU) the layer switches to them.
constexpr uint32_t kTokMajorMinRowsPerExpert = 32;
bool use_tokmajor(int device, uint64_t pairs, uint32_t routed_experts) {
  return g_tokmajor_ok[device] && pairs >= (uint64_t)kTokMajorMinRowsPerExpert * routed_experts;
}
constexpr uint32_t kWeightsMxfp4 = 2;   // value of weights_tiled: MXFP4 code blocks and scale atoms

}  // namespace

struct netra_moe_layer {
  netra_moe_layer_desc_t desc;
  netra_moe_workspace_layout_t lay;
  CUtensorMap tm_w13, tm_w2, tm_a1, tm_a32, tm_a64, tm_a128, tm_h32, tm_h64, tm_h128, tm_router;
  int sm_count;
  int device;
  uint32_t launches;
  uint32_t gemm_mode;     // 0: pick the GEMM form by size, 1: always the swap-AB (decode) kernels, 2: swap-AB, both projections in one launch
  uint32_t router_mode;   // 0: pick the router by size, 1: always the FP64 tensor-core router, 2: as 0 with every logit exact
  uint32_t partial_f16;   // 1: the token-major down projection writes FP16 partial rows (prefill contract)
  bool gather_rows_in_gemm;   // the token-major gate_up gathers its rows with four-row TMA gathers (slower; kept as a recorded tactic)
  bool prequantised;      // set for the duration of a call whose token rows were quantised by the fused norm kernel
  bool external_topk;     // set for the duration of a call that brings its own top-k: the sort then runs as a launch of its own
  uint32_t front_mode;    // 0: router, top-k + quantisation and sort are three launches; 1: one launch for calls of up to 1,024 tokens
};

namespace {
bool layer_merged_gemm(const netra_moe_layer* layer, uint32_t pairs);
}

extern "C" {

// ------------------------------------------------------------------ bridges
// load(): the kernels are linked in, so there is no code object to open; it runs the per-device set-up, which refuses a
// device that is not sm_100a - as the reference's load() refuses a wrong architecture.
#define NETRA_BRIDGE_COMMON(name)                                       \
  int name##_load(const char*) { return umma_setup(); }                 \
  int name##_unload(void) { return 0; }                                 \
  const char* name##_last_error(void) { return g_error; }

NETRA_BRIDGE_COMMON(netra_qwen36_router_bf16)
NETRA_BRIDGE_COMMON(netra_qwen36_shared_gate_append)
NETRA_BRIDGE_COMMON(netra_qwen36_moe_gate_up)
NETRA_BRIDGE_COMMON(netra_qwen36_moe_silu_mul_quant)
NETRA_BRIDGE_COMMON(netra_qwen36_moe_down_reduce)

int netra_qwen36_router_bf16_launch(void* out, const void* hidden, const void* weight, uint32_t rows, cudaStream_t stream) {
  if (!out || !hidden || !weight || rows == 0) return fail("router_bf16: null pointer or zero rows");
  dim3 grid((rows + 15) / 16, 8);
  netra_router_logits_bf16_sm100<<<grid, 256, 0, stream>>>((uint16_t*)out, (const uint16_t*)hidden, (const uint16_t*)weight, rows);
  return check_launch("router_bf16 launch");
}

int netra_qwen36_shared_gate_append_launch(void* out_ids, void* out_w, const void* hidden, const void* gate_w,
                                           const void* ids, const void* w, uint32_t rows, cudaStream_t stream) {
  if (!out_ids || !out_w || !hidden || !gate_w || !ids || !w || rows == 0) return fail("shared_gate_append: null pointer or zero rows");
  netra_qwen36_shared_gate_append_sm100<<<rows, 32, 0, stream>>>((int32_t*)out_ids, (float*)out_w, (const uint16_t*)hidden,
                                                                 (const uint16_t*)gate_w, (const int32_t*)ids, (const float*)w, rows);
  return check_launch("shared_gate_append launch");
}

int netra_qwen36_moe_gate_up_launch(const void* hidden_fp8, const float* hidden_scale, const void* w13, const float* w13_scale,
                                    const int32_t* topk_ids, float* out, int rows, cudaStream_t stream) {
  if (!hidden_fp8 || !hidden_scale || !w13 || !w13_scale || !topk_ids || !out || rows <= 0) return fail("gate_up: null pointer or bad rows");
  dim3 grid(2 * kInter / 64, rows * kSlots);
  netra_qwen36_moe_gate_up_fp8_sm100<<<grid, 256, 0, stream>>>((const uint8_t*)hidden_fp8, hidden_scale, (const uint8_t*)w13,
                                                               w13_scale, topk_ids, out, (uint32_t)rows);
  return check_launch("gate_up launch");
}

int netra_qwen36_moe_silu_mul_quant_launch(const float* in, void* out_fp8, float* out_scale, int rows, cudaStream_t stream) {
  if (!in || !out_fp8 || !out_scale || rows <= 0) return fail("silu_mul_quant: null pointer or bad rows");
  netra_qwen36_moe_silu_mul_quant_fp8_sm100<<<rows, 64, 0, stream>>>(in, (uint8_t*)out_fp8, out_scale, (uint32_t)rows);
  return check_launch("silu_mul_quant launch");
}

int netra_qwen36_moe_down_reduce_launch(const void* act_fp8, const float* act_scale, const void* w2, const float* w2_scale,
                                        const float* topk_w, const int32_t* topk_ids, void* out, int rows, cudaStream_t stream) {
  if (!act_fp8 || !act_scale || !w2 || !w2_scale || !topk_w || !topk_ids || !out || rows <= 0) return fail("down_reduce: null pointer or bad rows");
  dim3 grid(kHidden / 64, rows);
  netra_qwen36_moe_down_reduce_fp8_sm100<<<grid, 256, 0, stream>>>((const uint8_t*)act_fp8, act_scale, (const uint8_t*)w2, w2_scale,
                                                                   topk_w, topk_ids, (uint16_t*)out, (uint32_t)rows);
  return check_launch("down_reduce launch");
}

// group-quant bridge (runtime/gfx950/group_quant/verify/group_quant_assembly_bridge.h:21-31), at width 2048
int netra_group_quant_assembly_load(const char*, const char*, const char*, const char*, const char*, const char*) { return umma_setup(); }
int netra_group_quant_assembly_unload(void) { return 0; }
const char* netra_group_quant_assembly_last_error(void) { return g_error; }

int netra_add_rmsnorm_group_quant_n2048_launch(const void* input_bf16, const void* residual_bf16, const void* weight_f32,
                                               void* output_bf16, void* residual_out_bf16, void* output_fp8,
                                               void* output_scale_f32, uint32_t rows, float epsilon, cudaStream_t stream) {
  if (!input_bf16 || !residual_bf16 || !weight_f32 || !output_bf16 || !residual_out_bf16 || !output_fp8 || !output_scale_f32)
    return fail("add_rmsnorm_group_quant: pointers must be nonnull");
  if (rows == 0 || rows > (1u << 20)) return fail("add_rmsnorm_group_quant: rows out of range");
  if (!(epsilon > 0.0f)) return fail("add_rmsnorm_group_quant: epsilon must be positive");
  netra_add_rmsnorm_group_quant_n2048_sm100<<<(rows + 3) / 4, 128, 0, stream>>>(
      (const uint16_t*)input_bf16, (const uint16_t*)residual_bf16, (const float*)weight_f32, (uint16_t*)output_bf16,
      (uint16_t*)residual_out_bf16, (uint8_t*)output_fp8, (float*)output_scale_f32, rows, 0u, epsilon);
  return check_launch("add_rmsnorm_group_quant launch");
}

// ------------------------------------------------------------------ fused layer
const char* netra_moe_last_error(void) { return g_error; }

int netra_moe_workspace_layout_query(uint32_t tokens, netra_moe_workspace_layout_t* out) {
  if (out == nullptr || out->struct_size != sizeof(netra_moe_workspace_layout_t)) return fail("workspace_layout: bad struct_size");
  if (tokens == 0 || tokens > (1u << 20)) return fail("workspace_layout: tokens out of range");
  const uint64_t t = tokens, p = t * kTopK, rows = p + t;
  const uint64_t nseg = (p + kSortSegment - 1) / kSortSegment;
  uint64_t o = 0;
  auto take = [&](uint64_t bytes) { uint64_t at = o; o = align_up(o + bytes, 1024); return at; };
  out->tokens = tokens;
  out->logits_bf16 = take(t * kRouted * 2);
  out->topk_ids = take(t * kSlots * 4);
  out->topk_weights = take(t * kSlots * 4);
  out->perm = take(p * 4);
  out->inv_perm = take(p * 4);
  out->counts = take(kRouted * 4);
  out->offsets = take((kRouted + 2) * 4);
  out->seg_hist = take(nseg * kRouted * 4);
  out->a_fp8 = take(rows * kHidden);
  out->a_scale = take((rows + 128) * kHiddenBlocks * 4);   // +128 rows: scale tiles are copied 128 rows at a time
  out->h_fp8 = take(rows * kInter);
  out->h_scale = take((rows + 128) * kInterBlocks * 4);
  out->down_f32 = take(rows * kHidden * 4);
  out->status = take(16);
  out->logits_f32 = take(t * kRouted * 4);
  out->wnorm = take(kRouted * 4);
  out->router_stats = take(16);
  out->gemm_ready = take(kReadyWords * 4);
  out->front_counters = take(128 * 4);
  out->total_bytes = o;
  return 0;
}

int netra_moe_layer_create(const netra_moe_layer_desc_t* desc, netra_moe_layer_t** output) {
  if (desc == nullptr || output == nullptr || desc->struct_size != sizeof(netra_moe_layer_desc_t)) return fail("layer_create: bad struct_size");
  if (!desc->router_weight_bf16 || !desc->w13_fp8 || !desc->w13_scale_f32 || !desc->w2_fp8 || !desc->w2_scale_f32 || !desc->workspace)
    return fail("layer_create: null pointer");
  if (((uintptr_t)desc->workspace & 1023) != 0) return fail("layer_create: workspace must be 1024-byte aligned");
  netra_moe_workspace_layout_t lay;
  lay.struct_size = sizeof lay;
  if (int rc = netra_moe_workspace_layout_query(desc->max_tokens, &lay)) return rc;
  if (desc->workspace_bytes < lay.total_bytes) return fail("layer_create: workspace too small");
  int device = 0, major = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (major != 10) return fail("layer_create: this library targets sm_100a (compute capability 10.x)");
  if (int rc = umma_setup()) return rc;
  netra_moe_layer* layer = new (std::nothrow) netra_moe_layer;
  if (layer == nullptr) return fail("layer_create: out of host memory");
  layer->desc = *desc;
  layer->lay = lay;
  layer->sm_count = sms;
  layer->device = device;
  layer->launches = 9;  // stages of launch_stage()
  layer->gemm_mode = 0;
  layer->router_mode = 0;
  layer->partial_f16 = 0;
  layer->prequantised = false;
  layer->external_topk = false;
  layer->front_mode = 0;
  layer->gather_rows_in_gemm = false;
  const uint64_t slabs = desc->num_expert_slabs ? desc->num_expert_slabs : (uint64_t)(kRouted + 1);
  if (slabs > (uint64_t)(kRouted + 1)) { delete layer; return fail("layer_create: at most 257 expert slabs"); }
  uint8_t* ws = (uint8_t*)desc->workspace;
  const uint64_t rows = (uint64_t)desc->max_tokens * (kTopK + 1);
  int rc = 0;
  if (desc->weights_tiled > kWeightsMxfp4) { delete layer; return fail("layer_create: unknown weights_tiled value"); }
  if (desc->weights_tiled == kWeightsMxfp4) {   // blocks of 128 rows x 64 bytes of E2M1 codes, one after another
    rc = rc ? rc : encode_fp4_tiles(&layer->tm_w13, desc->w13_fp8, slabs * 2 * kInter * kHiddenBlocks);
    rc = rc ? rc : encode_fp4_tiles(&layer->tm_w2, desc->w2_fp8, slabs * kHidden * kInterBlocks);
  } else if (desc->weights_tiled) {   // tiles of 128 rows x 128 bytes, one after another
    rc = rc ? rc : encode_u8_2d(&layer->tm_w13, desc->w13_fp8, slabs * 2 * kInter * kHiddenBlocks, kBlock, 128);
    rc = rc ? rc : encode_u8_2d(&layer->tm_w2, desc->w2_fp8, slabs * kHidden * kInterBlocks, kBlock, 128);
  } else {
    rc = rc ? rc : encode_u8_2d(&layer->tm_w13, desc->w13_fp8, slabs * 2 * kInter, kHidden, 128);
    rc = rc ? rc : encode_u8_2d(&layer->tm_w2, desc->w2_fp8, slabs * kHidden, kInter, 128);
  }
  rc = rc ? rc : encode_u8_2d(&layer->tm_router, desc->router_weight_bf16, kRouted, kHidden * 2, 128);
  rc = rc ? rc : encode_u8_2d(&layer->tm_a1, ws + lay.a_fp8, rows, kHidden, 1);     // one-row box: four-row gathers
  rc = rc ? rc : encode_u8_2d(&layer->tm_a32, ws + lay.a_fp8, rows, kHidden, 32);
  rc = rc ? rc : encode_u8_2d(&layer->tm_a64, ws + lay.a_fp8, rows, kHidden, 64);
  rc = rc ? rc : encode_u8_2d(&layer->tm_a128, ws + lay.a_fp8, rows, kHidden, 128);
  rc = rc ? rc : encode_u8_2d(&layer->tm_h32, ws + lay.h_fp8, rows, kInter, 32);
  rc = rc ? rc : encode_u8_2d(&layer->tm_h64, ws + lay.h_fp8, rows, kInter, 64);
  rc = rc ? rc : encode_u8_2d(&layer->tm_h128, ws + lay.h_fp8, rows, kInter, 128);
  if (rc == 0) {
    e = cudaMemset(ws + lay.status, 0, 16);
    if (e == cudaSuccess) e = cudaMemset(ws + lay.router_stats, 0, 16);
    if (e == cudaSuccess) e = cudaMemset(ws + lay.front_counters, 0, 128 * 4);
    if (e != cudaSuccess) rc = fail_cuda("cudaMemset(status)", e);
  }
  if (rc != 0) { delete layer; return rc; }
  *output = layer;
  return 0;
}

uint32_t netra_moe_layer_launch_count(const netra_moe_layer_t* layer, uint32_t tokens) {
  if (layer == nullptr) return 0;
  uint32_t n = tokens <= (uint32_t)kSortSmallMaxRows ? layer->launches - 2 : layer->launches;
  if (tokens <= (uint32_t)kSortSmallMaxRows && layer->front_mode == 1) n -= 2;   // router, top-k + quantisation and sort are one launch
  if (layer_merged_gemm(layer, tokens * kTopK)) --n;   // both projections in one launch
  if (layer->gather_rows_in_gemm && layer->desc.weights_tiled != kWeightsMxfp4 && layer->gemm_mode != 2) --n;   // no row gather
  return n;
}

}  // extern "C" (reopened below)

namespace {
constexpr uint32_t kStageCount = 9;
constexpr uint32_t kRouterK8MaxRows = 1024;   // up to here the router runs on the FP64 tensor cores with eight K-slices per tile

// Calls above kRouterK8MaxRows rows take the BF16 tensor-core router (FP32 approximations, then FP64 only where
// the rounding is undecided) unless the layer was told to keep the FP64 router.
bool use_umma_router(const netra_moe_layer* layer, uint32_t tokens) {
  return tokens > kRouterK8MaxRows && layer->router_mode != 1;
}
bool layer_tokmajor(const netra_moe_layer* layer, uint32_t pairs) {
  return layer->gemm_mode == 0 && use_tokmajor(layer->device, pairs, kRouted);
}
// Recorded tactic (gemm_mode 2): both projections in one launch.  Measured at 256 tokens: 164.4 us per call against 160.4 us
// for two launches - every CTA reaches the boundary between the halves at the same time (the items are spread evenly), so
// the drained pipeline and the second set-up idle the HBM as long as the launch gap did.  (The work-item units fit the
// counter table up to 8,192 + 1,024 rows in 32-row chunks over 257 groups: 545 units.)
bool layer_merged_gemm(const netra_moe_layer* layer, uint32_t pairs) {
  return layer->gemm_mode == 2 && layer->desc.weights_tiled != kWeightsMxfp4 && pairs <= (uint32_t)kTokMajorMinRowsPerExpert * kRouted;
}
// FP16 partial rows are an output format of the E4M3 token-major down projection
bool use_f16_partials(const netra_moe_layer* layer, uint32_t pairs) {
  return layer->partial_f16 != 0 && layer->desc.weights_tiled != kWeightsMxfp4 && layer_tokmajor(layer, pairs);
}

// One launch of the layer's fixed sequence (same idea as the reference's per-operation launch,
// runtime/gfx950/engine/netra_engine.h:90-92).  Returns 0 or the code of a failed host-side step.
int launch_stage(netra_moe_layer* layer, uint32_t stage, const void* hidden, const float* shared_w, void* out,
                 uint32_t tokens, cudaStream_t stream) {
  const netra_moe_workspace_layout_t& L = layer->lay;
  uint8_t* ws = (uint8_t*)layer->desc.workspace;
  uint16_t* logits = (uint16_t*)(ws + L.logits_bf16);
  int32_t* ids9 = (int32_t*)(ws + L.topk_ids);
  float* w9 = (float*)(ws + L.topk_weights);
  int32_t* perm = (int32_t*)(ws + L.perm);
  int32_t* inv_perm = (int32_t*)(ws + L.inv_perm);
  int32_t* counts = (int32_t*)(ws + L.counts);
  int32_t* offsets = (int32_t*)(ws + L.offsets);
  int32_t* seg_hist = (int32_t*)(ws + L.seg_hist);
  uint8_t* a_fp8 = ws + L.a_fp8;
  float* a_scale = (float*)(ws + L.a_scale);
  uint8_t* h_fp8 = ws + L.h_fp8;
  float* h_scale = (float*)(ws + L.h_scale);
  float* down = (float*)(ws + L.down_f32);
  uint32_t* status = (uint32_t*)(ws + L.status);
  float* logits_f32 = (float*)(ws + L.logits_f32);
  float* wnorm = (float*)(ws + L.wnorm);
  uint32_t* router_stats = (uint32_t*)(ws + L.router_stats);
  const uint16_t* router_w = (const uint16_t*)layer->desc.router_weight_bf16;
  const uint32_t pairs = tokens * kTopK;
  const uint32_t nseg = (pairs + kSortSegment - 1) / kSortSegment;
  const bool tokmajor = layer_tokmajor(layer, pairs);
  const bool mxfp4 = layer->desc.weights_tiled == kWeightsMxfp4;
  const bool merged = layer_merged_gemm(layer, pairs);
  // Recorded tactic: the swap-AB gate_up on E4M3 weights fetches its token rows from token order itself (no expert-sorted
  // copy).  Measured: 169.5 us per 256-token call against 160.3 us with the copy (149.3 against 144.7 at 64 tokens, no
  // difference at 16): eight four-row gathers per K-block instead of one box.
  const bool swapab_gather = layer->gather_rows_in_gemm && !tokmajor && !mxfp4 && !merged;
  uint32_t* gemm_ready = (uint32_t*)(ws + L.gemm_ready);
  // Recorded tactic (front_mode 1): up to 1,024 tokens stage 0 is the whole routing front end and stages 1 and 2 launch
  // nothing (a call with an external top-k skips stages 0 and 1, so its sort stays a launch of its own).  Measured at 256
  // tokens: 164.6 us per call against 160.4 us - router, top-k and sort depend on each other whole, so one launch only
  // trades two launch gaps for two device-wide hand-offs, and its sort runs on sixteen warps instead of thirty-two.
  const bool front = tokens <= (uint32_t)kSortSmallMaxRows && layer->front_mode == 1 && !layer->external_topk;
  switch (stage) {
    case 0:
      if (front) {
        netra_moe_route_front_sm100<<<dim3((tokens + 15) / 16, 8), 512, 0, stream>>>(
            logits, (const uint16_t*)hidden, router_w, ids9, w9, layer->prequantised ? nullptr : a_fp8, a_scale,
            layer->desc.router_bias_f32, shared_w, perm, inv_perm, counts, offsets, (uint32_t*)(ws + L.front_counters), tokens, pairs);
      } else if (use_umma_router(layer, tokens)) {
        // the token rows are the caller's buffer of this call: their tensor map is encoded here (host work only)
        CUtensorMap tm_hidden;
        if (int rc = encode_u8_2d(&tm_hidden, hidden, tokens, kHidden * 2, 128)) return rc;
        const uint32_t tiles = 2 * ((tokens + kRtTile - 1) / kRtTile);
        netra_router_logits_f32_umma_sm100<<<tiles + kRtNormCtas, kRtThreads, router_umma_smem_bytes(), stream>>>(
            tm_hidden, layer->tm_router, logits_f32, wnorm, router_w, tokens, status + 2);
      } else if (tokens <= kRouterK8MaxRows) {
        netra_router_logits_bf16_k8_sm100<<<dim3((tokens + 15) / 16, 8), 512, 0, stream>>>(
            logits, (const uint16_t*)hidden, router_w, tokens);
      } else {
        netra_router_logits_bf16_sm100<<<dim3((tokens + 15) / 16, 8), 256, 0, stream>>>(
            logits, (const uint16_t*)hidden, router_w, tokens);
      }
      break;
    case 1: {
      if (front) break;
      uint8_t* q_rows = layer->prequantised ? nullptr : a_fp8;    // null: the fused norm kernel already wrote the token rows
      if (use_umma_router(layer, tokens))
        netra_moe_topk_quant_fix_sm100<<<(tokens + 3) / 4, 128, 0, stream>>>(
            ids9, w9, q_rows, a_scale, logits, logits_f32, wnorm, router_w, layer->desc.router_bias_f32, shared_w,
            (const uint16_t*)hidden, router_stats, tokens, pairs, layer->router_mode == 2 ? 1u : 0u);
      else
        netra_moe_topk_quant_sm100<<<(tokens + 3) / 4, 128, 0, stream>>>(
            ids9, w9, q_rows, a_scale, logits, layer->desc.router_bias_f32, shared_w, (const uint16_t*)hidden, tokens, pairs);
      break;
    }
    case 2:
      if (front) break;
      if (tokens <= (uint32_t)kSortSmallMaxRows)   // one block does the whole sort; stages 3 and 4 launch nothing
        netra_moe_sort_small_sm100<<<1, 1024, 0, stream>>>(perm, inv_perm, counts, offsets, ids9, tokens);
      else
        netra_moe_sort_hist_sm100<<<nseg, 256, 0, stream>>>(seg_hist, ids9, tokens);
      break;
    case 3:
      if (tokens > (uint32_t)kSortSmallMaxRows) netra_moe_sort_scan_sm100<<<1, 256, 0, stream>>>(seg_hist, counts, offsets, tokens, nseg);
      break;
    case 4:
      if (tokens > (uint32_t)kSortSmallMaxRows) netra_moe_sort_scatter_sm100<<<nseg, 256, 0, stream>>>(perm, inv_perm, seg_hist, ids9, tokens);
      break;
    case 5:   // the gathering gate_up fetches its token rows itself: no expert-sorted copy is made for it
      if (!(tokmajor && layer->gather_rows_in_gemm && !mxfp4) && !swapab_gather)
        netra_moe_gather_rows_sm100<<<(pairs + 7) / 8, 256, 0, stream>>>(a_fp8, a_scale, perm, tokens, merged ? gemm_ready : nullptr,
                                                                         (uint32_t)kReadyWords);
      break;
    case 6:
      if (swapab_gather)
        netra_moe_gate_up_umma_gather_sm100<<<layer->sm_count, kGemmThreads, gate_up_smem_bytes(), stream>>>(
            layer->tm_w13, layer->tm_a1, a_scale, layer->desc.w13_scale_f32, offsets, perm, h_fp8, h_scale, kRouted + 1,
            layer->desc.weights_tiled, pairs, status);
      else if (merged)
        netra_moe_gate_up_down_umma_sm100<<<layer->sm_count, kGemmThreads, gate_up_down_smem_bytes(), stream>>>(
            layer->tm_w13, layer->tm_a32, layer->tm_w2, layer->tm_h32, a_scale, layer->desc.w13_scale_f32, layer->desc.w2_scale_f32, offsets,
            h_fp8, h_scale, down, kRouted + 1, layer->desc.weights_tiled, gemm_ready, status);
      else if (mxfp4 && tokmajor)
        netra_moe_gate_up_mxfp4_tokmajor_sm100<<<layer->sm_count, kTmThreads, gate_up_mxfp4_tokmajor_smem_bytes(), stream>>>(
            layer->tm_w13, layer->tm_a128, a_scale, (const uint8_t*)layer->desc.w13_scale_f32, offsets, h_fp8, h_scale, kRouted + 1,
            status);
      else if (mxfp4)
        netra_moe_gate_up_mxfp4_umma_sm100<<<layer->sm_count, kGemmThreads, gate_up_mxfp4_smem_bytes(), stream>>>(
            layer->tm_w13, layer->tm_a32, layer->tm_a64, layer->tm_a128, a_scale, (const uint8_t*)layer->desc.w13_scale_f32, offsets,
            h_fp8, h_scale, kRouted + 1, status);
      else if (tokmajor && layer->gather_rows_in_gemm)
        // Measured at 8,192 tokens: 607 us against 240 us for the form below.  One four-row gather per lane and K-block is 32
        // TMA instructions where the sorted copy needs one; the copy engine's issue rate, not the bytes, sets the pace.
        netra_moe_gate_up_tokmajor_gather_sm100<<<layer->sm_count, kTmThreads, gate_up_tokmajor_smem_bytes(), stream>>>(
            layer->tm_w13, layer->tm_a1, a_scale, layer->desc.w13_scale_f32, offsets, perm, h_fp8, h_scale, kRouted + 1,
            layer->desc.weights_tiled, pairs, status);
      else if (tokmajor)
        netra_moe_gate_up_tokmajor_sm100<<<layer->sm_count, kTmThreads, gate_up_tokmajor_smem_bytes(), stream>>>(
            layer->tm_w13, layer->tm_a128, a_scale, layer->desc.w13_scale_f32, offsets, h_fp8, h_scale, kRouted + 1,
            layer->desc.weights_tiled, status);
      else
        netra_moe_gate_up_umma_sm100<<<layer->sm_count, kGemmThreads, gate_up_smem_bytes(), stream>>>(
            layer->tm_w13, layer->tm_a32, layer->tm_a64, layer->tm_a128, a_scale, layer->desc.w13_scale_f32, offsets, h_fp8,
            h_scale, kRouted + 1, layer->desc.weights_tiled, status);
      break;
    case 7:
      if (merged)
        break;      // the down projection ran inside stage 6's launch
      if (mxfp4 && tokmajor)
        netra_moe_down_mxfp4_tokmajor_sm100<<<layer->sm_count, kTmThreads, down_mxfp4_tokmajor_smem_bytes(), stream>>>(
            layer->tm_w2, layer->tm_h128, h_scale, (const uint8_t*)layer->desc.w2_scale_f32, offsets, down, kRouted + 1, status + 1);
      else if (mxfp4)
        netra_moe_down_mxfp4_umma_sm100<<<layer->sm_count, kGemmThreads, down_mxfp4_smem_bytes(), stream>>>(
            layer->tm_w2, layer->tm_h32, layer->tm_h64, layer->tm_h128, h_scale, (const uint8_t*)layer->desc.w2_scale_f32, offsets, down,
            kRouted + 1, status + 1);
      else if (tokmajor && layer->partial_f16)
        netra_moe_down_tokmajor_f16_sm100<<<layer->sm_count, kTmThreads, down_tokmajor_f16_smem_bytes(), stream>>>(
            layer->tm_w2, layer->tm_h128, h_scale, layer->desc.w2_scale_f32, offsets, down, kRouted + 1,
            layer->desc.weights_tiled, status + 1);
      else if (tokmajor)
        netra_moe_down_tokmajor_sm100<<<layer->sm_count, kTmThreads, down_tokmajor_smem_bytes(), stream>>>(
            layer->tm_w2, layer->tm_h128, h_scale, layer->desc.w2_scale_f32, offsets, down, kRouted + 1,
            layer->desc.weights_tiled, status + 1);
      else
        netra_moe_down_umma_sm100<<<layer->sm_count, kGemmThreads, down_smem_bytes(), stream>>>(
            layer->tm_w2, layer->tm_h32, layer->tm_h64, layer->tm_h128, h_scale, layer->desc.w2_scale_f32, offsets, down,
            kRouted + 1, layer->desc.weights_tiled, status + 1);
      break;
    default:
      if (use_f16_partials(layer, pairs))
        netra_moe_combine_f16_sm100<<<tokens, 256, 0, stream>>>((uint16_t*)out, (const __half*)down, w9, inv_perm, tokens);
      else
        netra_moe_combine_sm100<<<tokens, 256, 0, stream>>>((uint16_t*)out, down, w9, inv_perm, tokens);
      break;
  }
  return 0;
}
}  // namespace

extern "C" {

int netra_moe_layer_launch(netra_moe_layer_t* layer, const void* hidden, const float* shared_w, void* out, uint32_t tokens,
                           cudaStream_t stream) {
  if (layer == nullptr || hidden == nullptr || out == nullptr) return fail("layer_launch: null pointer");
  if (tokens == 0 || tokens > layer->desc.max_tokens) return fail("layer_launch: tokens exceed the bound capacity");
  for (uint32_t stage = 0; stage < kStageCount; ++stage)
    if (int rc = launch_stage(layer, stage, hidden, shared_w, out, tokens, stream)) return rc;
  return check_launch("layer launch");
}

int netra_moe_layer_launch_with_norm(netra_moe_layer_t* layer, const void* input, const void* residual, const float* norm_weight,
                                     float epsilon, void* hidden_out, void* residual_out, const float* shared_w, void* out,
                                     uint32_t tokens, cudaStream_t stream) {
  if (layer == nullptr || input == nullptr || residual == nullptr || norm_weight == nullptr || hidden_out == nullptr ||
      residual_out == nullptr || out == nullptr)
    return fail("layer_launch_with_norm: null pointer");
  if (tokens == 0 || tokens > layer->desc.max_tokens) return fail("layer_launch_with_norm: tokens exceed the bound capacity");
  const netra_moe_workspace_layout_t& L = layer->lay;
  uint8_t* ws = (uint8_t*)layer->desc.workspace;
  netra_add_rmsnorm_group_quant_n2048_sm100<<<(tokens + 3) / 4, 128, 0, stream>>>(
      (const uint16_t*)input, (const uint16_t*)residual, norm_weight, (uint16_t*)hidden_out, (uint16_t*)residual_out, ws + L.a_fp8,
      (float*)(ws + L.a_scale), tokens, tokens * kTopK, epsilon);
  layer->prequantised = true;
  int rc = 0;
  for (uint32_t stage = 0; stage < kStageCount && rc == 0; ++stage) rc = launch_stage(layer, stage, hidden_out, shared_w, out, tokens, stream);
  layer->prequantised = false;
  return rc ? rc : check_launch("layer launch with fused norm");
}

int netra_moe_layer_launch_with_topk(netra_moe_layer_t* layer, const void* hidden, const int32_t* topk_ids, const float* topk_weights,
                                     const float* shared_w, void* out, uint32_t tokens, cudaStream_t stream) {
  if (layer == nullptr || hidden == nullptr || out == nullptr || topk_ids == nullptr || topk_weights == nullptr)
    return fail("layer_launch_with_topk: null pointer");
  if (tokens == 0 || tokens > layer->desc.max_tokens) return fail("layer_launch_with_topk: tokens exceed the bound capacity");
  const netra_moe_workspace_layout_t& L = layer->lay;
  uint8_t* ws = (uint8_t*)layer->desc.workspace;
  netra_moe_import_topk_quant_sm100<<<(tokens + 3) / 4, 128, 0, stream>>>(
      (int32_t*)(ws + L.topk_ids), (float*)(ws + L.topk_weights), ws + L.a_fp8, (float*)(ws + L.a_scale), topk_ids, topk_weights,
      shared_w, (const uint16_t*)hidden, tokens, tokens * kTopK);
  layer->external_topk = true;
  int rc = 0;
  for (uint32_t stage = 2; stage < kStageCount && rc == 0; ++stage) rc = launch_stage(layer, stage, hidden, shared_w, out, tokens, stream);
  layer->external_topk = false;
  return rc ? rc : check_launch("layer launch with external top-k");
}

int netra_moe_layer_launch_stage(netra_moe_layer_t* layer, uint32_t stage, const void* hidden, const float* shared_w, void* out,
                                 uint32_t tokens, cudaStream_t stream) {
  if (layer == nullptr || hidden == nullptr || out == nullptr) return fail("layer_launch_stage: null pointer");
  if (tokens == 0 || tokens > layer->desc.max_tokens) return fail("layer_launch_stage: tokens exceed the bound capacity");
  if (stage >= kStageCount) return fail("layer_launch_stage: stage out of range");
  if (int rc = launch_stage(layer, stage, hidden, shared_w, out, tokens, stream)) return rc;
  return check_launch("layer stage launch");
}

int netra_moe_repack_tiles_launch(void* dst, const void* src, uint64_t total_rows, uint32_t k_bytes, cudaStream_t stream) {
  if (!dst || !src || dst == src) return fail("repack_tiles: null or aliased pointers");
  if (total_rows == 0 || total_rows % 128 != 0 || k_bytes == 0 || k_bytes % 128 != 0 || total_rows > (1ull << 31))
    return fail("repack_tiles: rows and row bytes must be positive multiples of 128");
  const uint64_t chunks = total_rows * k_bytes / 16;
  netra_moe_repack_tiles_sm100<<<(unsigned)((chunks + 255) / 256), 256, 0, stream>>>((uint4*)dst, (const uint4*)src,
                                                                                     (uint32_t)total_rows, k_bytes);
  return check_launch("repack_tiles launch");
}

int netra_moe_widen_scales_bf16_launch(float* dst_f32, const void* src_bf16, uint64_t count, cudaStream_t stream) {
  if (!dst_f32 || !src_bf16) return fail("widen_scales: null pointer");
  if (count == 0 || count > (1ull << 32)) return fail("widen_scales: count out of range");
  netra_moe_widen_scales_bf16_sm100<<<(unsigned)((count + 255) / 256), 256, 0, stream>>>(dst_f32, (const uint16_t*)src_bf16, count);
  return check_launch("widen_scales launch");
}

int netra_moe_mxfp4_expand_launch(void* dst_fp8, float* dst_scale, uint32_t* inexact, const void* packed, const void* scales_e8m0,
                                  uint64_t total_rows, uint32_t k, cudaStream_t stream) {
  if (!dst_fp8 || !dst_scale || !inexact || !packed || !scales_e8m0) return fail("mxfp4_expand: null pointer");
  if (total_rows == 0 || total_rows % 128 != 0 || k == 0 || k % 128 != 0 || total_rows / 128 > 65535u * 128u)
    return fail("mxfp4_expand: rows and k must be positive multiples of 128");
  if (total_rows / 128 > 65535) return fail("mxfp4_expand: at most 65,535 row tiles per call");
  netra_moe_mxfp4_expand_sm100<<<dim3(k / 128, (unsigned)(total_rows / 128)), 128, 0, stream>>>(
      (uint8_t*)dst_fp8, dst_scale, inexact, (const uint8_t*)packed, (const uint8_t*)scales_e8m0, k);
  return check_launch("mxfp4_expand launch");
}

int netra_moe_mxfp4_pack_launch(void* dst_codes, void* dst_scale_atoms, const void* packed, const void* scales_e8m0,
                                uint64_t total_rows, uint32_t k, uint32_t paired_half_rows, cudaStream_t stream) {
  if (!dst_codes || !dst_scale_atoms || !packed || !scales_e8m0 || dst_codes == packed || dst_scale_atoms == scales_e8m0)
    return fail("mxfp4_pack: null or aliased pointers");
  if (total_rows == 0 || total_rows % 128 != 0 || k == 0 || k % 128 != 0) return fail("mxfp4_pack: rows and k must be positive multiples of 128");
  if (total_rows / 128 > 65535) return fail("mxfp4_pack: at most 65,535 row tiles per call");
  if (paired_half_rows == 0 || paired_half_rows % 128 != 0 || total_rows % (2ull * paired_half_rows) != 0)
    return fail("mxfp4_pack: paired_half_rows must be a positive multiple of 128 and the rows whole groups of twice that");
  if ((((uintptr_t)dst_codes | (uintptr_t)packed) & 15) != 0 || (((uintptr_t)dst_scale_atoms | (uintptr_t)scales_e8m0) & 3) != 0)
    return fail("mxfp4_pack: code pointers must be 16-byte aligned, scale pointers 4-byte aligned");
  netra_moe_mxfp4_pack_sm100<<<dim3(k / 128, (unsigned)(total_rows / 128)), 128, 0, stream>>>(
      (uint8_t*)dst_codes, (uint8_t*)dst_scale_atoms, (const uint8_t*)packed, (const uint8_t*)scales_e8m0, k, paired_half_rows / 128);
  return check_launch("mxfp4_pack launch");
}

// ------------------------------------------------------------------ expert block (expert parallelism)
struct netra_moe_expert_block {
  netra_moe_expert_block_desc_t desc;
  CUtensorMap tm_w13, tm_w2, tm_a32, tm_a64, tm_a128, tm_h32, tm_h64, tm_h128;
  int sm_count;
};

int netra_moe_expert_block_create(const netra_moe_expert_block_desc_t* desc, netra_moe_expert_block_t** output) {
  if (!desc || !output || desc->struct_size != sizeof(netra_moe_expert_block_desc_t)) return fail("expert_block_create: bad struct_size");
  if (!desc->w13_fp8 || !desc->w13_scale_f32 || !desc->w2_fp8 || !desc->w2_scale_f32 || !desc->a_fp8 || !desc->a_scale_f32 ||
      !desc->h_fp8 || !desc->h_scale_f32 || !desc->down_f32 || !desc->offsets_i32 || !desc->status_u32)
    return fail("expert_block_create: null pointer");
  if (desc->num_groups == 0 || desc->num_groups > kRouted + 1 || desc->max_rows == 0) return fail("expert_block_create: bad group or row count");
  if (desc->weights_tiled > 1) return fail("expert_block_create: weights_tiled must be 0 or 1");
  int device = 0, major = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  if (major != 10) return fail("expert_block_create: this library targets sm_100a (compute capability 10.x)");
  if (int rc = umma_setup()) return rc;
  netra_moe_expert_block* b = new (std::nothrow) netra_moe_expert_block;
  if (!b) return fail("expert_block_create: out of host memory");
  b->desc = *desc;
  b->sm_count = sms;
  const uint64_t g = desc->num_groups, rows = desc->max_rows;
  int rc = 0;
  if (desc->weights_tiled) {
    rc = rc ? rc : encode_u8_2d(&b->tm_w13, desc->w13_fp8, g * 2 * kInter * kHiddenBlocks, kBlock, 128);
    rc = rc ? rc : encode_u8_2d(&b->tm_w2, desc->w2_fp8, g * kHidden * kInterBlocks, kBlock, 128);
  } else {
    rc = rc ? rc : encode_u8_2d(&b->tm_w13, desc->w13_fp8, g * 2 * kInter, kHidden, 128);
    rc = rc ? rc : encode_u8_2d(&b->tm_w2, desc->w2_fp8, g * kHidden, kInter, 128);
  }
  rc = rc ? rc : encode_u8_2d(&b->tm_a32, desc->a_fp8, rows, kHidden, 32);
  rc = rc ? rc : encode_u8_2d(&b->tm_a64, desc->a_fp8, rows, kHidden, 64);
  rc = rc ? rc : encode_u8_2d(&b->tm_a128, desc->a_fp8, rows, kHidden, 128);
  rc = rc ? rc : encode_u8_2d(&b->tm_h32, desc->h_fp8, rows, kInter, 32);
  rc = rc ? rc : encode_u8_2d(&b->tm_h64, desc->h_fp8, rows, kInter, 64);
  rc = rc ? rc : encode_u8_2d(&b->tm_h128, desc->h_fp8, rows, kInter, 128);
  if (rc) { delete b; return rc; }
  *output = b;
  return 0;
}

int netra_moe_expert_block_launch(netra_moe_expert_block_t* b, cudaStream_t stream) {
  if (!b) return fail("expert_block_launch: null handle");
  const netra_moe_expert_block_desc_t& d = b->desc;
  netra_moe_gate_up_umma_sm100<<<b->sm_count, kGemmThreads, gate_up_smem_bytes(), stream>>>(
      b->tm_w13, b->tm_a32, b->tm_a64, b->tm_a128, d.a_scale_f32, d.w13_scale_f32, d.offsets_i32, (uint8_t*)d.h_fp8,
      d.h_scale_f32, d.num_groups, d.weights_tiled, d.status_u32);
  netra_moe_down_umma_sm100<<<b->sm_count, kGemmThreads, down_smem_bytes(), stream>>>(
      b->tm_w2, b->tm_h32, b->tm_h64, b->tm_h128, d.h_scale_f32, d.w2_scale_f32, d.offsets_i32, d.down_f32, d.num_groups,
      d.weights_tiled, d.status_u32 + 1);
  return check_launch("expert_block launch");
}

int netra_moe_expert_block_destroy(netra_moe_expert_block_t* b) {
  delete b;
  return 0;
}

int netra_ep_regroup_launch(int32_t* src_base, int32_t* dst_base, int32_t* offsets, int32_t* index, const int32_t* counts,
                            uint32_t sources, uint32_t experts, uint32_t extra_rows, uint32_t index_rows, uint32_t slot_rows,
                            uint32_t shared_first, cudaStream_t stream) {
  if (!src_base || !dst_base || !offsets || !index || !counts) return fail("ep_regroup: null pointer");
  if (sources == 0 || experts == 0 || sources * experts > 1024) return fail("ep_regroup: sources * experts must be 1..1024");
  if (slot_rows && index_rows != sources * slot_rows) return fail("ep_regroup: with slots, index_rows must be sources * slot_rows");
  netra_ep_regroup_bases_sm100<<<1, 1024, 0, stream>>>(src_base, dst_base, offsets, counts, sources, experts, extra_rows, slot_rows,
                                                     shared_first);
  if (index_rows > 0)
    netra_ep_regroup_index_sm100<<<(index_rows + 255) / 256, 256, 0, stream>>>(index, src_base, dst_base, counts, sources * experts,
                                                                             index_rows);
  return check_launch("ep_regroup launch");
}

int netra_moe_move_rows_launch(void* dst, const void* src, const int32_t* index, uint32_t rows, uint32_t copy_bytes,
                               uint32_t dst_pitch, uint32_t src_pitch, uint32_t dst_col, uint32_t src_col, uint32_t scatter,
                               cudaStream_t stream) {
  if (!dst || !src || !index) return fail("move_rows: null pointer");
  if (copy_bytes == 0 || (copy_bytes | dst_pitch | src_pitch | dst_col | src_col) % 16 != 0)
    return fail("move_rows: sizes, pitches and column offsets must be multiples of 16");
  if (dst_col + copy_bytes > dst_pitch || src_col + copy_bytes > src_pitch) return fail("move_rows: copy exceeds a row pitch");
  if (rows == 0) return 0;
  netra_moe_move_rows_sm100<<<(rows + 7) / 8, 256, 0, stream>>>((uint8_t*)dst, (const uint8_t*)src, index, rows, copy_bytes, dst_pitch,
                                                               src_pitch, dst_col, src_col, scatter);
  return check_launch("move_rows launch");
}

int netra_ep_pack_rows_launch(void* send_slots, const void* a_fp8, const float* a_scale, const int32_t* offsets, uint32_t ranks,
                              uint32_t experts_per_rank, uint32_t slot_rows, uint32_t* overflow, cudaStream_t stream) {
  if (!send_slots || !a_fp8 || !a_scale || !offsets || !overflow) return fail("ep_pack_rows: null pointer");
  if (ranks == 0 || slot_rows == 0 || ranks * experts_per_rank != (uint32_t)kRouted) return fail("ep_pack_rows: ranks * experts_per_rank must be 256");
  netra_ep_pack_rows_sm100<<<dim3((slot_rows + 7) / 8, ranks), 256, 0, stream>>>((uint8_t*)send_slots, (const uint8_t*)a_fp8, a_scale,
                                                                                offsets, experts_per_rank, slot_rows, overflow);
  return check_launch("ep_pack_rows launch");
}

int netra_ep_unpack_rows_launch(float* down, const float* back_slots, const int32_t* offsets, uint32_t ranks,
                                uint32_t experts_per_rank, uint32_t slot_rows, cudaStream_t stream) {
  if (!down || !back_slots || !offsets) return fail("ep_unpack_rows: null pointer");
  if (ranks == 0 || slot_rows == 0 || ranks * experts_per_rank != (uint32_t)kRouted) return fail("ep_unpack_rows: ranks * experts_per_rank must be 256");
  netra_ep_unpack_rows_sm100<<<dim3((slot_rows + 7) / 8, ranks), 256, 0, stream>>>(down, back_slots, offsets, experts_per_rank, slot_rows);
  return check_launch("ep_unpack_rows launch");
}

int netra_moe_kernel_launch_info(uint32_t which, uint32_t* block_threads, uint32_t* dynamic_smem_bytes) {
  if (!block_threads || !dynamic_smem_bytes || which > 10) return fail("kernel_launch_info: bad argument");
  *block_threads = (which < 2 || which == 6 || which == 7 || which == 10) ? kGemmThreads : which == 5 ? kRtThreads : kTmThreads;
  const int bytes[11] = {gate_up_smem_bytes(), down_smem_bytes(), gate_up_tokmajor_smem_bytes(), down_tokmajor_smem_bytes(),
                         down_tokmajor_f16_smem_bytes(), router_umma_smem_bytes(), gate_up_mxfp4_smem_bytes(), down_mxfp4_smem_bytes(),
                         gate_up_mxfp4_tokmajor_smem_bytes(), down_mxfp4_tokmajor_smem_bytes(), gate_up_down_smem_bytes()};
  *dynamic_smem_bytes = (uint32_t)bytes[which];
  return 0;
}

int netra_moe_layer_set_gemm_mode(netra_moe_layer_t* layer, uint32_t mode) {
  if (layer == nullptr || mode > 2) return fail("layer_set_gemm_mode: null layer or unknown mode");
  layer->gemm_mode = mode;
  return 0;
}

int netra_moe_layer_set_front_mode(netra_moe_layer_t* layer, uint32_t mode) {
  if (layer == nullptr || mode > 1) return fail("layer_set_front_mode: null layer or unknown mode");
  layer->front_mode = mode;
  return 0;
}

int netra_moe_layer_set_row_gather(netra_moe_layer_t* layer, uint32_t in_gemm) {
  if (layer == nullptr || in_gemm > 1) return fail("layer_set_row_gather: null layer or unknown mode");
  layer->gather_rows_in_gemm = in_gemm != 0;
  return 0;
}

int netra_moe_layer_set_router_mode(netra_moe_layer_t* layer, uint32_t mode) {
  if (layer == nullptr || mode > 2) return fail("layer_set_router_mode: null layer or unknown mode");
  layer->router_mode = mode;
  return 0;
}

int netra_moe_layer_set_partial_format(netra_moe_layer_t* layer, uint32_t format) {
  if (layer == nullptr || format > 1) return fail("layer_set_partial_format: null layer or unknown format");
  layer->partial_f16 = format;
  return 0;
}

int netra_moe_layer_router_stats(netra_moe_layer_t* layer, uint32_t stats_out[4]) {
  if (layer == nullptr || stats_out == nullptr) return fail("layer_router_stats: null pointer");
  cudaError_t e = cudaMemcpy(stats_out, (uint8_t*)layer->desc.workspace + layer->lay.router_stats, 16, cudaMemcpyDeviceToHost);
  return e == cudaSuccess ? 0 : fail_cuda("cudaMemcpy(router_stats)", e);
}

int netra_moe_layer_status(netra_moe_layer_t* layer, uint32_t status_out[4]) {
  if (layer == nullptr || status_out == nullptr) return fail("layer_status: null pointer");
  cudaError_t e = cudaMemcpy(status_out, (uint8_t*)layer->desc.workspace + layer->lay.status, 16, cudaMemcpyDeviceToHost);
  return e == cudaSuccess ? 0 : fail_cuda("cudaMemcpy(status)", e);
}

int netra_moe_layer_destroy(netra_moe_layer_t* layer) {
  delete layer;
  return 0;
}

}  // extern "C"

// Expert parallelism over peer memory (kernels and host side; uses the helpers and launch_stage() above).
#include "ep_p2p.cu"

// Entry point with library-owned scratch (needs fail(), fail_cuda(), check_launch() from above).
#include "static_scratch_sort.cu"

// The reference's 768-row prefill bridge on this library's stages (needs launch_stage() from above).
#include "prefill_m768_bridge.cu"

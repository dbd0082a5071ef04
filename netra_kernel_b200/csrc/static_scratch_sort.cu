// Token sort for callers that cannot allocate device memory.
//
// Some callers of this library may not call cudaMalloc at all: a serving process that hands its
// whole device-memory budget to one framework allocator at start-up, a plugin running inside a
// host application whose policy forbids driver allocations after initialisation, or a step that
// runs while a stream is being captured (allocation is illegal there).  The regular sort needs a
// scratch table (one 256-entry histogram per 1024 routed pairs) that such a caller would have to
// carve out of memory it does not control.  This entry point keeps that table inside the
// library image instead: a fixed 128 KiB array in device memory that every GPU which loads the
// library holds until the process exits.  The caller passes only inputs and outputs.
//
// Limits and rules:
//   * at most kStaticSortMaxRows (16,384) token rows per call, i.e. 131,072 routed pairs and 128
//     histogram segments; larger calls are refused with an error, never truncated;
//   * the first call on each device resolves the device address of the table
//     (cudaGetSymbolAddress) - make that first call outside any stream capture;
//   * every call on a device shares the one table.  The histogram kernel rewrites all entries it
//     will read, so nothing has to be cleared between calls, but two calls that overlap on the
//     GPU (different streams, or one graph replayed concurrently) race on it - serialise them;
//   * no cudaMalloc, cudaFree or allocating library routine is called here.
#include <mutex>

namespace {

constexpr uint32_t kStaticSortMaxRows = 16384;
constexpr uint32_t kStaticSortMaxSegments = kStaticSortMaxRows * netra::kTopK / netra::kSortSegment;   // 128
constexpr int kStaticSortMaxDevices = 64;

// In host code this name is only a handle for the symbol, not a device address.
static __device__ __align__(256) int32_t g_static_sort_scratch[kStaticSortMaxSegments * netra::kRouted];

int32_t* g_static_sort_ptr[kStaticSortMaxDevices] = {};
std::mutex g_static_sort_mutex;

// Device address of the table on the current device, resolved once per device.
int static_sort_scratch(int32_t** out) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return fail_cuda("cudaGetDevice", e);
  if (device < 0 || device >= kStaticSortMaxDevices) return fail("sort_static_scratch: device index out of range");
  std::lock_guard<std::mutex> lock(g_static_sort_mutex);
  if (g_static_sort_ptr[device] == nullptr) {
    int32_t* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_static_sort_scratch);
    if (e != cudaSuccess) return fail_cuda("cudaGetSymbolAddress(static sort scratch)", e);
    if (ptr == nullptr) return fail("sort_static_scratch: symbol address is null");
    g_static_sort_ptr[device] = ptr;
  }
  *out = g_static_sort_ptr[device];
  return 0;
}

}  // namespace

extern "C" int netra_moe_sort_static_scratch_launch(const int32_t* topk_ids_i32, int32_t* perm_i32, int32_t* inv_perm_i32,
                                                    int32_t* counts_i32, int32_t* offsets_i32, uint32_t rows,
                                                    cudaStream_t stream) {
  if (!topk_ids_i32 || !perm_i32 || !inv_perm_i32 || !counts_i32 || !offsets_i32)
    return fail("sort_static_scratch: null pointer");
  if (rows == 0) return fail("sort_static_scratch: zero rows");
  if (rows > kStaticSortMaxRows)
    return fail("sort_static_scratch: rows exceed the built-in scratch capacity of 16384 token rows");
  int32_t* scratch = nullptr;
  if (int rc = static_sort_scratch(&scratch)) return rc;
  const uint32_t pairs = rows * netra::kTopK;
  const uint32_t nseg = (pairs + netra::kSortSegment - 1) / netra::kSortSegment;
  netra::netra_moe_sort_hist_sm100<<<nseg, 256, 0, stream>>>(scratch, topk_ids_i32, rows);
  netra::netra_moe_sort_scan_sm100<<<1, 256, 0, stream>>>(scratch, counts_i32, offsets_i32, rows, nseg);
  netra::netra_moe_sort_scatter_sm100<<<nseg, 256, 0, stream>>>(perm_i32, inv_perm_i32, scratch, topk_ids_i32, rows);
  return check_launch("sort_static_scratch launch");
}

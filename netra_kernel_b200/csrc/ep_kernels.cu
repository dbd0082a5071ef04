// Expert-parallel helpers: regrouping rows that arrive source-rank-major into expert-major order
// (and back), and a generic indexed row gather.  The reference has no expert parallelism (its
// 8-GPU mode is eight replicas, manifests/gfx950/models/qwen36-moe-m1-golden.json:11-12); these
// kernels serve the all-to-all dispatch / combine around the grouped GEMMs.
#include "common.cuh"

namespace netra {

// counts[s * experts + e] = rows that source rank s sends for local expert e (sources * experts <= 1024).
// Source-major order: all rows of source 0 (expert ascending), then source 1, ...
// Expert-major order: all rows of expert 0 (source ascending), then expert 1, ...
// Outputs: src_base / dst_base per (s, e) bucket, and offsets[experts + 2]: exclusive prefix over
// local experts, then offsets[experts] = total routed rows, offsets[experts + 1] = total + extra_rows
// (the rows of the shared expert, appended after the routed rows).  grid 1, block 1024.
extern "C" __global__ void __launch_bounds__(1024)
netra_ep_regroup_bases_sm100(int32_t* __restrict__ src_base, int32_t* __restrict__ dst_base, int32_t* __restrict__ offsets,
                             const int32_t* __restrict__ counts, uint32_t sources, uint32_t experts, uint32_t extra_rows) {
  __shared__ int cnt[1024];
  const int n = (int)(sources * experts);
  const int tid = threadIdx.x;
  cnt[tid] = tid < n ? counts[tid] : 0;
  __syncthreads();
  // source-major exclusive prefix: bucket index b = s * experts + e is already in that order
  // expert-major exclusive prefix: position of bucket (s, e) in the order (e, s)
  int src = 0, dst = 0;
  if (tid < n) {
    const int s = tid / (int)experts, e = tid % (int)experts;
    for (int b = 0; b < tid; ++b) src += cnt[b];
    for (int ee = 0; ee < e; ++ee)
      for (int ss = 0; ss < (int)sources; ++ss) dst += cnt[ss * (int)experts + ee];
    for (int ss = 0; ss < s; ++ss) dst += cnt[ss * (int)experts + e];
    src_base[tid] = src;
    dst_base[tid] = dst;
    if (s == 0) offsets[e] = dst;
    if (tid == n - 1) {
      offsets[experts] = src + cnt[tid];
      offsets[experts + 1] = src + cnt[tid] + (int)extra_rows;
    }
  }
}

// index[i] = expert-major position of source-major row i.  grid ceil(rows/256), block 256.
extern "C" __global__ void __launch_bounds__(256)
netra_ep_regroup_index_sm100(int32_t* __restrict__ index, const int32_t* __restrict__ src_base,
                             const int32_t* __restrict__ dst_base, uint32_t buckets, const int32_t* __restrict__ total_rows) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= *total_rows) return;
  int lo = 0, hi = (int)buckets;          // largest bucket with src_base <= i (empty buckets share a base: take the last)
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (src_base[mid] <= i) lo = mid; else hi = mid;
  }
  index[i] = dst_base[lo] + (i - src_base[lo]);
}

// dst row r <- src row (index ? index[r] : r) when scatter == 0; dst row index[r] <- src row r when scatter == 1.
// Rows are row_bytes long (a multiple of 16).  One warp per row.  grid ceil(rows/8), block 256.
extern "C" __global__ void __launch_bounds__(256)
netra_moe_move_rows_sm100(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, const int32_t* __restrict__ index,
                          const int32_t* __restrict__ rows_ptr, uint32_t max_rows, uint32_t row_bytes, uint32_t scatter) {
  const int rows = rows_ptr != nullptr ? min(*rows_ptr, (int)max_rows) : (int)max_rows;
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= rows) return;
  const size_t other = (size_t)index[r];
  const uint4* s = reinterpret_cast<const uint4*>(src + (scatter ? (size_t)r : other) * row_bytes);
  uint4* d = reinterpret_cast<uint4*>(dst + (scatter ? other : (size_t)r) * row_bytes);
  for (uint32_t c = lane; c < row_bytes / 16; c += 32) d[c] = s[c];
}

}  // namespace netra

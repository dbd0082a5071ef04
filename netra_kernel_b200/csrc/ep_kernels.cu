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
                             const int32_t* __restrict__ counts, uint32_t sources, uint32_t experts, uint32_t extra_rows,
                             uint32_t slot_rows, uint32_t shared_first) {
  __shared__ int cnt[1024];
  const int n = (int)(sources * experts);
  const int tid = threadIdx.x;
  cnt[tid] = tid < n ? counts[tid] : 0;
  __syncthreads();
  // A sender whose rows for this rank exceed a slot sent only the first slot_rows of them (and raised its
  // overflow word): count no more than that, so no index or offset ever points past the receive buffers.
  if (slot_rows && tid < (int)sources) {
    int room = (int)slot_rows;
    for (int e = 0; e < (int)experts; ++e) {
      const int c = min(cnt[tid * (int)experts + e], room);
      cnt[tid * (int)experts + e] = c;
      room -= c;
    }
  }
  __syncthreads();
  // source-major exclusive prefix: bucket index b = s * experts + e is already in that order
  // expert-major exclusive prefix: position of bucket (s, e) in the order (e, s)
  int src = 0, dst = 0;
  if (tid < n) {
    const int s = tid / (int)experts, e = tid % (int)experts;
    if (slot_rows) {            // fixed-capacity exchange: source s owns rows [s * slot_rows, (s + 1) * slot_rows)
      src = s * (int)slot_rows;
      for (int ee = 0; ee < e; ++ee) src += cnt[s * (int)experts + ee];
    } else {
      for (int b = 0; b < tid; ++b) src += cnt[b];
    }
    for (int ee = 0; ee < e; ++ee)
      for (int ss = 0; ss < (int)sources; ++ss) dst += cnt[ss * (int)experts + ee];
    for (int ss = 0; ss < s; ++ss) dst += cnt[ss * (int)experts + e];
    // shared_first: the extra (shared expert) rows are group 0 at rows [0, extra_rows), routed groups follow
    const int base = shared_first ? (int)extra_rows : 0;
    src_base[tid] = src;
    dst_base[tid] = dst + base;
    if (s == 0) offsets[e + (shared_first ? 1 : 0)] = dst + base;
    if (tid == n - 1) {
      int total = 0;
      for (int b = 0; b < n; ++b) total += cnt[b];
      if (shared_first) {
        offsets[0] = 0;
        offsets[experts + 1] = base + total;
      } else {
        offsets[experts] = total;
        offsets[experts + 1] = total + (int)extra_rows;
      }
    }
  }
}

// index[i] = expert-major position of source-major row i, or -1 for an unused slot row.
// grid ceil(rows/256), block 256.
extern "C" __global__ void __launch_bounds__(256)
netra_ep_regroup_index_sm100(int32_t* __restrict__ index, const int32_t* __restrict__ src_base,
                             const int32_t* __restrict__ dst_base, const int32_t* __restrict__ counts, uint32_t buckets,
                             uint32_t rows) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int)rows) return;
  int lo = 0, hi = (int)buckets;          // largest bucket with src_base <= i (empty buckets share a base: take the last)
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (src_base[mid] <= i) lo = mid; else hi = mid;
  }
  const int within = i - src_base[lo];
  index[i] = within < counts[lo] ? dst_base[lo] + within : -1;
}

// Row mover with independent pitches.  scatter == 0: dst row r <- src row index[r];
// scatter == 1: dst row index[r] <- src row r; rows with index[r] < 0 are skipped.  copy_bytes, both
// pitches and both column offsets are multiples of 16.  One warp per row.  grid ceil(rows/8), block 256.
extern "C" __global__ void __launch_bounds__(256)
netra_moe_move_rows_sm100(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, const int32_t* __restrict__ index,
                          uint32_t rows, uint32_t copy_bytes, uint32_t dst_pitch, uint32_t src_pitch, uint32_t dst_col,
                          uint32_t src_col, uint32_t scatter) {
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= (int)rows) return;
  const int other = index[r];
  if (other < 0) return;
  const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)(scatter ? r : other) * src_pitch + src_col);
  uint4* d = reinterpret_cast<uint4*>(dst + (size_t)(scatter ? other : r) * dst_pitch + dst_col);
  for (uint32_t c = lane; c < copy_bytes / 16; c += 32) d[c] = s[c];
}

// Fixed-capacity exchange, sender side: the rows this rank routes to rank g (sorted rows
// [offsets[g*E_l], offsets[(g+1)*E_l])) go to slot rows [g*slot_rows, ...) of the send buffer, each
// slot row = 2048 FP8 codes followed by 16 FP32 scales (2112 bytes).  A destination that would need
// more than slot_rows rows sets *overflow.  grid (ceil(slot_rows/8), ranks), block 256.
constexpr int kEpRowBytes = kHidden + kHiddenBlocks * 4;   // 2112

extern "C" __global__ void __launch_bounds__(256)
netra_ep_pack_rows_sm100(uint8_t* __restrict__ send, const uint8_t* __restrict__ a_fp8, const float* __restrict__ a_scale,
                         const int32_t* __restrict__ offsets, uint32_t experts_per_rank, uint32_t slot_rows,
                         uint32_t* __restrict__ overflow) {
  const int g = blockIdx.y;
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int first = offsets[g * (int)experts_per_rank];
  const int n = offsets[(g + 1) * (int)experts_per_rank] - first;
  if (n > (int)slot_rows && i == 0 && lane == 0) atomicMax(overflow, (uint32_t)n);
  if (i >= n || i >= (int)slot_rows) return;
  const uint4* src = reinterpret_cast<const uint4*>(a_fp8 + (size_t)(first + i) * kHidden);
  uint4* dst = reinterpret_cast<uint4*>(send + ((size_t)g * slot_rows + i) * kEpRowBytes);
#pragma unroll
  for (int c = 0; c < 4; ++c) dst[c * 32 + lane] = src[c * 32 + lane];
  if (lane < 4) dst[128 + lane] = reinterpret_cast<const uint4*>(a_scale + (size_t)(first + i) * kHiddenBlocks)[lane];
}

// Fixed-capacity exchange, return side: slot row (g, i) of the returned FP32 rows is this rank's
// sorted row offsets[g*E_l] + i.  grid (ceil(slot_rows/8), ranks), block 256.
extern "C" __global__ void __launch_bounds__(256)
netra_ep_unpack_rows_sm100(float* __restrict__ down, const float* __restrict__ back, const int32_t* __restrict__ offsets,
                           uint32_t experts_per_rank, uint32_t slot_rows) {
  const int g = blockIdx.y;
  const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int first = offsets[g * (int)experts_per_rank];
  const int n = min(offsets[(g + 1) * (int)experts_per_rank] - first, (int)slot_rows);
  if (i >= n) return;
  const uint4* src = reinterpret_cast<const uint4*>(back + ((size_t)g * slot_rows + i) * kHidden);
  uint4* dst = reinterpret_cast<uint4*>(down + (size_t)(first + i) * kHidden);
#pragma unroll
  for (int c = 0; c < 16; ++c) dst[c * 32 + lane] = src[c * 32 + lane];
}

}  // namespace netra

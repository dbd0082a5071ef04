// Routing front end of the routed-MoE layer: exact BF16 router logits, softmax /
// top-8 / renormalise with the shared slot appended, per-token FP8 input
// quantisation, the stable expert-major token sort, the row gather into sorted
// order, and the slot-ordered weighted combine.
//
// Behaviour replaced (paths inside the reference project):
//   kernels/gfx950/templates/routing/bf16_gemv.inc:16-89            router logits
//   runtime/gfx950/routing/decode/qwen36_shared_gate_append_bridge.h:10-23  slot 8
//   scripts/rocm/integrations/sglang/netra_gfx1151_sglang.py:1186-1209      sort
//   harness/gfx950/fp8/moe/decode/qwen36_moe_silu_mul_quant_fp8_gfx950.hip:57-94  quantiser
//   kernels/gfx950/templates/moe/prefill/route_reduce_splitk2_f16.inc:107-118     combine order
#include "common.cuh"

namespace netra {

// ------------------------------------------------------------------------------------------
// Router logits.  logits[t,e] = RNE_bf16(exact dot(hidden[t,:], w[e,:])): BF16 products are
// exact in FP64 and a 2048-term FP64 sum is far below half a BF16 ulp from the exact value, so
// the single FP64->BF16 rounding is order independent in practice and bit-reproducible here
// (fixed lane-strided order + xor tree).
// grid (ceil(rows/4), 4), block 256: a warp owns 4 tokens x 8 experts.
// ------------------------------------------------------------------------------------------
constexpr int kRtTok = 4;
constexpr int kRtExp = 8;

__device__ __forceinline__ uint16_t f64_to_bf16_bits(double d) {
  long long bits = __double_as_longlong(d);
  uint16_t sign = (uint16_t)(((unsigned long long)bits >> 63) << 15);
  long long mag = bits & 0x7fffffffffffffffLL;
  long long r = (mag + ((1LL << 44) - 1) + ((mag >> 45) & 1)) >> 45;
  r -= (896LL << 7);
  if (r < (1 << 7)) r = 0;
  return (uint16_t)(sign | (uint16_t)r);
}

extern "C" __global__ void __launch_bounds__(256)
netra_router_logits_bf16_sm100(uint16_t* __restrict__ logits, const uint16_t* __restrict__ hidden,
                               const uint16_t* __restrict__ weight, uint32_t rows) {
  __shared__ uint4 sh[kRtTok][kHidden / 8];
  const int tok0 = blockIdx.x * kRtTok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kRtTok * (kHidden / 8); i += blockDim.x) {
    int t = i / (kHidden / 8), c = i % (kHidden / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tok0 + t < (int)rows) v = reinterpret_cast<const uint4*>(hidden + (size_t)(tok0 + t) * kHidden)[c];
    sh[t][c] = v;
  }
  __syncthreads();
  const int e0 = blockIdx.y * 64 + warp * kRtExp;
  double acc[kRtTok][kRtExp];
#pragma unroll
  for (int t = 0; t < kRtTok; ++t)
#pragma unroll
    for (int e = 0; e < kRtExp; ++e) acc[t][e] = 0.0;
  for (int i = 0; i < kHidden / 256; ++i) {
    const int c = i * 32 + lane;  // 16-byte chunk (8 values) index along K
    uint4 hv[kRtTok];
#pragma unroll
    for (int t = 0; t < kRtTok; ++t) hv[t] = sh[t][c];
#pragma unroll
    for (int e = 0; e < kRtExp; ++e) {
      uint4 wv = __ldg(reinterpret_cast<const uint4*>(weight + (size_t)(e0 + e) * kHidden) + c);
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        double w_lo = (double)bf16_bits_to_f32(ww[q] & 0xffffu);
        double w_hi = (double)bf16_bits_to_f32(ww[q] >> 16);
#pragma unroll
        for (int t = 0; t < kRtTok; ++t) {
          const uint32_t hh = (&hv[t].x)[q];
          acc[t][e] = fma((double)bf16_bits_to_f32(hh & 0xffffu), w_lo, acc[t][e]);
          acc[t][e] = fma((double)bf16_bits_to_f32(hh >> 16), w_hi, acc[t][e]);
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < kRtTok; ++t)
#pragma unroll
    for (int e = 0; e < kRtExp; ++e) {
      double v = acc[t][e];
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
      if (lane == 0 && tok0 + t < (int)rows)
        logits[(size_t)(tok0 + t) * kRouted + e0 + e] = f64_to_bf16_bits(v);
    }
}

// ------------------------------------------------------------------------------------------
// Softmax / top-8 / renormalise + shared slot + per-token FP8 quantisation.  One warp per token.
// Selection key is (z desc, expert id asc) with z = f32(logit) + bias; weights are
// softmax(z)[id] renormalised over the 8 selected entries in slot order.
// The quantised row goes to row (row_base + t) of the activation buffer.
// grid ceil(rows/4), block 128.
// ------------------------------------------------------------------------------------------
extern "C" __global__ void __launch_bounds__(128)
netra_moe_topk_quant_sm100(int32_t* __restrict__ ids9, float* __restrict__ w9,
                           uint8_t* __restrict__ a_fp8, float* __restrict__ a_scale,
                           const uint16_t* __restrict__ logits, const float* __restrict__ bias,
                           const float* __restrict__ shared_w, const uint16_t* __restrict__ hidden,
                           uint32_t rows, uint32_t row_base) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= (int)rows) return;
  // lane owns experts lane*8 .. lane*8+7 (ascending id inside the lane)
  float z[8];
  {
    uint4 v = reinterpret_cast<const uint4*>(logits + (size_t)t * kRouted)[lane];
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      z[2 * q] = bf16_bits_to_f32(u[q] & 0xffffu);
      z[2 * q + 1] = bf16_bits_to_f32(u[q] >> 16);
    }
    if (bias != nullptr) {
#pragma unroll
      for (int i = 0; i < 8; ++i) z[i] = z[i] + bias[lane * 8 + i];
    }
  }
  float zmax = z[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) zmax = fmaxf(zmax, z[i]);
  zmax = warp_max(zmax);
  float p[8], part = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) { p[i] = expf(z[i] - zmax); part += p[i]; }
  const float denom = warp_sum(part);
  uint32_t taken = 0;
  float sel_p = 0.0f;   // lane k (< 8) keeps the probability of slot k
  int sel_id = 0;
#pragma unroll 1
  for (int k = 0; k < kTopK; ++k) {
    float bv = -INFINITY; int bi = 0x7fffffff; float bp = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      bool better = !((taken >> i) & 1u) && (bi == 0x7fffffff || z[i] > bv);
      if (better) { bv = z[i]; bi = lane * 8 + i; bp = p[i]; }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, d);
      int oi = __shfl_xor_sync(0xffffffffu, bi, d);
      float op = __shfl_xor_sync(0xffffffffu, bp, d);
      bool take = (oi != 0x7fffffff) && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi));
      if (take) { bv = ov; bi = oi; bp = op; }
    }
    if ((bi >> 3) == lane) taken |= 1u << (bi & 7);
    if (lane == k) { sel_p = bp / denom; sel_id = bi; }
  }
  float s = 0.0f;
#pragma unroll
  for (int k = 0; k < kTopK; ++k) s += __shfl_sync(0xffffffffu, sel_p, k);  // slot-order FP32 sum
  if (lane < kTopK) {
    ids9[t * kSlots + lane] = sel_id;
    w9[t * kSlots + lane] = sel_p / s;
  } else if (lane == kTopK) {
    ids9[t * kSlots + kTopK] = kRouted;
    w9[t * kSlots + kTopK] = shared_w != nullptr ? shared_w[t] : 1.0f;
  }
  // ---- per-128 FP8 quantisation of the hidden row: a lane owns 64 values, 2 lanes one group
  const uint4* src = reinterpret_cast<const uint4*>(hidden + (size_t)t * kHidden) + lane * 8;
  float x[64];
  float amax = amax_floor();
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 v = src[c];
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      x[c * 8 + 2 * q] = bf16_bits_to_f32(u[q] & 0xffffu);
      x[c * 8 + 2 * q + 1] = bf16_bits_to_f32(u[q] >> 16);
    }
  }
#pragma unroll
  for (int i = 0; i < 64; ++i) amax = fmaxf(amax, fabsf(x[i]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  const float scale = amax * inv448();
  const float inv = 1.0f / scale;
  const size_t row = (size_t)row_base + t;
  if ((lane & 1) == 0) a_scale[row * kHiddenBlocks + (lane >> 1)] = scale;
  uint4* dst = reinterpret_cast<uint4*>(a_fp8 + row * kHidden) + lane * 4;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t b = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) b |= (uint32_t)f32_to_e4m3(x[c * 16 + q * 4 + j] * inv) << (8 * j);
      w[q] = b;
    }
    dst[c] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// ------------------------------------------------------------------------------------------
// Stable expert-major sort of the rows*8 routed pairs (pair index = t*8 + slot).
// Three launches for any size: per-segment histograms, a scan over segments, and a stable
// scatter; a segment is 1024 consecutive pairs.  No atomics decide an output position.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ int pair_expert(const int32_t* ids9, int pair) {
  return ids9[(pair >> 3) * kSlots + (pair & 7)];
}

// grid nseg, block 256
extern "C" __global__ void __launch_bounds__(256)
netra_moe_sort_hist_sm100(int32_t* __restrict__ seg_hist, const int32_t* __restrict__ ids9, uint32_t rows) {
  __shared__ int hist[kRouted];
  const int pairs = (int)rows * kTopK;
  hist[threadIdx.x] = 0;
  __syncthreads();
  const int base = blockIdx.x * kSortSegment;
  for (int i = threadIdx.x; i < kSortSegment && base + i < pairs; i += blockDim.x)
    atomicAdd(&hist[pair_expert(ids9, base + i)], 1);   // counts only: order independent
  __syncthreads();
  seg_hist[blockIdx.x * kRouted + threadIdx.x] = hist[threadIdx.x];
}

// grid 1, block 256: counts, exclusive offsets, and per-segment bases (in place in seg_hist).
// offsets has 258 entries: [e] for routed experts, [256] = pairs (start of the token-order rows
// used by the shared expert) and [257] = pairs + rows.
extern "C" __global__ void __launch_bounds__(256)
netra_moe_sort_scan_sm100(int32_t* __restrict__ seg_hist, int32_t* __restrict__ counts,
                          int32_t* __restrict__ offsets, uint32_t rows, uint32_t nseg) {
  __shared__ int warp_tot[8];
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  int total = 0;
  for (uint32_t s = 0; s < nseg; ++s) total += seg_hist[s * kRouted + e];
  counts[e] = total;
  int incl = total;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int o = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += o;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  int before = 0;
  for (int w = 0; w < warp; ++w) before += warp_tot[w];
  int running = before + incl - total;   // exclusive offset of expert e
  offsets[e] = running;
  if (e == kRouted - 1) {
    offsets[kRouted] = running + total;
    offsets[kRouted + 1] = running + total + (int)rows;
  }
  for (uint32_t s = 0; s < nseg; ++s) {
    int c = seg_hist[s * kRouted + e];
    seg_hist[s * kRouted + e] = running;
    running += c;
  }
}

// grid nseg, block 256 (8 warps x 128 consecutive pairs)
extern "C" __global__ void __launch_bounds__(256)
netra_moe_sort_scatter_sm100(int32_t* __restrict__ perm, int32_t* __restrict__ inv_perm,
                             const int32_t* __restrict__ seg_base, const int32_t* __restrict__ ids9,
                             uint32_t rows) {
  __shared__ int wbase[8][kRouted];
  const int pairs = (int)rows * kTopK;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wstart = blockIdx.x * kSortSegment + warp * 128;
  for (int e = lane; e < kRouted; e += 32) wbase[warp][e] = 0;
  __syncwarp();
  int my_e[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    int pair = wstart + c * 32 + lane;
    my_e[c] = pair < pairs ? pair_expert(ids9, pair) : -1;
    if (my_e[c] >= 0) atomicAdd(&wbase[warp][my_e[c]], 1);
  }
  __syncthreads();
  {  // exclusive scan over the 8 warps for expert e = threadIdx.x, plus the segment base
    const int e = threadIdx.x;
    int running = seg_base[blockIdx.x * kRouted + e];
#pragma unroll
    for (int w = 0; w < 8; ++w) { int c = wbase[w][e]; wbase[w][e] = running; running += c; }
  }
  __syncthreads();
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int pair = wstart + c * 32 + lane;
    const int e = my_e[c];
    const unsigned active = __ballot_sync(0xffffffffu, e >= 0);
    if (e >= 0) {
      const unsigned same = __match_any_sync(active, e);
      const int rank = __popc(same & ((1u << lane) - 1u));
      const int pos = wbase[warp][e] + rank;
      perm[pos] = pair;
      inv_perm[pair] = pos;
      __syncwarp(active);
      if (rank == 0) wbase[warp][e] += __popc(same);
    }
    __syncwarp();
  }
}

// Gather quantised hidden rows into expert-sorted order: row pos <- row (row_base + perm[pos]/8).
// One warp per row (2048 B codes + 64 B scales).  grid ceil(pairs/8), block 256.
extern "C" __global__ void __launch_bounds__(256)
netra_moe_gather_rows_sm100(uint8_t* __restrict__ a_fp8, float* __restrict__ a_scale,
                            const int32_t* __restrict__ perm, uint32_t rows) {
  const int pairs = (int)rows * kTopK;
  const int pos = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (pos >= pairs) return;
  const size_t src_row = (size_t)pairs + (perm[pos] >> 3);
  const uint4* src = reinterpret_cast<const uint4*>(a_fp8 + src_row * kHidden);
  uint4* dst = reinterpret_cast<uint4*>(a_fp8 + (size_t)pos * kHidden);
#pragma unroll
  for (int c = 0; c < 4; ++c) dst[c * 32 + lane] = src[c * 32 + lane];
  if (lane < kHiddenBlocks) a_scale[(size_t)pos * kHiddenBlocks + lane] = a_scale[src_row * kHiddenBlocks + lane];
}

// ------------------------------------------------------------------------------------------
// Combine: out[t,n] = bf16( sum_{s=0..8} w[t,s] * down[pos(t,s), n] ), slot ascending, FP32,
// one multiply and one add per slot.  pos(t,s) = inv_perm[t*8+s] for routed slots and
// pairs + t for the shared slot.  grid rows, block 256 (8 columns per thread).
// ------------------------------------------------------------------------------------------
extern "C" __global__ void __launch_bounds__(256)
netra_moe_combine_sm100(uint16_t* __restrict__ out, const float* __restrict__ down,
                        const float* __restrict__ w9, const int32_t* __restrict__ inv_perm, uint32_t rows) {
  const int t = blockIdx.x;
  const int pairs = (int)rows * kTopK;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
#pragma unroll 1
  for (int s = 0; s < kSlots; ++s) {
    const size_t pos = s < kTopK ? (size_t)inv_perm[t * kTopK + s] : (size_t)pairs + t;
    const float w = w9[t * kSlots + s];
    const float4* src = reinterpret_cast<const float4*>(down + pos * kHidden) + threadIdx.x * 2;
    float4 a = src[0], b = src[1];
    acc[0] = __fadd_rn(acc[0], __fmul_rn(a.x, w)); acc[1] = __fadd_rn(acc[1], __fmul_rn(a.y, w));
    acc[2] = __fadd_rn(acc[2], __fmul_rn(a.z, w)); acc[3] = __fadd_rn(acc[3], __fmul_rn(a.w, w));
    acc[4] = __fadd_rn(acc[4], __fmul_rn(b.x, w)); acc[5] = __fadd_rn(acc[5], __fmul_rn(b.y, w));
    acc[6] = __fadd_rn(acc[6], __fmul_rn(b.z, w)); acc[7] = __fadd_rn(acc[7], __fmul_rn(b.w, w));
  }
  uint32_t pk[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    pk[i] = *reinterpret_cast<uint32_t*>(&v);
  }
  reinterpret_cast<uint4*>(out + (size_t)t * kHidden)[threadIdx.x] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
}

}  // namespace netra

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
// Router logits.  logits[t,e] = RNE_bf16(exact dot(hidden[t,:], w[e,:])).  BF16 values convert to
// FP64 exactly, their products are exact in FP64, and a 2048-term FP64 sum lies within 2^-42 of
// the exact value relative to the sum of magnitudes - far below half a BF16 ulp - so the single
// FP64->BF16 rounding gives the correctly rounded dot product whatever the summation order.
// The sums run on the FP64 tensor cores (mma.sync m8n8k4): a warp owns 16 tokens x 16 experts
// over one quarter of K; the four K-quarters are added in fixed order through shared memory.
// grid (ceil(rows/16), 8); see the two entry points below.
// ------------------------------------------------------------------------------------------
// exact BF16 -> FP64 with integer ops (the FP64 pipe is kept for the MMAs)
__device__ __forceinline__ double bf16_bits_to_f64(uint32_t b) {
  const uint32_t e = b & 0x7f80u;
  if (e != 0u && e != 0x7f80u)
    return __hiloint2double((int)(((b & 0x8000u) << 16) | (((b & 0x7fffu) << 13) + 0x38000000u)), 0);
  return (double)bf16_bits_to_f32(b);   // zero, subnormal, inf, nan
}

// The same conversion without a branch (zero, subnormal, infinity and NaN included), for code that is unrolled
// many times: a BF16 subnormal m * 2^-133 is normalised by hand, infinity and NaN keep their payload.
__device__ __forceinline__ double bf16_bits_to_f64_nobranch(uint32_t b) {
  const uint32_t e = b & 0x7f80u, m = b & 0x7fu;
  const int p = 31 - __clz((int)(m | 1u));                                        // position of the leading one (0 when m == 0)
  const uint32_t hi_sub = m != 0u ? (((890u + (uint32_t)p) << 20) | ((m << (20 - p)) & 0xfffffu)) : 0u;
  const uint32_t hi_norm = ((b & 0x7fffu) << 13) + 0x38000000u;
  const uint32_t hi = e == 0u ? hi_sub : (e == 0x7f80u ? (0x7ff00000u | (m << 13)) : hi_norm);
  return __hiloint2double((int)(((b & 0x8000u) << 16) | hi), 0);
}

__device__ __forceinline__ void dmma_m8n8k4(double& c0, double& c1, double a, double b) {
  asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
               : "+d"(c0), "+d"(c1) : "d"(a), "d"(b));
}

// kKSplit warps share one 16 x 16 output tile, each over 1 / kKSplit of K; block = 2 expert halves x kKSplit warps.
// part_mem: kKSplit * 4 KiB of shared memory for the K-slices' partial tiles.
template <int kKSplit>
__device__ __forceinline__ void router_logits_body(uint16_t* __restrict__ logits, const uint16_t* __restrict__ hidden,
                                                   const uint16_t* __restrict__ weight, uint32_t rows, double* part_mem) {
  double (*part)[2][16][16] = reinterpret_cast<double (*)[2][16][16]>(part_mem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kq = warp % kKSplit, eh = warp / kKSplit;   // K-slice, expert half
  const int tok0 = blockIdx.x * 16;
  const int exp0 = blockIdx.y * 32 + eh * 16;
  const int frow = lane >> 2, fk = lane & 3;         // fragment row (token or expert), K position
  double acc[2][2][2];                               // [token tile][expert tile][2 columns]
#pragma unroll
  for (int i = 0; i < 8; ++i) (&acc[0][0][0])[i] = 0.0;
  // Any permutation of K is valid as long as both operands use it: in MMA step j of a 32-wide
  // chunk, fragment position fk holds element k = chunk + 8*fk + j, so a lane needs 8 consecutive
  // BF16 (one 16-byte load) per row and chunk.
  const int kbase = kq * (kHidden / kKSplit);
  const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll 2
  for (int kc = 0; kc < kHidden / kKSplit; kc += 32) {
    const int k = kbase + kc + 8 * fk;
    uint4 hv[2], wv[2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      const int t = tok0 + m * 8 + frow;
      hv[m] = t < (int)rows ? __ldg(reinterpret_cast<const uint4*>(hidden + (size_t)t * kHidden + k)) : zero;
      wv[m] = __ldg(reinterpret_cast<const uint4*>(weight + (size_t)(exp0 + m * 8 + frow) * kHidden + k));
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      double a[2], b[2];
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        const uint32_t hw = (&hv[m].x)[j >> 1], ww = (&wv[m].x)[j >> 1];
        a[m] = bf16_bits_to_f64((j & 1) ? (hw >> 16) : (hw & 0xffffu));
        b[m] = bf16_bits_to_f64((j & 1) ? (ww >> 16) : (ww & 0xffffu));
      }
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int n = 0; n < 2; ++n) dmma_m8n8k4(acc[m][n][0], acc[m][n][1], a[m], b[n]);
    }
  }
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      part[kq][eh][m * 8 + frow][n * 8 + fk * 2] = acc[m][n][0];
      part[kq][eh][m * 8 + frow][n * 8 + fk * 2 + 1] = acc[m][n][1];
    }
  __syncthreads();
  // 16 tokens x 32 experts: a thread finishes two adjacent experts of one token, adding the K-slices in order
  if (threadIdx.x < 256) {
    const int t = threadIdx.x >> 4, e2 = (threadIdx.x & 15) * 2;
    if (tok0 + t < (int)rows) {
      uint32_t packed = 0;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int e = e2 + i;
        double v = part[0][e >> 4][t][e & 15];
#pragma unroll
        for (int q = 1; q < kKSplit; ++q) v += part[q][e >> 4][t][e & 15];
        packed |= (uint32_t)f64_to_bf16_bits(v) << (16 * i);
      }
      *reinterpret_cast<uint32_t*>(logits + (size_t)(tok0 + t) * kRouted + blockIdx.y * 32 + e2) = packed;
    }
  }
}

// grid (ceil(rows/16), 8), block 256: four K-quarters per output tile.
extern "C" __global__ void __launch_bounds__(256)
netra_router_logits_bf16_sm100(uint16_t* __restrict__ logits, const uint16_t* __restrict__ hidden,
                               const uint16_t* __restrict__ weight, uint32_t rows) {
  __shared__ double part[4 * 2 * 16 * 16];
  router_logits_body<4>(logits, hidden, weight, rows, part);
}

// The same with eight K-slices (block 512): twice the warps per SM for calls too small to fill the GPU
// with blocks (up to about 1,024 rows), where the FP64 pipe would otherwise wait on its own latency.
extern "C" __global__ void __launch_bounds__(512)
netra_router_logits_bf16_k8_sm100(uint16_t* __restrict__ logits, const uint16_t* __restrict__ hidden,
                                  const uint16_t* __restrict__ weight, uint32_t rows) {
  __shared__ double part[8 * 2 * 16 * 16];
  router_logits_body<8>(logits, hidden, weight, rows, part);
}

// One hidden row into registers, one warp per row: lane owns the 64 consecutive values [lane*64, +64).
__device__ __forceinline__ void load_hidden_row(float x[64], const uint16_t* __restrict__ hidden, int t, int lane) {
  const uint4* src = reinterpret_cast<const uint4*>(hidden + (size_t)t * kHidden) + lane * 8;
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
}

// Per-128 FP8 quantisation of a row held as above: two lanes share one group.
// The quantised row goes to row (row_base + t) of the activation buffer.
__device__ __forceinline__ void quantize_loaded_row(uint8_t* __restrict__ a_fp8, float* __restrict__ a_scale, const float x[64],
                                                    int t, uint32_t row_base, int lane) {
  float amax = amax_floor();
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
    for (int q = 0; q < 4; ++q)
      w[q] = f32x4_to_e4m3x4(x[c * 16 + q * 4] * inv, x[c * 16 + q * 4 + 1] * inv, x[c * 16 + q * 4 + 2] * inv,
                             x[c * 16 + q * 4 + 3] * inv);
    dst[c] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

__device__ __forceinline__ void quantize_hidden_row(uint8_t* __restrict__ a_fp8, float* __restrict__ a_scale,
                                                    const uint16_t* __restrict__ hidden, int t, uint32_t row_base, int lane) {
  float x[64];
  load_hidden_row(x, hidden, t, lane);
  quantize_loaded_row(a_fp8, a_scale, x, t, row_base, lane);
}

// ------------------------------------------------------------------------------------------
// Residual add + RMSNorm + per-128 FP8 quantisation of the normalised row, the fusion that feeds the layer
// (behaviour replaced: kernels/gfx950/templates/norm/verify/add_rmsnorm_group_quant_n5120.inc, ABI
// runtime/gfx950/group_quant/verify/group_quant_assembly_bridge.h:21-31, numerical id
// "residual_add_fp32_rms_bf16_round_then_fp8_rne_fixed"; here at this model's width 2048):
//   x = f32(input) + f32(residual)                       residual_out = bf16(x)
//   var = fl32( sum x^2 / 2048 )   (the sum of the exact squares in FP64: one rounding, any order)
//   y = bf16( (x * (1 / sqrt(var + eps))) * weight )       output_bf16 = y
//   per 128 columns: scale = max(amax |y|, 1e-10) * fl(1/448), code = e4m3_rne_sat(y * (1 / scale))
// The codes and scales go to row (row_base + t) of the buffers the grouped GEMMs read (scales row-major [rows, 16]).
// One warp per row: a lane owns 64 consecutive columns, two lanes one quantisation group.  grid ceil(rows/4), block 128.
// ------------------------------------------------------------------------------------------
extern "C" __global__ void __launch_bounds__(128)
netra_add_rmsnorm_group_quant_n2048_sm100(const uint16_t* __restrict__ input, const uint16_t* __restrict__ residual,
                                          const float* __restrict__ weight, uint16_t* __restrict__ output,
                                          uint16_t* __restrict__ residual_out, uint8_t* __restrict__ out_fp8,
                                          float* __restrict__ out_scale, uint32_t rows, uint32_t row_base, float epsilon) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= (int)rows) return;
  const uint4* in4 = reinterpret_cast<const uint4*>(input + (size_t)t * kHidden) + lane * 8;
  const uint4* res4 = reinterpret_cast<const uint4*>(residual + (size_t)t * kHidden) + lane * 8;
  uint4* resout4 = reinterpret_cast<uint4*>(residual_out + (size_t)t * kHidden) + lane * 8;
  float x[64];
  double sq = 0.0;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint4 a = in4[c], b = res4[c];
    const uint32_t ua[4] = {a.x, a.y, a.z, a.w}, ub[4] = {b.x, b.y, b.z, b.w};
    uint32_t pk[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float lo = __fadd_rn(bf16_bits_to_f32(ua[q] & 0xffffu), bf16_bits_to_f32(ub[q] & 0xffffu));
      const float hi = __fadd_rn(bf16_bits_to_f32(ua[q] >> 16), bf16_bits_to_f32(ub[q] >> 16));
      x[c * 8 + 2 * q] = lo;
      x[c * 8 + 2 * q + 1] = hi;
      sq = fma((double)lo, (double)lo, sq);
      sq = fma((double)hi, (double)hi, sq);
      const __nv_bfloat162 r = __floats2bfloat162_rn(lo, hi);
      pk[q] = *reinterpret_cast<const uint32_t*>(&r);
    }
    resout4[c] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, d);
  const float var = (float)(sq / (double)kHidden);
  const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, epsilon)));
  const float4* w4 = reinterpret_cast<const float4*>(weight) + lane * 16;
  uint4* out4 = reinterpret_cast<uint4*>(output + (size_t)t * kHidden) + lane * 8;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const float4 w0 = w4[2 * c], w1 = w4[2 * c + 1];
    const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    uint32_t pk[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float lo = bf16_round(__fmul_rn(__fmul_rn(x[c * 8 + 2 * q], inv), w[2 * q]));
      const float hi = bf16_round(__fmul_rn(__fmul_rn(x[c * 8 + 2 * q + 1], inv), w[2 * q + 1]));
      x[c * 8 + 2 * q] = lo;
      x[c * 8 + 2 * q + 1] = hi;
      pk[q] = (__float_as_uint(lo) >> 16) | (__float_as_uint(hi) & 0xffff0000u);
    }
    out4[c] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  }
  quantize_loaded_row(out_fp8, out_scale, x, t, row_base, lane);
}

// ------------------------------------------------------------------------------------------
// Softmax / top-8 / renormalise + shared slot + per-token FP8 quantisation.  One warp per token.
// Selection key is (z desc, expert id asc) with z = f32(logit) + bias; weights are
// softmax(z)[id] renormalised over the 8 selected entries in slot order.
// The quantised row goes to row (row_base + t) of the activation buffer.
// grid ceil(rows/4), block 128.
// ------------------------------------------------------------------------------------------
// Floats as unsigned keys whose integer order is the float order (-0 counts as +0, NaN sorts below everything).
__device__ __forceinline__ uint32_t order_key(float z) {
  const uint32_t u = __float_as_uint(z + 0.0f);
  if (z != z) return 1u;
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float order_key_value(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Selection for one token by one warp; lane holds z[i] = f32(logit) + bias of experts lane*8 + i.
// On return lane k < 8 holds slot k: expert id, softmax numerator exp(z - max z) and z of the k-th best
// under the key (z desc, id asc).  Each round is two warp-wide integer reductions (redux.sync): the largest
// remaining key, then the lowest expert id among the lanes that hold it.
__device__ __forceinline__ void softmax_top8_select(const float z[8], int lane, int& sel_id, float& sel_p, float& sel_z) {
  uint32_t key[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) key[i] = order_key(z[i]);
  uint32_t taken = 0, my_key = 0;
  sel_id = 0;
#pragma unroll 1
  for (int k = 0; k < kTopK; ++k) {
    uint32_t bk = 0; int bi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool better = !((taken >> i) & 1u) && key[i] > bk;    // strict: the lowest index of equal keys stays
      if (better) { bk = key[i]; bi = i; }
    }
    const uint32_t best = __reduce_max_sync(0xffffffffu, bk);
    const uint32_t winner = __reduce_min_sync(0xffffffffu, (bk == best && bk != 0u) ? (uint32_t)(lane * 8 + bi) : 0xffffffffu);
    if ((int)(winner >> 3) == lane) taken |= 1u << (winner & 7u);
    if (lane == k) { sel_id = (int)winner; my_key = best; }
  }
  // exp(z - zmax): the softmax numerators.  The softmax denominator cancels in the renormalisation over the eight
  // selected experts, so the weights depend on the selected logits only (slot 0 holds the largest z)
  const float zmax = order_key_value(__shfl_sync(0xffffffffu, my_key, 0));
  sel_z = order_key_value(my_key);
  sel_p = expf(sel_z - zmax);
}

// Renormalise over the eight selected probabilities (slot-order FP32 sum) and store ids / weights with the shared slot.
__device__ __forceinline__ void top8_store(int32_t* __restrict__ ids9, float* __restrict__ w9, int sel_id, float sel_p,
                                           const float* __restrict__ shared_w, int t, int lane) {
  float s = 0.0f;
#pragma unroll
  for (int k = 0; k < kTopK; ++k) s += __shfl_sync(0xffffffffu, sel_p, k);
  if (lane < kTopK) {
    ids9[t * kSlots + lane] = sel_id;
    w9[t * kSlots + lane] = sel_p / s;
  } else if (lane == kTopK) {
    ids9[t * kSlots + kTopK] = kRouted;
    w9[t * kSlots + kTopK] = shared_w != nullptr ? shared_w[t] : 1.0f;
  }
}

__device__ __forceinline__ void softmax_top8_store(int32_t* __restrict__ ids9, float* __restrict__ w9, const float z[8],
                                                   const float* __restrict__ shared_w, int t, int lane) {
  int sel_id; float sel_p, sel_z;
  softmax_top8_select(z, lane, sel_id, sel_p, sel_z);
  top8_store(ids9, w9, sel_id, sel_p, shared_w, t, lane);
}

// One token's softmax / top-8 / renormalise and FP8 quantisation by one warp.  kFromL2: the logits were written by other
// blocks of the same launch, so they are read around the L1.
template <bool kFromL2>
__device__ __forceinline__ void topk_quant_token(int32_t* __restrict__ ids9, float* __restrict__ w9,
                                                 uint8_t* __restrict__ a_fp8, float* __restrict__ a_scale,
                                                 const uint16_t* logits, const float* __restrict__ bias,
                                                 const float* __restrict__ shared_w, const uint16_t* __restrict__ hidden,
                                                 uint32_t row_base, int t, int lane) {
  // lane owns experts lane*8 .. lane*8+7 (ascending id inside the lane)
  float z[8];
  {
    const uint4* src = reinterpret_cast<const uint4*>(logits + (size_t)t * kRouted) + lane;
    uint4 v = kFromL2 ? __ldcg(src) : *src;
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
  softmax_top8_store(ids9, w9, z, shared_w, t, lane);
  if (a_fp8 != nullptr) quantize_hidden_row(a_fp8, a_scale, hidden, t, row_base, lane);   // null: the rows were quantised upstream
}

extern "C" __global__ void __launch_bounds__(128)
netra_moe_topk_quant_sm100(int32_t* __restrict__ ids9, float* __restrict__ w9,
                           uint8_t* __restrict__ a_fp8, float* __restrict__ a_scale,
                           const uint16_t* __restrict__ logits, const float* __restrict__ bias,
                           const float* __restrict__ shared_w, const uint16_t* __restrict__ hidden,
                           uint32_t rows, uint32_t row_base) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= (int)rows) return;
  topk_quant_token<false>(ids9, w9, a_fp8, a_scale, logits, bias, shared_w, hidden, row_base, t, lane);
}

// ------------------------------------------------------------------------------------------
// The same stage for calls whose logits come from the tensor-core router (router_umma.cu) as FP32
// approximations a[e].  The routing contract is the exact dot product rounded once to BF16.  The exact
// value lies within
//     bound[e] = kRouterErrScale * |hidden[t,:]|_2 * |w[e,:]|_2        (>= the approximation error)
// of a[e], so bf16(a[e]) is already the contract value unless a rounding boundary (the midpoint of two
// neighbouring BF16 values) lies inside that interval; such a logit is "undecided" and is recomputed in
// FP64 (exact products, accumulation error far below any BF16 spacing).  kRouterErrScale is an empirical
// bound of the tensor-core accumulation error relative to the product of the norms (which bounds the sum
// of the 2048 product magnitudes), eleven times the largest error seen over 7 million logits of the
// benchmark distributions; the GPU tests measure it again and compare every logit against the FP64 router.
//
// exact_all == 0 (default): only undecided logits that can reach the top 8 are recomputed.  Every
// contract logit differs from z = bf16(a) + bias by at most delta = max bound + two BF16 spacings of the
// largest logit, so the eight best approximate z prove that the true eighth-best z is at least
// v8 - delta, and an expert with z < v8 - 2 delta cannot be selected whatever its exact value.  The
// selected ids, their exact logits and therefore the routing weights are those of the contract; logits of
// experts out of reach keep bf16(a), within bound[e] plus one BF16 spacing of the contract value.
// exact_all != 0: every undecided logit is recomputed, and the logits array equals the contract everywhere.
// One warp per token.  stats[0] counts recomputed logits.  grid ceil(rows/4), block 128.
// ------------------------------------------------------------------------------------------
constexpr float kRouterErrScale = 3.8146973e-06f;   // 2^-18

// Exact dot product of one hidden row and one router row by one warp (every lane returns the sum): lane l owns the
// 16-byte chunks c*32 + l, so each of the sixteen loads is a fully coalesced 512-byte request and all are in flight
// together.  Fast path: the product of two BF16 values is exact in FP32 unless it leaves the normal range; the exact
// FP32 products are widened with integer operations and summed in FP64 (error far below any BF16 spacing).  A product
// that underflows or overflows FP32 sends the whole dot product to the slow path, which widens the operands first.
__device__ __noinline__ double exact_dot_slow(const uint4* __restrict__ hrow, const uint4* __restrict__ wrow, int lane) {
  double acc = 0.0;
  for (int c = 0; c < 8; ++c) {
    const uint4 hv = __ldg(hrow + c * 32 + lane), wv = __ldg(wrow + c * 32 + lane);
    const uint32_t x[4] = {hv.x, hv.y, hv.z, hv.w}, u[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      acc = fma(bf16_bits_to_f64_nobranch(x[q] & 0xffffu), bf16_bits_to_f64_nobranch(u[q] & 0xffffu), acc);
      acc = fma(bf16_bits_to_f64_nobranch(x[q] >> 16), bf16_bits_to_f64_nobranch(u[q] >> 16), acc);
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  return acc;
}

__device__ __forceinline__ double exact_dot(const uint4* __restrict__ hrow, const uint4* __restrict__ wrow, int lane) {
  uint4 hv[8], wv[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) { hv[c] = __ldg(hrow + c * 32 + lane); wv[c] = __ldg(wrow + c * 32 + lane); }
  double acc0 = 0.0, acc1 = 0.0;
  uint32_t bad = 0;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint32_t x[4] = {hv[c].x, hv[c].y, hv[c].z, hv[c].w}, u[4] = {wv[c].x, wv[c].y, wv[c].z, wv[c].w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint32_t xa = half ? (x[q] & 0xffff0000u) : (x[q] << 16), ub = half ? (u[q] & 0xffff0000u) : (u[q] << 16);
        const uint32_t pb = __float_as_uint(__fmul_rn(__uint_as_float(xa), __uint_as_float(ub)));
        const uint32_t pe = pb & 0x7f800000u;
        // exact unless the result left the normal range: zero with both factors nonzero (or subnormal), infinity, NaN
        bad |= (pe == 0x7f800000u) | ((pe == 0u) & ((xa << 1) != 0u) & ((ub << 1) != 0u));
        const uint32_t hi = pe != 0u ? ((pb & 0x80000000u) | (((pb & 0x7fffffffu) >> 3) + 0x38000000u)) : 0u;
        const double pd = __hiloint2double((int)hi, (int)(pe != 0u ? pb << 29 : 0u));
        if (half) acc1 += pd; else acc0 += pd;
      }
    }
  }
  if (__any_sync(0xffffffffu, bad != 0u)) return exact_dot_slow(hrow, wrow, lane);
  double acc = acc0 + acc1;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  return acc;
}

extern "C" __global__ void __launch_bounds__(128)
netra_moe_topk_quant_fix_sm100(int32_t* __restrict__ ids9, float* __restrict__ w9,
                               uint8_t* __restrict__ a_fp8, float* __restrict__ a_scale,
                               uint16_t* __restrict__ logits, const float* __restrict__ logits_f32,
                               const float* __restrict__ wnorm, const uint16_t* __restrict__ router_w,
                               const float* __restrict__ bias, const float* __restrict__ shared_w,
                               const uint16_t* __restrict__ hidden, uint32_t* __restrict__ stats,
                               uint32_t rows, uint32_t row_base, uint32_t exact_all) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= (int)rows) return;
  // The row is read three times instead of being held in registers (it would cost a third of the occupancy): here for
  // its norm (from DRAM), in the rare FP64 recomputation and for the quantisation at the end (from the caches).
  const uint4* hrow = reinterpret_cast<const uint4*>(hidden + (size_t)t * kHidden) + lane * 8;
  float hn = 0.0f;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint4 hv = __ldg(hrow + c);
    const uint32_t u[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float a = bf16_bits_to_f32(u[q] & 0xffffu), b = bf16_bits_to_f32(u[q] >> 16);
      hn = fmaf(a, a, hn);
      hn = fmaf(b, b, hn);
    }
  }
  hn = sqrtf(warp_sum(hn)) * 1.001f;
  float v[8], bs[8];      // contract candidates bf16(a) and the bias
  uint32_t pending = 0;
  float bmax = 0.0f, vmax = 0.0f;
  {
    const float4 a0 = reinterpret_cast<const float4*>(logits_f32 + (size_t)t * kRouted)[lane * 2];
    const float4 a1 = reinterpret_cast<const float4*>(logits_f32 + (size_t)t * kRouted)[lane * 2 + 1];
    const float4 n0 = reinterpret_cast<const float4*>(wnorm)[lane * 2];
    const float4 n1 = reinterpret_cast<const float4*>(wnorm)[lane * 2 + 1];
    const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const float n[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t bits = __float_as_uint(a[i]);
      const float ulp = __uint_as_float(bits & 0x7f800000u) * 1.1920929e-07f;        // spacing of FP32 at a[i]; 0 below the normals
      const float dist = fabsf((float)((int)(bits & 0xffffu) - 0x8000)) * ulp;         // to the rounding boundary of a[i]'s BF16 cell
      const float bound = kRouterErrScale * hn * n[i];
      // decided only when the boundary of this cell is out of reach AND the neighbouring cells' boundaries are
      // (they are at least a quarter of a BF16 spacing = 2^13 FP32 spacings away); NaN and infinity fail both tests
      const bool decided = dist > bound && bound < 8192.0f * ulp;
      if (!decided) pending |= 1u << i;
      v[i] = bf16_round(a[i]);
      bs[i] = bias != nullptr ? bias[lane * 8 + i] : 0.0f;
      bmax = fmaxf(bmax, bound);
      vmax = fmaxf(vmax, fabsf(v[i]));
    }
  }
  float z[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) z[i] = v[i] + bs[i];
  int sel_id; float sel_p, sel_z;
  bool selected = false;
  if (exact_all == 0u) {
    softmax_top8_select(z, lane, sel_id, sel_p, sel_z);
    selected = true;
    const float v8 = __shfl_sync(0xffffffffu, sel_z, kTopK - 1);
    // two BF16 spacings at the largest magnitude of the row cover the two roundings (of a and of the exact value, which
    // may sit one binade higher); 1.01 covers the FP32 roundings of this arithmetic and of the bias addition
    const float delta = (__uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(bmax))) +
                         __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(vmax))) * 0.015625f) * 1.01f;   // both are >= 0
    const float reach = v8 - 2.0f * delta;
    uint32_t cand = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (z[i] >= reach) cand |= 1u << i;
    pending &= cand;
  }
  uint32_t fixed = 0;
  for (;;) {
    const uint32_t any = __ballot_sync(0xffffffffu, pending != 0);
    if (any == 0) break;
    const int src = __ffs(any) - 1;
    const int i = __ffs(__shfl_sync(0xffffffffu, pending, src)) - 1;
    const double acc = exact_dot(reinterpret_cast<const uint4*>(hidden + (size_t)t * kHidden),
                                 reinterpret_cast<const uint4*>(router_w + (size_t)(src * 8 + i) * kHidden), lane);
    const float exact = bf16_bits_to_f32(f64_to_bf16_bits(acc));
    if (lane == src) {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k == i) { v[k] = exact; z[k] = exact + bs[k]; }
      pending &= ~(1u << i);
    }
    ++fixed;
  }
  if (stats != nullptr && lane == 0 && fixed != 0) atomicAdd(stats, fixed);
  {
    uint32_t pk[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) pk[q] = (__float_as_uint(v[2 * q]) >> 16) | (__float_as_uint(v[2 * q + 1]) & 0xffff0000u);
    reinterpret_cast<uint4*>(logits + (size_t)t * kRouted)[lane] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  }
  if (!selected || fixed != 0) softmax_top8_select(z, lane, sel_id, sel_p, sel_z);   // `fixed` is the same in every lane
  top8_store(ids9, w9, sel_id, sel_p, shared_w, t, lane);
  if (a_fp8 != nullptr) quantize_hidden_row(a_fp8, a_scale, hidden, t, row_base, lane);   // null: the rows were quantised upstream
}

// The same outputs from a top-k computed elsewhere (a serving stack that keeps its own fused top-k, the
// position of scripts/rocm/integrations/sglang/sglang-gfx1151-bf16-router.patch:64): copies ids [rows, 8] and
// weights [rows, 8] into the nine-slot arrays (slot 8 = shared expert), and quantises the hidden rows.
// Ids outside 0..255 are clamped so that no later stage can index out of range.  grid ceil(rows/4), block 128.
extern "C" __global__ void __launch_bounds__(128)
netra_moe_import_topk_quant_sm100(int32_t* __restrict__ ids9, float* __restrict__ w9, uint8_t* __restrict__ a_fp8,
                                  float* __restrict__ a_scale, const int32_t* __restrict__ ext_ids,
                                  const float* __restrict__ ext_w, const float* __restrict__ shared_w,
                                  const uint16_t* __restrict__ hidden, uint32_t rows, uint32_t row_base) {
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (t >= (int)rows) return;
  if (lane < kTopK) {
    ids9[t * kSlots + lane] = min(max(ext_ids[t * kTopK + lane], 0), kRouted - 1);
    w9[t * kSlots + lane] = ext_w[t * kTopK + lane];
  } else if (lane == kTopK) {
    ids9[t * kSlots + kTopK] = kRouted;
    w9[t * kSlots + kTopK] = shared_w != nullptr ? shared_w[t] : 1.0f;
  }
  quantize_hidden_row(a_fp8, a_scale, hidden, t, row_base, lane);
}

// ------------------------------------------------------------------------------------------
// Stable expert-major sort of the rows*8 routed pairs (pair index = t*8 + slot).
// Three launches for any size: per-segment histograms, a scan over segments, and a stable
// scatter; a segment is 1024 consecutive pairs.  No atomics decide an output position.
// ------------------------------------------------------------------------------------------
// Ids are clamped to 0..255: the sort kernels index shared-memory tables with them, and one entry point
// (netra_moe_sort_static_scratch_launch) takes ids produced by the caller.
__device__ __forceinline__ int pair_expert(const int32_t* ids9, int pair) {
  return min(max(ids9[(pair >> 3) * kSlots + (pair & 7)], 0), kRouted - 1);
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

// Whole sort in one block for up to 8192 pairs (rows <= 1024): each of the 32 warps owns a run of consecutive
// pairs (a multiple of 32, as short as the pair count allows so that all warps work: 64 at 256 rows, 256 at
// 1,024 rows).  Same result as the three-launch path; no global scratch.  grid 1, block 1024.
constexpr int kSortSmallMaxRows = 1024;

// kWarps warps of one block; wbase: [kWarps][256] ints and warp_tot: [8] ints of shared memory.  kFromL2: the ids were
// written by other blocks of the same launch.
template <int kWarps, bool kFromL2>
__device__ __forceinline__ void sort_small_body(int32_t* __restrict__ perm, int32_t* __restrict__ inv_perm, int32_t* __restrict__ counts,
                                                int32_t* __restrict__ offsets, const int32_t* ids9, uint32_t rows,
                                                int (*wbase)[kRouted], int* warp_tot) {
  constexpr int kThreads = kWarps * 32;
  constexpr int kMaxRounds = kSortSmallMaxRows * kTopK / kThreads;     // 32-pair rounds per warp at the largest call: 8 | 16
  const int pairs = (int)rows * kTopK;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kWarps * kRouted; i += kThreads) (&wbase[0][0])[i] = 0;
  __syncthreads();
  const int rounds = max(1, (pairs + kThreads - 1) / kThreads);
  const int wstart = warp * rounds * 32;
  int my_e[kMaxRounds];
#pragma unroll
  for (int c = 0; c < kMaxRounds; ++c) {
    const int pair = wstart + c * 32 + lane;
    int e = -1;
    if (c < rounds && pair < pairs) {
      const int32_t* src = ids9 + (pair >> 3) * kSlots + (pair & 7);
      e = min(max(kFromL2 ? __ldcg(src) : *src, 0), kRouted - 1);
    }
    my_e[c] = e;
    if (e >= 0) atomicAdd(&wbase[warp][e], 1);   // counts only: order independent
  }
  __syncthreads();
  if (threadIdx.x < kRouted) {
    const int e = threadIdx.x;
    int total = 0;
#pragma unroll 8
    for (int w = 0; w < kWarps; ++w) total += wbase[w][e];
    counts[e] = total;
    int incl = total;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += o;
    }
    if (lane == 31) warp_tot[warp] = incl;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    int running = before + incl - total;
    offsets[e] = running;
    if (e == kRouted - 1) {
      offsets[kRouted] = running + total;
      offsets[kRouted + 1] = running + total + (int)rows;
    }
#pragma unroll 8
    for (int w = 0; w < kWarps; ++w) { int c = wbase[w][e]; wbase[w][e] = running; running += c; }
  }
  __syncthreads();
#pragma unroll
  for (int c = 0; c < kMaxRounds; ++c) {
    if (c >= rounds) break;                                // uniform across the block
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

extern "C" __global__ void __launch_bounds__(1024)
netra_moe_sort_small_sm100(int32_t* __restrict__ perm, int32_t* __restrict__ inv_perm, int32_t* __restrict__ counts,
                           int32_t* __restrict__ offsets, const int32_t* __restrict__ ids9, uint32_t rows) {
  __shared__ int wbase[32][kRouted];
  __shared__ int warp_tot[8];
  sort_small_body<32, false>(perm, inv_perm, counts, offsets, ids9, rows, wbase, warp_tot);
}

// ------------------------------------------------------------------------------------------
// The routing front end of a call of up to 1,024 tokens in one launch: router logits, softmax / top-8 / renormalise +
// FP8 quantisation, expert sort - the three kernels above, handed from block to block by last-arriver counters (no block
// ever waits for another one):
//   every block          its 16 tokens x 32 experts of exactly rounded logits (FP64 tensor cores), then one arrival on
//                        its token tile's counter;
//   the eighth arrival   of a tile runs the top-8 + quantisation of the tile's 16 tokens, a warp per token, while other
//                        tiles' router blocks are still at work; then one arrival on the launch's counter;
//   the last tile        to finish sorts the call's pairs by expert (the single-block sort with sixteen warps) and
//                        returns the counters to zero for the next launch.
// counters: [1 + ceil(rows/16)] zeroed words, word 0 for the launch.  grid (ceil(rows/16), 8), block 512.
// ------------------------------------------------------------------------------------------
extern "C" __global__ void __launch_bounds__(512)
netra_moe_route_front_sm100(uint16_t* __restrict__ logits, const uint16_t* __restrict__ hidden, const uint16_t* __restrict__ weight,
                            int32_t* __restrict__ ids9, float* __restrict__ w9, uint8_t* __restrict__ a_fp8, float* __restrict__ a_scale,
                            const float* __restrict__ bias, const float* __restrict__ shared_w, int32_t* __restrict__ perm,
                            int32_t* __restrict__ inv_perm, int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                            uint32_t* __restrict__ counters, uint32_t rows, uint32_t row_base) {
  __shared__ __align__(16) double scratch[8 * 2 * 16 * 16];      // 32 KiB: the router's partial tiles, later the sort's tables
  __shared__ int warp_tot[8];
  __shared__ uint32_t arrived;
  router_logits_body<8>(logits, hidden, weight, rows, scratch);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) arrived = atomicAdd(&counters[1 + blockIdx.x], 1u);
  __syncthreads();
  if (arrived != gridDim.y - 1) return;
  __threadfence();
  {
    const int t = blockIdx.x * 16 + (threadIdx.x >> 5);
    if (t < (int)rows)
      topk_quant_token<true>(ids9, w9, a_fp8, a_scale, logits, bias, shared_w, hidden, row_base, t, threadIdx.x & 31);
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) arrived = atomicAdd(&counters[0], 1u);
  __syncthreads();
  if (arrived != gridDim.x - 1) return;
  __threadfence();
  sort_small_body<16, true>(perm, inv_perm, counts, offsets, ids9, rows, reinterpret_cast<int (*)[kRouted]>(scratch), warp_tot);
  for (uint32_t i = threadIdx.x; i <= gridDim.x; i += blockDim.x) counters[i] = 0;
}

// Gather quantised hidden rows into expert-sorted order: row pos <- row (row_base + perm[pos]/8).
// One warp per row (2048 B codes + 64 B scales).  grid ceil(pairs/8), block 256.
extern "C" __global__ void __launch_bounds__(256)
netra_moe_gather_rows_sm100(uint8_t* __restrict__ a_fp8, float* __restrict__ a_scale,
                            const int32_t* __restrict__ perm, uint32_t rows, uint32_t* __restrict__ ready, uint32_t ready_words) {
  // ready (may be null): the per-unit arrival counters of the launch that follows (both projections in one kernel) start at zero
  if (blockIdx.x == 0 && ready != nullptr)
    for (uint32_t i = threadIdx.x; i < ready_words; i += blockDim.x) ready[i] = 0;
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
// kFromL2: the rows were written by other GPUs while this kernel was already running, so they are read around the L1.
template <bool kFromL2>
__device__ __forceinline__ void combine_rows_body(uint16_t* __restrict__ out, const float* down, const float* __restrict__ w9,
                                                  const int32_t* __restrict__ inv_perm, uint32_t rows) {
  const int t = blockIdx.x;
  const int pairs = (int)rows * kTopK;
  // all nine rows are requested before the first is used; the sum itself stays slot-ascending
  float4 a[kSlots], b[kSlots];
  float w[kSlots];
#pragma unroll
  for (int s = 0; s < kSlots; ++s) {
    const size_t pos = s < kTopK ? (size_t)inv_perm[t * kTopK + s] : (size_t)pairs + t;
    w[s] = w9[t * kSlots + s];
    const float4* src = reinterpret_cast<const float4*>(down + pos * kHidden) + threadIdx.x * 2;
    a[s] = kFromL2 ? __ldcg(src) : src[0];
    b[s] = kFromL2 ? __ldcg(src + 1) : src[1];
  }
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
#pragma unroll
  for (int s = 0; s < kSlots; ++s) {
    acc[0] = __fadd_rn(acc[0], __fmul_rn(a[s].x, w[s])); acc[1] = __fadd_rn(acc[1], __fmul_rn(a[s].y, w[s]));
    acc[2] = __fadd_rn(acc[2], __fmul_rn(a[s].z, w[s])); acc[3] = __fadd_rn(acc[3], __fmul_rn(a[s].w, w[s]));
    acc[4] = __fadd_rn(acc[4], __fmul_rn(b[s].x, w[s])); acc[5] = __fadd_rn(acc[5], __fmul_rn(b[s].y, w[s]));
    acc[6] = __fadd_rn(acc[6], __fmul_rn(b[s].z, w[s])); acc[7] = __fadd_rn(acc[7], __fmul_rn(b[s].w, w[s]));
  }
  uint32_t pk[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    pk[i] = *reinterpret_cast<uint32_t*>(&v);
  }
  reinterpret_cast<uint4*>(out + (size_t)t * kHidden)[threadIdx.x] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
}

extern "C" __global__ void __launch_bounds__(256)
netra_moe_combine_sm100(uint16_t* __restrict__ out, const float* __restrict__ down,
                        const float* __restrict__ w9, const int32_t* __restrict__ inv_perm, uint32_t rows) {
  combine_rows_body<false>(out, down, w9, inv_perm, rows);
}

// The same combine over FP16 partial rows (written by netra_moe_down_tokmajor_f16_sm100 as sixteen column panels
// [rows * 9][128 halves] with the 16-byte chunks of a row permuted by the row index): each partial is widened to
// FP32, multiplied by its routing weight and added in slot order, one BF16 rounding at the end - the order of
// kernels/gfx950/templates/moe/prefill/route_reduce_splitk2_f16.inc:107-118.  grid rows, block 256 (8 columns per thread).
// kFromL2: the rows were written by other GPUs into this one's memory and are read around the L1.
template <bool kFromL2>
__device__ __forceinline__ void combine_f16_rows_body(uint16_t* __restrict__ out, const __half* down,
                                                      const float* __restrict__ w9, const int32_t* __restrict__ inv_perm, uint32_t rows) {
  const int t = blockIdx.x;
  const int pairs = (int)rows * kTopK;
  const size_t total = (size_t)pairs + rows;      // rows of every column panel
  uint4 v[kSlots];
  float w[kSlots];
#pragma unroll
  for (int s = 0; s < kSlots; ++s) {
    const size_t pos = s < kTopK ? (size_t)inv_perm[t * kTopK + s] : (size_t)pairs + t;
    w[s] = w9[t * kSlots + s];
    // panel threadIdx.x / 16 (128 columns), chunk threadIdx.x % 16 of the row, stored at chunk ^ (row & 15)
    const size_t chunk = ((size_t)(threadIdx.x >> 4) * total + pos) * 16 + ((threadIdx.x & 15u) ^ ((uint32_t)pos & 15u));
    const uint4* src = reinterpret_cast<const uint4*>(down) + chunk;
    v[s] = kFromL2 ? __ldcg(src) : *src;
  }
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
#pragma unroll
  for (int s = 0; s < kSlots; ++s) {
    const uint32_t u[4] = {v[s].x, v[s].y, v[s].z, v[s].w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[q]));
      acc[2 * q] = __fadd_rn(acc[2 * q], __fmul_rn(f.x, w[s]));
      acc[2 * q + 1] = __fadd_rn(acc[2 * q + 1], __fmul_rn(f.y, w[s]));
    }
  }
  uint32_t pk[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    pk[i] = *reinterpret_cast<uint32_t*>(&b);
  }
  reinterpret_cast<uint4*>(out + (size_t)t * kHidden)[threadIdx.x] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
}

extern "C" __global__ void __launch_bounds__(256)
netra_moe_combine_f16_sm100(uint16_t* __restrict__ out, const __half* __restrict__ down,
                            const float* __restrict__ w9, const int32_t* __restrict__ inv_perm, uint32_t rows) {
  combine_f16_rows_body<false>(out, down, w9, inv_perm, rows);
}

}  // namespace netra

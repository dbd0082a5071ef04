// Slot-order decode kernels with the argument contract of the reference's per-kernel bridges
// (runtime/gfx950/fp8/moe/qwen36_moe_silu_mul_quant_bridge.h:14-64): gate_up into FP32
// [rows*9, 1024], SiLU*up + per-128 FP8 requantisation, down projection with the slot-ordered
// weighted reduce.  They run on CUDA cores, take any row count, and serve two purposes: drop-in
// entry points for callers that keep the reference's three-launch boundary, and an independent
// GPU-side cross-check of the tensor-core grouped kernels.
#include "common.cuh"

namespace netra {

// grid (16, rows*9), block 256: a warp owns 8 of the block's 64 output columns.
// Lane l covers K-block l/2, half l%2 (64 bytes): per K-block partial -> (part*a_s)*w_s -> xor tree.
extern "C" __global__ void __launch_bounds__(256)
netra_qwen36_moe_gate_up_fp8_sm100(const uint8_t* __restrict__ hidden_fp8, const float* __restrict__ hidden_scale,
                                   const uint8_t* __restrict__ w13, const float* __restrict__ w13_scale,
                                   const int32_t* __restrict__ topk_ids, float* __restrict__ out, uint32_t rows) {
  const int route = blockIdx.y;
  if (route >= (int)rows * kSlots) return;
  const int t = route / kSlots;
  const int e = topk_ids[route];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb = lane >> 1, koff = kb * kBlock + (lane & 1) * 64;
  float a[64];
  {
    const uint4* src = reinterpret_cast<const uint4*>(hidden_fp8 + (size_t)t * kHidden + koff);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 v = src[c];
      e4m3x4_to_f32(v.x, a + c * 16); e4m3x4_to_f32(v.y, a + c * 16 + 4);
      e4m3x4_to_f32(v.z, a + c * 16 + 8); e4m3x4_to_f32(v.w, a + c * 16 + 12);
    }
  }
  const float a_s = hidden_scale[t * kHiddenBlocks + kb];
  const int n0 = blockIdx.x * 64 + warp * 8;
#pragma unroll 1
  for (int j = 0; j < 8; ++j) {
    const int n = n0 + j;
    const uint4* wsrc = reinterpret_cast<const uint4*>(w13 + ((size_t)e * 2 * kInter + n) * kHidden + koff);
    float part = 0.0f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint4 v = __ldg(wsrc + c);
      float w[16];
      e4m3x4_to_f32(v.x, w); e4m3x4_to_f32(v.y, w + 4); e4m3x4_to_f32(v.z, w + 8); e4m3x4_to_f32(v.w, w + 12);
#pragma unroll
      for (int i = 0; i < 16; ++i) part = fmaf(a[c * 16 + i], w[i], part);
    }
    part += __shfl_xor_sync(0xffffffffu, part, 1);
    const float w_s = w13_scale[((size_t)e * (2 * kInter / kBlock) + n / kBlock) * kHiddenBlocks + kb];
    float v = __fmul_rn(__fmul_rn(part, a_s), w_s);
#pragma unroll
    for (int d = 2; d < 32; d <<= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    if (lane == 0) out[(size_t)route * 2 * kInter + n] = v;
  }
}

// grid rows, block 64: a lane owns 8 contiguous values, a 16-lane subgroup one 128-value group.
extern "C" __global__ void __launch_bounds__(64)
netra_qwen36_moe_silu_mul_quant_fp8_sm100(const float* __restrict__ in, uint8_t* __restrict__ out_fp8,
                                          float* __restrict__ out_scale, uint32_t rows) {
  const int row = blockIdx.x;
  if (row >= (int)rows) return;
  const int lane = threadIdx.x;
  const float* gate = in + (size_t)row * 2 * kInter + lane * 8;
  const float* up = gate + kInter;
  float h[8];
  float amax = amax_floor();
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float g = gate[i];
    const float sig = 1.0f / (1.0f + expf(-g));
    h[i] = bf16_round(__fmul_rn(__fmul_rn(g, sig), up[i]));
    amax = fmaxf(amax, fabsf(h[i]));
  }
#pragma unroll
  for (int d = 8; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d, 16));
  const float scale = amax * inv448();
  const float inv = 1.0f / scale;
  if ((lane & 15) == 0) out_scale[(size_t)row * kInterBlocks + (lane >> 4)] = scale;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lo |= (uint32_t)f32_to_e4m3(h[i] * inv) << (8 * i);
    hi |= (uint32_t)f32_to_e4m3(h[4 + i] * inv) << (8 * i);
  }
  reinterpret_cast<uint2*>(out_fp8 + (size_t)row * kInter)[lane] = make_uint2(lo, hi);
}

// grid (32, rows), block 256: a warp owns 8 output columns; lane l covers 16 bytes of K
// (K-block l/8).  Per slot: K-blocks ascending, then acc += slot_out * w[slot], slots ascending.
extern "C" __global__ void __launch_bounds__(256)
netra_qwen36_moe_down_reduce_fp8_sm100(const uint8_t* __restrict__ act_fp8, const float* __restrict__ act_scale,
                                       const uint8_t* __restrict__ w2, const float* __restrict__ w2_scale,
                                       const float* __restrict__ topk_w, const int32_t* __restrict__ topk_ids,
                                       uint16_t* __restrict__ out, uint32_t rows) {
  const int t = blockIdx.y;
  if (t >= (int)rows) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb = lane >> 3;
  const int n0 = blockIdx.x * 64 + warp * 8;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll 1
  for (int s = 0; s < kSlots; ++s) {
    const int route = t * kSlots + s;
    const int e = topk_ids[route];
    const float w = topk_w[route];
    float a[16];
    {
      uint4 v = reinterpret_cast<const uint4*>(act_fp8 + (size_t)route * kInter)[lane];
      e4m3x4_to_f32(v.x, a); e4m3x4_to_f32(v.y, a + 4); e4m3x4_to_f32(v.z, a + 8); e4m3x4_to_f32(v.w, a + 12);
    }
    const float a_s = act_scale[route * kInterBlocks + kb];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int n = n0 + j;
      uint4 v = __ldg(reinterpret_cast<const uint4*>(w2 + ((size_t)e * kHidden + n) * kInter) + lane);
      float wv[16];
      e4m3x4_to_f32(v.x, wv); e4m3x4_to_f32(v.y, wv + 4); e4m3x4_to_f32(v.z, wv + 8); e4m3x4_to_f32(v.w, wv + 12);
      float part = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; ++i) part = fmaf(a[i], wv[i], part);
#pragma unroll
      for (int d = 1; d < 8; d <<= 1) part += __shfl_xor_sync(0xffffffffu, part, d);
      const float w_s = w2_scale[((size_t)e * (kHidden / kBlock) + n / kBlock) * kInterBlocks + kb];
      const float scaled = __fmul_rn(__fmul_rn(part, a_s), w_s);
      float slot = __shfl_sync(0xffffffffu, scaled, 0);
      slot = __fadd_rn(slot, __shfl_sync(0xffffffffu, scaled, 8));
      slot = __fadd_rn(slot, __shfl_sync(0xffffffffu, scaled, 16));
      slot = __fadd_rn(slot, __shfl_sync(0xffffffffu, scaled, 24));
      acc[j] = __fadd_rn(acc[j], __fmul_rn(slot, w));
    }
  }
  if (lane == 0) {
    uint32_t pk[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      pk[i] = *reinterpret_cast<uint32_t*>(&v);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * kHidden + n0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
  }
}

// Router bridge extras: shared-gate slot append (hidden . gate_w in BF16 -> sigmoid -> slot 8).
// grid rows, block 32.
extern "C" __global__ void __launch_bounds__(32)
netra_qwen36_shared_gate_append_sm100(int32_t* __restrict__ out_ids, float* __restrict__ out_w,
                                      const uint16_t* __restrict__ hidden, const uint16_t* __restrict__ gate_w,
                                      const int32_t* __restrict__ ids, const float* __restrict__ w, uint32_t rows) {
  const int t = blockIdx.x, lane = threadIdx.x;
  if (t >= (int)rows) return;
  // The gate is defined exactly so that it can be compared bit for bit: logit = the exact dot product rounded once to
  // BF16 (FP64 accumulation of exact products), gate = sigmoid(logit) evaluated in FP64 and rounded once to BF16.
  double part = 0.0;
  for (int k = lane; k < kHidden; k += 32)
    part = fma((double)bf16_bits_to_f32(hidden[(size_t)t * kHidden + k]), (double)bf16_bits_to_f32(gate_w[k]), part);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) part += __shfl_xor_sync(0xffffffffu, part, d);
  const double logit = (double)bf16_bits_to_f32(f64_to_bf16_bits(part));
  const float gate = bf16_bits_to_f32(f64_to_bf16_bits(1.0 / (1.0 + exp(-logit))));
  if (lane < kTopK) {
    out_ids[t * kSlots + lane] = ids[t * kTopK + lane];
    out_w[t * kSlots + lane] = w[t * kTopK + lane];
  } else if (lane == kTopK) {
    out_ids[t * kSlots + kTopK] = kRouted;
    out_w[t * kSlots + kTopK] = gate;
  }
}

}  // namespace netra

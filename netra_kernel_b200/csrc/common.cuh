// Shared device helpers and fixed model constants for the sm_100a routed-MoE kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace netra {

// Fixed contract (same role as the reference's assembler guards,
// kernels/gfx950/templates/moe/decode/gate_up_mfma.inc:13-20).
constexpr int kHidden = 2048;       // model width
constexpr int kInter = 512;         // expert intermediate width
constexpr int kRouted = 256;        // routed experts (global)
constexpr int kTopK = 8;            // routed slots per token
constexpr int kSlots = 9;           // routed slots + shared slot
constexpr int kBlock = 128;         // quantisation block along K
constexpr int kHiddenBlocks = kHidden / kBlock;  // 16
constexpr int kInterBlocks = kInter / kBlock;    // 4
constexpr int kSortSegment = 1024;  // routed pairs per sort segment

// fl32(1/448) and 1e-10f as bit patterns (kernels/gfx950/templates/moe/decode/silu_quant.inc:40-41).
__device__ __forceinline__ float inv448() { return __uint_as_float(0x3b124925u); }
__device__ __forceinline__ float amax_floor() { return __uint_as_float(0x2edbe6ffu); }

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// One rounding FP64 -> BF16 (nearest even).  Results below the smallest normal BF16 are flushed to zero
// (signed), results at or above 2^128 become infinity, NaN stays NaN (quiet, sign kept).
__device__ __forceinline__ uint16_t f64_to_bf16_bits(double d) {
  long long bits = __double_as_longlong(d);
  uint16_t sign = (uint16_t)(((unsigned long long)bits >> 63) << 15);
  long long mag = bits & 0x7fffffffffffffffLL;
  if (mag > 0x7ff0000000000000LL) return (uint16_t)(sign | 0x7fc0u);   // NaN
  long long r = (mag + ((1LL << 44) - 1) + ((mag >> 45) & 1)) >> 45;
  r -= (896LL << 7);
  if (r < (1 << 7)) r = 0;
  if (r > 0x7f80) r = 0x7f80;                                            // overflow and infinity
  return (uint16_t)(sign | (uint16_t)r);
}

__device__ __forceinline__ uint8_t f32_to_e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

// four floats -> four packed E4M3 codes (round to nearest even, saturating), two conversions
__device__ __forceinline__ uint32_t f32x4_to_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

__device__ __forceinline__ float e4m3_to_f32(uint8_t c) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
  return __half2float(__half(h));
}

// four packed E4M3 codes -> four floats
__device__ __forceinline__ void e4m3x4_to_f32(uint32_t packed, float out[4]) {
  __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(packed & 0xffffu), __NV_E4M3);
  __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(packed >> 16), __NV_E4M3);
  float2 a = __half22float2(__half2(lo));
  float2 b = __half22float2(__half2(hi));
  out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
}

// SiLU in FP32: x / (1 + exp(-x)) (kernels/gfx950/templates/moe/decode/silu_quant.inc:54-94)
__device__ __forceinline__ float silu_f32(float x) { return x * (1.0f / (1.0f + __expf(-x))); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

}  // namespace netra

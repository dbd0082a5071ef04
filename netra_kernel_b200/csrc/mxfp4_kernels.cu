// MXFP4 expert weights on the FP8 tensor-core path: a load-time expansion of E2M1 codes with one
// E8M0 scale per 32 K-elements into E4M3 codes with one power-of-two FP32 scale per 128 x 128
// tile - the operand format of the grouped GEMMs (umma_kernels.cu, umma_tokmajor.cu).
//
// Encoding (tools/checkpoint/quantize_qwen36_lm_head_mxfp4.py:58-67,
// tests/gfx1151/test_netra_mxfp4_sgl_decode.py:23-31): w = lut[c & 7] * (-1)^(c >> 3) * 2^(s - 127),
// lut = {0, .5, 1, 1.5, 2, 3, 4, 6}, byte = code[k even] | code[k odd] << 4.
//
// Per tile: s_ref = (largest scale byte of the tile) - 6 and tile scale T = 2^(s_ref - 127); an element
// becomes the E4M3 value lut * 2^(s - s_ref).  E4M3 holds lut * 2^j exactly for -8 <= j <= 6 (6 * 2^6 =
// 384 <= 448; 0.5 * 2^-8 = 2^-9 is its smallest subnormal), so the expansion is exact whenever the
// scales inside a tile span at most 15 binades; smaller elements are rounded to nearest and counted
// in *inexact so that the caller knows.  Products and sums of the expanded weights on the tensor
// cores are then exactly those of the MXFP4 weights.
#include "common.cuh"

namespace netra {

// grid (k / 128, rows / 128), block 128: thread r expands row (blockIdx.y * 128 + r), K-block blockIdx.x.
// packed [rows, k / 2], scales [rows, k / 32], dst [rows, k] E4M3, dst_scale [rows / 128, k / 128] FP32.
extern "C" __global__ void __launch_bounds__(128)
netra_moe_mxfp4_expand_sm100(uint8_t* __restrict__ dst, float* __restrict__ dst_scale, uint32_t* __restrict__ inexact,
                             const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales, uint32_t k) {
  __shared__ int s_max[4];
  const int kb = blockIdx.x, r = threadIdx.x;
  const size_t row = (size_t)blockIdx.y * 128 + r;
  const uint32_t sc4 = *reinterpret_cast<const uint32_t*>(scales + row * (k / 32) + kb * 4);   // four E8M0 bytes
  int mine = max(max((int)(sc4 & 255u), (int)((sc4 >> 8) & 255u)), max((int)((sc4 >> 16) & 255u), (int)(sc4 >> 24)));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) mine = max(mine, __shfl_xor_sync(0xffffffffu, mine, d));
  if ((r & 31) == 0) s_max[r >> 5] = mine;
  __syncthreads();
  const int s_ref = max(max(s_max[0], s_max[1]), max(s_max[2], s_max[3])) - 6;
  if (r == 0) dst_scale[(size_t)blockIdx.y * (k / 128) + kb] = ldexpf(1.0f, s_ref - 127);
  const uint4* src = reinterpret_cast<const uint4*>(packed + row * (k / 2) + kb * 64);
  uint4* out = reinterpret_cast<uint4*>(dst + row * k + kb * 128);
  uint32_t bad = 0;
#pragma unroll
  for (int q = 0; q < 4; ++q) {              // 16 packed bytes = 32 elements = one scale group
    const uint4 p = src[q];
    const int j = (int)((sc4 >> (8 * q)) & 255u) - s_ref;      // <= 6
    const float mul = ldexpf(1.0f, max(j, -30));
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v[8];
#pragma unroll
      for (int n = 0; n < 8; ++n) {
        const uint32_t c = (w[i] >> (4 * n)) & 15u;
        const uint32_t m = c & 7u;
        // lut = {0, .5, 1, 1.5, 2, 3, 4, 6}: codes 0-1 are 0.5 * m, above that (1 + (m & 1) / 2) * 2^((m >> 1) - 1)
        const float mag = m < 2u ? 0.5f * (float)m : ldexpf(1.0f + 0.5f * (float)(m & 1u), (int)(m >> 1) - 1);
        v[n] = (c & 8u) ? -mag * mul : mag * mul;
        bad += (m != 0u && j < -8) ? 1u : 0u;
      }
      o[2 * i] = f32x4_to_e4m3x4(v[0], v[1], v[2], v[3]);
      o[2 * i + 1] = f32x4_to_e4m3x4(v[4], v[5], v[6], v[7]);
    }
    out[2 * q] = make_uint4(o[0], o[1], o[2], o[3]);
    out[2 * q + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
  if (bad) atomicAdd(inexact, bad);
}

// MXFP4 slabs -> the operand layout of the native kernels (netra_moe_gate_up_mxfp4_sm100, netra_moe_down_mxfp4_sm100):
//   codes  one contiguous 8 KiB block per (128-row tile, K-block): row r of the block holds the 64 bytes
//          [kb * 64, +64) of source row tile * 128 + r
//   atoms  one 512-byte block per (tile, K-block) in the same order: the four scale bytes of row r and this
//          K-block sit at byte 16 * (r % 32) + 4 * (r / 32) - the order in which a 32-row x 16-byte copy
//          into TMEM puts row r's bytes into lane r % 32, column r / 32, the place the tensor core reads them
// The kernels fetch two blocks per copy - the two weight tiles one MMA stage consumes - so blocks are ordered (group,
// tile within the half, K-block, half): the rows come in groups of 2 * paired_half_tiles tiles whose two halves are
// consumed together (W13: 4, a gate tile next to its up tile; W2: 1, tiles 2p and 2p + 1).
// grid (k / 128, rows / 128), block 128: thread r moves row (blockIdx.y * 128 + r), K-block blockIdx.x.
extern "C" __global__ void __launch_bounds__(128)
netra_moe_mxfp4_pack_sm100(uint8_t* __restrict__ dst_codes, uint8_t* __restrict__ dst_atoms, const uint8_t* __restrict__ packed,
                           const uint8_t* __restrict__ scales, uint32_t k, uint32_t paired_half_tiles) {
  const uint32_t kb = blockIdx.x, r = threadIdx.x, kblocks = k / 128;
  const size_t row = (size_t)blockIdx.y * 128 + r;
  const uint32_t group_tiles = 2 * paired_half_tiles;
  const size_t group = blockIdx.y / group_tiles;
  const uint32_t t = blockIdx.y % group_tiles, half = t / paired_half_tiles, tile = t % paired_half_tiles;
  const size_t block = (((group * paired_half_tiles + tile) * kblocks + kb) * 2) + half;
  const uint4* src = reinterpret_cast<const uint4*>(packed + row * (k / 2) + kb * 64);
  uint4* out = reinterpret_cast<uint4*>(dst_codes + (block * 128 + r) * 64);
#pragma unroll
  for (int q = 0; q < 4; ++q) out[q] = src[q];
  const uint32_t sc4 = *reinterpret_cast<const uint32_t*>(scales + row * (k / 32) + kb * 4);
  *reinterpret_cast<uint32_t*>(dst_atoms + block * 512 + 16 * (r & 31u) + 4 * (r >> 5)) = sc4;
}

}  // namespace netra

// Block-scaled FP8 grouped GEMMs on the sm_100a tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Both expert projections run "swap-AB": the 128 weight rows of a tile are the MMA M dimension
// and the (few) token rows of an expert are the MMA N dimension, so a decode-sized expert
// (about 8 rows) streams its weights exactly once with no padded M work.
//
//   gate_up (replaces kernels/gfx950/templates/moe/decode/gate_up_mfma.inc:13-95 and
//            kernels/gfx950/templates/moe/decode/silu_quant.inc:54-169):
//     tile = expert x 128 intermediate channels: W13 gate rows [c*128, +128) and up rows
//     [512 + c*128, +128) against the expert's token rows; per K-block (128) the raw FP8 partial
//     sums leave TMEM and are promoted in FP32 as acc += (part * a_scale[row,kb]) * w_scale[kb]
//     (gfx950 order, kernels/gfx950/templates/common/mfma.inc:20-24); the epilogue forms
//     bf16(silu(gate) * up), takes the per-128 amax (the tile is exactly one quantisation
//     group per row), and stores FP8 codes + FP32 scale.
//   down (replaces kernels/gfx950/templates/moe/decode/down_reduce_mfma_2wave.inc:73-217,
//         the GEMM part): tile = expert x 128 output columns, K = 512, FP32 rows written in
//     expert-sorted order for the slot-ordered combine kernel.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (owns TMEM),
// warps 2..5 = promotion/epilogue (TMEM lane quadrant = warp id % 4).
// Every mbarrier wait is bounded; on expiry the CTA records a code in status[] and drains.
#include <cuda.h>

#include "common.cuh"

namespace netra {

constexpr int kTileRows = 128;          // weight rows per MMA (UMMA M)
constexpr int kTokMax = 64;             // token rows per work item (UMMA N <= 64)
constexpr int kWTileBytes = kTileRows * kBlock;   // 16 KiB: 128 rows x 128 K bytes
constexpr int kTokTileBytes = kTokMax * kBlock;   // 8 KiB
constexpr int kMaxGroups = 257;
constexpr uint32_t kSpinLimit = 1u << 22;

enum : uint32_t { kStatusOk = 0, kStatusProducerTimeout = 1, kStatusMmaTimeout = 2, kStatusEpilogueTimeout = 3 };

// ---------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: false when the limit ran out or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 0xff) == 0xff && *abort_flag != 0) return false;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float v[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// K-major, 128-byte-swizzled operand tile: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3ffffu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f8f6f4, E4M3 x E4M3 -> FP32, both operands K-major, M = 128.
__device__ __forceinline__ uint32_t make_idesc(uint32_t n) {
  return (1u << 4) | ((n >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);
}

// ---------------------------------------------------------------------------- work items
struct Item {
  int group;    // expert slab index
  int ntile;    // 128-row weight tile inside the slab
  int row0;     // first token row (expert-sorted row space)
  int m_valid;  // token rows in this item (1..64)
};

template <int kNTiles>
__device__ __forceinline__ Item decode_item(int item, const int* item_pre, const int* offs, int num_groups) {
  int lo = 0, hi = num_groups;            // largest idx with item_pre[idx] <= item
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (item_pre[mid] <= item) lo = mid; else hi = mid;
  }
  const int local = item - item_pre[lo];
  Item it;
  it.group = lo == 0 ? num_groups - 1 : lo - 1;   // the last group (shared expert) is scheduled first
  it.ntile = local % kNTiles;
  it.row0 = offs[it.group] + (local / kNTiles) * kTokMax;
  it.m_valid = min(kTokMax, offs[it.group + 1] - it.row0);
  return it;
}

// kGateUp: 2 weight tiles per stage (gate, up), K = 2048, FP8 epilogue.  else: 1 tile, K = 512, FP32 epilogue.
template <bool kGateUp>
struct Cfg {
  static constexpr int kATiles = kGateUp ? 2 : 1;
  static constexpr int kKBlocks = kGateUp ? kHiddenBlocks : kInterBlocks;
  static constexpr int kNTiles = kGateUp ? kInter / kTileRows : kHidden / kTileRows;   // 4 | 16
  static constexpr int kSlabRows = kGateUp ? 2 * kInter : kHidden;                     // 1024 | 2048
  static constexpr int kStages = kGateUp ? 4 : 6;
  static constexpr int kStageBytes = kATiles * kWTileBytes + kTokTileBytes;            // 40 KiB | 24 KiB
  static constexpr int kTmemCols = 2 * kATiles * kTokMax;                              // 256 | 128
  static constexpr int kEpiBytes = kGateUp ? kTokMax * 272 : kTokMax * 132 * 4;        // staging tile
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kEpiBytes + kTokMax * kKBlocks * 4 +
                                    kATiles * kKBlocks * 4 + 2 * 264 * 4 + 256;
};

template <bool kGateUp>
__device__ __forceinline__ void grouped_gemm_body(const CUtensorMap* tm_w, const CUtensorMap* tm_x32,
                                                  const CUtensorMap* tm_x64, const float* __restrict__ x_scale,
                                                  const float* __restrict__ w_scale, const int32_t* __restrict__ offsets,
                                                  uint8_t* __restrict__ h_fp8, float* __restrict__ h_scale,
                                                  float* __restrict__ down, uint32_t num_groups, uint32_t* status) {
  using C = Cfg<kGateUp>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint8_t* epi_tile = stage_base + C::kStages * C::kStageBytes;
  float* xs_tile = reinterpret_cast<float*>(epi_tile + C::kEpiBytes);            // [64][kKBlocks]
  float* ws_tile = xs_tile + kTokMax * C::kKBlocks;                              // [kATiles][kKBlocks]
  int* offs = reinterpret_cast<int*>(ws_tile + C::kATiles * C::kKBlocks);        // [264]
  int* item_pre = offs + 264;                                                    // [264]
  uint64_t* bars = reinterpret_cast<uint64_t*>(item_pre + 264);
  uint64_t* full_bar = bars;                       // [kStages]
  uint64_t* empty_bar = bars + C::kStages;         // [kStages]
  uint64_t* tfull_bar = bars + 2 * C::kStages;     // [2]
  uint64_t* tempty_bar = tfull_bar + 2;            // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = (int)num_groups;

  // ---- setup: offsets -> smem, item prefix (shared group first), barriers, TMEM
  for (int i = threadIdx.x; i <= groups; i += blockDim.x) offs[i] = offsets[i];
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&tfull_bar[a]), 1); mbar_init(smem_u32(&tempty_bar[a]), 4); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    // lane owns 9 consecutive schedule slots; slot 0 = last group, slot i = group i-1
    int cnt[9], sum = 0;
#pragma unroll
    for (int j = 0; j < 9; ++j) {
      const int idx = lane * 9 + j;
      int c = 0;
      if (idx < groups) {
        const int g = idx == 0 ? groups - 1 : idx - 1;
        const int m = offs[g + 1] - offs[g];
        c = ((m + kTokMax - 1) / kTokMax) * C::kNTiles;
      }
      cnt[j] = c; sum += c;
    }
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { int o = __shfl_up_sync(0xffffffffu, incl, d); if (lane >= d) incl += o; }
    int run = incl - sum;
#pragma unroll
    for (int j = 0; j < 9; ++j) {
      const int idx = lane * 9 + j;
      if (idx <= groups) item_pre[idx] = run;
      run += cnt[j];
    }
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_items = item_pre[groups];

  if (warp == 0) {
    // =========================== TMA producer ===========================
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tm_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tm_x32) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tm_x64) : "memory");
      uint32_t it = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const Item w = decode_item<C::kNTiles>(item, item_pre, offs, groups);
        const bool small = w.m_valid <= 32;
        const uint32_t bytes = C::kATiles * kWTileBytes + (small ? 32 : 64) * kBlock;
        const int wrow = w.group * C::kSlabRows + w.ntile * kTileRows;
        for (int kb = 0; kb < C::kKBlocks; ++kb, ++it) {
          const int s = it % C::kStages;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / C::kStages) & 1) ^ 1, abort_flag)) {
            status[0] = kStatusProducerTimeout; *abort_flag = 1; ok = false; break;
          }
          const uint32_t bar = smem_u32(&full_bar[s]);
          const uint32_t dst = smem_u32(stage_base + s * C::kStageBytes);
          mbar_expect_tx(bar, bytes);
          tma_load_2d(dst, tm_w, bar, kb * kBlock, wrow);
          if (kGateUp) tma_load_2d(dst + kWTileBytes, tm_w, bar, kb * kBlock, wrow + kInter);
          tma_load_2d(dst + C::kATiles * kWTileBytes, small ? tm_x32 : tm_x64, bar, kb * kBlock, w.row0);
        }
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      uint32_t it = 0, jt = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const Item w = decode_item<C::kNTiles>(item, item_pre, offs, groups);
        const uint32_t n_mma = (uint32_t)((w.m_valid + 15) & ~15);
        const uint32_t idesc = make_idesc(n_mma);
        for (int kb = 0; kb < C::kKBlocks; ++kb, ++it, ++jt) {
          const int s = it % C::kStages, a = jt & 1;
          if (!mbar_wait(smem_u32(&tempty_bar[a]), ((jt >> 1) & 1) ^ 1, abort_flag) ||
              !mbar_wait(smem_u32(&full_bar[s]), (it / C::kStages) & 1, abort_flag)) {
            status[0] = kStatusMmaTimeout; *abort_flag = 1; ok = false; break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(stage_base + s * C::kStageBytes);
          const uint64_t bdesc = make_smem_desc(sa + C::kATiles * kWTileBytes);
#pragma unroll
          for (int tile = 0; tile < C::kATiles; ++tile) {
            const uint64_t adesc = make_smem_desc(sa + tile * kWTileBytes);
            const uint32_t d = tmem_base + (uint32_t)(a * C::kATiles * kTokMax + tile * kTokMax);
#pragma unroll
            for (int k = 0; k < kBlock / 32; ++k) umma_f8(d, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0);
          }
          umma_commit(smem_u32(&empty_bar[s]));
          umma_commit(smem_u32(&tfull_bar[a]));
        }
      }
    }
  } else {
    // =========================== promotion + epilogue (128 threads) ===========================
    const int et = threadIdx.x - 64;         // 0..127
    const int quad = warp & 3;               // TMEM lane quadrant this warp may read
    const int r = quad * 32 + lane;          // weight row inside the tile == TMEM lane
    uint32_t jt = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
      const Item w = decode_item<C::kNTiles>(item, item_pre, offs, groups);
      const int n_mma = (w.m_valid + 15) & ~15;
      // scales of this item -> smem
      for (int i = et; i < kTokMax * C::kKBlocks; i += 128) {
        const int c = i / C::kKBlocks;
        xs_tile[i] = c < w.m_valid ? x_scale[(size_t)(w.row0 + c) * C::kKBlocks + (i % C::kKBlocks)] : 0.0f;
      }
      if (et < C::kATiles * C::kKBlocks) {
        const int tile = et / C::kKBlocks, kb = et % C::kKBlocks;
        const int nb = kGateUp ? tile * (kInter / kBlock) + w.ntile : w.ntile;
        ws_tile[et] = w_scale[((size_t)w.group * (C::kSlabRows / kBlock) + nb) * C::kKBlocks + kb];
      }
      epi_barrier();
      float acc[C::kATiles][kTokMax];
#pragma unroll
      for (int tile = 0; tile < C::kATiles; ++tile)
#pragma unroll
        for (int c = 0; c < kTokMax; ++c) acc[tile][c] = 0.0f;
      for (int kb = 0; kb < C::kKBlocks; ++kb, ++jt) {
        const int a = jt & 1;
        if (ok && !mbar_wait(smem_u32(&tfull_bar[a]), (jt >> 1) & 1, abort_flag)) {
          status[0] = kStatusEpilogueTimeout; *abort_flag = 1; ok = false;
        }
        if (!ok) continue;
        tc_fence_after();
        const uint32_t tbase = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * C::kATiles * kTokMax);
#pragma unroll
        for (int tile = 0; tile < C::kATiles; ++tile) {
          const float ws = ws_tile[tile * C::kKBlocks + kb];
#pragma unroll
          for (int sl = 0; sl < kTokMax / 16; ++sl) {
            if (sl * 16 < n_mma) {
              float v[16];
              tmem_ld16(tbase + (uint32_t)(tile * kTokMax + sl * 16), v);
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const float xs = xs_tile[(sl * 16 + i) * C::kKBlocks + kb];
                acc[tile][sl * 16 + i] = __fadd_rn(acc[tile][sl * 16 + i], __fmul_rn(__fmul_rn(v[i], xs), ws));
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[a]));
      }
      // ---- item epilogue
      if constexpr (kGateUp) {
        __nv_bfloat16* hs = reinterpret_cast<__nv_bfloat16*>(epi_tile);   // [64][136]
#pragma unroll
        for (int c = 0; c < kTokMax; ++c) {
          if (c < n_mma) {
            const float g = acc[0][c];
            const float sig = 1.0f / (1.0f + expf(-g));
            hs[c * 136 + r] = __float2bfloat16_rn(__fmul_rn(__fmul_rn(g, sig), acc[C::kATiles - 1][c]));
          }
        }
        epi_barrier();
        const int c = et >> 1, half = et & 1;   // 2 threads per token row, 64 channels each
        const bool valid = c < w.m_valid;
        float x[64];
        float amax = amax_floor();
        const uint4* src = reinterpret_cast<const uint4*>(hs + c * 136 + half * 64);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          uint4 v = src[q];
          const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            x[q * 8 + 2 * j] = bf16_bits_to_f32(u[j] & 0xffffu);
            x[q * 8 + 2 * j + 1] = bf16_bits_to_f32(u[j] >> 16);
          }
        }
#pragma unroll
        for (int i = 0; i < 64; ++i) amax = fmaxf(amax, fabsf(x[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        if (valid) {
          const float scale = amax * inv448();
          const float inv = 1.0f / scale;
          const size_t row = (size_t)(w.row0 + c);
          if (half == 0) h_scale[row * kInterBlocks + w.ntile] = scale;
          uint4* dst = reinterpret_cast<uint4*>(h_fp8 + row * kInter + w.ntile * kTileRows + half * 64);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint32_t pk[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t b = 0;
#pragma unroll
              for (int i = 0; i < 4; ++i) b |= (uint32_t)f32_to_e4m3(x[q * 16 + j * 4 + i] * inv) << (8 * i);
              pk[j] = b;
            }
            dst[q] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
      } else {
        float* ds = reinterpret_cast<float*>(epi_tile);   // [64][132]
#pragma unroll
        for (int c = 0; c < kTokMax; ++c)
          if (c < n_mma) ds[c * 132 + r] = acc[0][c];
        epi_barrier();
        const int ew = et >> 5;
        for (int c = ew; c < w.m_valid; c += 4) {
          float4 v = *reinterpret_cast<const float4*>(ds + c * 132 + lane * 4);
          *reinterpret_cast<float4*>(down + (size_t)(w.row0 + c) * kHidden + w.ntile * kTileRows + lane * 4) = v;
        }
      }
      epi_barrier();   // staging tile and scale tiles are free for the next item
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) __nanosleep(200000);   // let copies already in flight land before the CTA exits
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

extern "C" __global__ void __launch_bounds__(192, 1)
netra_moe_gate_up_umma_sm100(const __grid_constant__ CUtensorMap tm_w13, const __grid_constant__ CUtensorMap tm_a32,
                             const __grid_constant__ CUtensorMap tm_a64, const float* a_scale, const float* w13_scale,
                             const int32_t* offsets, uint8_t* h_fp8, float* h_scale, uint32_t num_groups,
                             uint32_t* status) {
  grouped_gemm_body<true>(&tm_w13, &tm_a32, &tm_a64, a_scale, w13_scale, offsets, h_fp8, h_scale, nullptr, num_groups, status);
}

extern "C" __global__ void __launch_bounds__(192, 1)
netra_moe_down_umma_sm100(const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_h32,
                          const __grid_constant__ CUtensorMap tm_h64, const float* h_scale, const float* w2_scale,
                          const int32_t* offsets, float* down, uint32_t num_groups, uint32_t* status) {
  grouped_gemm_body<false>(&tm_w2, &tm_h32, &tm_h64, h_scale, w2_scale, offsets, nullptr, nullptr, down, num_groups, status);
}

int gate_up_smem_bytes() { return Cfg<true>::kSmemBytes; }
int down_smem_bytes() { return Cfg<false>::kSmemBytes; }

}  // namespace netra

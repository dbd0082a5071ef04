// Router projection on the sm_100a tensor cores for calls with many rows (prefill, expert-parallel
// steps): FP32 logits[t, e] = sum_k hidden[t, k] * w[e, k], BF16 operands fed by TMA, FP32
// accumulators in TMEM (tcgen05.mma kind::f16).  The result is an APPROXIMATION of the exact dot
// product (the accumulation order and rounding inside the tensor core are not specified); the
// routing contract - BF16 logits that are the exact dot product rounded once - is restored by
// the kernel that consumes these values (netra_moe_topk_quant_fix_sm100, route_kernels.cu): it
// recomputes in FP64 every logit whose FP32 value lies so close to a BF16 rounding boundary
// that the approximation error could change the rounded result.
//
// Behaviour replaced: kernels/gfx950/templates/routing/bf16_gemv.inc:16-89 (one fixed FP32 order
// per logit on the vector units).
//
// Grid: tile CTAs (m_tile, n_half) = (blockIdx.x >> 1, blockIdx.x & 1), each 128 token rows x 128
// experts over all of K, followed by kRtNormCtas CTAs that write the router rows' Euclidean norms
// (used by the consumer's error bound).  192 threads: warp 0 = TMA producer, warp 1 = MMA issuer
// (owns TMEM), warps 2-5 = epilogue (TMEM lane quadrant = warp % 4).  Two CTAs fit on one SM.
// Every mbarrier wait is bounded; on expiry the CTA records a code in status[] and drains.
#include "common.cuh"

namespace netra {

constexpr int kRtThreads = 192;
constexpr int kRtTile = 128;                         // token rows and expert rows per tile
constexpr int kRtKBytes = kHidden * 2;               // 4096 bytes of BF16 per row
constexpr int kRtKBlocks = kRtKBytes / kBlock;       // 32 K-blocks of 64 BF16 (128 bytes)
constexpr int kRtStages = 3;
constexpr int kRtStageBytes = 2 * kRtTile * kBlock;  // 32 KiB: token tile, expert tile
constexpr int kRtTmemCols = 128;
constexpr int kRtNormCtas = 8;
constexpr int kRtSmemBytes = 1024 + kRtStages * kRtStageBytes + 256;

// kind::f16: BF16 x BF16 -> FP32, both operands K-major, M = 128.
__device__ __forceinline__ uint32_t make_idesc_bf16(uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((uint32_t)(kRtTile >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

extern "C" __global__ void __launch_bounds__(kRtThreads, 2)
netra_router_logits_f32_umma_sm100(const __grid_constant__ CUtensorMap tm_hidden, const __grid_constant__ CUtensorMap tm_weight,
                                   float* __restrict__ logits_f32, float* __restrict__ wnorm,
                                   const uint16_t* __restrict__ weight, uint32_t rows, uint32_t* status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = ((int)rows + kRtTile - 1) / kRtTile;
  if ((int)blockIdx.x >= 2 * m_tiles) {
    // ---- norm CTAs: wnorm[e] >= |w[e, :]|_2 (rounded up by a relative 1e-3)
    const int part = (int)blockIdx.x - 2 * m_tiles;
    for (int j = warp; j < kRouted / kRtNormCtas; j += kRtThreads / 32) {
      const int e = part * (kRouted / kRtNormCtas) + j;
      const uint4* src = reinterpret_cast<const uint4*>(weight + (size_t)e * kHidden);
      float s = 0.0f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 v = __ldg(src + c * 32 + lane);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float a = bf16_bits_to_f32(u[q] & 0xffffu), b = bf16_bits_to_f32(u[q] >> 16);
          s = fmaf(a, a, s);
          s = fmaf(b, b, s);
        }
      }
      s = warp_sum(s);
      if (lane == 0) wnorm[e] = sqrtf(s) * 1.001f;
    }
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_base + kRtStages * kRtStageBytes);
  uint64_t* full_bar = bars;                   // [kRtStages]
  uint64_t* empty_bar = bars + kRtStages;      // [kRtStages]
  uint64_t* tfull_bar = bars + 2 * kRtStages;  // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int m_tile = (int)blockIdx.x >> 1, n_half = (int)blockIdx.x & 1;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kRtStages; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
    mbar_init(smem_u32(tfull_bar), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_slot), kRtTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // =========================== TMA producer ===========================
      asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tm_hidden) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)&tm_weight) : "memory");
      const uint64_t pol = policy_evict_last();      // the token tile is read by two CTAs, the router rows by all
      for (int kb = 0; kb < kRtKBlocks; ++kb) {
        const int s = kb % kRtStages;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ((kb / kRtStages) & 1) ^ 1, abort_flag)) {
          status[0] = kStatusProducerTimeout; *abort_flag = 1; break;
        }
        const uint32_t bar = smem_u32(&full_bar[s]);
        const uint32_t dst = smem_u32(stage_base + s * kRtStageBytes);
        mbar_expect_tx(bar, kRtStageBytes);
        tma_load_2d(dst, &tm_hidden, bar, kb * kBlock, m_tile * kRtTile, pol);   // rows past `rows` read as zero
        tma_load_2d(dst + kRtTile * kBlock, &tm_weight, bar, kb * kBlock, n_half * kRtTile, pol);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // =========================== MMA issuer ===========================
      const uint32_t idesc = make_idesc_bf16(kRtTile);
      bool ok = true;
      for (int kb = 0; kb < kRtKBlocks; ++kb) {
        const int s = kb % kRtStages;
        if (!mbar_wait(smem_u32(&full_bar[s]), (kb / kRtStages) & 1, abort_flag)) {
          status[0] = kStatusMmaTimeout; *abort_flag = 1; ok = false; break;
        }
        tc_fence_after();
        const uint32_t sa = smem_u32(stage_base + s * kRtStageBytes);
        const uint64_t adesc = make_smem_desc(sa);                       // 128 token rows
        const uint64_t bdesc = make_smem_desc(sa + kRtTile * kBlock);    // 128 router rows
#pragma unroll
        for (int k = 0; k < kBlock / 32; ++k)                            // 16 BF16 (32 bytes) per MMA
          umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
        umma_commit(smem_u32(&empty_bar[s]));
      }
      if (ok) umma_commit(smem_u32(tfull_bar));
    }
  } else {
    // =========================== epilogue: TMEM -> FP32 rows ===========================
    const int quad = warp & 3;
    const int token = m_tile * kRtTile + quad * 32 + lane;
    if (mbar_wait(smem_u32(tfull_bar), 0, abort_flag)) {
      tc_fence_after();
      float* dst = logits_f32 + (size_t)token * kRouted + n_half * kRtTile;
#pragma unroll 1
      for (int c = 0; c < kRtTile / 32; ++c) {
        uint32_t v[32];
        tmem_ld32_nowait(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(c * 32), v);
        tmem_ld_wait();
        if (token < (int)rows) {
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(v[i]);
#pragma unroll
          for (int q = 0; q < 4; ++q) st_global_v8(dst + c * 32 + 8 * q, &f[8 * q]);
        }
      }
    } else {
      status[0] = kStatusEpilogueTimeout; *abort_flag = 1;
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (*abort_flag != 0) __nanosleep(200000);   // let copies already in flight land before the CTA exits
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kRtTmemCols);
  }
}

int router_umma_smem_bytes() { return kRtSmemBytes; }

}  // namespace netra

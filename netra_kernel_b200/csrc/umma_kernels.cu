// Block-scaled FP8 grouped GEMMs on the sm_100a tensor cores (tcgen05 + TMEM), fed by TMA.
//
// Both expert projections run "swap-AB": the 128 weight rows of a tile are the MMA M dimension
// and the token rows of an expert are the MMA N dimension (16 or 32), so a decode-sized expert
// (about 8 rows) streams its weights exactly once with no padded M work.
//
//   gate_up (replaces kernels/gfx950/templates/moe/decode/gate_up_mfma.inc:13-95 and
//            kernels/gfx950/templates/moe/decode/silu_quant.inc:54-169):
//     tile = expert x 128 intermediate channels: W13 gate rows [c*128, +128) and up rows
//     [512 + c*128, +128) against the expert's token rows; per K-block (128) the raw FP8 partial
//     sums leave TMEM and are promoted in FP32 as acc = fma(part, a_scale[row,kb] * w_scale[kb], acc)
//     (the order of kernels/gfx950/templates/moe/prefill/fused_splitk2/gate_up.inc:275-300); the epilogue forms
//     bf16(silu(gate) * up), takes the per-128 amax (the tile is exactly one quantisation
//     group per row), and stores FP8 codes + FP32 scale.
//   down (replaces kernels/gfx950/templates/moe/decode/down_reduce_mfma_2wave.inc:73-217,
//         the GEMM part): tile = expert x 128 output columns, K = 512, FP32 rows written in
//     expert-sorted order for the slot-ordered combine kernel.
//
// Warp roles (320 threads): warp 0 = TMA producer, warp 1 = MMA issuer (owns TMEM),
// warps 2..9 = promotion/epilogue (TMEM lane quadrant = warp id % 4; warps 2..5 own token
// first half of an item's token columns, warps 6..9 the second half).
// Weight tiles come either from the checkpoint's row-major layout or from the tiled layout
// written by netra_moe_repack_tiles_sm100 (one contiguous 16 KiB block per tile and K-block).
// Every mbarrier wait is bounded; on expiry the CTA records a code in status[] and drains.
#include <cuda.h>

#include "common.cuh"

namespace netra {

constexpr int kTileRows = 128;          // weight rows per MMA (UMMA M)
constexpr int kWTileBytes = kTileRows * kBlock;   // 16 KiB: 128 rows x 128 K bytes
constexpr int kGemmThreads = 320;
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
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y), "l"(policy) : "memory");
}
// Four rows of a 2-D tensor (box = 128 bytes x 1 row) chosen by index, written as four consecutive 128-byte rows
// of a swizzled tile: the token rows of a work item are fetched straight from token order, without a sorted copy.
__device__ __forceinline__ void tma_gather4_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int r0, int r1, int r2, int r3,
                                               uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2], %8;"
      ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "l"(policy) : "memory");
}

// contiguous global -> shared copy; both addresses 16-byte aligned, size a multiple of 16
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"((uint64_t)src), "r"(bytes), "r"(bar) : "memory");
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
// kind::mxf8f6f4 with block scaling: every 32 K-elements of a row of A (B) are multiplied by one UE8M0 scale byte that
// the tensor core reads from TMEM columns sfa (sfb); the byte used inside each 32-bit column is part of idesc.
__device__ __forceinline__ void umma_mxf8f6f4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa,
                                              uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
}
// shared memory -> TMEM: 32 rows of 16 bytes land in lanes 0..31 of four consecutive columns and are repeated in the
// other three lane quadrants (each quadrant of the tensor core reads its own copy of the scales)
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// the calling warp's 32 lanes x 4 columns <- one 32-bit value
__device__ __forceinline__ void tmem_fill4(uint32_t taddr, uint32_t v) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %1, %1, %1};" ::"r"(taddr), "r"(v) : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns; the caller issues tmem_ld_wait() before reading r[]
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t r[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld8_nowait(uint32_t taddr, uint32_t r[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 1/x for a normal positive x: hardware approximation plus one Newton step (the reference's quantiser does
// the same, kernels/gfx950/templates/moe/decode/silu_quant.inc:140-150)
__device__ __forceinline__ float rcp_newton(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return fmaf(r, fmaf(-x, r, 1.0f), r);
}
// barrier among the 128 threads of one epilogue warp group (ids 1 and 2)
__device__ __forceinline__ void group_barrier(int group) {
  if (group == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
  else asm volatile("bar.sync 2, 128;" ::: "memory");
}

// K-major, 128-byte-swizzled operand tile: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3ffffu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// kind::f8f6f4, E4M3 x E4M3 -> FP32, both operands K-major, M = 128.
__device__ __forceinline__ uint32_t make_idesc(uint32_t n) {
  return (1u << 4) | ((n >> 3) << 17) | ((uint32_t)(kTileRows >> 4) << 24);
}

// 512-byte scale atom: 32 rows of 16 bytes, unswizzled, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t make_scale_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3ffffu) >> 4) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}
// kind::mxf8f6f4.block_scale, A = E2M1 (MXFP4 weight rows), B = E4M3 (token rows), UE8M0 scales, FP32 accumulators,
// both operands K-major, M = 128; a_scale_byte selects the byte of the A-scale columns (the 32-element group of
// the 128-element K-block this instruction covers), B always uses byte 0.
__device__ __forceinline__ uint32_t make_idesc_mxfp4(uint32_t n, uint32_t a_scale_byte) {
  return (5u << 7) | ((n >> 3) << 17) | (1u << 23) | ((uint32_t)(kTileRows >> 4) << 24) | (a_scale_byte << 29);
}

// ---------------------------------------------------------------------------- work items
struct Item {
  int group;    // expert slab index
  int ntile;    // first 128-row weight tile of the item inside the slab
  int row0;     // first token row (expert-sorted row space)
  int m_valid;  // token rows in this item (1..64)
};

template <int kNTiles, int kSubTiles, int kTokMax>
__device__ __forceinline__ Item decode_item(int item, const int* item_pre, const int* offs, int num_groups) {
  int lo = 0, hi = num_groups;            // largest idx with item_pre[idx] <= item
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (item_pre[mid] <= item) lo = mid; else hi = mid;
  }
  const int local = item - item_pre[lo];
  Item it;
  it.group = lo == 0 ? num_groups - 1 : lo - 1;   // the last group (shared expert) is scheduled first
  it.ntile = (local % kNTiles) * kSubTiles;
  it.row0 = offs[it.group] + (local / kNTiles) * kTokMax;
  it.m_valid = min(kTokMax, offs[it.group + 1] - it.row0);
  return it;
}

// kGateUp: K = 2048, a stage holds a gate tile and its up tile, FP8 epilogue.  else: K = 512, a stage holds two
// neighbouring W2 tiles (an item is 256 output columns), FP32 epilogue.
// kFp4: the weight tiles are MXFP4 (E2M1 codes, 64 bytes per row and K-block in memory, expanded by the copy engine
// to one byte per element in shared memory) and each tile brings a 512-byte atom of UE8M0 scales.  The copy engine
// reaches the HBM rate on four-bit rows only with boxes of 256 rows (16 KiB of codes; boxes of 128 rows stop at about
// 5 TB/s however many are in flight), so a stage is filled by one such box: the gate and the up tile of a K-block, or
// two neighbouring W2 tiles, which the pack step stored next to each other.
template <bool kGateUp, bool kFp4 = false>
struct Cfg {
  static constexpr int kATiles = 2;   // weight tiles per stage: a gate tile and its up tile | two neighbouring W2 tiles
  // token rows per work item (UMMA N).  32 for both: 64-row items (the shared expert at decode sizes) ran a longer
  // epilogue than the four TMEM stages could hide, and the CTAs that held them finished 8 us after the rest
  static constexpr int kTokMax = 32;
  static constexpr int kColsPerGroup = kTokMax / 2;       // token columns owned by one epilogue warp group
  static constexpr int kSlices = kColsPerGroup / 8;       // 8-column TMEM loads per group and tile
  static constexpr int kTokTileBytes = kTokMax * kBlock;  // 4 KiB
  static constexpr int kScaleSlots = kGateUp ? 2 : 4;
  static constexpr int kKBlocks = kGateUp ? kHiddenBlocks : kInterBlocks;
  // consecutive tile pairs per work item (same token rows).  down: two, i.e. 512 output columns per item - with 256
  // the per-item costs (scale tile, drained pipeline, epilogue) showed: 52.4 us against 49.7 us at 256 tokens
  static constexpr int kSubTiles = (kGateUp || kFp4) ? 1 : 2;
  static constexpr int kNTiles = (kGateUp ? kInter / kTileRows : kHidden / kTileRows / kATiles) / kSubTiles;   // items per slab and chunk: 4 | 4 (MXFP4 down: 8)
  static constexpr int kSlabRows = kGateUp ? 2 * kInter : kHidden;                     // 1024 | 2048
  static constexpr int kSlabTiles = kSlabRows / kTileRows;                             // 8 | 16
  static constexpr int kKbPerStep = (kGateUp || kFp4) ? 1 : 2;   // K-blocks the MMA warp issues per accumulator hand-off
  static constexpr int kAccCols = kKbPerStep * kATiles * kTokMax;                      // TMEM columns per hand-off: 64 | 128
  static constexpr int kScaleCols = kFp4 ? 4 * kATiles + 4 : 0;                        // TMEM columns of the A and B scales
  static constexpr int kAccStages = (512 - kScaleCols) / kAccCols;                     // 8 | 4 (MXFP4: 7 | 3)
  static constexpr int kKbPerLoad = 1;                                                 // K-blocks per shared-memory stage
  static constexpr int kStages = kFp4 ? 5 : 6;
  static constexpr int kStageTiles = kKbPerLoad * kATiles;                             // weight tiles per stage
  static constexpr int kStageBytes = kKbPerLoad * (kATiles * kWTileBytes + kTokTileBytes);   // 36 KiB | 20 KiB (MXFP4 down: 40 KiB)
  static constexpr int kWTxBytes = kFp4 ? kWTileBytes / 2 : kWTileBytes;               // bytes one weight-tile copy reports
  static constexpr int kScaleAtomBytes = 512;                                          // 128 rows x 4 groups of 32
  static constexpr int kScaleStageBytes = kFp4 ? kStageTiles * kScaleAtomBytes : 0;
  static_assert(!kFp4 || kStageTiles == 2, "an MXFP4 stage is one 256-row box");
  static_assert(kKbPerStep % kKbPerLoad == 0 && kKBlocks % kKbPerLoad == 0, "stages must tile an accumulator step");
  static constexpr int kTmemCols = 512;
  static constexpr int kXsBytes = kTokMax * kKBlocks * 4;                              // 4 KiB | 1 KiB
  static constexpr int kWsBytes = kKBlocks * 4;                                        // 64 B | 16 B per tile
  static constexpr int kItemList = 128;                                                // work items of this CTA decoded once
  static constexpr int kScaleSlotBytes = kXsBytes + 128;                               // xs, then ws tiles
  static constexpr int kSmemBytes = 1024 + kStages * (kStageBytes + kScaleStageBytes) + kScaleSlots * kScaleSlotBytes +
                                    2 * 4 * kColsPerGroup * 4 + 2 * 264 * 4 + kItemList * 16 + 512;
};

// kChain: 0 = a kernel of its own.  1 and 2 = the two halves of netra_moe_gate_up_down_umma_sm100, one launch for both
// projections: the gate_up half (1) counts, per unit of four work items (an expert's token chunk), the epilogue groups
// that have written their part of the intermediate rows (`ready[unit]`, two per item); the down half (2), whose units
// are the same chunks in the same order, makes its producer wait for the eight arrivals of a unit before it fetches that
// unit's rows.  Every CTA finishes its gate_up items before it starts on down items and nothing in the gate_up half waits
// for another CTA, so with all CTAs resident (grid <= SM count, one CTA per SM) the wait always ends; it is bounded anyway.
// Returns false when this CTA gave up on a wait.
// kGatherX (gate_up on E4M3 weights): the item's token rows are not read from an expert-sorted copy but gathered from token
// order: sorted position p holds token-order row tok_row_base + (perm[p] >> 3) (positions from tok_row_base on are
// token-order rows already: the shared expert).  tm_x32 then is a map with a one-row box over the same buffer and x_scale
// its scales.
template <bool kGateUp, bool kFp4 = false, int kChain = 0, bool kGatherX = false>
__device__ __forceinline__ bool grouped_gemm_body(const CUtensorMap* tm_w, const CUtensorMap* tm_x32,
                                                  const CUtensorMap* tm_x64, const CUtensorMap* tm_x128,
                                                  const float* __restrict__ x_scale, const float* __restrict__ w_scale,
                                                  const uint8_t* __restrict__ w_scale_atoms,
                                                  const int32_t* __restrict__ offsets, uint8_t* __restrict__ h_fp8,
                                                  float* __restrict__ h_scale, float* __restrict__ down,
                                                  float* const* __restrict__ row_ptr, uint32_t num_groups, uint32_t w_tiled,
                                                  uint32_t* status, uint32_t* __restrict__ ready = nullptr,
                                                  uint32_t* tmem_chain = nullptr, const int32_t* __restrict__ perm = nullptr,
                                                  uint32_t tok_row_base = 0) {
  static_assert(!kGatherX || (kGateUp && !kFp4 && kChain == 0), "the gathering producer serves the stand-alone E4M3 gate_up");
  // tmem_chain (chained halves): a CTA may allocate TMEM only until it gives up its permit, so the first half allocates
  // and hands the base address on, the second half frees it
  using C = Cfg<kGateUp, kFp4>;
  static_assert(kChain == 0 || (!kFp4 && C::kNTiles == 4), "the chained halves share units of four work items");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint8_t* scale_base = stage_base + C::kStages * C::kStageBytes;                // 2 slots
  uint8_t* atom_base = scale_base + C::kScaleSlots * C::kScaleSlotBytes;         // [kStages][kATiles] scale atoms (MXFP4)
  uint32_t* red = reinterpret_cast<uint32_t*>(atom_base + C::kStages * C::kScaleStageBytes);       // [2 groups][4 warps][64]
  int* offs = reinterpret_cast<int*>(red + 2 * 4 * C::kColsPerGroup);               // [264]
  int* item_pre = offs + 264;                                                    // [264]
  int4* item_list = reinterpret_cast<int4*>(item_pre + 264);                     // [kItemList]
  uint64_t* bars = reinterpret_cast<uint64_t*>(item_list + C::kItemList);
  uint64_t* full_bar = bars;                       // [kStages]
  uint64_t* empty_bar = bars + C::kStages;         // [kStages]
  uint64_t* tfull_bar = bars + 2 * C::kStages;     // [C::kAccStages]
  uint64_t* tempty_bar = tfull_bar + C::kAccStages;   // [C::kAccStages]
  uint64_t* sfull_bar = tempty_bar + C::kAccStages;   // [kScaleSlots]
  uint64_t* sempty_bar = sfull_bar + C::kScaleSlots;
  uint64_t* hdone_bar = sempty_bar + C::kScaleSlots;  // [4] (chained gate_up half): both epilogue groups have stored an item's rows
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(hdone_bar + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = (int)num_groups;

  // ---- setup: offsets -> smem, item prefix (shared group first), barriers, TMEM
  for (int i = threadIdx.x; i <= groups; i += blockDim.x) offs[i] = offsets[i];
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
    for (int a = 0; a < C::kAccStages; ++a) { mbar_init(smem_u32(&tfull_bar[a]), 1); mbar_init(smem_u32(&tempty_bar[a]), 8); }
    for (int a = 0; a < C::kScaleSlots; ++a) { mbar_init(smem_u32(&sfull_bar[a]), 1); mbar_init(smem_u32(&sempty_bar[a]), 8); }
    for (int a = 0; a < 4; ++a) mbar_init(smem_u32(&hdone_bar[a]), 2);
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
        c = ((m + C::kTokMax - 1) / C::kTokMax) * C::kNTiles;
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
  if (kChain != 2 && warp == 1) tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = kChain == 2 ? *tmem_chain : *tmem_slot;
  if constexpr (kChain == 1) *tmem_chain = tmem_base;
  const uint32_t tmem_scale = tmem_base + (uint32_t)(C::kAccStages * C::kAccCols);   // A scales per tile, then the B scales
  if constexpr (kFp4) {
    // the token rows carry FP32 scales that the promotion step applies: inside the MMA they count as 2^0 (0x7f)
    if (warp >= 2 && warp < 6) tmem_fill4(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(C::kAccStages * C::kAccCols + 4 * C::kATiles), 0x7f7f7f7fu);
    tc_fence_before();
  }
  const int total_items = item_pre[groups];
  // Work items all cost about the same, so the launch is balanced when every participating CTA gets the
  // same count: with R = ceil(items / grid) rounds only ceil(items / R) CTAs take part (e.g. 130 of 148 for
  // 1040 items); the memory system, not the SM count, bounds these kernels.
  const int rounds = (total_items + (int)gridDim.x - 1) / (int)gridDim.x;
  const int stride = rounds > 0 ? (total_items + rounds - 1) / rounds : 1;
  const int first_item = (int)blockIdx.x < stride ? (int)blockIdx.x : total_items;
  // this CTA's first kItemList work items, decoded once for all roles
  for (int n = threadIdx.x; n < C::kItemList; n += blockDim.x) {
    const int item = first_item + n * stride;
    if (item < total_items) {
      const Item w = decode_item<C::kNTiles, C::kSubTiles, C::kTokMax>(item, item_pre, offs, groups);
      item_list[n] = make_int4(w.group, w.ntile, w.row0, w.m_valid);
    }
  }
  __syncthreads();
  auto get_item = [&](int n, int item) -> Item {
    if (n < C::kItemList) { const int4 v = item_list[n]; Item w; w.group = v.x; w.ntile = v.y; w.row0 = v.z; w.m_valid = v.w; return w; }
    return decode_item<C::kNTiles, C::kSubTiles, C::kTokMax>(item, item_pre, offs, groups);
  };

  if (warp == 0) {
    if (kChain == 1 && lane == 1) {
      // =========================== publisher (chained gate_up half) ===========================
      // item n's rows are in memory once both epilogue groups have arrived; release them to the other CTAs' down halves
      uint32_t n_item = 0;
      for (int item = first_item; item < total_items; item += stride, ++n_item) {
        if (!mbar_wait(smem_u32(&hdone_bar[n_item & 3]), (n_item >> 2) & 1, abort_flag)) {
          status[0] = kStatusEpilogueTimeout; *abort_flag = 1; break;
        }
        asm volatile("red.release.gpu.global.add.u32 [%0], 2;" ::"l"(ready + (item >> 2)) : "memory");
      }
    }
    if constexpr (kGatherX) {
      // =========================== TMA producer, token rows gathered (whole warp) ===========================
      // Lanes 0..7 own four rows each of the 32-row token tile: they look up where those sorted positions live in token
      // order once per item and fetch them with one four-row gather per K-block; every lane copies one row of token
      // scales; lane 0 also does the waits, the byte counts and the weight tiles.
      if (lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tm_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tm_x32) : "memory");
      }
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      uint32_t it = 0, n_item = 0;
      bool ok = true;
      for (int item = first_item; ok && item < total_items; item += stride, ++n_item) {
        const Item w = get_item((int)n_item, item);
        auto source_row = [&](int r) {       // rows past the item's end repeat its last row
          const int pos = w.row0 + min(r, w.m_valid - 1);
          return pos >= (int)tok_row_base ? pos : (int)tok_row_base + (__ldg(perm + pos) >> 3);
        };
        int src[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) src[j] = source_row(4 * (lane & 7) + j);
        const int my_scale_row = source_row(lane);
        const int slot = n_item % C::kScaleSlots;
        const uint32_t sbar = smem_u32(&sfull_bar[slot]);
        const uint32_t sdst = smem_u32(scale_base + slot * C::kScaleSlotBytes);
        bool good = true;
        if (lane == 0) {
          good = mbar_wait(smem_u32(&sempty_bar[slot]), ((n_item / C::kScaleSlots) & 1) ^ 1, abort_flag);
          if (good) {
            mbar_expect_tx(sbar, C::kXsBytes + C::kATiles * C::kWsBytes);
            const float* wsrc = w_scale + ((size_t)w.group * C::kSlabTiles + w.ntile) * C::kKBlocks;
            bulk_load(sdst + C::kXsBytes, wsrc, C::kWsBytes, sbar);
            bulk_load(sdst + C::kXsBytes + C::kWsBytes, wsrc + (kInter / kBlock) * C::kKBlocks, C::kWsBytes, sbar);
          } else {
            status[0] = kStatusProducerTimeout; *abort_flag = 1;
          }
        }
        good = __shfl_sync(0xffffffffu, good ? 1 : 0, 0) != 0;
        if (!good) { ok = false; break; }
        bulk_load(sdst + (uint32_t)lane * C::kKBlocks * 4, x_scale + (size_t)my_scale_row * C::kKBlocks, C::kKBlocks * 4, sbar);
        for (int kb = 0; kb < C::kKBlocks; ++kb, ++it) {
          const int s = it % C::kStages;
          const uint32_t bar = smem_u32(&full_bar[s]);
          const uint32_t dst = smem_u32(stage_base + s * C::kStageBytes);
          if (lane == 0) {
            good = mbar_wait(smem_u32(&empty_bar[s]), ((it / C::kStages) & 1) ^ 1, abort_flag);
            if (good) {
              mbar_expect_tx(bar, C::kATiles * kWTileBytes + C::kTokTileBytes);
              int wx, wy0, wy1;
              if (w_tiled) {
                wx = 0;
                wy0 = ((w.group * C::kSlabTiles + w.ntile) * C::kKBlocks + kb) * kTileRows;
                wy1 = wy0 + (kInter / kTileRows) * C::kKBlocks * kTileRows;
              } else {
                wx = kb * kBlock;
                wy0 = w.group * C::kSlabRows + w.ntile * kTileRows;
                wy1 = wy0 + kInter;
              }
              tma_load_2d(dst, tm_w, bar, wx, wy0, pol_w);
              tma_load_2d(dst + kWTileBytes, tm_w, bar, wx, wy1, pol_w);
            } else {
              status[0] = kStatusProducerTimeout; *abort_flag = 1;
            }
          }
          good = __shfl_sync(0xffffffffu, good ? 1 : 0, 0) != 0;      // also orders the lanes' gathers after lane 0's wait
          if (!good) { ok = false; break; }
          if (lane < 8)
            tma_gather4_2d(dst + C::kATiles * kWTileBytes + (uint32_t)lane * 4 * kBlock, tm_x32, bar, kb * kBlock, src[0], src[1], src[2],
                           src[3], pol_x);
        }
      }
    } else
    // =========================== TMA producer ===========================
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tm_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tm_x32) : "memory");
      const uint64_t pol_w = policy_evict_first();     // weights are read once per launch
      const uint64_t pol_x = policy_evict_last();      // token rows are re-read by every tile of the expert
      uint32_t it = 0, n_item = 0;
      bool ok = true;
      for (int item = first_item; ok && item < total_items; item += stride, ++n_item) {
        const Item w = get_item((int)n_item, item);
        if constexpr (kChain == 2) {
          // the unit's intermediate rows and their scales were written by other CTAs' epilogues: wait for all eight
          // epilogue groups, then order the copy engine's reads after what this thread has now observed
          const uint32_t* flag = ready + (item >> 2);
          uint32_t seen = 0, spin = 0;
          for (; spin < kSpinLimit; ++spin) {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
            if (seen >= 8u) break;
            if ((spin & 0xff) == 0xff && *abort_flag != 0) break;
            __nanosleep(64);
          }
          if (seen < 8u) { status[0] = kStatusProducerTimeout; *abort_flag = 1; ok = false; break; }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        const int box = (C::kTokMax == 32 || w.m_valid <= 32) ? 32 : 64;
        const CUtensorMap* tm_x = box == 32 ? tm_x32 : tm_x64;
        const uint32_t bytes = C::kStageTiles * C::kWTxBytes + C::kKbPerLoad * box * kBlock + C::kScaleStageBytes;
        // scales of this item: token-row scales [128][KB] and the tile's weight scales
        {
          const int slot = n_item % C::kScaleSlots;
          if (!mbar_wait(smem_u32(&sempty_bar[slot]), ((n_item / C::kScaleSlots) & 1) ^ 1, abort_flag)) {
            status[0] = kStatusProducerTimeout; *abort_flag = 1; ok = false; break;
          }
          const uint32_t sbar = smem_u32(&sfull_bar[slot]);
          const uint32_t sdst = smem_u32(scale_base + slot * C::kScaleSlotBytes);
          mbar_expect_tx(sbar, C::kXsBytes + (kFp4 ? 0 : C::kATiles * C::kSubTiles * C::kWsBytes));
          bulk_load(sdst, x_scale + (size_t)w.row0 * C::kKBlocks, C::kXsBytes, sbar);
          if constexpr (!kFp4) {
            if (kGateUp) {     // gate tile ntile, up tile 4 + ntile
              const float* wsrc = w_scale + ((size_t)w.group * C::kSlabTiles + w.ntile) * C::kKBlocks;
              bulk_load(sdst + C::kXsBytes, wsrc, C::kWsBytes, sbar);
              bulk_load(sdst + C::kXsBytes + C::kWsBytes, wsrc + (kInter / kBlock) * C::kKBlocks, C::kWsBytes, sbar);
            } else {           // tiles 2 * ntile and 2 * ntile + 1: consecutive scale rows
              const float* wsrc = w_scale + ((size_t)w.group * C::kSlabTiles + 2 * w.ntile) * C::kKBlocks;
              bulk_load(sdst + C::kXsBytes, wsrc, C::kSubTiles * 2 * C::kWsBytes, sbar);
            }
          }
        }
        for (int sub = 0; ok && sub < C::kSubTiles; ++sub)
        for (int kb = 0; kb < C::kKBlocks; kb += C::kKbPerLoad, ++it) {
          const int s = it % C::kStages;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / C::kStages) & 1) ^ 1, abort_flag)) {
            status[0] = kStatusProducerTimeout; *abort_flag = 1; ok = false; break;
          }
          const uint32_t bar = smem_u32(&full_bar[s]);
          const uint32_t dst = smem_u32(stage_base + s * C::kStageBytes);
          mbar_expect_tx(bar, bytes);
          if constexpr (kFp4) {
            // one box of 256 code rows = two 8 KiB blocks that the pack step stored next to each other: blocks are
            // ordered (slab, tile pair, K-block, tile of the pair) - W13 pairs a gate tile with its up tile, W2 pairs
            // tiles 2p and 2p + 1; the 512-byte scale atoms follow the same order, so the stage's two are one 1 KiB copy
            const int wy = (((w.group * C::kNTiles * C::kSubTiles + w.ntile + sub) * C::kKBlocks + kb) * 2) * kTileRows;
            tma_load_2d(dst, tm_w, bar, 0, wy, pol_w);
#pragma unroll
            for (int j = 0; j < C::kKbPerLoad; ++j)
              tma_load_2d(dst + C::kStageTiles * kWTileBytes + j * C::kTokTileBytes, tm_x, bar, (kb + j) * kBlock, w.row0, pol_x);
            bulk_load(smem_u32(atom_base + s * C::kScaleStageBytes), w_scale_atoms + (size_t)wy * 4, C::kScaleStageBytes, bar);
            continue;
          }
          // the stage's two weight tiles: gate tile ntile and up tile 4 + ntile | W2 tiles 2 ntile and 2 ntile + 1
          const int tile0 = kGateUp ? w.ntile + sub : 2 * (w.ntile + sub);
          const int tile_step = kGateUp ? kInter / kTileRows : 1;
          int wx, wy0, wy1;
          if (w_tiled) {   // one contiguous 16 KiB block per (slab tile, K-block)
            wx = 0;
            wy0 = ((w.group * C::kSlabTiles + tile0) * C::kKBlocks + kb) * kTileRows;
            wy1 = wy0 + tile_step * C::kKBlocks * kTileRows;
          } else {
            wx = kb * kBlock;
            wy0 = w.group * C::kSlabRows + tile0 * kTileRows;
            wy1 = wy0 + tile_step * kTileRows;
          }
          tma_load_2d(dst, tm_w, bar, wx, wy0, pol_w);
          tma_load_2d(dst + kWTileBytes, tm_w, bar, wx, wy1, pol_w);
          tma_load_2d(dst + C::kATiles * kWTileBytes, tm_x, bar, kb * kBlock, w.row0, pol_x);
        }
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    if (lane == 0) {
      uint32_t it = 0, jt = 0, n_item = 0;
      bool ok = true;
      for (int item = first_item; ok && item < total_items; item += stride, ++n_item) {
        const Item w = get_item((int)n_item, item);
        const uint32_t n_mma = (uint32_t)((w.m_valid + 15) & ~15);
        const uint32_t idesc = make_idesc(n_mma);
        for (int step = 0; ok && step < C::kSubTiles * C::kKBlocks / C::kKbPerStep; ++step, ++jt) {
          const int a = jt % C::kAccStages;
          if (!mbar_wait(smem_u32(&tempty_bar[a]), ((jt / C::kAccStages) & 1) ^ 1, abort_flag)) {
            status[0] = kStatusMmaTimeout; *abort_flag = 1; ok = false; break;
          }
#pragma unroll 1
          for (int q = 0; q < C::kKbPerStep; q += C::kKbPerLoad, ++it) {
            const int s = it % C::kStages;
            if (!mbar_wait(smem_u32(&full_bar[s]), (it / C::kStages) & 1, abort_flag)) {
              status[0] = kStatusMmaTimeout; *abort_flag = 1; ok = false; break;
            }
            tc_fence_after();
            const uint32_t sa = smem_u32(stage_base + s * C::kStageBytes);
#pragma unroll
            for (int j = 0; j < C::kKbPerLoad; ++j) {      // K-blocks held by this stage
              const uint32_t sw = sa + (uint32_t)(j * C::kATiles * kWTileBytes);            // their weight tiles
              const uint64_t bdesc = make_smem_desc(sa + C::kStageTiles * kWTileBytes + j * C::kTokTileBytes);
              const uint32_t d0 = tmem_base + (uint32_t)(a * C::kAccCols + (q + j) * C::kATiles * C::kTokMax);
              // the two tiles accumulate into different TMEM columns: alternate them so that consecutive
              // MMAs never depend on each other
              if constexpr (kFp4) {
                // scale atoms -> TMEM; the tensor-core pipe runs copies and MMAs of one thread in issue order, so the
                // MMAs of the previous K-block have read these columns before they are overwritten
#pragma unroll
                for (int tile = 0; tile < C::kATiles; ++tile)
                  tmem_cp_32x128b_warpx4(tmem_scale + (uint32_t)(4 * tile),
                                         make_scale_desc(smem_u32(atom_base + s * C::kScaleStageBytes + (j * C::kATiles + tile) * C::kScaleAtomBytes)));
#pragma unroll
                for (int k = 0; k < kBlock / 32; ++k) {
#pragma unroll
                  for (int tile = 0; tile < C::kATiles; ++tile)
                    umma_mxf8f6f4(d0 + (uint32_t)(tile * C::kTokMax), make_smem_desc(sw + tile * kWTileBytes) + 2 * k, bdesc + 2 * k,
                                  make_idesc_mxfp4(n_mma, (uint32_t)k), (tmem_scale + (uint32_t)(4 * tile)) | ((uint32_t)k << 30),
                                  tmem_scale + (uint32_t)(4 * C::kATiles), k > 0);
                }
              } else {
#pragma unroll
                for (int k = 0; k < kBlock / 32; ++k) {
#pragma unroll
                  for (int tile = 0; tile < C::kATiles; ++tile)
                    umma_f8(d0 + (uint32_t)(tile * C::kTokMax), make_smem_desc(sw + tile * kWTileBytes) + 2 * k, bdesc + 2 * k, idesc, k > 0);
                }
              }
            }
            umma_commit(smem_u32(&empty_bar[s]));
          }
          if (ok) umma_commit(smem_u32(&tfull_bar[a]));
        }
      }
    }
  } else {
    // =========================== promotion + epilogue (2 groups x 128 threads) ===========================
    const int grp = (warp - 2) >> 2;         // the two groups split an item's token columns in halves
    const int gw = (warp - 2) & 3;           // warp inside the group
    const int quad = warp & 3;               // TMEM lane quadrant this warp may read
    const int r = quad * 32 + lane;          // weight row inside the tile == TMEM lane
    uint32_t jt = 0, n_item = 0;
    bool ok = true;
    for (int item = first_item; item < total_items; item += stride, ++n_item) {
      const Item w = get_item((int)n_item, item);
      const int n_mma = (w.m_valid + 15) & ~15;
      const int col_base = grp * (n_mma >> 1);   // this group's first column; it owns n_mma/2 columns
      const int nsl = n_mma >> 4;                // ... in 8-column slices: 1..4
      const int slot = n_item % C::kScaleSlots;
      const float* xs_tile = reinterpret_cast<const float*>(scale_base + slot * C::kScaleSlotBytes);
      const float* ws_tile = xs_tile + C::kTokMax * C::kKBlocks;
      if (ok && !mbar_wait(smem_u32(&sfull_bar[slot]), (n_item / C::kScaleSlots) & 1, abort_flag)) {
        status[0] = kStatusEpilogueTimeout; *abort_flag = 1; ok = false;
      }
      const int my_cols = min(n_mma >> 1, w.m_valid - col_base);         // columns holding real rows; may be <= 0
#pragma unroll 1
      for (int sub = 0; sub < C::kSubTiles; ++sub) {
      const int ntile = w.ntile + sub;
      float acc[C::kATiles][C::kColsPerGroup];
#pragma unroll
      for (int tile = 0; tile < C::kATiles; ++tile)
#pragma unroll
        for (int c = 0; c < C::kColsPerGroup; ++c) acc[tile][c] = 0.0f;
      for (int step = 0; step < C::kKBlocks / C::kKbPerStep; ++step, ++jt) {
        const int a = jt % C::kAccStages;
        if (ok && !mbar_wait(smem_u32(&tfull_bar[a]), (jt / C::kAccStages) & 1, abort_flag)) {
          status[0] = kStatusEpilogueTimeout; *abort_flag = 1; ok = false;
        }
        if (!ok) continue;
        tc_fence_after();
#pragma unroll
        for (int q = 0; q < C::kKbPerStep; ++q) {
        const int kb = step * C::kKbPerStep + q;
        const uint32_t tbase = tmem_base + ((uint32_t)(quad * 32) << 16) +
                               (uint32_t)(a * C::kAccCols + q * C::kATiles * C::kTokMax + col_base);
        // all TMEM loads of this K-block are issued before the single wait
        uint32_t v[C::kATiles][C::kSlices][8];
#pragma unroll
        for (int sl = 0; sl < C::kSlices; ++sl)
          if (sl < nsl) {
#pragma unroll
            for (int tile = 0; tile < C::kATiles; ++tile) tmem_ld8_nowait(tbase + (uint32_t)(tile * C::kTokMax + sl * 8), v[tile][sl]);
          }
        tmem_ld_wait();
        if (q == C::kKbPerStep - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[a]));   // the partials now live in registers
        }
        float ws[C::kATiles];   // MXFP4: the weight scales were applied inside the MMA
#pragma unroll
        for (int tile = 0; tile < C::kATiles; ++tile) ws[tile] = kFp4 ? 1.0f : ws_tile[((kGateUp ? sub : 2 * sub) + tile) * C::kKBlocks + kb];
#pragma unroll
        for (int sl = 0; sl < C::kSlices; ++sl)
          if (sl < nsl) {
            const float* xs = xs_tile + (col_base + sl * 8) * C::kKBlocks + kb;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float x = xs[i * C::kKBlocks];
#pragma unroll
              for (int tile = 0; tile < C::kATiles; ++tile)
                acc[tile][sl * 8 + i] = fmaf(__uint_as_float(v[tile][sl][i]), __fmul_rn(x, ws[tile]), acc[tile][sl * 8 + i]);
            }
          }
        }   // K-block of the step
      }
      if (sub == C::kSubTiles - 1) {
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sempty_bar[slot]));   // the scale tiles were last read above
      }
      // ---- tile epilogue (columns of this group that hold real rows), eight columns at a time
      if constexpr (kGateUp) {
        uint32_t* my_red = red + (grp * 4 + gw) * C::kColsPerGroup;
#pragma unroll
        for (int c0 = 0; c0 < C::kColsPerGroup; c0 += 8) {
          if (c0 < my_cols) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {     // independent chains first ...
              const float g = acc[0][c0 + j];
              const float silu = __fdividef(g, 1.0f + __expf(-g));
              acc[0][c0 + j] = bf16_round(__fmul_rn(silu, acc[C::kATiles - 1][c0 + j]));
            }
            uint32_t mine = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {     // ... then the warp reductions back to back
              const uint32_t m = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(acc[0][c0 + j])));
              if (lane == j) mine = m;
            }
            if (lane < 8) my_red[c0 + lane] = mine;
          }
        }
        group_barrier(grp);
        const uint32_t* g_red = red + grp * 4 * C::kColsPerGroup;
#pragma unroll
        for (int c0 = 0; c0 < C::kColsPerGroup; c0 += 8) {
          if (c0 < my_cols) {
            uint8_t q[8];
            float scale[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int c = c0 + j;
              const uint32_t m = max(max(g_red[c], g_red[C::kColsPerGroup + c]), max(g_red[2 * C::kColsPerGroup + c], g_red[3 * C::kColsPerGroup + c]));
              scale[j] = fmaxf(__uint_as_float(m), amax_floor()) * inv448();
              q[j] = f32_to_e4m3(acc[0][c] * rcp_newton(scale[j]));
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (c0 + j < my_cols) {
                const size_t row = (size_t)(w.row0 + col_base + c0 + j);
                h_fp8[row * kInter + ntile * kTileRows + r] = q[j];
                if (r == 0) h_scale[row * kInterBlocks + ntile] = scale[j];
              }
            }
          }
        }
        group_barrier(grp);   // red[] is free for the next item
        if constexpr (kChain == 1) {
          // every thread of the group has issued its stores of this item's rows before the barrier above; the publication
          // (a device-wide release) is left to an idle lane of warp 0 so that it does not hold up the next item's hand-offs
          if (gw == 0 && lane == 0) mbar_arrive(smem_u32(&hdone_bar[n_item & 3]));
        }
      } else {
        // row_ptr (expert parallelism): each output row goes to its own destination, possibly a peer GPU's memory
#pragma unroll
        for (int c = 0; c < C::kColsPerGroup; ++c)
          if (c < my_cols) {
            const int row = w.row0 + col_base + c;
            float* dst = row_ptr != nullptr ? row_ptr[row] : down + (size_t)row * kHidden;
#pragma unroll
            for (int tile = 0; tile < C::kATiles; ++tile) dst[(ntile * C::kATiles + tile) * kTileRows + r] = acc[tile][c];
          }
      }
      }   // sub tile
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  const bool gave_up = *abort_flag != 0;
  if (gave_up) __nanosleep(200000);   // let copies already in flight land before the CTA exits
  if (warp == 1 && (kChain != 1 || gave_up)) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if constexpr (kChain == 1) {
    // the shared memory is about to be carved up again: retire this half's barriers first
    if (threadIdx.x == 0)
      for (int b = 0; b < 2 * C::kStages + 2 * C::kAccStages + 2 * C::kScaleSlots + 4; ++b)
        asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(&bars[b])) : "memory");
    __syncthreads();
  }
  return !gave_up;
}

extern "C" __global__ void __launch_bounds__(kGemmThreads, 1)
netra_moe_gate_up_umma_sm100(const __grid_constant__ CUtensorMap tm_w13, const __grid_constant__ CUtensorMap tm_a32,
                             const __grid_constant__ CUtensorMap tm_a64, const __grid_constant__ CUtensorMap tm_a128,
                             const float* a_scale, const float* w13_scale, const int32_t* offsets, uint8_t* h_fp8,
                             float* h_scale, uint32_t num_groups, uint32_t w_tiled, uint32_t* status) {
  grouped_gemm_body<true>(&tm_w13, &tm_a32, &tm_a64, &tm_a128, a_scale, w13_scale, nullptr, offsets, h_fp8, h_scale, nullptr, nullptr,
                          num_groups, w_tiled, status);
}

extern "C" __global__ void __launch_bounds__(kGemmThreads, 1)
netra_moe_down_umma_sm100(const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_h32,
                          const __grid_constant__ CUtensorMap tm_h64, const __grid_constant__ CUtensorMap tm_h128,
                          const float* h_scale, const float* w2_scale, const int32_t* offsets, float* down,
                          uint32_t num_groups, uint32_t w_tiled, uint32_t* status) {
  grouped_gemm_body<false>(&tm_w2, &tm_h32, &tm_h64, &tm_h128, h_scale, w2_scale, nullptr, offsets, nullptr, nullptr, down, nullptr,
                           num_groups, w_tiled, status);
}

// The same two projections on MXFP4 expert weights (E2M1 codes with one UE8M0 scale per 32 K-elements; semantics of
// kernels/gfx1151/mxfp4/prefill/mxfp4_prefill_gate_wmma_gfx1151.s:3-8 and mxfp4_prefill_down_wmma_gfx1151.s:3-5, call
// sequence of runtime/gfx1151/mxfp4/decode/runtime.h:10-47) through tcgen05.mma.kind::mxf8f6f4.block_scale: the
// weight tiles stay 4-bit in memory (tm_w*: tiles of 128 rows x 64 bytes written by netra_moe_mxfp4_pack_sm100) and
// their scales reach the tensor core through TMEM; the token rows are E4M3 with their FP32 per-128 scales applied
// in the promotion step, as in the FP8 kernels above.
extern "C" __global__ void __launch_bounds__(kGemmThreads, 1)
netra_moe_gate_up_mxfp4_umma_sm100(const __grid_constant__ CUtensorMap tm_w13, const __grid_constant__ CUtensorMap tm_a32,
                              const __grid_constant__ CUtensorMap tm_a64, const __grid_constant__ CUtensorMap tm_a128,
                              const float* a_scale, const uint8_t* w13_scale_atoms, const int32_t* offsets, uint8_t* h_fp8,
                              float* h_scale, uint32_t num_groups, uint32_t* status) {
  grouped_gemm_body<true, true>(&tm_w13, &tm_a32, &tm_a64, &tm_a128, a_scale, nullptr, w13_scale_atoms, offsets, h_fp8, h_scale,
                                nullptr, nullptr, num_groups, 1u, status);
}

extern "C" __global__ void __launch_bounds__(kGemmThreads, 1)
netra_moe_down_mxfp4_umma_sm100(const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_h32,
                           const __grid_constant__ CUtensorMap tm_h64, const __grid_constant__ CUtensorMap tm_h128,
                           const float* h_scale, const uint8_t* w2_scale_atoms, const int32_t* offsets, float* down,
                           uint32_t num_groups, uint32_t* status) {
  grouped_gemm_body<false, true>(&tm_w2, &tm_h32, &tm_h64, &tm_h128, h_scale, nullptr, w2_scale_atoms, offsets, nullptr, nullptr, down,
                                 nullptr, num_groups, 1u, status);
}

// Repack row-major slabs [groups * slab_rows, k_bytes] into tiles: destination row
// ((slab_tile * kblocks + kb) * 128 + r) holds bytes [kb*128, +128) of source row slab_tile*128 + r.
// One thread moves 16 bytes.  grid = total_bytes / 16 / 256.
extern "C" __global__ void __launch_bounds__(256)
netra_moe_repack_tiles_sm100(uint4* __restrict__ dst, const uint4* __restrict__ src, uint32_t total_rows, uint32_t k_bytes) {
  const uint32_t kblocks = k_bytes / kBlock;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;      // 16-byte chunk of the destination
  const size_t total = (size_t)total_rows * k_bytes / 16;
  if (idx >= total) return;
  const uint32_t chunk = idx & 7;                 // 16-byte chunk inside the 128-byte row
  const size_t drow = idx >> 3;
  const uint32_t r = drow % kTileRows;
  const size_t t = drow / kTileRows;              // slab_tile * kblocks + kb
  const uint32_t kb = t % kblocks;
  const size_t slab_tile = t / kblocks;
  const size_t srow = slab_tile * kTileRows + r;
  dst[idx] = src[(srow * k_bytes + (size_t)kb * kBlock) / 16 + chunk];
}

// Block scales stored as BF16 in a checkpoint -> the FP32 scales the kernels read (exact widening).  grid ceil(count/256).
extern "C" __global__ void __launch_bounds__(256)
netra_moe_widen_scales_bf16_sm100(float* __restrict__ dst, const uint16_t* __restrict__ src, uint64_t count) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) dst[i] = bf16_bits_to_f32(src[i]);
}

// Both projections in one launch (decode sizes, E4M3 weights): see kChain above.  ready: one zeroed word per unit
// (at most kReadyWords); zeroed by netra_moe_gather_rows_sm100, the launch before this one.
constexpr int kReadyWords = 1024;
extern "C" __global__ void __launch_bounds__(kGemmThreads, 1)
netra_moe_gate_up_down_umma_sm100(const __grid_constant__ CUtensorMap tm_w13, const __grid_constant__ CUtensorMap tm_a32,
                                  const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_h32,
                                  const float* a_scale, const float* w13_scale, const float* w2_scale, const int32_t* offsets,
                                  uint8_t* h_fp8, float* h_scale, float* down, uint32_t num_groups, uint32_t w_tiled, uint32_t* ready,
                                  uint32_t* status) {
  uint32_t tmem = 0;
  if (!grouped_gemm_body<true, false, 1>(&tm_w13, &tm_a32, &tm_a32, &tm_a32, a_scale, w13_scale, nullptr, offsets, h_fp8, h_scale, nullptr,
                                         nullptr, num_groups, w_tiled, status, ready, &tmem))
    return;
  grouped_gemm_body<false, false, 2>(&tm_w2, &tm_h32, &tm_h32, &tm_h32, h_scale, w2_scale, nullptr, offsets, nullptr, nullptr, down, nullptr,
                                     num_groups, w_tiled, status + 1, ready, &tmem);
}

// gate_up with the token rows gathered from token order (no expert-sorted copy of the quantised rows is made for it):
// tm_tok1 is a one-row-box map over the quantised-row buffer, tok_scale its scales [rows, 16], perm the sorted
// position -> pair index table, tok_row_base the first token-order row of that buffer.
extern "C" __global__ void __launch_bounds__(kGemmThreads, 1)
netra_moe_gate_up_umma_gather_sm100(const __grid_constant__ CUtensorMap tm_w13, const __grid_constant__ CUtensorMap tm_tok1,
                                    const float* tok_scale, const float* w13_scale, const int32_t* offsets, const int32_t* perm,
                                    uint8_t* h_fp8, float* h_scale, uint32_t num_groups, uint32_t w_tiled, uint32_t tok_row_base,
                                    uint32_t* status) {
  grouped_gemm_body<true, false, 0, true>(&tm_w13, &tm_tok1, &tm_tok1, &tm_tok1, tok_scale, w13_scale, nullptr, offsets, h_fp8, h_scale,
                                          nullptr, nullptr, num_groups, w_tiled, status, nullptr, nullptr, perm, tok_row_base);
}

int gate_up_down_smem_bytes() { return Cfg<true>::kSmemBytes > Cfg<false>::kSmemBytes ? Cfg<true>::kSmemBytes : Cfg<false>::kSmemBytes; }
int gate_up_smem_bytes() { return Cfg<true>::kSmemBytes; }
int down_smem_bytes() { return Cfg<false>::kSmemBytes; }
int gate_up_mxfp4_smem_bytes() { return Cfg<true, true>::kSmemBytes; }
int down_mxfp4_smem_bytes() { return Cfg<false, true>::kSmemBytes; }

}  // namespace netra

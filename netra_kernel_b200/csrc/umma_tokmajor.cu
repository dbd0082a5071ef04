// Token-major block-scaled FP8 grouped GEMMs for experts with many rows (prefill, or the blocks of
// an expert-parallel rank): 128 token rows are the MMA M dimension and 256 weight rows the MMA N
// dimension, so one tcgen05.mma does four times the work of the 64-column swap-AB form used for
// decode (umma_kernels.cu) and the tensor pipe, not the per-instruction issue cost, sets the pace.
//
//   gate_up: item = expert x 128 token rows x 128 intermediate channels; the B operand stacks the
//            channel tile's 128 gate rows and 128 up rows of W13 (two TMA boxes, adjacent in shared
//            memory, one N = 256 descriptor).  A thread of the epilogue owns one token row (TMEM lane):
//            gate and up of a channel sit in the same thread, so SiLU*up, the row's amax over the 128
//            channels (exactly one quantisation group) and the FP8 requantisation need no shuffles.
//   down:    item = expert x 128 token rows x 256 output columns (two W2 tiles), K = 512, FP32 rows
//            written to the sorted row space (or to per-row destinations, see row_ptr).
// Same numerics as the swap-AB kernels (and the same reference order,
// kernels/gfx950/templates/moe/prefill/fused_splitk2/gate_up.inc:275-300): per 128-wide K-block the raw FP8
// partial sums leave TMEM and are promoted as acc = fma(part, a_scale[row,kb] * w_scale[tile,kb], acc).
//
// 384 threads: warp 0 = TMA producer, warps 1-2 = MMA issuers (alternate K-blocks; warp 1 owns TMEM), warp 3 idle, warps 4-11 =
// two epilogue warpgroups that split the 256 accumulator columns (TMEM lane quadrant = warp % 4).
// Registers are re-balanced with setmaxnreg: 40 for the first warpgroup, 232 for the epilogue.
// Every mbarrier wait is bounded; on expiry the CTA records a code in status[] and drains.
#include "common.cuh"

namespace netra {

constexpr int kTmThreads = 384;
// Register re-balancing.  setmaxnreg.inc waits, without any bound, until the CTA's pool holds the registers it
// asks for, and the pool only ever receives what setmaxnreg.dec released: the two epilogue warpgroups can be
// served only if 128 * (launch - low) >= 2 * 128 * (high - launch).  (A 640-thread variant with four epilogue
// warpgroups that broke this rule never left its first instruction.)  The launch allocation of a 384-thread
// kernel is 168 registers per thread (65,536 / 384, rounded down to a multiple of 8); the host refuses to launch
// these kernels if the built code reports anything else.
constexpr int kTmRegsLaunch = 168;
constexpr int kTmRegsLow = 40;
constexpr int kTmRegsHigh = 232;
constexpr int kTmEpiGroups = 2;
static_assert(128 * (kTmRegsLaunch - kTmRegsLow) >= kTmEpiGroups * 128 * (kTmRegsHigh - kTmRegsLaunch),
              "the epilogue warpgroups would wait forever for registers nobody releases");

// one 32-byte store (a full sector) of eight consecutive floats; p is 32-byte aligned
__device__ __forceinline__ void st_global_v8(float* p, const float* v) {
  asm volatile("st.global.v8.f32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]),
               "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]) : "memory");
}

__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t r[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}

// ask the L2 for a TMA box ahead of the load that will need it (no shared memory is reserved)
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"((uint64_t)map), "r"(x), "r"(y) : "memory");
}

// barrier among the 256 epilogue threads
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 3, 256;" ::: "memory"); }

// kF16Out (down only): the output rows are FP16 partials staged in shared memory and written with one bulk copy per row
// kFp4: the weight rows are MXFP4 (E2M1 codes + one UE8M0 scale per 32 along K) multiplied by
//   tcgen05.mma.kind::mxf8f6f4.block_scale; the two weight tiles of a K-block are one 256-row box of code blocks that the
//   pack step stored next to each other, and their two 512-byte scale atoms one 1 KiB copy.  The scales take TMEM columns
//   (4 for the token rows' unit scales, 8 for the 256 weight rows), which leaves room for one 256-column accumulator
//   stage instead of two: the MMAs of a K-block start when the previous K-block's partial sums have left TMEM.
template <bool kGateUp, bool kF16Out = false, bool kFp4 = false>
struct TmCfg {
  static constexpr int kTokTile = 128;                                  // token rows per item (UMMA M)
  static constexpr int kLanes = kTokTile;
  static constexpr int kKBlocks = kGateUp ? kHiddenBlocks : kInterBlocks;   // 16 | 4
  static constexpr int kNTiles = kGateUp ? kInter / kTileRows : kHidden / (2 * kTileRows);   // items per slab and token tile: 4 | 8
  static constexpr int kSlabTiles = kGateUp ? 2 * kInter / kTileRows : kHidden / kTileRows;  // 8 | 16
  static constexpr int kSlabRows = kGateUp ? 2 * kInter : kHidden;
  static constexpr int kStages = kF16Out ? 3 : 4;                       // the FP16 staging rows take the fourth stage's room
  static constexpr int kPrefetch = 4;                                   // K-blocks between an L2 prefetch and its load (kStages..kKBlocks)
  static constexpr int kStageBytes = kTokTile * kBlock + 2 * kWTileBytes;   // 48 KiB: tokens, weight tile 0, weight tile 1
  static constexpr int kAccCols = 256;
  static constexpr int kAccStages = kFp4 ? 1 : 2;
  static constexpr int kScaleCol = kAccStages * kAccCols;                   // MXFP4: token-row scales, then weight-row scales
  static constexpr int kWTxBytes = kFp4 ? kWTileBytes / 2 : kWTileBytes;    // bytes one weight-tile copy reports
  static constexpr int kAtomStageBytes = kFp4 ? 1024 : 0;                   // the two tiles' scale atoms
  static constexpr int kTmemCols = 512;
  static constexpr int kXsBytes = kTokTile * kKBlocks * 4;                  // 8 KiB | 2 KiB
  static constexpr int kWsBytes = kKBlocks * 4;                             // per weight tile
  static constexpr int kScaleSlots = 2;
  static constexpr int kScaleSlotBytes = kXsBytes + 128;
  static constexpr int kItemList = 256;
  static constexpr int kEpiGroups = 2;                                      // epilogue warpgroups
  // FP16 output staging: one tile of 128 rows x 128 halves per epilogue warpgroup, rows 256 bytes apart; the 16-byte
  // chunks of a row are permuted (chunk j sits at j ^ (row & 15)), which keeps the 16-byte shared-memory stores of a
  // quarter warp on different banks and is the layout the rows keep in global memory
  static constexpr int kOutRowBytes = 256;
  static constexpr int kOutStageBytes = kF16Out ? kEpiGroups * kLanes * kOutRowBytes : 0;
  static constexpr int kSmemBytes = 1024 + kStages * (kStageBytes + kAtomStageBytes) + kScaleSlots * kScaleSlotBytes + kOutStageBytes +
                                    2 * kEpiGroups * kLanes * 4 + 2 * 264 * 4 + kItemList * 16 + 512;
  static_assert(!(kFp4 && kF16Out), "the MXFP4 down projection writes FP32 rows");
  static_assert(kSmemBytes <= 232448, "exceeds the shared memory of one SM");
};

// kind::mxf8f6f4.block_scale, A = E4M3 token rows (unit scales), B = E2M1 weight rows, N = 256, M = 128, both K-major;
// b_scale_byte selects the byte of the weight-scale columns that belongs to this instruction's 32-element K-group.
__device__ __forceinline__ uint32_t make_idesc_mxfp4_b(uint32_t b_scale_byte) {
  return (b_scale_byte << 4) | (5u << 10) | ((256u >> 3) << 17) | (1u << 23) | ((uint32_t)(128 >> 4) << 24);
}

// Where the FP16 partial rows of a block go when they are not kept in this GPU's panels (expert parallelism): block row r
// belongs to sorted row row_dst[r].y of rank row_dst[r].x (x < 0: nowhere), whose panels start at base[x] and hold
// nine rows per token of that rank (tokens_of_rank[x * tokens_pitch]).
struct F16RowReturn {
  const int2* row_dst;
  const int32_t* tokens_of_rank;
  uint32_t tokens_pitch;
  uint8_t* base[16];
};

// kGatherX (gate_up only): the item's token rows are not read from an expert-sorted copy but gathered from token order:
// sorted position p holds token-order row tok_row_base + (perm[p] >> 3) (positions from tok_row_base on are token-order
// rows already: the shared expert).  tm_x128 then is a map with a one-row box over the same buffer, x_scale its scales.
template <bool kGateUp, bool kF16Out = false, bool kGatherX = false, bool kFp4 = false>
__device__ __forceinline__ void tokmajor_gemm_body(const CUtensorMap* tm_w, const CUtensorMap* tm_x128,
                                                   const float* __restrict__ x_scale, const float* __restrict__ w_scale,
                                                   const int32_t* __restrict__ offsets, uint8_t* __restrict__ h_fp8,
                                                   float* __restrict__ h_scale, float* __restrict__ down,
                                                   float* const* __restrict__ row_ptr, uint32_t num_groups, uint32_t w_tiled,
                                                   uint32_t* status, const int32_t* __restrict__ perm = nullptr, uint32_t tok_row_base = 0,
                                                   const F16RowReturn* ret = nullptr) {
  static_assert(!(kGateUp && kF16Out), "FP16 partial rows are an output format of the down projection");
  static_assert(kGateUp || !kGatherX, "only the gate_up projection reads token rows");
  using C = TmCfg<kGateUp, kF16Out, kFp4>;
  static_assert(!kGatherX || C::kTokTile == 128, "a warp of 32 lanes gathers 4 rows each");
  static_assert(!(kGatherX && kFp4), "the gathering producer exists for E4M3 weights only");
  // MXFP4: w_scale points at the scale atoms (bytes), in the order of the code blocks
  const uint8_t* w_scale_atoms = reinterpret_cast<const uint8_t*>(w_scale);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* stage_base = smem;
  uint8_t* scale_base = stage_base + C::kStages * C::kStageBytes;
  uint8_t* atom_base = scale_base + C::kScaleSlots * C::kScaleSlotBytes;                            // [kStages][2 atoms] (MXFP4 only)
  uint8_t* out_stage = atom_base + C::kStages * C::kAtomStageBytes;                                 // [2 groups][128 rows][272 B] (FP16 output only)
  uint32_t* red = reinterpret_cast<uint32_t*>(out_stage + C::kOutStageBytes);                       // [2 parities][2 groups][128 rows]
  int* offs = reinterpret_cast<int*>(red + 2 * C::kEpiGroups * C::kLanes);                    // [264]
  int* item_pre = offs + 264;                                                     // [264]
  int4* item_list = reinterpret_cast<int4*>(item_pre + 264);                      // [kItemList]
  uint64_t* bars = reinterpret_cast<uint64_t*>(item_list + C::kItemList);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + C::kStages;
  uint64_t* tfull_bar = bars + 2 * C::kStages;
  uint64_t* tempty_bar = tfull_bar + C::kAccStages;
  uint64_t* sfull_bar = tempty_bar + C::kAccStages;
  uint64_t* sempty_bar = sfull_bar + C::kScaleSlots;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sempty_bar + C::kScaleSlots);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = (int)num_groups;

  for (int i = threadIdx.x; i <= groups; i += blockDim.x) offs[i] = offsets[i];
  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
    for (int a = 0; a < C::kAccStages; ++a) { mbar_init(smem_u32(&tfull_bar[a]), 1); mbar_init(smem_u32(&tempty_bar[a]), 4 * C::kEpiGroups); }
    for (int a = 0; a < C::kScaleSlots; ++a) { mbar_init(smem_u32(&sfull_bar[a]), 1); mbar_init(smem_u32(&sempty_bar[a]), 4 * C::kEpiGroups); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    // item prefix over the schedule order (slot 0 = last group, slot i = group i - 1); a lane owns 9 slots
    int cnt[9], sum = 0;
#pragma unroll
    for (int j = 0; j < 9; ++j) {
      const int idx = lane * 9 + j;
      int c = 0;
      if (idx < groups) {
        const int g = idx == 0 ? groups - 1 : idx - 1;
        const int m = offs[g + 1] - offs[g];
        c = ((m + C::kTokTile - 1) / C::kTokTile) * C::kNTiles;
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
  const uint32_t tmem_scale = tmem_base + (uint32_t)C::kScaleCol;
  if constexpr (kFp4) {
    // the token rows carry FP32 scales that the promotion step applies: inside the MMA they count as 2^0 (0x7f)
    if (warp >= 4 && warp < 8) tmem_fill4(tmem_scale + ((uint32_t)((warp & 3) * 32) << 16), 0x7f7f7f7fu);
    tc_fence_before();
  }
  const int total_items = item_pre[groups];
  const int rounds = (total_items + (int)gridDim.x - 1) / (int)gridDim.x;
  const int stride = rounds > 0 ? (total_items + rounds - 1) / rounds : 1;
  const int first_item = (int)blockIdx.x < stride ? (int)blockIdx.x : total_items;
  for (int n = threadIdx.x; n < C::kItemList; n += blockDim.x) {
    const int item = first_item + n * stride;
    if (item < total_items) {
      const Item w = decode_item<C::kNTiles, 1, C::kTokTile>(item, item_pre, offs, groups);
      item_list[n] = make_int4(w.group, w.ntile, w.row0, w.m_valid);
    }
  }
  __syncthreads();
  auto get_item = [&](int n, int item) -> Item {
    if (n < C::kItemList) { const int4 v = item_list[n]; Item w; w.group = v.x; w.ntile = v.y; w.row0 = v.z; w.m_valid = v.w; return w; }
    return decode_item<C::kNTiles, 1, C::kTokTile>(item, item_pre, offs, groups);
  };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kTmRegsLow));
    if (kGatherX && warp == 0) {
      // =========================== TMA producer, token rows gathered (whole warp) ===========================
      // Lane l owns rows 4l .. 4l+3 of the 128-row tile: it looks up where those sorted positions live in token order once
      // per item and fetches them with one four-row gather per K-block (and their scale rows with four small bulk copies);
      // lane 0 also does the waits, the byte counts and the weight tiles.
      if (lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tm_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tm_x128) : "memory");
      }
      const uint64_t pol_w = policy_evict_last();
      const uint64_t pol_x = policy_evict_last();
      uint32_t it = 0, n_item = 0;
      bool ok = true;
      for (int item = first_item; ok && item < total_items; item += stride, ++n_item) {
        const Item w = get_item((int)n_item, item);
        int src[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int pos = w.row0 + min(4 * lane + j, w.m_valid - 1);       // rows past the item's end repeat its last row
          src[j] = pos >= (int)tok_row_base ? pos : (int)tok_row_base + (__ldg(perm + pos) >> 3);
        }
        const int slot = n_item % C::kScaleSlots;
        const uint32_t sbar = smem_u32(&sfull_bar[slot]);
        const uint32_t sdst = smem_u32(scale_base + slot * C::kScaleSlotBytes);
        bool good = true;
        if (lane == 0) {
          good = mbar_wait(smem_u32(&sempty_bar[slot]), ((n_item / C::kScaleSlots) & 1) ^ 1, abort_flag);
          if (good) {
            mbar_expect_tx(sbar, C::kXsBytes + 2 * C::kWsBytes);
            const float* wsrc = w_scale + ((size_t)w.group * C::kSlabTiles + w.ntile) * C::kKBlocks;
            bulk_load(sdst + C::kXsBytes, wsrc, C::kWsBytes, sbar);
            bulk_load(sdst + C::kXsBytes + C::kWsBytes, wsrc + (kInter / kTileRows) * C::kKBlocks, C::kWsBytes, sbar);
          } else {
            status[0] = kStatusProducerTimeout; *abort_flag = 1;
          }
        }
        good = __shfl_sync(0xffffffffu, good ? 1 : 0, 0) != 0;
        if (!good) { ok = false; break; }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          bulk_load(sdst + (uint32_t)(4 * lane + j) * C::kKBlocks * 4, x_scale + (size_t)src[j] * C::kKBlocks, C::kKBlocks * 4, sbar);
        const bool have_next = item + stride < total_items;
        const Item wn = have_next ? get_item((int)n_item + 1, item + stride) : w;
        for (int kb = 0; kb < C::kKBlocks; ++kb, ++it) {
          const int s = it % C::kStages;
          const uint32_t bar = smem_u32(&full_bar[s]);
          const uint32_t dst = smem_u32(stage_base + s * C::kStageBytes);
          if (lane == 0) {
            // weight boxes of K-block kb + kPrefetch (in this item or the next) are pulled into the L2 now
            const int pk = kb + C::kPrefetch;
            const Item& wp = pk < C::kKBlocks ? w : wn;
            if (pk < C::kKBlocks || have_next) {
              const int kp = pk < C::kKBlocks ? pk : pk - C::kKBlocks;
              const int wx = w_tiled ? 0 : kp * kBlock;
              const int wy0 = w_tiled ? ((wp.group * C::kSlabTiles + wp.ntile) * C::kKBlocks + kp) * kTileRows
                                      : wp.group * C::kSlabRows + wp.ntile * kTileRows;
              const int wy1 = wy0 + (w_tiled ? (kInter / kTileRows) * C::kKBlocks * kTileRows : kInter);
              tma_prefetch_2d(tm_w, wx, wy0);
              tma_prefetch_2d(tm_w, wx, wy1);
            }
            good = mbar_wait(smem_u32(&empty_bar[s]), ((it / C::kStages) & 1) ^ 1, abort_flag);
            if (good) {
              mbar_expect_tx(bar, C::kStageBytes);
              const int wx = w_tiled ? 0 : kb * kBlock;
              const int wy0 = w_tiled ? ((w.group * C::kSlabTiles + w.ntile) * C::kKBlocks + kb) * kTileRows
                                      : w.group * C::kSlabRows + w.ntile * kTileRows;
              const int wy1 = wy0 + (w_tiled ? (kInter / kTileRows) * C::kKBlocks * kTileRows : kInter);
              tma_load_2d(dst + C::kTokTile * kBlock, tm_w, bar, wx, wy0, pol_w);
              tma_load_2d(dst + C::kTokTile * kBlock + kWTileBytes, tm_w, bar, wx, wy1, pol_w);
            } else {
              status[0] = kStatusProducerTimeout; *abort_flag = 1;
            }
          }
          good = __shfl_sync(0xffffffffu, good ? 1 : 0, 0) != 0;      // also orders the lanes' gathers after lane 0's wait
          if (!good) { ok = false; break; }
          tma_gather4_2d(dst + (uint32_t)lane * 4 * kBlock, tm_x128, bar, kb * kBlock, src[0], src[1], src[2], src[3], pol_x);
        }
      }
    } else if (!kGatherX && warp == 0 && lane == 0) {
      // =========================== TMA producer ===========================
      asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tm_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)tm_x128) : "memory");
      const uint64_t pol_w = policy_evict_last();      // a weight tile is re-read by every token tile of the expert
      const uint64_t pol_x = policy_evict_last();      // token rows are re-read by every channel tile
      uint32_t it = 0, n_item = 0;
      bool ok = true;
      for (int item = first_item; ok && item < total_items; item += stride, ++n_item) {
        const Item w = get_item((int)n_item, item);
        {
          const int slot = n_item % C::kScaleSlots;
          if (!mbar_wait(smem_u32(&sempty_bar[slot]), ((n_item / C::kScaleSlots) & 1) ^ 1, abort_flag)) {
            status[0] = kStatusProducerTimeout; *abort_flag = 1; ok = false; break;
          }
          const uint32_t sbar = smem_u32(&sfull_bar[slot]);
          const uint32_t sdst = smem_u32(scale_base + slot * C::kScaleSlotBytes);
          mbar_expect_tx(sbar, C::kXsBytes + (kFp4 ? 0 : 2 * C::kWsBytes));
          bulk_load(sdst, x_scale + (size_t)w.row0 * C::kKBlocks, C::kXsBytes, sbar);
          if constexpr (kFp4) {
            // the weight scales travel with the weight tiles, stage by stage
          } else if (kGateUp) {     // gate tile ntile, up tile 4 + ntile
            const float* wsrc = w_scale + ((size_t)w.group * C::kSlabTiles + w.ntile) * C::kKBlocks;
            bulk_load(sdst + C::kXsBytes, wsrc, C::kWsBytes, sbar);
            bulk_load(sdst + C::kXsBytes + C::kWsBytes, wsrc + (kInter / kTileRows) * C::kKBlocks, C::kWsBytes, sbar);
          } else {           // tiles 2 * ntile and 2 * ntile + 1 are consecutive
            const float* wsrc = w_scale + ((size_t)w.group * C::kSlabTiles + 2 * w.ntile) * C::kKBlocks;
            bulk_load(sdst + C::kXsBytes, wsrc, 2 * C::kWsBytes, sbar);
          }
        }
        const int tile0 = kGateUp ? w.ntile : 2 * w.ntile;
        const int tile_step = kGateUp ? kInter / kTileRows : 1;
        auto weight_xy = [&](const Item& wi, int t0, int kb, int& wx, int& wy0, int& wy1) {
          if constexpr (kFp4) {
            // code blocks in (slab, tile pair, K-block, tile of the pair) order: the item's two tiles are one 256-row box
            wx = 0;
            wy0 = (((wi.group * C::kNTiles + wi.ntile) * C::kKBlocks + kb) * 2) * kTileRows;
            wy1 = wy0 + kTileRows;
          } else if (w_tiled) {
            wx = 0;
            wy0 = ((wi.group * C::kSlabTiles + t0) * C::kKBlocks + kb) * kTileRows;
            wy1 = wy0 + tile_step * C::kKBlocks * kTileRows;
          } else {
            wx = kb * kBlock;
            wy0 = wi.group * C::kSlabRows + t0 * kTileRows;
            wy1 = wy0 + tile_step * kTileRows;
          }
        };
        // The shared-memory ring holds under two microseconds of MMA work, less than a DRAM round trip under
        // load, so the boxes of K-block kb + kPrefetch (in this item or the next) are pulled into the L2 now.
        const bool have_next = item + stride < total_items;
        const Item wn = have_next ? get_item((int)n_item + 1, item + stride) : w;
        const int tile0_next = kGateUp ? wn.ntile : 2 * wn.ntile;
        for (int kb = 0; kb < C::kKBlocks; ++kb, ++it) {
          {
            const int pk = kb + C::kPrefetch;
            int wx, wy0, wy1;
            if (pk < C::kKBlocks) {
              weight_xy(w, tile0, pk, wx, wy0, wy1);
              tma_prefetch_2d(tm_w, wx, wy0);
              if (!kFp4) tma_prefetch_2d(tm_w, wx, wy1);
              tma_prefetch_2d(tm_x128, pk * kBlock, w.row0);
            } else if (have_next) {
              weight_xy(wn, tile0_next, pk - C::kKBlocks, wx, wy0, wy1);
              tma_prefetch_2d(tm_w, wx, wy0);
              if (!kFp4) tma_prefetch_2d(tm_w, wx, wy1);
              tma_prefetch_2d(tm_x128, (pk - C::kKBlocks) * kBlock, wn.row0);
            }
          }
          const int s = it % C::kStages;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / C::kStages) & 1) ^ 1, abort_flag)) {
            status[0] = kStatusProducerTimeout; *abort_flag = 1; ok = false; break;
          }
          const uint32_t bar = smem_u32(&full_bar[s]);
          const uint32_t dst = smem_u32(stage_base + s * C::kStageBytes);
          mbar_expect_tx(bar, C::kTokTile * kBlock + 2 * C::kWTxBytes + C::kAtomStageBytes);
          int wx, wy0, wy1;
          weight_xy(w, tile0, kb, wx, wy0, wy1);
          tma_load_2d(dst, tm_x128, bar, kb * kBlock, w.row0, pol_x);
          tma_load_2d(dst + C::kTokTile * kBlock, tm_w, bar, wx, wy0, pol_w);
          if constexpr (kFp4)
            bulk_load(smem_u32(atom_base + s * C::kAtomStageBytes), w_scale_atoms + (size_t)wy0 * 4, C::kAtomStageBytes, bar);
          else
            tma_load_2d(dst + C::kTokTile * kBlock + kWTileBytes, tm_w, bar, wx, wy1, pol_w);
        }
      }
    } else if ((warp == 1 || warp == 2) && lane == 0) {
      // =========================== MMA issuers ===========================
      // Two threads take alternate K-blocks (warp 1 the even ones into TMEM stage 0, warp 2 the odd ones into
      // stage 1): while one is blocked feeding its four MMAs to the tensor pipe, the other has already passed its
      // barrier waits, so the pipe does not drain between K-blocks.  The K-blocks are independent (own shared-memory
      // stage, own TMEM stage) and a commit covers the MMAs of the thread that issues it.
      // (MXFP4: one accumulator stage, so warp 1 issues every K-block and warp 2 has nothing to do)
      const uint32_t idesc = make_idesc(256);
      const uint32_t par = (uint32_t)(warp - 1);
      bool ok = !(kFp4 && warp == 2);
      uint32_t it = 0;
      for (int item = first_item; ok && item < total_items; item += stride) {
        for (int kb = 0; kb < C::kKBlocks; ++kb, ++it) {
          if (!kFp4 && (it & 1u) != par) continue;
          const int a = kFp4 ? 0 : (int)par;
          if (!mbar_wait(smem_u32(&tempty_bar[a]), ((it / C::kAccStages) & 1) ^ 1, abort_flag)) {
            status[0] = kStatusMmaTimeout; *abort_flag = 1; ok = false; break;
          }
          const int s = it % C::kStages;
          if (!mbar_wait(smem_u32(&full_bar[s]), (it / C::kStages) & 1, abort_flag)) {
            status[0] = kStatusMmaTimeout; *abort_flag = 1; ok = false; break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(stage_base + s * C::kStageBytes);
          const uint64_t adesc = make_smem_desc(sa);                              // 128 token rows
          const uint64_t bdesc = make_smem_desc(sa + C::kTokTile * kBlock);       // 256 weight rows
          const uint32_t d0 = tmem_base + (uint32_t)(a * C::kAccCols);
          if constexpr (kFp4) {
            // the two tiles' scale atoms -> eight TMEM columns (weight row n: lane n % 32, column n / 32); copies and
            // MMAs of one thread run in issue order, so the previous K-block's MMAs have read the columns by now
            const uint32_t at = smem_u32(atom_base + s * C::kAtomStageBytes);
            tmem_cp_32x128b_warpx4(tmem_scale + 4, make_scale_desc(at));
            tmem_cp_32x128b_warpx4(tmem_scale + 8, make_scale_desc(at + 512));
#pragma unroll
            for (int k = 0; k < kBlock / 32; ++k)
              umma_mxf8f6f4(d0, adesc + 2 * k, bdesc + 2 * k, make_idesc_mxfp4_b((uint32_t)k), tmem_scale,
                            (tmem_scale + 4) | ((uint32_t)k << 30), k > 0);
          } else {
#pragma unroll
            for (int k = 0; k < kBlock / 32; ++k) umma_f8(d0, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0);
          }
          umma_commit(smem_u32(&empty_bar[s]));
          umma_commit(smem_u32(&tfull_bar[a]));
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kTmRegsHigh));
    // =========================== promotion + epilogue (2 warpgroups x 128 threads) ===========================
    const int wg = (warp - 4) >> 2;          // which half of the accumulator columns
    const int quad = warp & 3;               // TMEM lane quadrant this warp may read
    const int r = quad * 32 + lane;          // token row inside the item == TMEM lane
    // two 64-column segments per thread.  gate_up: gate channels [wg*64, +64) and their up partners;
    // down: output columns [wg*128, +128) (all of weight tile wg)
    const int seg_col0 = kGateUp ? wg * 64 : wg * 128;
    const int seg_col1 = kGateUp ? 128 + wg * 64 : wg * 128 + 64;
    const int ws0 = kGateUp ? 0 : wg, ws1 = kGateUp ? 1 : wg;
    const int total_rows = offs[groups];     // rows of this call: the row count of every FP16 output panel
    uint32_t it = 0, n_item = 0;
    bool ok = true;
    for (int item = first_item; item < total_items; item += stride, ++n_item) {
      const Item w = get_item((int)n_item, item);
      const int slot = n_item % C::kScaleSlots;
      const float* xs_tile = reinterpret_cast<const float*>(scale_base + slot * C::kScaleSlotBytes);
      const float* ws_tile = xs_tile + C::kTokTile * C::kKBlocks;
      if (ok && !mbar_wait(smem_u32(&sfull_bar[slot]), (n_item / C::kScaleSlots) & 1, abort_flag)) {
        status[0] = kStatusEpilogueTimeout; *abort_flag = 1; ok = false;
      }
      float acc0[64], acc1[64];
#pragma unroll
      for (int c = 0; c < 64; ++c) { acc0[c] = 0.0f; acc1[c] = 0.0f; }
      for (int kb = 0; kb < C::kKBlocks; ++kb, ++it) {
        const int a = it % C::kAccStages;
        if (ok && !mbar_wait(smem_u32(&tfull_bar[a]), (it / C::kAccStages) & 1, abort_flag)) {
          status[0] = kStatusEpilogueTimeout; *abort_flag = 1; ok = false;
        }
        if (!ok) continue;
        tc_fence_after();
        if (kFp4 && quad * 32 >= w.m_valid) {
          // no row of this item lives in this warp's TMEM lanes (the tail tile of an expert): nothing to promote, the
          // warp only keeps step with the hand-off
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[a]));
          continue;
        }
        const uint32_t tbase = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * C::kAccCols);
        uint32_t v[2][32];
        tmem_ld32_nowait(tbase + (uint32_t)seg_col0, v[0]);
        tmem_ld32_nowait(tbase + (uint32_t)(seg_col0 + 32), v[1]);
        const float x = xs_tile[r * C::kKBlocks + kb];
        // MXFP4: the weight scales were applied inside the MMA
        const float s0 = kFp4 ? x : __fmul_rn(x, ws_tile[ws0 * C::kKBlocks + kb]);
        const float s1 = kFp4 ? x : __fmul_rn(x, ws_tile[ws1 * C::kKBlocks + kb]);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          acc0[c] = fmaf(__uint_as_float(v[0][c]), s0, acc0[c]);
          acc0[32 + c] = fmaf(__uint_as_float(v[1][c]), s0, acc0[32 + c]);
        }
        tmem_ld32_nowait(tbase + (uint32_t)seg_col1, v[0]);
        tmem_ld32_nowait(tbase + (uint32_t)(seg_col1 + 32), v[1]);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[a]));   // the partials now live in registers
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          acc1[c] = fmaf(__uint_as_float(v[0][c]), s1, acc1[c]);
          acc1[32 + c] = fmaf(__uint_as_float(v[1][c]), s1, acc1[32 + c]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sempty_bar[slot]));   // the scale tiles were last read above
      const bool live = r < w.m_valid;
      const size_t row = (size_t)(w.row0 + r);
      if constexpr (kGateUp) {
        float amax = 0.0f;
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const float g = acc0[c];
          const float silu = __fdividef(g, 1.0f + __expf(-g));
          acc0[c] = bf16_round(__fmul_rn(silu, acc1[c]));
          amax = fmaxf(amax, fabsf(acc0[c]));
        }
        uint32_t* my_red = red + (n_item & 1) * C::kEpiGroups * C::kLanes;     // double-buffered by item parity: one barrier per item
        my_red[wg * C::kLanes + r] = __float_as_uint(amax);
        epilogue_barrier();
        const float m = fmaxf(__uint_as_float(my_red[r]), __uint_as_float(my_red[C::kLanes + r]));
        const float scale = fmaxf(m, amax_floor()) * inv448();
        const float inv = rcp_newton(scale);
        if (live) {
          // the thread's 64 bytes as two 32-byte stores: a lane owns a row, so every store is a sector of its own, and
          // a full one (16-byte stores half-fill each sector twice)
          float* dst = reinterpret_cast<float*>(h_fp8 + row * kInter + w.ntile * kTileRows + wg * 64);
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            float p[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int c = q * 32 + j * 4;
              p[j] = __uint_as_float(f32x4_to_e4m3x4(acc0[c] * inv, acc0[c + 1] * inv, acc0[c + 2] * inv, acc0[c + 3] * inv));
            }
            st_global_v8(dst + 8 * q, p);
          }
          if (wg == 0) h_scale[row * kInterBlocks + w.ntile] = scale;
        }
      } else if constexpr (kF16Out) {
        // FP16 partial rows (the reference's prefill contract, kernels/gfx950/templates/moe/prefill/fused_splitk2/down_partial.inc:435-458).
        // Layout in global memory: sixteen column panels of 128 halves, panel p = [total rows][256 bytes], the sixteen
        // 16-byte chunks of a row permuted by the row's index (chunk j at position j ^ (row & 15); the reducer
        // netra_moe_combine_f16_sm100 reads them back the same way).  A warpgroup's item is then one contiguous block
        // of its panel: the threads stage their rows in shared memory in exactly that image and ONE bulk copy of
        // m_valid x 256 bytes writes it - the copy engine's cost is per copy (one 256-byte copy per thread took
        // 3,500 of an item's 8,700 cycles), not per byte.
        uint8_t* tile = out_stage + (size_t)wg * (C::kLanes * C::kOutRowBytes);
        const bool elected = quad == 0 && lane == 0;
        // the copies of the previous item have read the tile (with a return table any thread may have issued one)
        if (elected || ret != nullptr) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        group_barrier(wg);
        // With a return table the row goes to another rank's panels (or this rank's own): it is staged with the
        // permutation of its destination row, and every run of rows that lands on consecutive rows of one rank - the
        // rows one source sent to one expert - leaves as one bulk copy, over NVLink while the next items are computed.
        // A run starts where the destination is not the previous row's plus one; its length is the distance to the next
        // start or to the first row without a destination, found from the warps' ballots (four words per warpgroup in
        // the area the amax exchange of gate_up uses, which is idle here).
        uint32_t* brk_masks = red + wg * 4;
        int2 mine = make_int2(-1, -1);
        bool head = false;
        uint32_t my_brk = 0;
        if (ret != nullptr) {
          if (live) mine = ret->row_dst[row];
          int2 prev;
          prev.x = __shfl_up_sync(0xffffffffu, mine.x, 1);
          prev.y = __shfl_up_sync(0xffffffffu, mine.y, 1);
          if (lane == 0) prev = (r > 0 && live) ? ret->row_dst[row - 1] : make_int2(-1, -1);
          head = mine.x >= 0 && (r == 0 || prev.x != mine.x || prev.y + 1 != mine.y);
          my_brk = __ballot_sync(0xffffffffu, head || mine.x < 0);
          if (lane == 0) brk_masks[quad] = my_brk;
        }
        const uint32_t key = (ret != nullptr ? (uint32_t)max(mine.y, 0) : (uint32_t)(w.row0 + r)) & 15u;
        uint8_t* my_row = tile + (size_t)r * C::kOutRowBytes;
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          const float* a = q < 8 ? &acc0[8 * q] : &acc1[8 * (q - 8)];
          uint32_t pk[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __half2 h = __floats2half2_rn(a[2 * j], a[2 * j + 1]);
            pk[j] = *reinterpret_cast<const uint32_t*>(&h);
          }
          *reinterpret_cast<uint4*>(my_row + 16 * ((uint32_t)q ^ key)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        group_barrier(wg);
        if (ret == nullptr) {
          if (elected) {
            __half* gdst = reinterpret_cast<__half*>(down) + ((size_t)(w.ntile * 2 + wg) * (size_t)total_rows + (size_t)w.row0) * kTileRows;
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(tile)),
                         "r"((uint32_t)w.m_valid * (uint32_t)C::kOutRowBytes) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        } else {
          if (head) {
            int len;
            const uint32_t above = lane < 31 ? my_brk >> (lane + 1) : 0u;
            if (above != 0u) {
              len = __ffs(above);
            } else {
              len = 32 - lane;
              for (int q2 = quad + 1; q2 < 4; ++q2) {
                const uint32_t m = brk_masks[q2];
                if (m != 0u) { len += __ffs(m) - 1; break; }
                len += 32;
              }
            }
            const size_t dst_total = (size_t)ret->tokens_of_rank[(size_t)mine.x * ret->tokens_pitch] * kSlots;
            uint8_t* gdst = ret->base[mine.x] + ((size_t)(w.ntile * 2 + wg) * dst_total + (size_t)mine.y) * (size_t)C::kOutRowBytes;
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(my_row)),
                         "r"((uint32_t)len * (uint32_t)C::kOutRowBytes) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
      } else {
        if (live) {
          // a lane owns a whole row, so a warp's stores touch 32 rows: 256-bit stores fill one 32-byte sector each
          float* base = (row_ptr != nullptr ? row_ptr[row] : down + row * kHidden) + w.ntile * 2 * kTileRows + wg * kTileRows;
#pragma unroll
          for (int q = 0; q < 8; ++q) st_global_v8(base + 8 * q, &acc0[8 * q]);
#pragma unroll
          for (int q = 0; q < 8; ++q) st_global_v8(base + 64 + 8 * q, &acc1[8 * q]);
        }
      }
    }
    if constexpr (kF16Out) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // this thread's row copies are complete
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

extern "C" __global__ void __launch_bounds__(kTmThreads, 1)
netra_moe_gate_up_tokmajor_sm100(const __grid_constant__ CUtensorMap tm_w13, const __grid_constant__ CUtensorMap tm_a128,
                                 const float* a_scale, const float* w13_scale, const int32_t* offsets, uint8_t* h_fp8,
                                 float* h_scale, uint32_t num_groups, uint32_t w_tiled, uint32_t* status) {
  tokmajor_gemm_body<true>(&tm_w13, &tm_a128, a_scale, w13_scale, offsets, h_fp8, h_scale, nullptr, nullptr, num_groups, w_tiled,
                           status);
}

extern "C" __global__ void __launch_bounds__(kTmThreads, 1)
netra_moe_down_tokmajor_sm100(const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_h128,
                              const float* h_scale, const float* w2_scale, const int32_t* offsets, float* down,
                              uint32_t num_groups, uint32_t w_tiled, uint32_t* status) {
  tokmajor_gemm_body<false>(&tm_w2, &tm_h128, h_scale, w2_scale, offsets, nullptr, nullptr, down, nullptr, num_groups, w_tiled,
                            status);
}

// gate_up with the token rows gathered from token order (no expert-sorted copy of the quantised rows is needed):
// tm_tok1 is a one-row-box map over the quantised-row buffer, tok_scale its scales [rows, 16], perm the sorted
// position -> pair index table, tok_row_base the first token-order row of that buffer.
extern "C" __global__ void __launch_bounds__(kTmThreads, 1)
netra_moe_gate_up_tokmajor_gather_sm100(const __grid_constant__ CUtensorMap tm_w13, const __grid_constant__ CUtensorMap tm_tok1,
                                        const float* tok_scale, const float* w13_scale, const int32_t* offsets, const int32_t* perm,
                                        uint8_t* h_fp8, float* h_scale, uint32_t num_groups, uint32_t w_tiled, uint32_t tok_row_base,
                                        uint32_t* status) {
  tokmajor_gemm_body<true, false, true>(&tm_w13, &tm_tok1, tok_scale, w13_scale, offsets, h_fp8, h_scale, nullptr, nullptr, num_groups,
                                        w_tiled, status, perm, tok_row_base);
}

// The down projection writing FP16 partial rows [rows, 2048] (half the bytes of the FP32 rows; consumed by
// netra_moe_combine_f16_sm100).  Same accumulation as above, one rounding to FP16 per output element.
extern "C" __global__ void __launch_bounds__(kTmThreads, 1)
netra_moe_down_tokmajor_f16_sm100(const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_h128,
                                  const float* h_scale, const float* w2_scale, const int32_t* offsets, void* down_f16,
                                  uint32_t num_groups, uint32_t w_tiled, uint32_t* status) {
  tokmajor_gemm_body<false, true>(&tm_w2, &tm_h128, h_scale, w2_scale, offsets, nullptr, nullptr, reinterpret_cast<float*>(down_f16),
                                  nullptr, num_groups, w_tiled, status);
}

// The two projections on MXFP4 expert weights (E2M1 codes, one UE8M0 scale per 32 K-elements; semantics of
// kernels/gfx1151/mxfp4/prefill/mxfp4_prefill_gate_wmma_gfx1151.s:3-8, mxfp4_prefill_up_silu_wmma_gfx1151.s:3-8 and
// mxfp4_prefill_down_wmma_gfx1151.s:3-5; decode call sequence runtime/gfx1151/mxfp4/decode/runtime.h:10-47): the weights
// stay four-bit in memory (tm_w*: code blocks of 128 rows x 64 bytes written by netra_moe_mxfp4_pack_sm100, fetched two at
// a time) and their scales reach the tensor core through TMEM.  For calls whose experts hold many rows; the swap-AB
// forms (umma_kernels.cu) serve decode sizes.
extern "C" __global__ void __launch_bounds__(kTmThreads, 1)
netra_moe_gate_up_mxfp4_tokmajor_sm100(const __grid_constant__ CUtensorMap tm_w13, const __grid_constant__ CUtensorMap tm_a128,
                              const float* a_scale, const uint8_t* w13_scale_atoms, const int32_t* offsets, uint8_t* h_fp8,
                              float* h_scale, uint32_t num_groups, uint32_t* status) {
  tokmajor_gemm_body<true, false, false, true>(&tm_w13, &tm_a128, a_scale, reinterpret_cast<const float*>(w13_scale_atoms), offsets, h_fp8,
                                               h_scale, nullptr, nullptr, num_groups, 1u, status);
}

extern "C" __global__ void __launch_bounds__(kTmThreads, 1)
netra_moe_down_mxfp4_tokmajor_sm100(const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_h128,
                           const float* h_scale, const uint8_t* w2_scale_atoms, const int32_t* offsets, float* down,
                           uint32_t num_groups, uint32_t* status) {
  tokmajor_gemm_body<false, false, false, true>(&tm_w2, &tm_h128, h_scale, reinterpret_cast<const float*>(w2_scale_atoms), offsets, nullptr,
                                                nullptr, down, nullptr, num_groups, 1u, status);
}

int gate_up_mxfp4_tokmajor_smem_bytes() { return TmCfg<true, false, true>::kSmemBytes; }
int down_mxfp4_tokmajor_smem_bytes() { return TmCfg<false, false, true>::kSmemBytes; }
int gate_up_tokmajor_smem_bytes() { return TmCfg<true>::kSmemBytes; }
int down_tokmajor_smem_bytes() { return TmCfg<false>::kSmemBytes; }
int down_tokmajor_f16_smem_bytes() { return TmCfg<false, true>::kSmemBytes; }

}  // namespace netra

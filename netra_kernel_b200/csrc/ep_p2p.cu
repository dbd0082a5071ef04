// Expert parallelism over peer memory: every exchange of the expert-parallel layer is done by this
// library's own kernels with plain stores into the peers' windows (NVLink through NVSwitch) and
// epoch-valued flags, so one layer call is a fixed sequence of kernel launches with no host
// read-back and no library collective.  The reference has no expert parallelism (its 8-GPU mode is
// eight replicas, manifests/gfx950/models/qwen36-moe-m1-golden.json:11-12); this is new design.
//
// Rank r owns routed experts [r * E_l, (r + 1) * E_l), E_l = 256 / world, plus a copy of the shared
// expert.  Per call, on every rank:
//   publish  the rank's 256 per-expert pair counts and its token count go to every peer    (flag 0)
//   plan     wait for all count rows; from the full count matrix every rank derives where each of
//            its sorted rows lands in the owner's expert-major block, the group offsets of its own
//            block, and for each block row the (rank, sorted row) it is returned to
//   push     each sorted row (2048 FP8 codes + 16 scales) is stored straight into its expert-major
//            position in the owner's activation block; the rank's own tokens become the shared
//            expert's rows (group 0); the same launch builds the table "block row -> where its
//            result goes"                                                                   (flag 1)
//   gate_up  waits for the pushed rows, then the grouped GEMM over E_l + 1 slabs
//   down     grouped GEMM whose epilogue stores each FP32 row straight into the sending rank's
//            sorted-order buffer (the return overlaps the remaining tiles)                   (flag 2)
//   combine  waits for the returned rows, then the slot-ordered combine of the one-GPU layer
// One call is nine stages; a real multi-GPU call runs publish and plan as one launch (eight launches up to
// 1,024 tokens).  Ranks emulated on one GPU are driven stage by stage instead, so that every wait finds its
// flags raised (two kernels that wait on one another must never be in flight on one GPU).
// A flag holds the epoch (call number) of its writer; a wait spins until the flag reaches the
// current epoch or a time limit passes, in which case a status word records it and the kernel
// returns.  Buffer reuse is ordered by the flags themselves: a rank's next push follows its wait for
// flag 2, which each peer raises only after its GEMMs have read the previous rows.
#include "common.cuh"

namespace netra {

constexpr int kEpMaxRanks = 16;
constexpr int kEpMatrixPitch = 264;          // ints per count row: 256 counts, [256] = tokens, rest spare
constexpr int kEpFlagPitch = 32;             // uint32 per phase
constexpr int kEpTableBlocks = 296;          // blocks of the push launch that also build the return table

struct EpPeers {
  uint8_t* win[kEpMaxRanks];
};

struct EpWindowLayout {                      // byte offsets inside one rank's window
  uint64_t flags, matrix, blk_a, blk_as, down, total;
};

struct EpTables {                            // per-rank device tables (local memory)
  int32_t offsets[kRouted + 2];              // group offsets of this rank's block (E_l + 2 used)
  int32_t push_base[kRouted];                // global expert -> first row, in the owner's block, of this rank's rows
  int32_t blk_start[kRouted + 1];            // bucket (local expert j, source s) = j * world + s -> first block row
  int32_t ret_row[kRouted];                  // bucket -> first sorted row at source s
  uint32_t epoch, done_push, done_ret, pad;
  uint32_t status[4];                        // gate_up wait, down wait, rows needed beyond capacity, wait time-outs
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Spin until flag >= epoch (wrapping compare) or timeout_ns passes.  Returns false on time-out.
__device__ __forceinline__ bool ep_wait_flag(const uint32_t* flag, uint32_t epoch, uint64_t timeout_ns) {
  if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
      __nanosleep(64);
    }
    if (global_timer_ns() - t0 > timeout_ns) return false;
  }
}

// publish: this rank's counts row -> every peer's matrix, then flag 0.  One block of at least 288 threads.
__device__ __forceinline__ void ep_publish_body(const EpPeers& peers, const EpWindowLayout& lay, EpTables* __restrict__ tab,
                                                const int32_t* __restrict__ counts, uint32_t tokens, uint32_t world, uint32_t rank) {
  __shared__ uint32_t s_epoch;
  const int tid = threadIdx.x;
  if (tid == 0) {
    s_epoch = tab->epoch + 1;
    tab->epoch = s_epoch;
  }
  __syncthreads();
  if (tid < 257) {
    const int32_t v = tid < kRouted ? counts[tid] : (int32_t)tokens;
    for (uint32_t g = 0; g < world; ++g)
      reinterpret_cast<int32_t*>(peers.win[g] + lay.matrix)[rank * kEpMatrixPitch + tid] = v;
  }
  __syncthreads();                 // the release stores below are cumulative over the block's stores
  if (tid < (int)world) st_release_sys(reinterpret_cast<uint32_t*>(peers.win[tid] + lay.flags) + 0 * kEpFlagPitch + rank, s_epoch);
}

// grid 1, block 288
extern "C" __global__ void __launch_bounds__(288)
netra_ep_publish_counts_sm100(EpPeers peers, EpWindowLayout lay, EpTables* __restrict__ tab, const int32_t* __restrict__ counts,
                              uint32_t tokens, uint32_t world, uint32_t rank) {
  ep_publish_body(peers, lay, tab, counts, tokens, world, rank);
}

// wait for one phase's flags from every rank.  grid 1, block 32.
extern "C" __global__ void __launch_bounds__(32)
netra_ep_wait_sm100(const uint8_t* __restrict__ window, EpWindowLayout lay, EpTables* __restrict__ tab, uint32_t phase,
                    uint32_t world, uint64_t timeout_ns) {
  const int tid = threadIdx.x;
  if (tid < (int)world) {
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(window + lay.flags) + phase * kEpFlagPitch + tid;
    if (!ep_wait_flag(flag, tab->epoch, timeout_ns)) atomicOr(&tab->status[3], (1u << (8 * phase)) << min(tid, 7));
  }
}

// plan: wait for flag 0 of every rank, then derive all row placements from the count matrix.  One block of 1,024 threads.
__device__ __forceinline__ void ep_plan_body(const uint8_t* __restrict__ window, const EpWindowLayout& lay, EpTables* __restrict__ tab,
                                             uint32_t world, uint32_t rank, uint32_t capacity, uint64_t timeout_ns) {
  __shared__ int C[kEpMaxRanks][kRouted];    // C[s][e]: pairs of rank s for global expert e
  __shared__ int rowpre[kEpMaxRanks][kRouted];
  __shared__ int colsum[kRouted];
  __shared__ int colpre[kRouted];
  __shared__ int exp_base[kRouted];          // first row of expert e in its owner's block
  __shared__ int tok[kEpMaxRanks];
  const int tid = threadIdx.x;
  const int e_l = kRouted / (int)world;
  if (tid < (int)world) {
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(window + lay.flags) + tid;
    if (!ep_wait_flag(flag, tab->epoch, timeout_ns)) atomicOr(&tab->status[3], 1u << min(tid, 7));
  }
  __syncthreads();
  const int32_t* matrix = reinterpret_cast<const int32_t*>(window + lay.matrix);
  for (int i = tid; i < (int)world * kRouted; i += 1024) {
    const int s = i / kRouted, e = i % kRouted;
    // a count row is trusted only inside its own bounds: negative or oversized values are clamped
    C[s][e] = min(max(__ldcg(matrix + s * kEpMatrixPitch + e), 0), (int)capacity);
  }
  if (tid < (int)world) tok[tid] = min(max(__ldcg(matrix + tid * kEpMatrixPitch + kRouted), 0), (int)capacity);
  __syncthreads();
  // rowpre[s][e] = pairs of source s for experts below e (its sorted row of expert e): one warp per source,
  // eight experts per lane, shuffle scan across the lanes
  {
    const int w = tid >> 5, lane = tid & 31;
    if (w < (int)world) {
      int v[8], sum = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) { v[k] = C[w][lane * 8 + k]; sum += v[k]; }
      int incl = sum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += o;
      }
      int run = incl - sum;
#pragma unroll
      for (int k = 0; k < 8; ++k) { rowpre[w][lane * 8 + k] = run; run += v[k]; }
    }
  }
  if (tid < kRouted) {
    int sum = 0;
    for (int s = 0; s < (int)world; ++s) sum += C[s][tid];
    colsum[tid] = sum;
  }
  __syncthreads();
  if (tid < 32) {                            // colpre[e] = rows of all experts below e, over all sources
    int v[8], sum = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) { v[k] = colsum[tid * 8 + k]; sum += v[k]; }
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (tid >= d) incl += o;
    }
    int run = incl - sum;
#pragma unroll
    for (int k = 0; k < 8; ++k) { colpre[tid * 8 + k] = run; run += v[k]; }
  }
  __syncthreads();
  if (tid < kRouted) {
    const int g = tid / e_l;
    const int base = tok[g] + colpre[tid] - colpre[g * e_l];
    exp_base[tid] = base;
    int mine = base;
    for (int s = 0; s < (int)rank; ++s) mine += C[s][tid];
    tab->push_base[tid] = mine;
  }
  __syncthreads();
  if (tid < kRouted) {
    // buckets of this rank's block in block order: local expert j major, source s minor
    const int j = tid / (int)world, s = tid % (int)world, e = (int)rank * e_l + j;
    int start = exp_base[e];
    for (int ss = 0; ss < s; ++ss) start += C[ss][e];
    tab->blk_start[tid] = start;
    tab->ret_row[tid] = rowpre[s][e];
  }
  if (tid < e_l) tab->offsets[1 + tid] = min(exp_base[(int)rank * e_l + tid], (int)capacity);
  if (tid == 0) {
    const int last = (int)rank * e_l + e_l - 1;
    const int total = exp_base[last] + colsum[last];
    tab->offsets[0] = 0;
    tab->offsets[e_l + 1] = min(total, (int)capacity);
    tab->blk_start[kRouted] = total;
  }
  if (tid < (int)world) {                    // every rank sees every block's size: all report the same overflow
    const int last = tid * e_l + e_l - 1;
    const int total = exp_base[last] + colsum[last];
    if (total > (int)capacity) atomicMax(&tab->status[2], (uint32_t)total);
  }
}

// grid 1, block 1024
extern "C" __global__ void __launch_bounds__(1024)
netra_ep_plan_sm100(const uint8_t* __restrict__ window, EpWindowLayout lay, EpTables* __restrict__ tab, uint32_t world,
                    uint32_t rank, uint32_t capacity, uint64_t timeout_ns) {
  ep_plan_body(window, lay, tab, world, rank, capacity, timeout_ns);
}

// publish and plan in one launch, for ranks that live on GPUs of their own (the wait inside would never end for ranks
// emulated one after another on one GPU).  grid 1, block 1024.
extern "C" __global__ void __launch_bounds__(1024)
netra_ep_publish_plan_sm100(EpPeers peers, EpWindowLayout lay, EpTables* __restrict__ tab, const int32_t* __restrict__ counts,
                            uint32_t tokens, uint32_t world, uint32_t rank, uint32_t capacity, uint64_t timeout_ns) {
  ep_publish_body(peers, lay, tab, counts, tokens, world, rank);
  __syncthreads();
  ep_plan_body(peers.win[rank], lay, tab, world, rank, capacity, timeout_ns);
}

// Signal a phase to every peer once all blocks of the calling kernel have fenced their stores.
__device__ __forceinline__ void ep_signal_when_last(const EpPeers& peers, const EpWindowLayout& lay, EpTables* tab, uint32_t* counter,
                                                    uint32_t phase, uint32_t world, uint32_t rank) {
  __shared__ uint32_t s_last;
  // Each block orders its stores before its count at GPU scope (thread 0's fence is cumulative over the
  // block's stores after the barrier); the last block alone pays for the system-scope fence, which is
  // cumulative over everything it has observed, before it raises the flags.  A system-scope fence per
  // block costs several microseconds per kernel on this part.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = atomicAdd(counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) {
      *counter = 0;
      __threadfence_system();
    }
    __syncthreads();
    if (threadIdx.x < world)
      st_release_sys(reinterpret_cast<uint32_t*>(peers.win[threadIdx.x] + lay.flags) + phase * kEpFlagPitch + rank, tab->epoch);
  }
}

__device__ __forceinline__ void ep_build_return_table(const EpPeers& peers, const EpWindowLayout& lay, const EpTables* __restrict__ tab,
                                                      float** __restrict__ row_ptr, float* __restrict__ blk_down, uint32_t tokens,
                                                      uint32_t max_tokens, uint32_t world, uint32_t rank, uint32_t capacity, uint32_t as_pairs);

// push: sorted row i (i < pairs) of this rank -> its expert-major row in the owner's block;
// rows pairs .. pairs + tokens - 1 are the rank's own tokens -> rows [0, tokens) of its own block.
// a_fp8 / a_scale hold the per-token quantised rows at row (pairs + t).  One warp per two rows (i and i + half): the two
// chains of dependent index loads (perm -> ids -> push_base / offsets) run side by side, and the sixteen 16-byte loads of
// both rows are in flight before the first store.  The first blocks also build the return table.
// grid ceil(ceil((pairs + tokens) / 2) / 8), block 256.
extern "C" __global__ void __launch_bounds__(256)
netra_ep_push_rows_sm100(EpPeers peers, EpWindowLayout lay, EpTables* __restrict__ tab, const uint8_t* __restrict__ a_fp8,
                         const float* __restrict__ a_scale, const int32_t* __restrict__ perm, const int32_t* __restrict__ ids9,
                         const int32_t* __restrict__ sorted_offsets, uint32_t tokens, uint32_t world, uint32_t rank,
                         uint32_t capacity, float** __restrict__ row_ptr, float* __restrict__ blk_down, uint32_t max_tokens,
                         uint32_t table_as_pairs) {
  if (blockIdx.x < kEpTableBlocks)
    ep_build_return_table(peers, lay, tab, row_ptr, blk_down, tokens, max_tokens, world, rank, capacity, table_as_pairs);
  const int pairs = (int)tokens * kTopK;
  const int rows = pairs + (int)tokens, half = (rows + 1) / 2;
  const int i0 = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (i0 < half) {
    int t[2], g[2], dst_row[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int i = i0 + k * half;
      t[k] = 0; g[k] = (int)rank; dst_row[k] = -1;
      if (i < pairs) {
        const int pair = perm[i];
        t[k] = pair >> 3;
        const int e = ids9[t[k] * kSlots + (pair & 7)];
        g[k] = e / (kRouted / (int)world);
        dst_row[k] = tab->push_base[e] + (i - sorted_offsets[e]);
      } else if (i < rows) {
        t[k] = i - pairs;
        dst_row[k] = t[k];
      }
      if (dst_row[k] >= (int)capacity) dst_row[k] = -1;
    }
    uint4 v[2][4], sc[2];
#pragma unroll
    for (int k = 0; k < 2; ++k)
      if (dst_row[k] >= 0) {
        const size_t src_row = (size_t)pairs + t[k];
        const uint4* src = reinterpret_cast<const uint4*>(a_fp8 + src_row * kHidden);
#pragma unroll
        for (int c = 0; c < 4; ++c) v[k][c] = src[c * 32 + lane];
        if (lane < 4) sc[k] = reinterpret_cast<const uint4*>(a_scale + src_row * kHiddenBlocks)[lane];
      }
#pragma unroll
    for (int k = 0; k < 2; ++k)
      if (dst_row[k] >= 0) {
        uint4* dst = reinterpret_cast<uint4*>(peers.win[g[k]] + lay.blk_a + (size_t)dst_row[k] * kHidden);
#pragma unroll
        for (int c = 0; c < 4; ++c) dst[c * 32 + lane] = v[k][c];
        if (lane < 4) reinterpret_cast<uint4*>(peers.win[g[k]] + lay.blk_as + (size_t)dst_row[k] * (kHiddenBlocks * 4))[lane] = sc[k];
      }
  }
  ep_signal_when_last(peers, lay, tab, &tab->done_push, 1, world, rank);
}

// The return table: row_ptr[r] = where block row r's FP32 down row goes - the sorted-order buffer of the rank it came
// from, or this rank's own shared rows (pairs + t) for the shared group.  Rows without a valid destination point at the
// local block buffer.  as_pairs: the same 8 bytes per row hold (rank, sorted row) instead, (-1, -1) without a valid
// destination - the form the FP16 return takes.  Grid-stride over the block rows, block 256; needs only what the plan wrote.
__device__ __forceinline__ void ep_build_return_table(const EpPeers& peers, const EpWindowLayout& lay, const EpTables* __restrict__ tab,
                                                      float** __restrict__ row_ptr, float* __restrict__ blk_down, uint32_t tokens,
                                                      uint32_t max_tokens, uint32_t world, uint32_t rank, uint32_t capacity, uint32_t as_pairs) {
  __shared__ int s_start[kRouted + 1];
  for (int i = threadIdx.x; i <= kRouted; i += blockDim.x) s_start[i] = tab->blk_start[i];
  __syncthreads();
  const int total = min(s_start[kRouted], (int)capacity);
  const int table_blocks = min((int)gridDim.x, kEpTableBlocks);
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < total; r += table_blocks * blockDim.x) {
    int g, dst_row;
    if (r < (int)tokens) {
      g = (int)rank;
      dst_row = (int)tokens * kTopK + r;
    } else {
      int lo = 0, hi = kRouted;              // last bucket whose first row is <= r
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_start[mid] <= r) lo = mid; else hi = mid;
      }
      g = lo % (int)world;
      dst_row = tab->ret_row[lo] + (r - s_start[lo]);
    }
    const bool valid = dst_row >= 0 && dst_row < (int)max_tokens * kSlots;
    if (as_pairs)
      reinterpret_cast<int2*>(row_ptr)[r] = valid ? make_int2(g, dst_row) : make_int2(-1, -1);
    else
      row_ptr[r] = valid ? reinterpret_cast<float*>(peers.win[g] + lay.down) + (size_t)dst_row * kHidden : blk_down + (size_t)r * kHidden;
  }
}

// Every thread below `world` waits for one rank's flag of `phase` in this rank's window; the block then goes on together,
// with the copy engine's later reads ordered after what the waiting threads observed.
__device__ __forceinline__ void ep_block_wait_phase(const uint8_t* __restrict__ window, const EpWindowLayout& lay, EpTables* __restrict__ tab,
                                                    uint32_t phase, uint32_t world, uint64_t timeout_ns) {
  if (threadIdx.x < world) {
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(window + lay.flags) + phase * kEpFlagPitch + threadIdx.x;
    if (!ep_wait_flag(flag, tab->epoch, timeout_ns)) atomicOr(&tab->status[3], (1u << (8 * phase)) << min((int)threadIdx.x, 7));
  }
  __syncthreads();
  asm volatile("fence.proxy.async;" ::: "memory");
}

// gate_up over the rows the peers pushed: every CTA waits for flag 1 of every rank (bounded), then runs the grouped GEMM.
extern "C" __global__ void __launch_bounds__(kGemmThreads, 1)
netra_ep_gate_up_umma_sm100(const __grid_constant__ CUtensorMap tm_w13, const __grid_constant__ CUtensorMap tm_a32,
                            const __grid_constant__ CUtensorMap tm_a64, const __grid_constant__ CUtensorMap tm_a128,
                            const float* a_scale, const float* w13_scale, const int32_t* offsets, uint8_t* h_fp8, float* h_scale,
                            uint32_t num_groups, uint32_t w_tiled, uint32_t* status, const uint8_t* window, EpWindowLayout lay,
                            EpTables* tab, uint32_t world, uint64_t timeout_ns) {
  ep_block_wait_phase(window, lay, tab, 1, world, timeout_ns);
  grouped_gemm_body<true>(&tm_w13, &tm_a32, &tm_a64, &tm_a128, a_scale, w13_scale, nullptr, offsets, h_fp8, h_scale, nullptr, nullptr,
                          num_groups, w_tiled, status);
}

extern "C" __global__ void __launch_bounds__(kTmThreads, 1)
netra_ep_gate_up_tokmajor_sm100(const __grid_constant__ CUtensorMap tm_w13, const __grid_constant__ CUtensorMap tm_a128,
                                const float* a_scale, const float* w13_scale, const int32_t* offsets, uint8_t* h_fp8, float* h_scale,
                                uint32_t num_groups, uint32_t w_tiled, uint32_t* status, const uint8_t* window, EpWindowLayout lay,
                                EpTables* tab, uint32_t world, uint64_t timeout_ns) {
  ep_block_wait_phase(window, lay, tab, 1, world, timeout_ns);
  tokmajor_gemm_body<true>(&tm_w13, &tm_a128, a_scale, w13_scale, offsets, h_fp8, h_scale, nullptr, nullptr, num_groups, w_tiled, status);
}

// The slot-ordered combine over the rows the peers returned: every block waits for flag 2 of every rank (bounded) first.
// grid rows, block 256.
extern "C" __global__ void __launch_bounds__(256)
netra_ep_combine_sm100(uint16_t* __restrict__ out, const float* down, const float* __restrict__ w9, const int32_t* __restrict__ inv_perm,
                       uint32_t rows, const uint8_t* window, EpWindowLayout lay, EpTables* tab, uint32_t world, uint64_t timeout_ns) {
  ep_block_wait_phase(window, lay, tab, 2, world, timeout_ns);
  combine_rows_body<true>(out, down, w9, inv_perm, rows);
}

// The down projection with the return fused in: every FP32 output row is stored straight to row_ptr[row]
// (a peer's sorted-order buffer over NVLink, overlapping the remaining tiles), and the last CTA to finish
// raises flag 2 at every peer.
extern "C" __global__ void __launch_bounds__(kGemmThreads, 1)
netra_ep_down_return_umma_sm100(const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_h32,
                                const __grid_constant__ CUtensorMap tm_h64, const __grid_constant__ CUtensorMap tm_h128,
                                const float* h_scale, const float* w2_scale, const int32_t* offsets, float* const* row_ptr,
                                uint32_t num_groups, uint32_t w_tiled, uint32_t* status, EpPeers peers, EpWindowLayout lay,
                                EpTables* tab, uint32_t world, uint32_t rank) {
  grouped_gemm_body<false>(&tm_w2, &tm_h32, &tm_h64, &tm_h128, h_scale, w2_scale, nullptr, offsets, nullptr, nullptr, nullptr, row_ptr,
                           num_groups, w_tiled, status);
  ep_signal_when_last(peers, lay, tab, &tab->done_ret, 2, world, rank);
}

// The same for the token-major form (blocks whose experts hold many rows).
extern "C" __global__ void __launch_bounds__(kTmThreads, 1)
netra_ep_down_return_tokmajor_sm100(const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_h128,
                                    const float* h_scale, const float* w2_scale, const int32_t* offsets, float* const* row_ptr,
                                    uint32_t num_groups, uint32_t w_tiled, uint32_t* status, EpPeers peers, EpWindowLayout lay,
                                    EpTables* tab, uint32_t world, uint32_t rank) {
  tokmajor_gemm_body<false>(&tm_w2, &tm_h128, h_scale, w2_scale, offsets, nullptr, nullptr, nullptr, row_ptr, num_groups, w_tiled,
                            status);
  ep_signal_when_last(peers, lay, tab, &tab->done_ret, 2, world, rank);
}

// The down projection of the prefill contract with the return fused in: every run of FP16 partial rows that one source
// sent to one expert leaves the epilogue's staging tile as one bulk copy into that source's panels (its own sorted
// order), over NVLink while the next items are computed; the last CTA raises flag 2 at every peer.
extern "C" __global__ void __launch_bounds__(kTmThreads, 1)
netra_ep_down_return_tokmajor_f16_sm100(const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_h128,
                                        const float* h_scale, const float* w2_scale, const int32_t* offsets,
                                        const __grid_constant__ F16RowReturn ret, uint32_t num_groups, uint32_t w_tiled, uint32_t* status,
                                        EpPeers peers, EpWindowLayout lay, EpTables* tab, uint32_t world, uint32_t rank) {
  tokmajor_gemm_body<false, true>(&tm_w2, &tm_h128, h_scale, w2_scale, offsets, nullptr, nullptr, nullptr, nullptr, num_groups, w_tiled,
                                  status, nullptr, 0, &ret);
  ep_signal_when_last(peers, lay, tab, &tab->done_ret, 2, world, rank);
}

// The reducer over FP16 partial rows that the peers returned: every block waits for flag 2 of every rank (bounded) first.
extern "C" __global__ void __launch_bounds__(256)
netra_ep_combine_f16_sm100(uint16_t* __restrict__ out, const __half* down, const float* __restrict__ w9,
                           const int32_t* __restrict__ inv_perm, uint32_t rows, const uint8_t* window, EpWindowLayout lay,
                           EpTables* tab, uint32_t world, uint64_t timeout_ns) {
  ep_block_wait_phase(window, lay, tab, 2, world, timeout_ns);
  combine_f16_rows_body<true>(out, down, w9, inv_perm, rows);
}

}  // namespace netra

// ------------------------------------------------------------------ host side (C ABI, include/netra_moe.h)
// Included by api.cu after the single-GPU layer: uses its fail()/check_launch()/encode_u8_2d()/launch_stage().
using namespace netra;

struct netra_ep_layer {
  netra_ep_layer_desc_t desc;
  netra_moe_layer* route;          // routing stages run on the single-GPU layer's workspace layout
  EpPeers peers;
  EpWindowLayout wl;
  uint8_t* window;                 // this rank's own window
  uint8_t* blk_h;
  float* blk_hs;
  float* blk_down;
  float** row_ptr;
  EpTables* tab;
  CUtensorMap tm_w13, tm_w2, tm_a32, tm_a64, tm_a128, tm_h32, tm_h64, tm_h128;
  int sm_count;
  uint32_t e_l;
  bool tokmajor_ok;                // the fused-return token-major kernel was built with the register allocation it assumes
  bool partial_f16;                // calls served by the token-major GEMMs return FP16 partial rows (the prefill contract)
};

namespace {

constexpr uint32_t kEpStageCount = 9;

EpWindowLayout ep_window_layout(uint32_t world, uint32_t max_tokens, uint32_t capacity) {
  EpWindowLayout l;
  uint64_t o = 0;
  auto take = [&](uint64_t bytes) { uint64_t at = o; o = align_up(o + bytes, 1024); return at; };
  l.flags = take(3 * kEpFlagPitch * 4);
  l.matrix = take((uint64_t)world * kEpMatrixPitch * 4);
  l.blk_a = take((uint64_t)capacity * kHidden);
  l.blk_as = take(((uint64_t)capacity + 128) * kHiddenBlocks * 4);
  l.down = take((uint64_t)max_tokens * kSlots * kHidden * 4);
  l.total = o;
  return l;
}

struct EpWorkspaceLayout {
  uint64_t route, blk_h, blk_hs, blk_down, row_ptr, tables, total;
};

int ep_workspace_layout(uint32_t max_tokens, uint32_t capacity, EpWorkspaceLayout* out) {
  netra_moe_workspace_layout_t lay;
  lay.struct_size = sizeof lay;
  if (int rc = netra_moe_workspace_layout_query(max_tokens, &lay)) return rc;
  uint64_t o = 0;
  auto take = [&](uint64_t bytes) { uint64_t at = o; o = align_up(o + bytes, 1024); return at; };
  out->route = take(lay.total_bytes);
  out->blk_h = take((uint64_t)capacity * kInter);
  out->blk_hs = take(((uint64_t)capacity + 128) * kInterBlocks * 4);
  out->blk_down = take((uint64_t)capacity * kHidden * 4);
  out->row_ptr = take((uint64_t)capacity * 8);
  out->tables = take(sizeof(EpTables));
  out->total = o;
  return 0;
}

int ep_check_shape(uint32_t world, uint32_t max_tokens, uint32_t capacity) {
  if (world == 0 || world > (uint32_t)kEpMaxRanks || kRouted % world != 0) return fail("expert parallelism: world must divide 256 and be at most 16");
  if (max_tokens == 0 || max_tokens > (1u << 20)) return fail("expert parallelism: max_tokens out of range");
  if (capacity < max_tokens || capacity > (1u << 24)) return fail("expert parallelism: row_capacity must hold at least the rank's own tokens");
  return 0;
}

// FP16 partial rows are a contract of the token-major GEMM form (calls whose experts hold many rows), as in the one-GPU layer
bool ep_f16_call(const netra_ep_layer* L, uint32_t pairs) {
  return L->partial_f16 && L->tokmajor_ok && use_tokmajor(L->route->device, (uint64_t)L->desc.world * pairs, kRouted);
}

int ep_launch_stage(netra_ep_layer* L, uint32_t stage, const void* hidden, const float* shared_w, void* out, uint32_t tokens,
                    cudaStream_t stream) {
  const netra_ep_layer_desc_t& d = L->desc;
  const netra_moe_workspace_layout_t& R = L->route->lay;
  uint8_t* ws = (uint8_t*)L->route->desc.workspace;
  const uint32_t pairs = tokens * kTopK;
  switch (stage) {
    case 0: return launch_stage(L->route, 0, hidden, shared_w, out, tokens, stream);
    case 1: return launch_stage(L->route, 1, hidden, shared_w, out, tokens, stream);
    case 2:
      for (uint32_t s = 2; s <= 4; ++s)
        if (int rc = launch_stage(L->route, s, hidden, shared_w, out, tokens, stream)) return rc;
      break;
    case 3:
      netra_ep_publish_counts_sm100<<<1, 288, 0, stream>>>(L->peers, L->wl, L->tab, (const int32_t*)(ws + R.counts), tokens, d.world, d.rank);
      break;
    case 4:
      netra_ep_plan_sm100<<<1, 1024, 0, stream>>>(L->window, L->wl, L->tab, d.world, d.rank, d.row_capacity, d.wait_timeout_ns);
      break;
    case 5:
      netra_ep_push_rows_sm100<<<((pairs + tokens + 1) / 2 + 7) / 8, 256, 0, stream>>>(
          L->peers, L->wl, L->tab, ws + R.a_fp8, (const float*)(ws + R.a_scale), (const int32_t*)(ws + R.perm),
          (const int32_t*)(ws + R.topk_ids), (const int32_t*)(ws + R.offsets), tokens, d.world, d.rank, d.row_capacity, L->row_ptr,
          L->blk_down, d.max_tokens, ep_f16_call(L, pairs) ? 1u : 0u);
      break;
    case 6:
      // the pairs of all ranks (equal token counts assumed) spread over 256 routed experts decide the GEMM form
      if (L->tokmajor_ok && use_tokmajor(L->route->device, (uint64_t)d.world * pairs, kRouted))
        netra_ep_gate_up_tokmajor_sm100<<<L->sm_count, kTmThreads, gate_up_tokmajor_smem_bytes(), stream>>>(
            L->tm_w13, L->tm_a128, (const float*)(L->window + L->wl.blk_as), d.w13_scale_f32, L->tab->offsets, L->blk_h, L->blk_hs,
            L->e_l + 1, d.weights_tiled, L->tab->status, L->window, L->wl, L->tab, d.world, d.wait_timeout_ns);
      else
        netra_ep_gate_up_umma_sm100<<<L->sm_count, kGemmThreads, gate_up_smem_bytes(), stream>>>(
            L->tm_w13, L->tm_a32, L->tm_a64, L->tm_a128, (const float*)(L->window + L->wl.blk_as), d.w13_scale_f32, L->tab->offsets,
            L->blk_h, L->blk_hs, L->e_l + 1, d.weights_tiled, L->tab->status, L->window, L->wl, L->tab, d.world, d.wait_timeout_ns);
      break;
    case 7:
      if (ep_f16_call(L, pairs)) {
        // the prefill contract: the token-major kernel of the one-GPU layer, its FP16 rows leaving run by run for their senders
        F16RowReturn ret;
        memset(&ret, 0, sizeof ret);
        ret.row_dst = reinterpret_cast<const int2*>(L->row_ptr);
        ret.tokens_of_rank = reinterpret_cast<const int32_t*>(L->window + L->wl.matrix) + kRouted;
        ret.tokens_pitch = kEpMatrixPitch;
        for (uint32_t g = 0; g < d.world; ++g) ret.base[g] = L->peers.win[g] + L->wl.down;
        netra_ep_down_return_tokmajor_f16_sm100<<<L->sm_count, kTmThreads, down_tokmajor_f16_smem_bytes(), stream>>>(
            L->tm_w2, L->tm_h128, L->blk_hs, d.w2_scale_f32, L->tab->offsets, ret, L->e_l + 1, d.weights_tiled, L->tab->status + 1,
            L->peers, L->wl, L->tab, d.world, d.rank);
        break;
      }
      // Across GPUs the swap-AB form is kept for the FP32-row down projection whatever the size: its epilogue stores 128
      // contiguous bytes of one row per warp instruction, while a token-major thread owns a whole row and a warp
      // instruction scatters 32-byte pieces over 32 rows - over NVLink that took three times as long (8 GPUs,
      // 64 rows per expert: 77 us against 25 us of GEMM time).
      if (L->tokmajor_ok && d.world == 1 && use_tokmajor(L->route->device, (uint64_t)d.world * pairs, kRouted))
        netra_ep_down_return_tokmajor_sm100<<<L->sm_count, kTmThreads, down_tokmajor_smem_bytes(), stream>>>(
            L->tm_w2, L->tm_h128, L->blk_hs, d.w2_scale_f32, L->tab->offsets, L->row_ptr, L->e_l + 1, d.weights_tiled,
            L->tab->status + 1, L->peers, L->wl, L->tab, d.world, d.rank);
      else
        netra_ep_down_return_umma_sm100<<<L->sm_count, kGemmThreads, down_smem_bytes(), stream>>>(
            L->tm_w2, L->tm_h32, L->tm_h64, L->tm_h128, L->blk_hs, d.w2_scale_f32, L->tab->offsets, L->row_ptr, L->e_l + 1,
            d.weights_tiled, L->tab->status + 1, L->peers, L->wl, L->tab, d.world, d.rank);
      break;
    default:
      if (ep_f16_call(L, pairs)) {
        netra_ep_combine_f16_sm100<<<tokens, 256, 0, stream>>>((uint16_t*)out, (const __half*)(L->window + L->wl.down),
                                                               (const float*)(ws + R.topk_weights), (const int32_t*)(ws + R.inv_perm),
                                                               tokens, L->window, L->wl, L->tab, d.world, d.wait_timeout_ns);
        break;
      }
      netra_ep_combine_sm100<<<tokens, 256, 0, stream>>>((uint16_t*)out, (const float*)(L->window + L->wl.down),
                                                         (const float*)(ws + R.topk_weights), (const int32_t*)(ws + R.inv_perm), tokens,
                                                         L->window, L->wl, L->tab, d.world, d.wait_timeout_ns);
      break;
  }
  return 0;
}

}  // namespace

extern "C" {

int netra_ep_sizes_query(uint32_t world, uint32_t max_tokens, uint32_t row_capacity, uint64_t* workspace_bytes, uint64_t* window_bytes) {
  if (!workspace_bytes || !window_bytes) return fail("ep_sizes_query: null pointer");
  if (int rc = ep_check_shape(world, max_tokens, row_capacity)) return rc;
  EpWorkspaceLayout w;
  if (int rc = ep_workspace_layout(max_tokens, row_capacity, &w)) return rc;
  *workspace_bytes = w.total;
  *window_bytes = ep_window_layout(world, max_tokens, row_capacity).total;
  return 0;
}

int netra_ep_window_create(uint64_t bytes, void** window, void* ipc_handle_64) {
  if (!window || !ipc_handle_64 || bytes == 0) return fail("ep_window_create: null pointer or zero size");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the exported handle is 64 bytes");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return fail_cuda("ep_window_create: cudaMalloc", e);
  e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) { cudaFree(p); return fail_cuda("ep_window_create: cudaMemset", e); }
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaFree(p); return fail_cuda("ep_window_create: cudaIpcGetMemHandle", e); }
  memcpy(ipc_handle_64, &h, 64);
  *window = p;
  return 0;
}

int netra_ep_window_open(const void* ipc_handle_64, void** window) {
  if (!ipc_handle_64 || !window) return fail("ep_window_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle_64, 64);
  cudaError_t e = cudaIpcOpenMemHandle(window, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : fail_cuda("ep_window_open: cudaIpcOpenMemHandle", e);
}

int netra_ep_window_close(void* window) {
  if (!window) return 0;
  cudaError_t e = cudaIpcCloseMemHandle(window);
  return e == cudaSuccess ? 0 : fail_cuda("ep_window_close: cudaIpcCloseMemHandle", e);
}

int netra_ep_window_destroy(void* window) {
  if (!window) return 0;
  cudaError_t e = cudaFree(window);
  return e == cudaSuccess ? 0 : fail_cuda("ep_window_destroy: cudaFree", e);
}

int netra_ep_layer_create(const netra_ep_layer_desc_t* desc, netra_ep_layer_t** output) {
  if (!desc || !output || desc->struct_size != sizeof(netra_ep_layer_desc_t)) return fail("ep_layer_create: bad struct_size");
  if (int rc = ep_check_shape(desc->world, desc->max_tokens, desc->row_capacity)) return rc;
  if (desc->rank >= desc->world) return fail("ep_layer_create: rank out of range");
  if (!desc->router_weight_bf16 || !desc->w13_fp8 || !desc->w13_scale_f32 || !desc->w2_fp8 || !desc->w2_scale_f32 || !desc->workspace ||
      !desc->windows)
    return fail("ep_layer_create: null pointer");
  if (desc->weights_tiled > 1) return fail("ep_layer_create: weights_tiled must be 0 or 1 (the expert-parallel kernels take E4M3 weights)");
  if (desc->wait_timeout_ns == 0) return fail("ep_layer_create: wait_timeout_ns must be positive (every wait is bounded)");
  for (uint32_t g = 0; g < desc->world; ++g)
    if (!desc->windows[g] || ((uintptr_t)desc->windows[g] & 1023) != 0) return fail("ep_layer_create: every window must be a 1024-byte aligned pointer");
  EpWorkspaceLayout wsl;
  if (int rc = ep_workspace_layout(desc->max_tokens, desc->row_capacity, &wsl)) return rc;
  const EpWindowLayout wl = ep_window_layout(desc->world, desc->max_tokens, desc->row_capacity);
  if (desc->workspace_bytes < wsl.total) return fail("ep_layer_create: workspace too small (netra_ep_sizes_query)");
  if (desc->window_bytes < wl.total) return fail("ep_layer_create: windows too small (netra_ep_sizes_query)");
  if (((uintptr_t)desc->workspace & 1023) != 0) return fail("ep_layer_create: workspace must be 1024-byte aligned");
  netra_ep_layer* L = new (std::nothrow) netra_ep_layer;
  if (!L) return fail("ep_layer_create: out of host memory");
  L->desc = *desc;
  L->desc.windows = nullptr;       // the pointers are copied below; the caller's array need not outlive this call
  L->e_l = kRouted / desc->world;
  L->partial_f16 = false;
  L->wl = wl;
  memset(&L->peers, 0, sizeof L->peers);
  for (uint32_t g = 0; g < desc->world; ++g) L->peers.win[g] = (uint8_t*)desc->windows[g];
  L->window = L->peers.win[desc->rank];
  uint8_t* ws = (uint8_t*)desc->workspace;
  L->blk_h = ws + wsl.blk_h;
  L->blk_hs = (float*)(ws + wsl.blk_hs);
  L->blk_down = (float*)(ws + wsl.blk_down);
  L->row_ptr = (float**)(ws + wsl.row_ptr);
  L->tab = (EpTables*)(ws + wsl.tables);
  L->route = nullptr;
  netra_moe_layer_desc_t rd;
  memset(&rd, 0, sizeof rd);
  rd.struct_size = sizeof rd;
  rd.max_tokens = desc->max_tokens;
  rd.router_weight_bf16 = desc->router_weight_bf16;
  rd.router_bias_f32 = desc->router_bias_f32;
  rd.w13_fp8 = desc->w13_fp8;
  rd.w13_scale_f32 = desc->w13_scale_f32;
  rd.w2_fp8 = desc->w2_fp8;
  rd.w2_scale_f32 = desc->w2_scale_f32;
  rd.workspace = ws + wsl.route;
  rd.workspace_bytes = wsl.blk_h - wsl.route;
  rd.weights_tiled = desc->weights_tiled;
  rd.num_expert_slabs = L->e_l + 1;
  int rc = netra_moe_layer_create(&rd, &L->route);
  if (rc) { delete L; return rc; }
  L->sm_count = L->route->sm_count;
  {
    cudaError_t e = cudaFuncSetAttribute(netra_ep_down_return_umma_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, down_smem_bytes());
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(netra_ep_gate_up_umma_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, gate_up_smem_bytes());
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(netra_ep_gate_up_tokmajor_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, gate_up_tokmajor_smem_bytes());
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(netra_ep_down_return_tokmajor_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, down_tokmajor_smem_bytes());
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(netra_ep_down_return_tokmajor_f16_sm100, cudaFuncAttributeMaxDynamicSharedMemorySize, down_tokmajor_f16_smem_bytes());
    cudaFuncAttributes attr, attr_gate_up, attr_f16;
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr_f16, netra_ep_down_return_tokmajor_f16_sm100);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr, netra_ep_down_return_tokmajor_sm100);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr_gate_up, netra_ep_gate_up_tokmajor_sm100);
    if (e != cudaSuccess) { netra_moe_layer_destroy(L->route); delete L; return fail_cuda("cudaFuncSetAttribute(down_return)", e); }
    L->tokmajor_ok = g_tokmajor_ok[L->route->device] && attr.numRegs == kTmRegsLaunch && attr_gate_up.numRegs == kTmRegsLaunch &&
                     attr_f16.numRegs == kTmRegsLaunch;
  }
  const uint64_t g = L->e_l + 1, rows = desc->row_capacity;
  if (desc->weights_tiled) {
    rc = rc ? rc : encode_u8_2d(&L->tm_w13, desc->w13_fp8, g * 2 * kInter * kHiddenBlocks, kBlock, 128);
    rc = rc ? rc : encode_u8_2d(&L->tm_w2, desc->w2_fp8, g * kHidden * kInterBlocks, kBlock, 128);
  } else {
    rc = rc ? rc : encode_u8_2d(&L->tm_w13, desc->w13_fp8, g * 2 * kInter, kHidden, 128);
    rc = rc ? rc : encode_u8_2d(&L->tm_w2, desc->w2_fp8, g * kHidden, kInter, 128);
  }
  uint8_t* blk_a = L->window + wl.blk_a;
  rc = rc ? rc : encode_u8_2d(&L->tm_a32, blk_a, rows, kHidden, 32);
  rc = rc ? rc : encode_u8_2d(&L->tm_a64, blk_a, rows, kHidden, 64);
  rc = rc ? rc : encode_u8_2d(&L->tm_a128, blk_a, rows, kHidden, 128);
  rc = rc ? rc : encode_u8_2d(&L->tm_h32, L->blk_h, rows, kInter, 32);
  rc = rc ? rc : encode_u8_2d(&L->tm_h64, L->blk_h, rows, kInter, 64);
  rc = rc ? rc : encode_u8_2d(&L->tm_h128, L->blk_h, rows, kInter, 128);
  if (rc == 0) {
    cudaError_t e = cudaMemset(L->tab, 0, sizeof(EpTables));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) rc = fail_cuda("ep_layer_create: cudaMemset(tables)", e);
  }
  if (rc) { netra_moe_layer_destroy(L->route); delete L; return rc; }
  *output = L;
  return 0;
}

uint32_t netra_ep_layer_stage_count(void) { return kEpStageCount; }

uint32_t netra_ep_layer_launch_count(const netra_ep_layer_t* L, uint32_t tokens) {
  if (!L) return 0;
  // a whole call runs publish and plan as one launch; above 1,024 tokens the sort is three launches
  if (tokens > (uint32_t)kSortSmallMaxRows) return kEpStageCount - 1 + 2;
  return kEpStageCount - 1 - (L->route->front_mode == 1 ? 2 : 0);                       // router, top-k and sort as one launch
}

int netra_ep_layer_launch(netra_ep_layer_t* L, const void* hidden, const float* shared_w, void* out, uint32_t tokens, cudaStream_t stream) {
  if (!L || !hidden || !out) return fail("ep_layer_launch: null pointer");
  if (tokens == 0 || tokens > L->desc.max_tokens) return fail("ep_layer_launch: tokens exceed the bound capacity");
  for (uint32_t s = 0; s < kEpStageCount; ++s) {
    if (s == 3) {      // publish and plan in one launch: this rank's GPU is its own, the peers' flags arrive while it waits
      const netra_ep_layer_desc_t& d = L->desc;
      const uint8_t* ws = (const uint8_t*)L->route->desc.workspace;
      netra_ep_publish_plan_sm100<<<1, 1024, 0, stream>>>(L->peers, L->wl, L->tab, (const int32_t*)(ws + L->route->lay.counts), tokens,
                                                          d.world, d.rank, d.row_capacity, d.wait_timeout_ns);
      ++s;             // stage 4 (plan) is done
      continue;
    }
    if (int rc = ep_launch_stage(L, s, hidden, shared_w, out, tokens, stream)) return rc;
  }
  return check_launch("ep_layer launch");
}

int netra_ep_layer_launch_stage(netra_ep_layer_t* L, uint32_t stage, const void* hidden, const float* shared_w, void* out,
                                uint32_t tokens, cudaStream_t stream) {
  if (!L || !hidden || !out) return fail("ep_layer_launch_stage: null pointer");
  if (tokens == 0 || tokens > L->desc.max_tokens) return fail("ep_layer_launch_stage: tokens exceed the bound capacity");
  if (stage >= kEpStageCount) return fail("ep_layer_launch_stage: stage out of range");
  if (int rc = ep_launch_stage(L, stage, hidden, shared_w, out, tokens, stream)) return rc;
  return check_launch("ep_layer stage launch");
}

int netra_ep_layer_set_partial_format(netra_ep_layer_t* L, uint32_t format) {
  if (L == nullptr || format > 1) return fail("ep_layer_set_partial_format: null layer or unknown format");
  L->partial_f16 = format == 1;
  return 0;
}

int netra_ep_layer_status(netra_ep_layer_t* L, uint32_t status_out[4]) {
  if (!L || !status_out) return fail("ep_layer_status: null pointer");
  cudaError_t e = cudaMemcpy(status_out, L->tab->status, 16, cudaMemcpyDeviceToHost);
  return e == cudaSuccess ? 0 : fail_cuda("ep_layer_status: cudaMemcpy", e);
}

int netra_ep_layer_destroy(netra_ep_layer_t* L) {
  if (L) {
    netra_moe_layer_destroy(L->route);
    delete L;
  }
  return 0;
}

}  // extern "C"

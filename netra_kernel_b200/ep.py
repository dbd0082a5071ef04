"""Expert parallelism for the routed-MoE layer: contiguous blocks of ``256 / G`` routed experts per
GPU, router and shared expert replicated, tokens block-sharded, one all-to-all each way.

The reference has no expert parallelism (its 8-GPU mode is eight replicas,
``manifests/gfx950/models/qwen36-moe-m1-golden.json:11-12``); this module is new design.

Per layer call on rank r (``T_l`` local tokens, ``P_l = 8 T_l`` pairs, ``E_l = 256 / G``):

1. route locally over all 256 experts (router, top-8, sort, gather): the sorted rows are already
   grouped by owner rank because experts are owned in contiguous blocks;
2. exchange per-expert counts (all-to-all of ``[G, E_l]`` int32), read the split sizes on the host;
3. dispatch the sorted FP8 rows and their scales (all-to-all, variable splits);
4. regroup the received rows from source-major to expert-major, append the local tokens as the
   shared expert's rows, run the grouped gate_up and down kernels over ``E_l + 1`` slabs;
5. return the FP32 down rows in the order they arrived (all-to-all), which is the sender's own
   sorted order, and combine them slot by slot exactly as on one GPU.

``ExpertParallelPlan`` holds the host logic and the collectives and works on CPU tensors (gloo) as
well; ``ExpertParallelMoELayer`` adds the sm_100a kernels.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from .synth import HIDDEN, INTER, N_ROUTED, TOPK


@dataclass
class Splits:
    send: list[int]        # rows this rank sends to each rank
    recv: list[int]        # rows this rank receives from each rank

    @property
    def total_recv(self) -> int:
        return sum(self.recv)


class ExpertParallelPlan:
    """Ownership, count exchange, variable all-to-all and the source-major -> expert-major index."""

    def __init__(self, world_size: int, rank: int, group=None, n_routed: int = N_ROUTED):
        if world_size < 1 or n_routed % world_size:
            raise ValueError("the routed experts must divide evenly over the ranks")
        if not 0 <= rank < world_size:
            raise ValueError("rank out of range")
        self.world, self.rank, self.group = world_size, rank, group
        self.n_routed = n_routed
        self.experts_per_rank = n_routed // world_size

    def owner(self, expert: int) -> int:
        return expert // self.experts_per_rank

    def local_expert_range(self) -> range:
        return range(self.rank * self.experts_per_rank, (self.rank + 1) * self.experts_per_rank)

    # ------------------------------------------------------------------ collectives
    def exchange_counts(self, counts: torch.Tensor) -> torch.Tensor:
        """counts int32 [n_routed] (pairs of this rank per global expert) -> int32 [world, E_l]:
        row s = pairs that rank s sends here, per local expert."""
        if counts.numel() != self.n_routed or counts.dtype != torch.int32:
            raise ValueError("counts must be int32 [n_routed]")
        recv = torch.empty(self.world * self.experts_per_rank, dtype=torch.int32, device=counts.device)
        if self.world == 1:
            recv.copy_(counts)
        else:
            dist.all_to_all_single(recv, counts.contiguous(), group=self.group)
        return recv.view(self.world, self.experts_per_rank)

    def splits(self, counts: torch.Tensor, recv_counts: torch.Tensor) -> Splits:
        """Host split sizes (one device->host read).  Validates them before any payload collective."""
        both = torch.stack([counts.view(self.world, self.experts_per_rank).sum(1), recv_counts.sum(1)]).cpu()
        send, recv = both[0].tolist(), both[1].tolist()
        if min(send + recv) < 0:
            raise ValueError("negative row count in the expert-parallel exchange")
        return Splits([int(v) for v in send], [int(v) for v in recv])

    def all_to_all_rows(self, rows: torch.Tensor, send: list[int], recv: list[int], out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """rows [sum(send), B] -> [sum(recv), B]; rank-major on both sides."""
        if rows.shape[0] != sum(send):
            raise ValueError(f"payload has {rows.shape[0]} rows but the split sizes add up to {sum(send)}")
        total = sum(recv)
        if out is None:
            out = torch.empty((total,) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
        elif out.shape[0] != total:
            raise ValueError("output buffer does not match the receive split sizes")
        if self.world == 1:
            out.copy_(rows)
        else:
            dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=recv, input_split_sizes=send, group=self.group)
        return out

    # ------------------------------------------------------------------ index math (torch reference)
    def regroup_reference(self, recv_counts: torch.Tensor, extra_rows: int):
        """Same result as ``netra_ep_regroup_launch``: (index [R] source-major -> expert-major,
        offsets [E_l + 2])."""
        c = recv_counts.to(torch.int64).cpu()                       # [world, E_l]
        flat = c.reshape(-1)
        src_base = torch.cumsum(flat, 0) - flat
        per_expert = c.sum(0)
        expert_base = torch.cumsum(per_expert, 0) - per_expert
        within = torch.cumsum(c, 0) - c                              # rows of earlier sources, same expert
        dst_base = (expert_base[None, :] + within).reshape(-1)
        total = int(flat.sum())
        bucket = torch.repeat_interleave(torch.arange(flat.numel()), flat)
        index = dst_base[bucket] + (torch.arange(total) - src_base[bucket])
        offsets = torch.cat([expert_base, torch.tensor([total, total + extra_rows])])
        return index.to(torch.int32), offsets.to(torch.int32)


class ExpertParallelMoELayer:
    """One rank of the expert-parallel layer on a B200.  ``w13`` etc. hold this rank's
    ``E_l`` routed slabs followed by the (replicated) shared expert's slab."""

    def __init__(self, plan: ExpertParallelPlan, router_w, w13, w13_scale, w2, w2_scale, max_local_tokens: int,
                 router_bias=None, tiled: bool = True, max_recv_rows: Optional[int] = None):
        from . import abi
        from .moe import RoutedMoELayer
        self.plan, self.abi, self.lib = plan, abi, abi.load()
        e_l = plan.experts_per_rank
        if w13.shape[0] != e_l + 1:
            raise ValueError(f"this rank holds {e_l} routed slabs + the shared slab, got {w13.shape[0]}")
        dev = router_w.device
        self.device, self.t_max = dev, int(max_local_tokens)
        # routing stages (0-5) and the combine (8) of the single-GPU layer, on the local tokens
        self.route = RoutedMoELayer(router_w, w13, w13_scale, w2, w2_scale, self.t_max, router_bias, tiled=tiled,
                                    routing_only=True)
        w13, w2 = self.route._keep[1], self.route._keep[3]           # the copies the kernels read (tile order if tiled)
        pairs = self.t_max * TOPK
        # worst case every pair of every rank lands here; callers with tighter knowledge pass max_recv_rows
        self.r_max = int(max_recv_rows) if max_recv_rows else pairs * plan.world
        rows = self.r_max + self.t_max
        u8, f32, i32 = torch.uint8, torch.float32, torch.int32
        self.blk_a = torch.zeros(rows, HIDDEN, dtype=u8, device=dev)
        self.blk_as = torch.zeros(rows + 64, HIDDEN // 128, dtype=f32, device=dev)
        self.blk_h = torch.zeros(rows, INTER, dtype=u8, device=dev)
        self.blk_hs = torch.zeros(rows + 64, INTER // 128, dtype=f32, device=dev)
        self.blk_down = torch.zeros(rows, HIDDEN, dtype=f32, device=dev)
        self.recv_a = torch.empty(self.r_max, HIDDEN, dtype=u8, device=dev)
        self.recv_as = torch.empty(self.r_max, HIDDEN // 128, dtype=f32, device=dev)
        self.back = torch.empty(self.r_max, HIDDEN, dtype=f32, device=dev)
        n_bucket = plan.world * e_l
        self.src_base = torch.zeros(n_bucket, dtype=i32, device=dev)
        self.dst_base = torch.zeros(n_bucket, dtype=i32, device=dev)
        self.offsets = torch.zeros(e_l + 2, dtype=i32, device=dev)
        self.index = torch.zeros(self.r_max, dtype=i32, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        desc = abi.ExpertBlockDesc()
        desc.struct_size = ctypes.sizeof(desc)
        desc.num_groups, desc.max_rows, desc.weights_tiled = e_l + 1, rows, int(tiled)
        desc.w13_fp8, desc.w13_scale_f32 = w13.data_ptr(), w13_scale.data_ptr()
        desc.w2_fp8, desc.w2_scale_f32 = w2.data_ptr(), w2_scale.data_ptr()
        desc.a_fp8, desc.a_scale_f32 = self.blk_a.data_ptr(), self.blk_as.data_ptr()
        desc.h_fp8, desc.h_scale_f32 = self.blk_h.data_ptr(), self.blk_hs.data_ptr()
        desc.down_f32, desc.offsets_i32, desc.status_u32 = self.blk_down.data_ptr(), self.offsets.data_ptr(), self.status.data_ptr()
        handle = ctypes.c_void_p()
        abi.check(self.lib.netra_moe_expert_block_create(ctypes.byref(desc), ctypes.byref(handle)), "expert_block_create")
        self.block = handle
        self._keep = (w13, w13_scale, w2, w2_scale)
        self.last_splits: Optional[Splits] = None

    def _stream(self) -> int:
        return torch.cuda.current_stream().cuda_stream

    def _move(self, dst, src, index, rows: int, row_bytes: int, scatter: bool) -> None:
        self.abi.check(self.lib.netra_moe_move_rows_launch(dst.data_ptr(), src.data_ptr(), index.data_ptr(), rows, row_bytes,
                                                           int(scatter), self._stream()), "move_rows_launch")

    def __call__(self, hidden: torch.Tensor, shared_weight: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        plan, route = self.plan, self.route
        t_l = hidden.shape[0]
        p_l = t_l * TOPK
        if t_l > self.t_max:
            raise ValueError("more local tokens than the layer was sized for")
        if out is None:
            out = torch.empty_like(hidden)
        for stage in range(6):                                        # router .. gather, local tokens, 256 experts
            route.launch_stage(stage, hidden, out, shared_weight)
        launches = route.launches_per_call(t_l) - 3                   # this library's kernels launched by the call
        inter = route.intermediates(t_l)
        recv_counts = plan.exchange_counts(inter["counts"])
        splits = plan.splits(inter["counts"], recv_counts)            # the one host read-back of the call
        self.last_splits = splits
        r = splits.total_recv
        if r > self.r_max:
            raise RuntimeError(f"{r} rows arrive but the receive buffers hold {self.r_max}")
        # dispatch: the sorted rows are already grouped by owner rank
        plan.all_to_all_rows(inter["a_fp8"][:p_l], splits.send, splits.recv, out=self.recv_a[:r])
        plan.all_to_all_rows(inter["a_scale"][:p_l], splits.send, splits.recv, out=self.recv_as[:r])
        self.abi.check(self.lib.netra_ep_regroup_launch(self.src_base.data_ptr(), self.dst_base.data_ptr(), self.offsets.data_ptr(),
                                                        self.index.data_ptr(), recv_counts.data_ptr(), plan.world,
                                                        plan.experts_per_rank, t_l, r, self._stream()), "ep_regroup_launch")
        launches += 2 if r else 1
        if r:
            self._move(self.blk_a, self.recv_a, self.index, r, HIDDEN, scatter=True)
            self._move(self.blk_as, self.recv_as, self.index, r, HIDDEN // 128 * 4, scatter=True)
            launches += 3
        self.blk_a[r:r + t_l].copy_(inter["a_fp8"][p_l:p_l + t_l])    # the shared expert's rows: the local tokens
        self.blk_as[r:r + t_l].copy_(inter["a_scale"][p_l:p_l + t_l])
        self.abi.check(self.lib.netra_moe_expert_block_launch(self.block, self._stream()), "expert_block_launch")
        # return: back into the order the rows arrived in, which is each sender's own sorted order
        if r:
            self._move(self.back, self.blk_down, self.index, r, HIDDEN * 4, scatter=False)
        plan.all_to_all_rows(self.back[:r], splits.recv, splits.send, out=inter["down"][:p_l])
        inter["down"][p_l:p_l + t_l].copy_(self.blk_down[r:r + t_l])
        route.launch_stage(8, hidden, out, shared_weight)             # slot-ordered combine, as on one GPU
        self.launches_last_call = launches + 3                        # gate_up, down, combine
        return out

    def launch_expert_block(self) -> None:
        """The two grouped GEMMs over the rows of the last call (for isolated timing)."""
        self.abi.check(self.lib.netra_moe_expert_block_launch(self.block, self._stream()), "expert_block_launch")

    def check_status(self) -> None:
        words = self.status.cpu().tolist()
        if any(words):
            raise self.abi.NetraError(f"device status words {words}: a bounded wait expired inside a grouped GEMM")

    def close(self) -> None:
        if getattr(self, "block", None):
            self.lib.netra_moe_expert_block_destroy(self.block)
            self.block = None
        self.route.close()


def shard_expert_weights(weights, plan: ExpertParallelPlan):
    """(w13, w13_scale, w2, w2_scale) with 257 slabs -> this rank's E_l routed slabs + the shared slab."""
    lo, hi = plan.local_expert_range().start, plan.local_expert_range().stop
    return tuple(torch.cat([t[lo:hi], t[-1:]]).contiguous() for t in weights)

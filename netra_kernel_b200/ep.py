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
    def regroup_reference(self, recv_counts: torch.Tensor, extra_rows: int, slot_rows: int = 0, shared_first: bool = False):
        """Same result as ``netra_ep_regroup_launch``: (index source-major -> expert-major with -1 for
        unused slot rows, offsets [E_l + 2])."""
        c = recv_counts.to(torch.int64).cpu()                       # [world, E_l]
        world, e_l = c.shape
        if slot_rows:                                                # a sender never delivers more than one slot
            start = torch.cumsum(c, 1) - c
            c = torch.clamp(torch.clamp(start + c, max=slot_rows) - torch.clamp(start, max=slot_rows), min=0)
        per_expert = c.sum(0)
        base = extra_rows if shared_first else 0
        expert_base = torch.cumsum(per_expert, 0) - per_expert + base
        within_expert = torch.cumsum(c, 0) - c                       # rows of earlier sources, same expert
        dst_base = expert_base[None, :] + within_expert              # [world, E_l]
        total = int(c.sum())
        rows = world * slot_rows if slot_rows else total
        index = torch.full((rows,), -1, dtype=torch.int64)
        pos = 0
        for s in range(world):
            if slot_rows:
                pos = s * slot_rows
            for e in range(e_l):
                n = int(c[s, e])
                index[pos:pos + n] = dst_base[s, e] + torch.arange(n)
                pos += n
        if shared_first:
            offsets = torch.cat([torch.tensor([0]), expert_base, torch.tensor([base + total])])
        else:
            offsets = torch.cat([expert_base, torch.tensor([total, total + extra_rows])])
        return index.to(torch.int32), offsets.to(torch.int32)

    def slot_rows_for(self, local_tokens: int, headroom: float = 8.0) -> int:
        """Fixed capacity per (source, destination) pair: the mean of near-uniform routing plus
        ``headroom`` standard deviations, rounded up to 64 rows and never more than all pairs."""
        pairs = local_tokens * TOPK
        if self.world == 1:
            return pairs
        p = 1.0 / self.world
        mean, sd = pairs * p, (pairs * p * (1 - p)) ** 0.5
        return min(pairs, int(-(-(mean + headroom * sd + 32) // 64) * 64))


EP_ROW_BYTES = HIDDEN + HIDDEN // 128 * 4      # FP8 codes followed by the 16 FP32 scales


class ExpertParallelMoELayer:
    """One rank of the expert-parallel layer on a B200.  ``w13`` etc. hold the (replicated) shared
    expert's slab FIRST, then this rank's ``E_l`` routed slabs (``shard_expert_weights``).

    ``exchange="fixed"`` (default) moves a fixed number of slot rows per rank pair, so a call is
    enqueued without any host read-back and can be captured into a CUDA graph; a destination that
    would need more rows than a slot holds is reported by ``check_status``.  ``exchange="exact"``
    reads the split sizes on the host once per call and moves exactly the routed rows."""

    def __init__(self, plan: ExpertParallelPlan, router_w, w13, w13_scale, w2, w2_scale, max_local_tokens: int,
                 router_bias=None, tiled: bool = True, exchange: str = "fixed", slot_rows: Optional[int] = None):
        from . import abi
        from .moe import RoutedMoELayer
        if exchange not in ("fixed", "exact"):
            raise ValueError("exchange must be 'fixed' or 'exact'")
        self.plan, self.abi, self.lib, self.exchange = plan, abi, abi.load(), exchange
        e_l, world = plan.experts_per_rank, plan.world
        if w13.shape[0] != e_l + 1:
            raise ValueError(f"this rank holds the shared slab + {e_l} routed slabs, got {w13.shape[0]}")
        dev = router_w.device
        self.device, self.t_max = dev, int(max_local_tokens)
        # routing stages (0-5) and the combine (8) of the single-GPU layer, on the local tokens (NCCL arm)
        self.route = RoutedMoELayer(router_w, w13, w13_scale, w2, w2_scale, self.t_max, router_bias, tiled=tiled,
                                    routing_only=True)
        w13, w2 = self.route._keep[1], self.route._keep[3]           # the copies the kernels read (tile order if tiled)
        pairs = self.t_max * TOPK
        self.slot_rows = int(slot_rows) if slot_rows else (plan.slot_rows_for(self.t_max) if exchange == "fixed" else pairs)
        self.r_max = self.slot_rows * world                          # rows that can arrive here
        rows = self.r_max + self.t_max
        u8, f32, i32 = torch.uint8, torch.float32, torch.int32
        self.blk_a = torch.zeros(rows, HIDDEN, dtype=u8, device=dev)
        self.blk_as = torch.zeros(rows + 64, HIDDEN // 128, dtype=f32, device=dev)
        self.blk_h = torch.zeros(rows, INTER, dtype=u8, device=dev)
        self.blk_hs = torch.zeros(rows + 64, INTER // 128, dtype=f32, device=dev)
        self.blk_down = torch.zeros(rows, HIDDEN, dtype=f32, device=dev)
        self.send = torch.zeros(self.r_max, EP_ROW_BYTES, dtype=u8, device=dev)
        self.recv = torch.zeros(self.r_max, EP_ROW_BYTES, dtype=u8, device=dev)
        self.back = torch.zeros(self.r_max, HIDDEN, dtype=f32, device=dev)
        self.back_recv = torch.zeros(self.r_max, HIDDEN, dtype=f32, device=dev)
        self.recv_counts = torch.zeros(world * e_l, dtype=i32, device=dev)
        n_bucket = world * e_l
        self.src_base = torch.zeros(n_bucket, dtype=i32, device=dev)
        self.dst_base = torch.zeros(n_bucket, dtype=i32, device=dev)
        self.offsets = torch.zeros(e_l + 2, dtype=i32, device=dev)
        self.index = torch.full((self.r_max,), -1, dtype=i32, device=dev)
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)   # [gate_up, down, slot overflow, unused]
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
        self.launches_last_call = 0

    def _stream(self) -> int:
        return torch.cuda.current_stream().cuda_stream

    def _move(self, dst, src, rows, copy_bytes, dst_pitch, src_pitch, dst_col, src_col, scatter) -> None:
        self.abi.check(self.lib.netra_moe_move_rows_launch(dst.data_ptr(), src.data_ptr(), self.index.data_ptr(), rows, copy_bytes,
                                                           dst_pitch, src_pitch, dst_col, src_col, int(scatter), self._stream()),
                       "move_rows_launch")

    def __call__(self, hidden: torch.Tensor, shared_weight: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        plan, route, lib, check = self.plan, self.route, self.lib, self.abi.check
        world, e_l = plan.world, plan.experts_per_rank
        t_l = hidden.shape[0]
        p_l = t_l * TOPK
        if t_l > self.t_max:
            raise ValueError("more local tokens than the layer was sized for")
        if out is None:
            out = torch.empty_like(hidden)
        for stage in range(6):                                        # router .. gather, local tokens, 256 experts
            route.launch_stage(stage, hidden, out, shared_weight)
        inter = route.intermediates(t_l)
        fixed = self.exchange == "fixed"
        slot = self.slot_rows if fixed else 0
        # ---- dispatch
        recv_counts = plan.exchange_counts(inter["counts"])
        if fixed:
            check(lib.netra_ep_pack_rows_launch(self.send.data_ptr(), inter["a_fp8"].data_ptr(), inter["a_scale"].data_ptr(),
                                                inter["offsets"].data_ptr(), world, e_l, slot, self.status[2:].data_ptr(),
                                                self._stream()), "ep_pack_rows_launch")
            equal = [slot] * world
            plan.all_to_all_rows(self.send, equal, equal, out=self.recv)
            arrived = self.r_max
        else:
            splits = plan.splits(inter["counts"], recv_counts)        # the one host read-back of the call
            self.last_splits = splits
            arrived = splits.total_recv
            if arrived > self.r_max:
                raise RuntimeError(f"{arrived} rows arrive but the receive buffers hold {self.r_max}")
            packed = torch.cat([inter["a_fp8"][:p_l], inter["a_scale"][:p_l].view(torch.uint8).view(p_l, -1)], dim=1)
            plan.all_to_all_rows(packed, splits.send, splits.recv, out=self.recv[:arrived])
        # ---- regroup source-major -> expert-major; the shared expert's rows (local tokens) are group 0
        check(lib.netra_ep_regroup_launch(self.src_base.data_ptr(), self.dst_base.data_ptr(), self.offsets.data_ptr(),
                                          self.index.data_ptr(), recv_counts.data_ptr(), world, e_l, t_l, arrived, slot, 1,
                                          self._stream()), "ep_regroup_launch")
        if arrived:
            self._move(self.blk_a, self.recv, arrived, HIDDEN, HIDDEN, EP_ROW_BYTES, 0, 0, scatter=True)
            self._move(self.blk_as, self.recv, arrived, HIDDEN // 128 * 4, HIDDEN // 128 * 4, EP_ROW_BYTES, 0, HIDDEN, scatter=True)
        self.blk_a[:t_l].copy_(inter["a_fp8"][p_l:p_l + t_l])
        self.blk_as[:t_l].copy_(inter["a_scale"][p_l:p_l + t_l])
        check(lib.netra_moe_expert_block_launch(self.block, self._stream()), "expert_block_launch")
        # ---- return the FP32 rows in arrival order, which is each sender's own sorted order
        if arrived:
            self._move(self.back, self.blk_down, arrived, HIDDEN * 4, HIDDEN * 4, HIDDEN * 4, 0, 0, scatter=False)
        if fixed:
            equal = [slot] * world
            plan.all_to_all_rows(self.back, equal, equal, out=self.back_recv)
            check(lib.netra_ep_unpack_rows_launch(inter["down"].data_ptr(), self.back_recv.data_ptr(), inter["offsets"].data_ptr(),
                                                  world, e_l, slot, self._stream()), "ep_unpack_rows_launch")
        else:
            plan.all_to_all_rows(self.back[:arrived], splits.recv, splits.send, out=inter["down"][:p_l])
        inter["down"][p_l:p_l + t_l].copy_(self.blk_down[:t_l])
        route.launch_stage(8, hidden, out, shared_weight)             # slot-ordered combine, as on one GPU
        self.launches_last_call = route.launches_per_call(t_l) - 2 + 2 + (3 if arrived else 0) + (2 if fixed else 0) + 2
        return out

    def launch_expert_block(self) -> None:
        """The two grouped GEMMs over the rows of the last call (for isolated timing)."""
        self.abi.check(self.lib.netra_moe_expert_block_launch(self.block, self._stream()), "expert_block_launch")

    def check_status(self) -> None:
        words = self.status.cpu().tolist()
        if words[2]:
            raise self.abi.NetraError(f"a destination rank needed {words[2]} rows but a slot holds {self.slot_rows}: "
                                      "construct the layer with a larger slot_rows or exchange='exact'")
        if any(words[:2]):
            raise self.abi.NetraError(f"device status words {words}: a bounded wait expired inside a grouped GEMM")

    def close(self) -> None:
        if getattr(self, "block", None):
            self.lib.netra_moe_expert_block_destroy(self.block)
            self.block = None
        self.route.close()


def shard_expert_weights(weights, plan: ExpertParallelPlan):
    """(w13, w13_scale, w2, w2_scale) with 257 slabs -> the shared slab followed by this rank's E_l routed slabs."""
    lo, hi = plan.local_expert_range().start, plan.local_expert_range().stop
    return tuple(torch.cat([t[-1:], t[lo:hi]]).contiguous() for t in weights)


# ---------------------------------------------------------------------------------------------
# Expert parallelism over peer memory: the library's own kernels move the rows (NVLink stores
# into the peers' windows, epoch flags), no NCCL collective and no host read-back in a call.
# ---------------------------------------------------------------------------------------------
class PeerWindow:
    """Device memory that peer ranks write into.  ``handle`` (64 bytes) lets another process on
    the node open it; ranks in the same process use ``ptr`` directly."""

    def __init__(self, nbytes: int):
        from . import abi
        self.abi, self.lib = abi, abi.load()
        ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        abi.check(self.lib.netra_ep_window_create(nbytes, ctypes.byref(ptr), handle), "ep_window_create")
        self.ptr, self.handle, self.nbytes = ptr.value, handle.raw, nbytes
        self.opened: list[int] = []

    def open_peer(self, handle: bytes) -> int:
        ptr = ctypes.c_void_p()
        self.abi.check(self.lib.netra_ep_window_open(ctypes.create_string_buffer(handle, 64), ctypes.byref(ptr)), "ep_window_open")
        self.opened.append(ptr.value)
        return ptr.value

    def close(self) -> None:
        for p in self.opened:
            self.lib.netra_ep_window_close(p)
        self.opened = []
        if self.ptr:
            self.lib.netra_ep_window_destroy(self.ptr)
            self.ptr = None


def ep_sizes(world: int, max_tokens: int, row_capacity: int) -> tuple[int, int]:
    """(local workspace bytes, window bytes) of one rank."""
    from . import abi
    ws, win = ctypes.c_uint64(), ctypes.c_uint64()
    abi.check(abi.load().netra_ep_sizes_query(world, max_tokens, row_capacity, ctypes.byref(ws), ctypes.byref(win)), "ep_sizes_query")
    return ws.value, win.value


def default_row_capacity(world: int, max_tokens: int, headroom: Optional[float] = None) -> int:
    """Rows of one rank's expert block: its own tokens plus the routed rows of all ranks for its experts.
    Without ``headroom`` this is the worst case (every pair of every rank routed here), which can never
    overflow; with it, the mean of near-uniform routing plus ``headroom`` standard deviations."""
    pairs = world * max_tokens * TOPK
    if world == 1 or headroom is None:
        return max_tokens + pairs
    p = 1.0 / world
    mean, sd = pairs * p, (pairs * p * (1 - p)) ** 0.5
    return max_tokens + min(pairs, int(-(-(mean + headroom * sd + 64) // 64) * 64))


class PeerExpertParallelLayer:
    """One rank of the expert-parallel layer with peer-memory exchange (``netra_ep_layer_*``).

    ``w13`` etc. hold the shared expert's slab first, then this rank's routed slabs
    (``shard_expert_weights``).  ``windows`` is the list of all ranks' window pointers (this rank's
    own at index ``plan.rank``); when it is None the layer creates its window and exchanges the
    handles through ``torch.distributed`` (one process per GPU).  A call enqueues a fixed sequence
    of kernels and may be captured into a CUDA graph; all ranks must make the same calls."""

    def __init__(self, plan: ExpertParallelPlan, router_w, w13, w13_scale, w2, w2_scale, max_local_tokens: int,
                 router_bias=None, tiled: bool = True, row_capacity: Optional[int] = None, wait_timeout_s: float = 2.0,
                 windows: Optional[list[int]] = None, share_with: Optional["PeerExpertParallelLayer"] = None):
        """``share_with``: another layer of the same shape on this rank whose windows, workspace and epoch tables this
        one uses as well - the layers of a stack, which run one after the other on one stream and whose exchanges the
        epoch flags already order exactly as they order repeated calls of one layer.  Create every layer of such a
        group (on every rank) before the first call of any of them."""
        from . import abi
        self.plan, self.abi, self.lib = plan, abi, abi.load()
        world, e_l = plan.world, plan.experts_per_rank
        if w13.shape[0] != e_l + 1:
            raise ValueError(f"this rank holds the shared slab + {e_l} routed slabs, got {w13.shape[0]}")
        dev = router_w.device
        self.device, self.t_max = dev, int(max_local_tokens)
        if share_with is not None:
            if (share_with.t_max, share_with.plan.world, share_with.plan.rank) != (self.t_max, world, plan.rank):
                raise ValueError("layers that share buffers must have the same shape, world and rank")
            row_capacity = share_with.row_capacity
            windows = list(share_with._windows)
        self.row_capacity = int(row_capacity) if row_capacity else default_row_capacity(world, self.t_max)
        ws_bytes, win_bytes = ep_sizes(world, self.t_max, self.row_capacity)
        self.window_bytes = win_bytes
        self.own_window: Optional[PeerWindow] = None
        if windows is None:
            self.own_window = PeerWindow(win_bytes)
            if world > 1:
                handles: list = [None] * world
                dist.all_gather_object(handles, self.own_window.handle, group=plan.group)
                windows = [self.own_window.ptr if g == plan.rank else self.own_window.open_peer(handles[g]) for g in range(world)]
                dist.barrier(group=plan.group)          # every window exists and is zeroed before anyone's first call
            else:
                windows = [self.own_window.ptr]
        if len(windows) != world:
            raise ValueError("one window pointer per rank is required")
        if tiled:
            w13, w2 = self._repack(w13), self._repack(w2)
        self.workspace = share_with.workspace if share_with is not None else torch.zeros(ws_bytes + 1024, dtype=torch.uint8, device=dev)
        base = (self.workspace.data_ptr() + 1023) // 1024 * 1024
        desc = abi.EpLayerDesc()
        desc.struct_size = ctypes.sizeof(desc)
        desc.world, desc.rank, desc.max_tokens, desc.row_capacity = world, plan.rank, self.t_max, self.row_capacity
        desc.weights_tiled, desc.wait_timeout_ns = int(tiled), int(wait_timeout_s * 1e9)
        desc.router_weight_bf16 = router_w.data_ptr()
        desc.router_bias_f32 = router_bias.data_ptr() if router_bias is not None else None
        desc.w13_fp8, desc.w13_scale_f32 = w13.data_ptr(), w13_scale.data_ptr()
        desc.w2_fp8, desc.w2_scale_f32 = w2.data_ptr(), w2_scale.data_ptr()
        desc.workspace, desc.workspace_bytes = base, ws_bytes
        self._windows = (ctypes.c_void_p * world)(*windows)
        desc.windows, desc.window_bytes = self._windows, win_bytes
        handle = ctypes.c_void_p()
        torch.cuda.synchronize(dev)
        abi.check(self.lib.netra_ep_layer_create(ctypes.byref(desc), ctypes.byref(handle)), "ep_layer_create")
        self.handle = handle
        self._keep = (router_w, w13, w13_scale, w2, w2_scale, router_bias)
        self.stage_count = int(self.lib.netra_ep_layer_stage_count())

    def _repack(self, w: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(w)
        self.abi.check(self.lib.netra_moe_repack_tiles_launch(out.data_ptr(), w.data_ptr(), w.shape[0] * w.shape[1],
                                                              w.shape[2] * w.element_size(), torch.cuda.current_stream().cuda_stream),
                       "repack_tiles_launch")
        return out

    def launches_per_call(self, tokens: int) -> int:
        return int(self.lib.netra_ep_layer_launch_count(self.handle, tokens))

    def set_partial_format(self, fmt: int) -> None:
        """1: calls served by the token-major GEMMs return FP16 partial rows (the reference's prefill contract; half the
        NVLink bytes); 0: FP32 rows.  Every rank of the world must use the same format."""
        self.abi.check(self.lib.netra_ep_layer_set_partial_format(self.handle, fmt), "ep_layer_set_partial_format")

    def _args(self, hidden, shared_weight, out):
        if hidden.dtype != torch.bfloat16 or hidden.dim() != 2 or hidden.shape[1] != HIDDEN or not hidden.is_contiguous():
            raise ValueError("hidden must be contiguous BF16 [tokens, 2048]")
        if hidden.shape[0] > self.t_max:
            raise ValueError("more local tokens than the layer was sized for")
        if out is None:
            out = torch.empty_like(hidden)
        sw = shared_weight.data_ptr() if shared_weight is not None else None
        return hidden.data_ptr(), sw, out, hidden.shape[0], torch.cuda.current_stream().cuda_stream

    def __call__(self, hidden: torch.Tensor, shared_weight: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        h, sw, out, tokens, stream = self._args(hidden, shared_weight, out)
        self.abi.check(self.lib.netra_ep_layer_launch(self.handle, h, sw, out.data_ptr(), tokens, stream), "ep_layer_launch")
        return out

    def launch_stage(self, stage: int, hidden: torch.Tensor, out: torch.Tensor, shared_weight: Optional[torch.Tensor] = None) -> None:
        h, sw, out, tokens, stream = self._args(hidden, shared_weight, out)
        self.abi.check(self.lib.netra_ep_layer_launch_stage(self.handle, stage, h, sw, out.data_ptr(), tokens, stream), "ep_layer_launch_stage")

    def status(self) -> list[int]:
        words = (ctypes.c_uint32 * 4)()
        self.abi.check(self.lib.netra_ep_layer_status(self.handle, ctypes.byref(words)), "ep_layer_status")
        return list(words)

    def check_status(self) -> None:
        words = self.status()
        if words[2]:
            raise self.abi.NetraError(f"an expert block needed {words[2]} rows but row_capacity is {self.row_capacity}")
        if words[3]:
            raise self.abi.NetraError(f"a wait for a peer's flag timed out (mask {words[3]:#x}): a rank is missing or late")
        if any(words[:2]):
            raise self.abi.NetraError(f"device status words {words}: a bounded wait expired inside a grouped GEMM")

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.netra_ep_layer_destroy(self.handle)
            self.handle = None
        if self.own_window is not None:
            self.own_window.close()
            self.own_window = None

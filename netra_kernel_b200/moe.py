"""Host-side mirror of the routed-MoE boundary: torch tensors for device memory and streams,
every computation through the C ABI (``abi.py``).

``RoutedMoELayer.__call__(hidden)`` plays the role of the reference's serving adapter call
``apply(layer, hidden, topk_w, topk_ids)`` (``scripts/rocm/integrations/sglang/netra_gfx1151_sglang.py:1297-1311``)
with routing included; the ``bridge_*`` functions mirror the reference's per-kernel bridges
(``runtime/gfx950/fp8/moe/qwen36_moe_silu_mul_quant_bridge.h:14-64``).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import abi
from .synth import HIDDEN, INTER, N_ROUTED, SLOTS, TOPK


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise ValueError("operands must be contiguous CUDA tensors")


def workspace_layout(tokens: int) -> abi.WorkspaceLayout:
    lay = abi.WorkspaceLayout()
    lay.struct_size = ctypes.sizeof(lay)
    abi.check(abi.load().netra_moe_workspace_layout_query(tokens, ctypes.byref(lay)), "workspace_layout_query")
    return lay


def _f16_rows_from_panels(raw: "torch.Tensor", rows: int) -> "torch.Tensor":
    """Row-major [rows, 2048] copy of the FP16 partial rows, which the down projection stores as sixteen column panels
    [rows, 128] whose 16-byte chunks are permuted by the row index (chunk j of row p sits at position j ^ (p & 15))."""
    panels = raw.view(HIDDEN // 128, rows, 16, 8)
    pos = torch.arange(16, device=raw.device)[None, :] ^ (torch.arange(rows, device=raw.device)[:, None] & 15)   # [rows, chunk j] -> position
    idx = pos[None, :, :, None].expand(HIDDEN // 128, rows, 16, 8)
    return panels.gather(2, idx).permute(1, 0, 2, 3).reshape(rows, HIDDEN)


class RoutedMoELayer:
    """One routed-MoE layer bound to persistent device weights and a private workspace."""

    def __init__(self, router_w: torch.Tensor, w13: torch.Tensor, w13_scale: torch.Tensor,
                 w2: torch.Tensor, w2_scale: torch.Tensor, max_tokens: int,
                 router_bias: Optional[torch.Tensor] = None, tiled: bool = True, routing_only: bool = False,
                 pretiled: bool = False, workspace: Optional[torch.Tensor] = None, mxfp4: bool = False):
        """``w13`` / ``w2`` are the checkpoint's row-major slabs.  With ``tiled`` (default) they are
        rewritten once into the tile order the grouped GEMMs stream best and only that copy is kept
        by the layer; the caller may drop the row-major tensors.  ``pretiled`` says the tensors are
        already in tile order (another layer's ``tiled_weights()``), so nothing is copied.
        ``workspace`` lets several layers that never run concurrently (the layers of a stack on one
        stream) share one scratch buffer: a uint8 CUDA tensor of at least ``workspace_layout(max_tokens).total_bytes
        + 1024`` bytes.
        ``mxfp4``: the slabs are MXFP4 instead - ``w13`` / ``w2`` the packed E2M1 codes (u8 ``[S, 1024, 1024]`` /
        ``[S, 2048, 256]``, low nibble = even k) and ``w13_scale`` / ``w2_scale`` the E8M0 scales (u8 ``[S, 1024, 64]`` /
        ``[S, 2048, 16]``).  They are packed once (``pack_mxfp4``) and stay four-bit in memory: the grouped GEMMs
        multiply them on the tensor cores' block-scaled path.  With ``pretiled`` the four tensors are already the
        packed code blocks and scale atoms."""
        _require_cuda(router_w, w13, w13_scale, w2, w2_scale, router_bias)
        if tuple(router_w.shape) != (N_ROUTED, HIDDEN) or router_w.dtype != torch.bfloat16:
            raise ValueError("router weight must be bf16 [256, 2048]")
        slabs = w13.shape[0]
        if not routing_only and slabs != N_ROUTED + 1:
            raise ValueError("a full layer needs 257 expert slabs (slab 256 = shared expert)")
        self.mxfp4 = bool(mxfp4)
        if self.mxfp4:
            if any(t.dtype != torch.uint8 for t in (w13, w13_scale, w2, w2_scale)):
                raise ValueError("MXFP4 slabs and scales must be uint8")
            if tuple(w13.shape) != (slabs, 2 * INTER, HIDDEN // 2) or tuple(w2.shape) != (slabs, HIDDEN, INTER // 2):
                raise ValueError("MXFP4 expert slabs must be [S, 1024, 1024] and [S, 2048, 256] bytes")
            if tuple(w13_scale.shape) != (slabs, 2 * INTER, HIDDEN // 32) or tuple(w2_scale.shape) != (slabs, HIDDEN, INTER // 32):
                raise ValueError("MXFP4 scales must be u8 [S, 1024, 64] and [S, 2048, 16]")
        else:
            if tuple(w13.shape) != (slabs, 2 * INTER, HIDDEN) or tuple(w2.shape) != (slabs, HIDDEN, INTER):
                raise ValueError("expert slabs must be [S, 1024, 2048] and [S, 2048, 512]")
            if tuple(w13_scale.shape) != (slabs, 8, 16) or tuple(w2_scale.shape) != (slabs, 16, 4):
                raise ValueError("block scales must be f32 [S, 8, 16] and [S, 16, 4]")
        self.routing_only = routing_only
        self.lib = abi.load()
        self.tiled = bool(tiled)
        if self.mxfp4:
            self.tiled = True
            if not pretiled:
                (w13, w13_scale), (w2, w2_scale) = pack_mxfp4(w13, w13_scale, paired_half_rows=INTER), pack_mxfp4(w2, w2_scale, paired_half_rows=128)
        elif pretiled:
            self.tiled = True
        elif self.tiled:
            w13, w2 = self._repack(w13), self._repack(w2)
        self.max_tokens = int(max_tokens)
        self.layout = workspace_layout(self.max_tokens)
        self._keep = (router_w, w13, w13_scale, w2, w2_scale, router_bias)
        if workspace is None:
            raw = torch.zeros(self.layout.total_bytes + 1024, dtype=torch.uint8, device=router_w.device)
        else:
            _require_cuda(workspace)
            if workspace.dtype != torch.uint8 or workspace.numel() < self.layout.total_bytes + 1024:
                raise ValueError("a shared workspace must be a uint8 tensor of total_bytes + 1024 bytes")
            raw = workspace
        shift = (-raw.data_ptr()) % 1024
        self.workspace = raw[shift:shift + self.layout.total_bytes]
        self._raw = raw
        desc = abi.LayerDesc()
        desc.struct_size = ctypes.sizeof(desc)
        desc.max_tokens = self.max_tokens
        desc.router_weight_bf16 = router_w.data_ptr()
        desc.router_bias_f32 = _ptr(router_bias)
        desc.w13_fp8, desc.w13_scale_f32 = w13.data_ptr(), w13_scale.data_ptr()
        desc.w2_fp8, desc.w2_scale_f32 = w2.data_ptr(), w2_scale.data_ptr()
        desc.workspace, desc.workspace_bytes = self.workspace.data_ptr(), self.layout.total_bytes
        desc.weights_tiled, desc.num_expert_slabs = (2 if self.mxfp4 else int(self.tiled)), int(w13.shape[0])
        handle = ctypes.c_void_p()
        abi.check(self.lib.netra_moe_layer_create(ctypes.byref(desc), ctypes.byref(handle)), "layer_create")
        self.handle = handle
        self.device = router_w.device
        self.partial_f16 = False

    def _repack(self, w: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(w)
        abi.check(self.lib.netra_moe_repack_tiles_launch(out.data_ptr(), w.data_ptr(), w.shape[0] * w.shape[1],
                                                         w.shape[2] * w.element_size(), _stream()), "repack_tiles_launch")
        return out

    @classmethod
    def from_operands(cls, ops, max_tokens: Optional[int] = None, device="cuda"):
        dev = torch.device(device)
        bias = None if ops.router_bias is None else ops.router_bias.to(dev)
        return cls(ops.router_w.to(dev), ops.w13.to(dev), ops.w13_scale.to(dev), ops.w2.to(dev),
                   ops.w2_scale.to(dev), max_tokens or ops.tokens, bias)

    def tiled_weights(self):
        """(w13, w2) as the layer streams them (tile order when ``tiled``), for another layer's ``pretiled`` use."""
        return self._keep[1], self._keep[3]

    def set_gemm_mode(self, mode: int) -> None:
        """0: the layer picks the grouped-GEMM form by token count (token-major from 1,024 tokens); 1: always swap-AB;
        2: swap-AB with both projections in one launch up to 1,024 tokens (same results, slower: a recorded tactic)."""
        abi.check(self.lib.netra_moe_layer_set_gemm_mode(self.handle, mode), "layer_set_gemm_mode")

    def set_front_mode(self, mode: int) -> None:
        """1: calls of up to 1,024 tokens run router, top-8 + quantisation and sort in one launch (stage 0; stages 1 and 2
        then launch nothing); 0 (default): three launches.  Same results; the one-launch form measured slower."""
        abi.check(self.lib.netra_moe_layer_set_front_mode(self.handle, mode), "layer_set_front_mode")

    def set_row_gather(self, in_gemm: bool) -> None:
        """True: the token-major gate_up gathers its token rows with four-row TMA gathers instead of reading an
        expert-sorted copy (same results, slower: a recorded tactic)."""
        abi.check(self.lib.netra_moe_layer_set_row_gather(self.handle, int(bool(in_gemm))), "layer_set_row_gather")

    def set_router_mode(self, mode: int) -> None:
        """0: calls above 1,024 rows take the BF16 tensor-core router with exact FP64 recomputation of the undecided logits
        that can reach the top 8 (routing identical to the exact logits'); 2: the same with every undecided logit
        recomputed (the whole logits array exact); 1: every logit on the FP64 tensor cores."""
        abi.check(self.lib.netra_moe_layer_set_router_mode(self.handle, mode), "layer_set_router_mode")

    def set_partial_format(self, fmt: int) -> None:
        """0: FP32 down rows (decode contract); 1: FP16 partial rows where the token-major kernels run (prefill contract)."""
        abi.check(self.lib.netra_moe_layer_set_partial_format(self.handle, fmt), "layer_set_partial_format")
        self.partial_f16 = bool(fmt)

    def router_stats(self):
        words = (ctypes.c_uint32 * 4)()
        abi.check(self.lib.netra_moe_layer_router_stats(self.handle, ctypes.byref(words)), "layer_router_stats")
        return list(words)

    def launches_per_call(self, tokens: int) -> int:
        return int(self.lib.netra_moe_layer_launch_count(self.handle, tokens))

    def __call__(self, hidden: torch.Tensor, shared_weight: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _require_cuda(hidden, shared_weight, out)
        if hidden.dtype != torch.bfloat16 or hidden.dim() != 2 or hidden.shape[1] != HIDDEN:
            raise ValueError("hidden must be bf16 [tokens, 2048]")
        if self.routing_only:
            raise RuntimeError("this layer object only serves the routing stages (expert-parallel use)")
        tokens = hidden.shape[0]
        if out is None:
            out = torch.empty_like(hidden)
        abi.check(self.lib.netra_moe_layer_launch(self.handle, hidden.data_ptr(), _ptr(shared_weight),
                                                  out.data_ptr(), tokens, _stream()), "layer_launch")
        return out

    def forward_with_norm(self, x: torch.Tensor, residual: torch.Tensor, norm_weight: torch.Tensor, epsilon: float = 1e-6,
                          shared_weight: Optional[torch.Tensor] = None):
        """Residual add + RMSNorm + input quantisation fused in front of the layer
        (``netra_moe_layer_launch_with_norm``).  Returns (layer output, updated residual, normalised hidden)."""
        _require_cuda(x, residual, norm_weight, shared_weight)
        if x.dtype != torch.bfloat16 or residual.dtype != torch.bfloat16 or x.shape != residual.shape or x.shape[1] != HIDDEN:
            raise ValueError("input and residual must be bf16 [tokens, 2048]")
        if norm_weight.dtype != torch.float32 or norm_weight.numel() != HIDDEN:
            raise ValueError("norm weight must be float32 [2048]")
        hidden, res_out, out = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
        abi.check(self.lib.netra_moe_layer_launch_with_norm(self.handle, x.data_ptr(), residual.data_ptr(), norm_weight.data_ptr(),
                                                            float(epsilon), hidden.data_ptr(), res_out.data_ptr(), _ptr(shared_weight),
                                                            out.data_ptr(), x.shape[0], _stream()), "layer_launch_with_norm")
        return out, res_out, hidden

    def apply(self, hidden: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
              shared_weight: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The layer with a top-k computed by the caller (argument order of the reference's
        ``apply(layer, hidden, topk_weights, topk_ids)``, ``scripts/rocm/integrations/sglang/netra_gfx1151_sglang.py:1297-1311``):
        ``topk_ids`` int32 ``[tokens, 8]``, ``topk_weights`` float32 ``[tokens, 8]`` (normalised by the caller)."""
        _require_cuda(hidden, topk_weights, topk_ids, shared_weight, out)
        tokens = hidden.shape[0]
        if hidden.dtype != torch.bfloat16 or hidden.dim() != 2 or hidden.shape[1] != HIDDEN or not hidden.is_contiguous():
            raise ValueError("hidden must be contiguous bf16 [tokens, 2048]")
        if topk_ids.dtype != torch.int32 or tuple(topk_ids.shape) != (tokens, 8) or not topk_ids.is_contiguous():
            raise ValueError("topk_ids must be contiguous int32 [tokens, 8]")
        if topk_weights.dtype != torch.float32 or tuple(topk_weights.shape) != (tokens, 8) or not topk_weights.is_contiguous():
            raise ValueError("topk_weights must be contiguous float32 [tokens, 8]")
        if self.routing_only:
            raise RuntimeError("this layer object only serves the routing stages (expert-parallel use)")
        if out is None:
            out = torch.empty_like(hidden)
        abi.check(self.lib.netra_moe_layer_launch_with_topk(self.handle, hidden.data_ptr(), topk_ids.data_ptr(), topk_weights.data_ptr(),
                                                            _ptr(shared_weight), out.data_ptr(), tokens, _stream()),
                  "layer_launch_with_topk")
        return out

    STAGES = ("router_logits", "topk_quant", "sort_hist", "sort_scan", "sort_scatter", "gather_rows",
              "gate_up", "down", "combine")

    def launch_stage(self, stage: int, hidden: torch.Tensor, out: torch.Tensor,
                     shared_weight: Optional[torch.Tensor] = None) -> None:
        """Launch one stage of the layer sequence on the current stream."""
        abi.check(self.lib.netra_moe_layer_launch_stage(self.handle, stage, hidden.data_ptr(), _ptr(shared_weight),
                                                        out.data_ptr(), hidden.shape[0], _stream()), "layer_launch_stage")

    def status(self):
        words = (ctypes.c_uint32 * 4)()
        abi.check(self.lib.netra_moe_layer_status(self.handle, ctypes.byref(words)), "layer_status")
        return list(words)

    def check_status(self) -> None:
        words = self.status()
        if any(words):
            raise abi.NetraError(f"device status words {words}: a bounded wait expired inside a grouped GEMM")

    def intermediates(self, tokens: int) -> dict:
        """Views of the workspace tensors written by the last call with ``tokens`` rows."""
        lay, ws = self.layout, self.workspace
        pairs, rows = tokens * TOPK, tokens * SLOTS

        def view(offset, count, dtype):
            nbytes = count * torch.empty((), dtype=dtype).element_size()
            return ws[offset:offset + nbytes].view(dtype)

        return {
            "logits": view(lay.logits_bf16, tokens * N_ROUTED, torch.bfloat16).view(tokens, N_ROUTED),
            "topk_ids": view(lay.topk_ids, tokens * SLOTS, torch.int32).view(tokens, SLOTS),
            "topk_w": view(lay.topk_weights, tokens * SLOTS, torch.float32).view(tokens, SLOTS),
            "perm": view(lay.perm, pairs, torch.int32),
            "inv_perm": view(lay.inv_perm, pairs, torch.int32),
            "counts": view(lay.counts, N_ROUTED, torch.int32),
            "offsets": view(lay.offsets, N_ROUTED + 2, torch.int32),
            "a_fp8": view(lay.a_fp8, rows * HIDDEN, torch.uint8).view(rows, HIDDEN),
            "a_scale": view(lay.a_scale, rows * 16, torch.float32).view(rows, 16),
            "h_fp8": view(lay.h_fp8, rows * INTER, torch.uint8).view(rows, INTER),
            "h_scale": view(lay.h_scale, rows * 4, torch.float32).view(rows, 4),
            "down": view(lay.down_f32, rows * HIDDEN, torch.float32).view(rows, HIDDEN),
            "down_f16": _f16_rows_from_panels(view(lay.down_f32, rows * HIDDEN, torch.float16), rows),
            "logits_f32": view(lay.logits_f32, tokens * N_ROUTED, torch.float32).view(tokens, N_ROUTED),
            "wnorm": view(lay.wnorm, N_ROUTED, torch.float32),
        }

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.netra_moe_layer_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def pack_mxfp4(packed: torch.Tensor, scales: torch.Tensor, paired_half_rows: int = 128):
    """MXFP4 slabs (packed E2M1 ``[G, N, K/2]`` u8, E8M0 scales ``[G, N, K/32]`` u8, on the GPU) -> the operand layout of
    the native MXFP4 kernels, same shapes and sizes: code blocks (8 KiB per 128-row tile and K-block) and scale atoms
    (512 bytes per tile and K-block).  ``paired_half_rows``: 128 for W2 (tiles 2p and 2p + 1 side by side), 512 for W13
    (a gate tile's block next to its up tile's).  ``netra_moe_mxfp4_pack_launch``."""
    _require_cuda(packed, scales)
    g, n, half_k = packed.shape
    k = half_k * 2
    if packed.dtype != torch.uint8 or scales.dtype != torch.uint8 or scales.shape != (g, n, k // 32):
        raise ValueError("packed must be u8 [G, N, K/2] and scales u8 [G, N, K/32]")
    codes, atoms = torch.empty_like(packed), torch.empty_like(scales)
    lib = abi.load()
    tiles_per_call = 65535 // (n // 128) * (n // 128)        # whole slabs, at most 65,535 row tiles per launch
    rows_per_call = tiles_per_call * 128
    total = g * n
    src_c, src_s = packed.view(total, half_k), scales.view(total, k // 32)
    dst_c, dst_s = codes.view(total, half_k), atoms.view(total, k // 32)
    for r0 in range(0, total, rows_per_call):
        r1 = min(total, r0 + rows_per_call)
        abi.check(lib.netra_moe_mxfp4_pack_launch(dst_c[r0:r1].data_ptr(), dst_s[r0:r1].data_ptr(), src_c[r0:r1].data_ptr(),
                                                  src_s[r0:r1].data_ptr(), r1 - r0, k, paired_half_rows, _stream()), "mxfp4_pack_launch")
    return codes, atoms


def expand_mxfp4(packed: torch.Tensor, scales: torch.Tensor):
    """MXFP4 slabs (packed E2M1 ``[G, N, K/2]`` u8, E8M0 scales ``[G, N, K/32]`` u8, on the GPU) -> the layer's
    FP8 operands: (E4M3 codes ``[G, N, K]`` as float8, tile scales ``[G, N/128, K/128]`` FP32, count of elements
    that could not be held exactly).  ``netra_moe_mxfp4_expand_launch``."""
    _require_cuda(packed, scales)
    g, n, half_k = packed.shape
    k = half_k * 2
    if packed.dtype != torch.uint8 or scales.dtype != torch.uint8 or scales.shape != (g, n, k // 32):
        raise ValueError("packed must be u8 [G, N, K/2] and scales u8 [G, N, K/32]")
    codes = torch.empty(g, n, k, dtype=torch.uint8, device=packed.device)
    tile_scale = torch.empty(g, n // 128, k // 128, dtype=torch.float32, device=packed.device)
    inexact = torch.zeros(1, dtype=torch.int32, device=packed.device)
    abi.check(abi.load().netra_moe_mxfp4_expand_launch(codes.data_ptr(), tile_scale.data_ptr(), inexact.data_ptr(),
                                                      packed.contiguous().data_ptr(), scales.contiguous().data_ptr(), g * n, k, _stream()),
              "mxfp4_expand_launch")
    return codes.view(torch.float8_e4m3fn), tile_scale, int(inexact.item())


# ----------------------------------------------------------------------------- per-kernel bridges
def bridge_router_bf16(hidden: torch.Tensor, router_w: torch.Tensor) -> torch.Tensor:
    _require_cuda(hidden, router_w)
    out = torch.empty(hidden.shape[0], N_ROUTED, dtype=torch.bfloat16, device=hidden.device)
    abi.check(abi.load().netra_qwen36_router_bf16_launch(out.data_ptr(), hidden.data_ptr(), router_w.data_ptr(),
                                                         hidden.shape[0], _stream()), "router_bf16_launch")
    return out


def bridge_shared_gate_append(hidden, gate_w, ids8, w8):
    _require_cuda(hidden, gate_w, ids8, w8)
    rows = hidden.shape[0]
    ids9 = torch.empty(rows, SLOTS, dtype=torch.int32, device=hidden.device)
    w9 = torch.empty(rows, SLOTS, dtype=torch.float32, device=hidden.device)
    abi.check(abi.load().netra_qwen36_shared_gate_append_launch(
        ids9.data_ptr(), w9.data_ptr(), hidden.data_ptr(), gate_w.data_ptr(), ids8.data_ptr(), w8.data_ptr(),
        rows, _stream()), "shared_gate_append_launch")
    return ids9, w9


def bridge_gate_up(hidden_fp8, hidden_scale, w13, w13_scale, topk_ids9) -> torch.Tensor:
    _require_cuda(hidden_fp8, hidden_scale, w13, w13_scale, topk_ids9)
    rows = hidden_fp8.shape[0]
    out = torch.empty(rows * SLOTS, 2 * INTER, dtype=torch.float32, device=hidden_fp8.device)
    abi.check(abi.load().netra_qwen36_moe_gate_up_launch(
        hidden_fp8.data_ptr(), hidden_scale.data_ptr(), w13.data_ptr(), w13_scale.data_ptr(),
        topk_ids9.data_ptr(), out.data_ptr(), rows, _stream()), "gate_up_launch")
    return out


def bridge_silu_mul_quant(gate_up_f32: torch.Tensor):
    _require_cuda(gate_up_f32)
    rows = gate_up_f32.shape[0]
    q = torch.empty(rows, INTER, dtype=torch.uint8, device=gate_up_f32.device)
    s = torch.empty(rows, INTER // 128, dtype=torch.float32, device=gate_up_f32.device)
    abi.check(abi.load().netra_qwen36_moe_silu_mul_quant_launch(
        gate_up_f32.data_ptr(), q.data_ptr(), s.data_ptr(), rows, _stream()), "silu_mul_quant_launch")
    return q, s


def bridge_down_reduce(act_fp8, act_scale, w2, w2_scale, topk_w9, topk_ids9) -> torch.Tensor:
    _require_cuda(act_fp8, act_scale, w2, w2_scale, topk_w9, topk_ids9)
    rows = topk_ids9.shape[0]
    out = torch.empty(rows, HIDDEN, dtype=torch.bfloat16, device=act_fp8.device)
    abi.check(abi.load().netra_qwen36_moe_down_reduce_launch(
        act_fp8.data_ptr(), act_scale.data_ptr(), w2.data_ptr(), w2_scale.data_ptr(), topk_w9.data_ptr(),
        topk_ids9.data_ptr(), out.data_ptr(), rows, _stream()), "down_reduce_launch")
    return out


def bridge_add_rmsnorm_group_quant(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, epsilon: float = 1e-6):
    """``netra_add_rmsnorm_group_quant_n2048_launch``: (normalised BF16, updated residual BF16, FP8 codes u8, scales f32 [rows, 16])."""
    _require_cuda(x, residual, weight)
    rows = x.shape[0]
    out, res_out = torch.empty_like(x), torch.empty_like(x)
    q = torch.empty(rows, HIDDEN, dtype=torch.uint8, device=x.device)
    s = torch.empty(rows, HIDDEN // 128, dtype=torch.float32, device=x.device)
    abi.check(abi.load().netra_add_rmsnorm_group_quant_n2048_launch(x.data_ptr(), residual.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                                                     res_out.data_ptr(), q.data_ptr(), s.data_ptr(), rows, float(epsilon),
                                                                     _stream()), "add_rmsnorm_group_quant_launch")
    return out, res_out, q, s

"""ctypes binding of libnetra_sm100.so (the C ABI in include/netra_moe.h).

The library is the product path: if it is missing or cannot be loaded this module raises —
there is no Python or CPU fallback.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "csrc" / "libnetra_sm100.so"

c_void_p, c_int, c_u32, c_u64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32, ctypes.c_uint64


class WorkspaceLayout(ctypes.Structure):
    _fields_ = [("struct_size", c_u32), ("tokens", c_u32), ("total_bytes", c_u64)] + [
        (name, c_u64) for name in (
            "logits_bf16", "topk_ids", "topk_weights", "perm", "inv_perm", "counts", "offsets",
            "seg_hist", "a_fp8", "a_scale", "h_fp8", "h_scale", "down_f32", "status", "logits_f32", "wnorm",
            "router_stats", "gemm_ready", "front_counters")]


class LayerDesc(ctypes.Structure):
    _fields_ = [("struct_size", c_u32), ("max_tokens", c_u32),
                ("router_weight_bf16", c_void_p), ("router_bias_f32", c_void_p),
                ("w13_fp8", c_void_p), ("w13_scale_f32", c_void_p),
                ("w2_fp8", c_void_p), ("w2_scale_f32", c_void_p),
                ("workspace", c_void_p), ("workspace_bytes", c_u64),
                ("weights_tiled", c_u32), ("num_expert_slabs", c_u32)]


class ExpertBlockDesc(ctypes.Structure):
    _fields_ = [("struct_size", c_u32), ("num_groups", c_u32), ("max_rows", c_u32), ("weights_tiled", c_u32)] + [
        (name, c_void_p) for name in ("w13_fp8", "w13_scale_f32", "w2_fp8", "w2_scale_f32", "a_fp8", "a_scale_f32",
                                      "h_fp8", "h_scale_f32", "down_f32", "offsets_i32", "status_u32")]


class EpLayerDesc(ctypes.Structure):
    _fields_ = [("struct_size", c_u32), ("world", c_u32), ("rank", c_u32), ("max_tokens", c_u32), ("row_capacity", c_u32),
                ("weights_tiled", c_u32), ("wait_timeout_ns", c_u64),
                ("router_weight_bf16", c_void_p), ("router_bias_f32", c_void_p),
                ("w13_fp8", c_void_p), ("w13_scale_f32", c_void_p), ("w2_fp8", c_void_p), ("w2_scale_f32", c_void_p),
                ("workspace", c_void_p), ("workspace_bytes", c_u64),
                ("windows", ctypes.POINTER(c_void_p)), ("window_bytes", c_u64)]


BRIDGES = ("netra_qwen36_router_bf16", "netra_qwen36_shared_gate_append", "netra_qwen36_moe_gate_up",
           "netra_qwen36_moe_silu_mul_quant", "netra_qwen36_moe_down_reduce")

# every symbol include/netra_moe.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "netra_qwen36_router_bf16_launch": (c_int, [c_void_p, c_void_p, c_void_p, c_u32, c_void_p]),
    "netra_qwen36_shared_gate_append_launch": (c_int, [c_void_p] * 6 + [c_u32, c_void_p]),
    "netra_qwen36_moe_gate_up_launch": (c_int, [c_void_p] * 6 + [c_int, c_void_p]),
    "netra_qwen36_moe_silu_mul_quant_launch": (c_int, [c_void_p] * 3 + [c_int, c_void_p]),
    "netra_qwen36_moe_down_reduce_launch": (c_int, [c_void_p] * 7 + [c_int, c_void_p]),
    "netra_group_quant_assembly_load": (c_int, [ctypes.c_char_p] * 6),
    "netra_group_quant_assembly_unload": (c_int, []),
    "netra_group_quant_assembly_last_error": (ctypes.c_char_p, []),
    "netra_add_rmsnorm_group_quant_n2048_launch": (c_int, [c_void_p] * 7 + [c_u32, ctypes.c_float, c_void_p]),
    "netra_moe_layer_launch_with_norm": (c_int, [c_void_p] * 4 + [ctypes.c_float] + [c_void_p] * 4 + [c_u32, c_void_p]),
    "netra_moe_prefill_m768_load": (c_int, [ctypes.c_char_p, ctypes.c_char_p]),
    "netra_moe_prefill_m768_launch": (c_int, [c_void_p] * 15),
    "netra_moe_prefill_m768_status": (c_int, [ctypes.POINTER(c_u32 * 4)]),
    "netra_moe_prefill_m768_unload": (c_int, []),
    "netra_moe_prefill_m768_last_error": (ctypes.c_char_p, []),
    "netra_moe_workspace_layout_query": (c_int, [c_u32, ctypes.POINTER(WorkspaceLayout)]),
    "netra_moe_layer_create": (c_int, [ctypes.POINTER(LayerDesc), ctypes.POINTER(c_void_p)]),
    "netra_moe_layer_launch": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_u32, c_void_p]),
    "netra_moe_layer_launch_with_topk": (c_int, [c_void_p] * 6 + [c_u32, c_void_p]),
    "netra_moe_layer_launch_stage": (c_int, [c_void_p, c_u32, c_void_p, c_void_p, c_void_p, c_u32, c_void_p]),
    "netra_moe_repack_tiles_launch": (c_int, [c_void_p, c_void_p, c_u64, c_u32, c_void_p]),
    "netra_moe_widen_scales_bf16_launch": (c_int, [c_void_p, c_void_p, c_u64, c_void_p]),
    "netra_moe_mxfp4_expand_launch": (c_int, [c_void_p] * 5 + [c_u64, c_u32, c_void_p]),
    "netra_moe_mxfp4_pack_launch": (c_int, [c_void_p] * 4 + [c_u64, c_u32, c_u32, c_void_p]),
    "netra_moe_expert_block_create": (c_int, [ctypes.POINTER(ExpertBlockDesc), ctypes.POINTER(c_void_p)]),
    "netra_moe_expert_block_launch": (c_int, [c_void_p, c_void_p]),
    "netra_moe_expert_block_destroy": (c_int, [c_void_p]),
    "netra_ep_regroup_launch": (c_int, [c_void_p] * 5 + [c_u32] * 6 + [c_void_p]),
    "netra_moe_move_rows_launch": (c_int, [c_void_p] * 3 + [c_u32] * 7 + [c_void_p]),
    "netra_ep_pack_rows_launch": (c_int, [c_void_p] * 4 + [c_u32] * 3 + [c_void_p, c_void_p]),
    "netra_ep_unpack_rows_launch": (c_int, [c_void_p] * 3 + [c_u32] * 3 + [c_void_p]),
    "netra_ep_sizes_query": (c_int, [c_u32, c_u32, c_u32, ctypes.POINTER(c_u64), ctypes.POINTER(c_u64)]),
    "netra_ep_window_create": (c_int, [c_u64, ctypes.POINTER(c_void_p), c_void_p]),
    "netra_ep_window_open": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "netra_ep_window_close": (c_int, [c_void_p]),
    "netra_ep_window_destroy": (c_int, [c_void_p]),
    "netra_ep_layer_create": (c_int, [ctypes.POINTER(EpLayerDesc), ctypes.POINTER(c_void_p)]),
    "netra_ep_layer_launch": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_u32, c_void_p]),
    "netra_ep_layer_launch_stage": (c_int, [c_void_p, c_u32, c_void_p, c_void_p, c_void_p, c_u32, c_void_p]),
    "netra_ep_layer_stage_count": (c_u32, []),
    "netra_ep_layer_launch_count": (c_u32, [c_void_p, c_u32]),
    "netra_ep_layer_status": (c_int, [c_void_p, ctypes.POINTER(c_u32 * 4)]),
    "netra_ep_layer_destroy": (c_int, [c_void_p]),
    "netra_ep_layer_set_partial_format": (c_int, [c_void_p, c_u32]),
    "netra_moe_kernel_launch_info": (c_int, [c_u32, ctypes.POINTER(c_u32), ctypes.POINTER(c_u32)]),
    "netra_moe_layer_set_gemm_mode": (c_int, [c_void_p, c_u32]),
    "netra_moe_layer_set_front_mode": (c_int, [c_void_p, c_u32]),
    "netra_moe_layer_set_row_gather": (c_int, [c_void_p, c_u32]),
    "netra_moe_layer_set_router_mode": (c_int, [c_void_p, c_u32]),
    "netra_moe_layer_set_partial_format": (c_int, [c_void_p, c_u32]),
    "netra_moe_layer_router_stats": (c_int, [c_void_p, ctypes.POINTER(c_u32 * 4)]),
    "netra_moe_layer_status": (c_int, [c_void_p, ctypes.POINTER(c_u32 * 4)]),
    "netra_moe_layer_launch_count": (c_u32, [c_void_p, c_u32]),
    "netra_moe_layer_destroy": (c_int, [c_void_p]),
    "netra_moe_last_error": (ctypes.c_char_p, []),
    "netra_moe_sort_static_scratch_launch": (c_int, [c_void_p] * 5 + [c_u32, c_void_p]),
}
for _b in BRIDGES:
    SIGNATURES[_b + "_load"] = (c_int, [ctypes.c_char_p])
    SIGNATURES[_b + "_unload"] = (c_int, [])
    SIGNATURES[_b + "_last_error"] = (ctypes.c_char_p, [])

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library and type every exported symbol.  Raises if it is absent."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m netra_kernel_b200.csrc.build` "
                "(there is no fallback path)")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)          # AttributeError if the export is missing
            fn.restype, fn.argtypes = restype, argtypes
        _lib = lib
    return _lib


class NetraError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        message = load().netra_moe_last_error().decode(errors="replace")
        raise NetraError(f"{what} failed (code {rc}): {message}")

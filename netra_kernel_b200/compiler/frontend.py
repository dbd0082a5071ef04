"""Model manifest -> graph.  One family is built: ``routed_moe_layer`` (router logits, top-8 with
the shared slot and input quantisation, token sort, row gather, grouped gate_up, grouped down,
combine).  Role of the reference's ``compiler/netra_compiler/frontends/model_json.py:22-47`` and
``frontends/qwen.py``; the operation list is fixed by the family, its shapes by the profile."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any

from .contracts import KernelSemantics
from .ir import Graph, Operation, Tensor
from .profiles import ShapeProfile
from .types import TARGET, ValidationError

MODEL_FORMAT = "netra-model-1"
REQUIRED_CONSTANTS = ("hidden", "intermediate", "routed_experts", "top_k", "shared_experts", "scale_block", "sm_count")
SORT_SINGLE_BLOCK_MAX_ROWS = 1024
SORT_SEGMENT_PAIRS = 1024
ROUTER_FP64_MAX_ROWS = 1024      # above: BF16 tensor-core router + exact recomputation of the selectable undecided logits


def load_model(path: Path) -> dict[str, Any]:
    try:
        doc = json.loads(Path(path).read_text(encoding="utf-8"))
    except (OSError, json.JSONDecodeError) as exc:
        raise ValidationError(f"cannot read model manifest {path}: {exc}") from exc
    if doc.get("format") != MODEL_FORMAT:
        raise ValidationError(f"{path}: not a {MODEL_FORMAT} manifest")
    if doc.get("target") != TARGET:
        raise ValidationError(f"{path}: target must be {TARGET}")
    if doc.get("family") != "routed_moe_layer":
        raise ValidationError(f"{path}: unsupported model family {doc.get('family')!r}")
    constants = doc.get("constants", {})
    for key in REQUIRED_CONSTANTS:
        if not isinstance(constants.get(key), int) or isinstance(constants.get(key), bool) or constants[key] <= 0:
            raise ValidationError(f"{path}: constant {key} must be a positive integer")
    if constants["shared_experts"] != 1:
        raise ValidationError(f"{path}: exactly one shared expert is supported")
    deployment = doc.setdefault("deployment", {})
    deployment.setdefault("tensor_parallel", 1)
    deployment.setdefault("data_parallel_workers", 1)
    options = doc.setdefault("options", {})
    options.setdefault("router_bias", False)
    options.setdefault("shared_weight", False)
    options.setdefault("weight_layout", "tiles128")
    if options["weight_layout"] not in ("tiles128", "row_major", "mxfp4_paired_blocks"):
        raise ValidationError(f"{path}: weight_layout must be tiles128, row_major or mxfp4_paired_blocks")
    if (options["weight_layout"] == "mxfp4_paired_blocks") != (doc.get("quantization") == "mxfp4_block32"):
        raise ValidationError(f"{path}: the mxfp4_paired_blocks layout and the mxfp4_block32 quantization go together")
    # rows between the down projection and the combine where the token-major kernels run: "f32" (decode contract) or
    # "f16" (the reference's prefill contract: FP16 partial rows, kernels/gfx950/templates/moe/prefill/route_reduce_splitk2_f16.inc)
    options.setdefault("prefill_partials", "f32")
    if options["prefill_partials"] not in ("f32", "f16"):
        raise ValidationError(f"{path}: prefill_partials must be f32 or f16")
    return doc


def semantics(abi: str, dtypes: str, quantization: str, layouts: str, numerical: str) -> dict[str, str]:
    return KernelSemantics(abi, dtypes, quantization, layouts, numerical).to_dict()


def token_rows(profile: ShapeProfile) -> int:
    """Rows the routed layer sees.  A verify / speculative profile fixes ``route_rows`` (= m draft positions x batch, the
    reference's ``manifests/gfx950/profiles/verify_m12_b64_routes768.json``); any other profile's rows are its ``m``."""
    if any(key == "route_rows" for key, _ in profile.guards):
        rows = profile.exact_value("route_rows")
        if rows != profile.exact_value("m") * profile.exact_value("batch"):
            raise ValidationError(f"profile {profile.name!r}: route_rows must equal m * batch")
        return rows
    return profile.exact_value("m")


def dimensions_for(model: dict[str, Any], profile: ShapeProfile) -> dict[str, int]:
    m = token_rows(profile)
    c = model["constants"]
    pairs = m * c["top_k"]
    return {"m": m, "pairs": pairs, "rows": pairs + m, "nseg": -(-pairs // SORT_SEGMENT_PAIRS)}


def options_for(model: dict[str, Any]) -> dict[str, int]:
    c = model["constants"]
    return {"groups": c["routed_experts"] + c["shared_experts"], "sm_count": c["sm_count"],
            "w_tiled": 1 if model["options"]["weight_layout"] == "tiles128" else 0}


MXFP4 = "mxfp4_block32"      # model quantization: E2M1 expert weights with one UE8M0 scale per 32 along K; FP8 activations


def routed_moe_layer_graph(model: dict[str, Any], profile: ShapeProfile) -> Graph:
    c = model["constants"]
    opt = model["options"]
    d = dimensions_for(model, profile)
    m, pairs, rows, nseg = d["m"], d["pairs"], d["rows"], d["nseg"]
    hidden, inter, experts, slots = c["hidden"], c["intermediate"], c["routed_experts"], c["top_k"] + 1
    groups = experts + 1
    kb_h, kb_i = hidden // c["scale_block"], inter // c["scale_block"]
    segmented = m > SORT_SINGLE_BLOCK_MAX_ROWS

    mxfp4 = model.get("quantization") == MXFP4
    if mxfp4 and opt["weight_layout"] != "mxfp4_paired_blocks":
        raise ValidationError("an MXFP4 model streams its weights in the mxfp4_paired_blocks layout")
    if mxfp4 and opt.get("prefill_partials", "f32") != "f32":
        raise ValidationError("FP16 partial rows are an output format of the E4M3 kernels")
    if mxfp4:      # codes two per byte, scales one byte per 32 weights; both re-ordered by the pack step (layout plan)
        expert_tensors = [
            Tensor("w13", "e2m1x2", (groups, 2 * inter, hidden // 2), "weight", groups * 2 * inter * hidden // 2),
            Tensor("w13_scale", "ue8m0", (groups, 2 * inter, hidden // 32), "weight", groups * 2 * inter * hidden // 32),
            Tensor("w2", "e2m1x2", (groups, hidden, inter // 2), "weight", groups * hidden * inter // 2),
            Tensor("w2_scale", "ue8m0", (groups, hidden, inter // 32), "weight", groups * hidden * inter // 32)]
    else:
        expert_tensors = [
            Tensor("w13", "fp8_e4m3", (groups, 2 * inter, hidden), "weight", groups * 2 * inter * hidden),
            Tensor("w13_scale", "fp32", (groups, 2 * inter // c["scale_block"], kb_h), "weight", groups * (2 * inter // c["scale_block"]) * kb_h * 4),
            Tensor("w2", "fp8_e4m3", (groups, hidden, inter), "weight", groups * hidden * inter),
            Tensor("w2_scale", "fp32", (groups, kb_h, kb_i), "weight", groups * kb_h * kb_i * 4)]
    tensors = [
        Tensor("hidden", "bf16", (m, hidden), "input", m * hidden * 2),
        Tensor("output", "bf16", (m, hidden), "output", m * hidden * 2),
        Tensor("router_weight", "bf16", (experts, hidden), "weight", experts * hidden * 2),
        *expert_tensors,
        Tensor("logits", "bf16", (m, experts), "workspace", m * experts * 2),
        Tensor("topk_ids", "int32", (m, slots), "workspace", m * slots * 4),
        Tensor("topk_weights", "fp32", (m, slots), "workspace", m * slots * 4),
        Tensor("perm", "int32", (pairs,), "workspace", pairs * 4),
        Tensor("inv_perm", "int32", (pairs,), "workspace", pairs * 4),
        Tensor("counts", "int32", (experts,), "workspace", experts * 4),
        Tensor("offsets", "int32", (experts + 2,), "workspace", (experts + 2) * 4),
        Tensor("a_fp8", "fp8_e4m3", (rows, hidden), "workspace", rows * hidden),
        # scale tiles are copied 64 rows at a time: 128 spare rows keep the last copy inside the buffer
        Tensor("a_scale", "fp32", (rows + 128, kb_h), "workspace", (rows + 128) * kb_h * 4),
        Tensor("h_fp8", "fp8_e4m3", (rows, inter), "workspace", rows * inter),
        Tensor("h_scale", "fp32", (rows + 128, kb_i), "workspace", (rows + 128) * kb_i * 4),
        Tensor("down_f32", "fp32", (rows, hidden), "workspace", rows * hidden * 4),
        Tensor("status", "uint32", (4,), "workspace", 16),
    ]
    if opt["router_bias"]:
        tensors.append(Tensor("router_bias", "fp32", (experts,), "weight", experts * 4))
    if opt["shared_weight"]:
        tensors.append(Tensor("shared_weight", "fp32", (m,), "input", m * 4))
    if segmented:
        tensors.append(Tensor("seg_hist", "int32", (nseg, experts), "workspace", nseg * experts * 4))
    tensor_core_router = m > ROUTER_FP64_MAX_ROWS
    if tensor_core_router:
        tensors += [Tensor("logits_f32", "fp32", (m, experts), "workspace", m * experts * 4),
                    Tensor("wnorm", "fp32", (experts,), "workspace", experts * 4),
                    Tensor("router_stats", "uint32", (4,), "workspace", 16)]

    routing_constants = {"hidden": hidden, "routed_experts": experts}
    gemm_constants = {"hidden": hidden, "intermediate": inter, "scale_block": c["scale_block"], "tile_rows": 128}

    # grouped-GEMM form: token-major (128 token rows x 256 weight rows per MMA) from an average of 32 rows per routed expert
    token_major = m * c["top_k"] >= 32 * experts
    form = ("token_major" if token_major else "swap_ab") + ".sorted_rows." + (
        "mxfp4_paired_blocks" if mxfp4 else "tiles128" if opt["weight_layout"] == "tiles128" else "row_major")
    maps = "tmap2" if token_major else "tmap4"
    # the MXFP4 kernels take no weight-layout flag (one u32 fewer) and apply the weight scales inside the MMA
    gemm_abi = ("{}_grouped." + maps + "_ptr{}_u32_ptr.mxfp4.v1") if mxfp4 else ("{}_grouped." + maps + "_ptr{}_u32x2_ptr.v1")
    gemm_dtypes = "fp8e4m3_e2m1_to_{}" if mxfp4 else "fp8e4m3_fp8e4m3_to_{}"
    gemm_quant = "mxfp4_w1x32_ue8m0.a_fp8_e4m3_1x128_amax448" if mxfp4 else "fp8_e4m3_w128x128_a1x128_amax448"
    f16_rows = token_major and opt["prefill_partials"] == "f16"   # the rows keep the down_f32 buffer (half of it is used)

    def op(name, family, operation, inputs, outputs, constants, sem):
        return Operation(name, "fixed_kernel", family, operation, tuple(inputs), tuple(outputs),
                         {"constants": constants, "semantics": sem, "fallback": f"framework.{operation}"})

    optional_inputs = [t for t, on in (("router_bias", opt["router_bias"]), ("shared_weight", opt["shared_weight"])) if on]
    if tensor_core_router:
        ops = [
            op("router_logits", "moe_routing", "router_logits_tensor_core", ["hidden", "router_weight"], ["logits_f32", "wnorm", "status"],
               routing_constants,
               semantics("router_umma.tmap2_ptr3_u32_ptr.v1", "bf16_bf16_to_f32", "none", "row_major", "tcgen05_f16_fp32_accumulate.approximate.v1")),
            op("topk_quant", "moe_routing", "softmax_top8_exact_fixup_fp8_quant",
               ["logits_f32", "wnorm", "router_weight", "hidden", *optional_inputs],
               ["logits", "topk_ids", "topk_weights", "a_fp8", "a_scale", "router_stats"],
               {**routing_constants, "top_k": c["top_k"], "scale_block": c["scale_block"]},
               semantics("topk_quant_fix.ptr12_u32x3.v1", "f32_bf16_to_bf16_i32_f32_fp8e4m3_f32", "fp8_e4m3_per_token_block128_amax448",
                         "slot9_shared_last.token_rows_after_pairs",
                         "exact_dot_rne_bf16_for_selectable.logit_desc_id_asc.fp32_softmax_renorm.v1")),
        ]
    else:
        ops = [
            op("router_logits", "moe_routing", "router_logits", ["hidden", "router_weight"], ["logits"], routing_constants,
               semantics("router_logits.ptr3_u32.v1", "bf16_bf16_to_bf16", "none", "row_major", "exact_dot_rne_bf16.v1")),
            op("topk_quant", "moe_routing", "softmax_top8_shared_slot_fp8_quant",
               ["logits", "hidden", *optional_inputs], ["topk_ids", "topk_weights", "a_fp8", "a_scale"],
               {**routing_constants, "top_k": c["top_k"], "scale_block": c["scale_block"]},
               semantics("topk_quant.ptr8_u32x2.v1", "bf16_to_i32_f32_fp8e4m3_f32", "fp8_e4m3_per_token_block128_amax448",
                         "slot9_shared_last.token_rows_after_pairs", "logit_desc_id_asc.fp32_softmax_renorm.v1")),
        ]
    if segmented:
        ops += [
            op("sort_hist", "moe_sort", "sort_histogram", ["topk_ids"], ["seg_hist"], {"routed_experts": experts, "top_k": c["top_k"]},
               semantics("sort_hist.ptr2_u32.v1", "i32", "none", "segments_of_1024_pairs", "counting.v1")),
            op("sort_scan", "moe_sort", "sort_scan", ["seg_hist"], ["seg_hist", "counts", "offsets"], {"routed_experts": experts, "top_k": c["top_k"]},
               semantics("sort_scan.ptr3_u32x2.v1", "i32", "none", "offsets258_shared_group_last", "exclusive_prefix.v1")),
            op("sort_scatter", "moe_sort", "sort_scatter", ["seg_hist", "topk_ids"], ["perm", "inv_perm"], {"routed_experts": experts, "top_k": c["top_k"]},
               semantics("sort_scatter.ptr4_u32.v1", "i32", "none", "pair_index_t8_plus_slot", "stable_expert_major.v1")),
        ]
    else:
        ops.append(op("token_sort", "moe_sort", "token_sort", ["topk_ids"], ["perm", "inv_perm", "counts", "offsets"],
                      {"routed_experts": experts, "top_k": c["top_k"]},
                      semantics("token_sort.ptr5_u32.v1", "i32", "none", "pair_index_t8_plus_slot.offsets258_shared_group_last",
                                "stable_expert_major.v1")))
    ops += [
        op("gather_rows", "moe_sort", "gather_quantized_rows", ["perm", "a_fp8", "a_scale"], ["a_fp8", "a_scale"],
           {"hidden": hidden, "top_k": c["top_k"], "scale_block": c["scale_block"]},
           semantics("gather_rows.ptr3_u32_ptr_u32.v1", "fp8e4m3_f32", "fp8_e4m3_per_token_block128_amax448",
                     "sorted_rows_first.token_rows_after_pairs", "copy.v1")),
        op("gate_up", "moe_fp8_grouped_gemm", "gate_up_silu_requant", ["a_fp8", "a_scale", "w13", "w13_scale", "offsets"],
           ["h_fp8", "h_scale", "status"], gemm_constants,
           semantics(gemm_abi.format("gate_up", 5), gemm_dtypes.format("fp8e4m3_f32"), gemm_quant,
                     form, "kblock_fma_ascending.silu_fp32.bf16_round_then_amax.v1")),
        op("down", "moe_fp8_grouped_gemm", "down_projection", ["h_fp8", "h_scale", "w2", "w2_scale", "offsets"],
           ["down_f32", "status"], gemm_constants,
           semantics(gemm_abi.format("down", 4), gemm_dtypes.format("f16" if f16_rows else "f32"), gemm_quant, form,
                     "kblock_fma_ascending.f16_partial_rows.v1" if f16_rows else "kblock_fma_ascending.v1")),
        op("combine", "moe_combine", "weighted_slot_combine", ["down_f32", "topk_weights", "inv_perm"], ["output"],
           {"hidden": hidden, "top_k": c["top_k"]},
           semantics("combine.ptr4_u32.v1", "f16_f32_to_bf16" if f16_rows else "f32_f32_to_bf16", "none",
                     "sorted_rows_first.token_rows_after_pairs",
                     "slot_ascending_widen_mul_add_fp32_rne_bf16.v1" if f16_rows else "slot_ascending_mul_add_fp32_rne_bf16.v1")),
    ]
    return Graph(f"{model['name']}@{profile.name}", tuple(tensors), tuple(ops))

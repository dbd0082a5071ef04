"""CPU tests of the compiler slice (contracts, profiles, catalog, planner, memory plan, engine
emitter, validator), modelled on the reference's tests/compiler/*."""
import ctypes
import dataclasses
import json
import shutil
from pathlib import Path

import numpy as np
import pytest

from netra_kernel_b200 import abi
from netra_kernel_b200.compiler import compile_engine, validate_engine_directory
from netra_kernel_b200.compiler import catalog, contracts, engine, expr, frontend, layouts, memory, planner, profiles
from netra_kernel_b200.compiler.library import KernelLibrary
from netra_kernel_b200.compiler.types import TARGET, Maturity, ValidationError, canonical_json, stable_hash
from tests import helpers

LIB_ROOT = KernelLibrary.discover().root
MODEL = LIB_ROOT / "manifests" / TARGET / "models" / "routed-moe-layer-fp8.json"
MODEL_ZIPF = LIB_ROOT / "manifests" / TARGET / "models" / "routed-moe-layer-fp8-zipf.json"


# ------------------------------------------------------------------ hashing / contracts
def test_canonical_json_and_stable_hash_match_the_reference_compiler():
    kat = json.loads((helpers.GOLDEN / "compiler_hash_kat.json").read_text(encoding="utf-8"))
    for value, text, digest in zip(kat["values"], kat["canonical"], kat["sha256"]):
        assert canonical_json(value) == text
        assert stable_hash(value) == digest
    # the reference's contract id is "nk_" + first 24 hex digits of the identity hash
    assert "nk_" + stable_hash(kat["contract_identity"])[:24] == kat["contract_id"]


def _contract(**overrides):
    base = dict(target=TARGET, wave_size=32, operation="op", family="fam", constants=(("hidden", 2048),),
                specialization=(("m", 256),), semantics=contracts.KernelSemantics("a.v1", "d", "q", "l", "n.v1"),
                kernarg_size=32, symbol="sym", launch=contracts.Launch((4, 1, 1), (128, 1, 1)))
    base.update(overrides)
    return contracts.FixedKernelContract(**base)


def test_contract_ids_are_stable_and_ignore_the_symbol():
    a, b = _contract(), _contract(symbol="other_name")
    assert a.stable_id == b.stable_id and a.stable_id.startswith("nk_") and len(a.stable_id) == 27
    assert _contract(specialization=(("m", 16),)).stable_id != a.stable_id
    assert _contract(launch=contracts.Launch((5, 1, 1), (128, 1, 1))).stable_id != a.stable_id
    with pytest.raises(dataclasses.FrozenInstanceError):
        a.symbol = "x"


@pytest.mark.parametrize("bad", [
    dict(target="gfx950"), dict(wave_size=64), dict(kernarg_size=30), dict(symbol=""),
    dict(constants=(("m", 1),), specialization=(("m", 2),)),
])
def test_invalid_contracts_are_refused(bad):
    with pytest.raises(ValidationError):
        _contract(**bad)


def test_launch_and_semantics_validation():
    with pytest.raises(ValidationError):
        contracts.Launch((1, 1), (32, 1, 1))
    with pytest.raises(ValidationError):
        contracts.Launch((1, 1, 1), (1025, 1, 1))
    with pytest.raises(ValidationError):
        contracts.Launch((1, 1, 1), (32, 1, 1), 0, 300000)
    with pytest.raises(ValidationError):
        contracts.KernelSemantics("qwen36.abi", "d", "q", "l", "n")
    with pytest.raises(ValidationError):
        contracts.KernelSemantics("abi with space", "d", "q", "l", "n")


# ------------------------------------------------------------------ profiles
def test_profile_registry_selection_and_tensor_parallel_binding():
    reg = profiles.load_profile_registry(LIB_ROOT, TARGET, tensor_parallel=1)
    names = [p.name for p in reg]
    assert names == sorted(names) and {"cpu_t16", "decode_t256", "prefill_t8192"} <= set(names)
    dims = {"m": 256, "batch": 1, "sequence": 0}
    hit = profiles.select_profile(reg, dims, quantization="fp8_block128", tensor_parallel=1)
    assert hit.supported and hit.profile.name == "decode_t256"
    assert not profiles.select_profile(reg, {**dims, "m": 255}, quantization="fp8_block128", tensor_parallel=1).supported
    assert not profiles.select_profile(reg, dims, quantization="mxfp4", tensor_parallel=1).supported
    assert not profiles.select_profile(reg, dims, quantization="fp8_block128", tensor_parallel=2).supported
    reg2 = profiles.load_profile_registry(LIB_ROOT, TARGET, tensor_parallel=2)
    assert profiles.select_profile(reg2, dims, quantization="fp8_block128", tensor_parallel=2).supported
    with pytest.raises(ValidationError):
        profiles.DimensionGuard(5, 4)
    bounded = profiles.ShapeProfile("b", (("m", profiles.DimensionGuard(1, 16)),))
    assert bounded.matches({"m": 16}, quantization="fp8_block128", tensor_parallel=1)
    with pytest.raises(ValidationError):
        bounded.exact_value("m")


# ------------------------------------------------------------------ expressions and memory plan
def test_expression_language_is_closed():
    env = {"m": 256, "pairs": 2048}
    assert expr.evaluate("ceil_div(m,16)", env) == 16 and expr.evaluate("align(pairs+1, 1024)", env) == 3072
    assert expr.evaluate(7, env) == 7 and expr.evaluate("max(m//3, 2)*2", env) == 170
    for bad in ("__import__('os')", "m.real", "m**2", "unknown+1", "m//0", "1-2", "ceil_div(m)", "[1]"):
        with pytest.raises(ValidationError):
            expr.evaluate(bad, env)


def test_memory_plan_reuses_dead_buffers_and_never_overlaps_live_ones():
    R = memory.BufferRequest
    placed, total = memory.plan_buffers([R("a", 4000, 1024, 0, 1), R("b", 3000, 1024, 1, 2), R("c", 4096, 1024, 2, 3),
                                         R("keep", 100, 1024, 0, 0, True)])
    by = {p.name: p for p in placed}
    assert by["c"].offset == by["a"].offset            # a is dead when c is born
    assert by["b"].offset >= by["a"].offset + 4000
    for x in placed:
        for y in placed:
            if x.name < y.name and not (x.last_use < y.first_use or y.last_use < x.first_use) or "keep" in (x.name, y.name) and x.name != y.name:
                assert x.offset + x.bytes <= y.offset or y.offset + y.bytes <= x.offset
    assert total % 1024 == 0 and all(p.offset % 1024 == 0 for p in placed)
    with pytest.raises(ValidationError):
        memory.checked_mul(1 << 40, 1 << 40)
    with pytest.raises(ValidationError):
        memory.align_up(10, 3)


# ------------------------------------------------------------------ catalog and planner
def test_catalog_is_locked_to_the_kernel_sources_and_model_independent(tmp_path):
    tactics = catalog.load_fixed_tactic_catalog(LIB_ROOT, TARGET)
    assert len(tactics) >= 12 and all(t.rank >= 0 for t in tactics)
    assert any(t.maturity is Maturity.REJECTED for t in tactics)
    # a changed kernel source invalidates the catalog
    root = tmp_path / "lib"
    shutil.copytree(LIB_ROOT / "manifests", root / "manifests")
    (root / "csrc").mkdir()
    for rel in ("common.cuh", "route_kernels.cu", "bridge_kernels.cu", "umma_kernels.cu", "umma_tokmajor.cu", "router_umma.cu", "kernels_cubin.cu"):
        shutil.copyfile(LIB_ROOT / "csrc" / rel, root / "csrc" / rel)
    catalog.load_fixed_tactic_catalog(root, TARGET)
    with open(root / "csrc" / "umma_kernels.cu", "a") as f:
        f.write("// edit\n")
    with pytest.raises(ValidationError, match="changed since the catalog was locked"):
        catalog.load_fixed_tactic_catalog(root, TARGET)


def test_catalog_launch_constants_match_the_built_library():
    lib = abi.load()
    tactics = {t.name: t for t in catalog.load_fixed_tactic_catalog(LIB_ROOT, TARGET)}
    for which, name in ((0, "gate_up_silu_requant_umma_swapab_tiles128"), (1, "down_projection_umma_swapab_tiles128"),
                        (2, "gate_up_silu_requant_umma_tokmajor_tiles128"), (3, "down_projection_umma_tokmajor_row_major"),
                        (4, "down_projection_umma_tokmajor_f16_tiles128"), (5, "router_logits_f32_bf16_umma"),
                        (6, "gate_up_silu_requant_mxfp4_block_scaled_swapab"), (7, "down_projection_mxfp4_block_scaled_swapab"),
                        (8, "gate_up_silu_requant_mxfp4_block_scaled_tokmajor"), (9, "down_projection_mxfp4_block_scaled_tokmajor")):
        block, smem = ctypes.c_uint32(), ctypes.c_uint32()
        assert lib.netra_moe_kernel_launch_info(which, ctypes.byref(block), ctypes.byref(smem)) == 0
        assert tactics[name].launch["block"][0] == block.value
        assert tactics[name].launch["dynamic_lds_bytes"] == smem.value


def test_prefill_profile_selects_the_tensor_core_router_and_the_fp16_row_tactics(tmp_path):
    """Above 1,024 rows the router pair changes (tensor-core pass + exact fix-up); the prefill model manifest asks for FP16
    partial rows, which only the token-major profiles can serve - the decode profile of the same model keeps FP32 rows."""
    prefill = LIB_ROOT / "manifests" / TARGET / "models" / "routed-moe-layer-fp8-prefill.json"
    picked = {o["name"]: o["tactic"] for o in compile_engine(prefill, "prefill_t8192", tmp_path / "p", copy_cubin=False)["operations"]}
    assert picked["router_logits"] == "router_logits_f32_bf16_umma" and picked["topk_quant"] == "softmax_top8_quant_exact_fixup"
    assert picked["down"] == "down_projection_umma_tokmajor_f16_tiles128" and picked["combine"] == "combine_slot_ordered_f16_partials"
    decode = {o["name"]: o["tactic"] for o in compile_engine(prefill, "decode_t256", tmp_path / "d", copy_cubin=False)["operations"]}
    assert decode["router_logits"] == "router_logits_bf16_fp64_mma_k8" and decode["combine"] == "combine_slot_ordered_fp32"
    plain = {o["name"]: o["tactic"] for o in compile_engine(MODEL, "prefill_t8192", tmp_path / "q", copy_cubin=False)["operations"]}
    assert plain["down"] == "down_projection_umma_tokmajor_tiles128" and plain["combine"] == "combine_slot_ordered_fp32"
    contracts_p = json.loads((tmp_path / "p" / "contracts.json").read_text())["contracts"]
    contracts_q = json.loads((tmp_path / "q" / "contracts.json").read_text())["contracts"]
    numerical = lambda cs, op: next(c["semantics"]["numerical"] for c in cs if c["operation"] == op)
    assert numerical(contracts_p, "down_projection") != numerical(contracts_q, "down_projection")     # a numerical id of its own


def test_mxfp4_model_selects_the_block_scaled_tactics_and_a_pack_step(tmp_path):
    """An MXFP4 model manifest: the two grouped GEMMs resolve to the block-scaled kernels (swap-AB at decode size, token-major
    at prefill size), the four-bit weight tensor maps are described as such, the layout plan names the pack entry point, and
    an FP8 profile cannot serve the model."""
    model = LIB_ROOT / "manifests" / TARGET / "models" / "routed-moe-layer-mxfp4.json"
    dec = compile_engine(model, "decode_t256_mxfp4", tmp_path / "d", copy_cubin=False)
    picked = {o["name"]: o["tactic"] for o in dec["operations"]}
    assert picked["gate_up"] == "gate_up_silu_requant_mxfp4_block_scaled_swapab"
    assert picked["down"] == "down_projection_mxfp4_block_scaled_swapab"
    assert picked["router_logits"] == "router_logits_bf16_fp64_mma_k8" and picked["combine"] == "combine_slot_ordered_fp32"
    pre = compile_engine(model, "prefill_t8192_mxfp4", tmp_path / "p", copy_cubin=False)
    picked = {o["name"]: o["tactic"] for o in pre["operations"]}
    assert picked["gate_up"] == "gate_up_silu_requant_mxfp4_block_scaled_tokmajor"
    assert picked["down"] == "down_projection_mxfp4_block_scaled_tokmajor"
    engine = json.loads((tmp_path / "d" / "engine.json").read_text())
    gate_up = next(o for o in engine["operations"] if o["name"] == "gate_up")
    w13_map = gate_up["arguments"][0]["tensor_map"]
    assert w13_map == {"rows": 257 * 1024 * 16, "row_bytes": 64, "box_rows": 256, "box_bytes": 128, "swizzle": "128B", "element": "e2m1"}
    assert "element" not in gate_up["arguments"][1]["tensor_map"]
    plan = json.loads((tmp_path / "d" / "layout_plan.json").read_text())
    assert [s["entry_point"] for s in plan["steps"]] == ["netra_moe_mxfp4_pack_launch"] * 2
    assert [s["paired_half_rows"] for s in plan["steps"]] == [512, 128]
    assert plan["weights"][0]["steps"][0]["operation"] == "mxfp4_pair_blocks"
    with pytest.raises(ValidationError):
        compile_engine(model, "decode_t256", tmp_path / "x", copy_cubin=False)          # an FP8 profile
    with pytest.raises(ValidationError):
        compile_engine(MODEL, "decode_t256_mxfp4", tmp_path / "y", copy_cubin=False)    # an FP8 model


def test_binding_sets_replicate_the_profile_over_one_workspace(tmp_path):
    """binding_sets = 2: two profile ids with the same guards (their own pointers and graph at run time), one operation
    list, one workspace; the directory still validates."""
    one = compile_engine(MODEL, "decode_t256", tmp_path / "one", copy_cubin=False)
    two = compile_engine(MODEL, "decode_t256", tmp_path / "two", binding_sets=2)
    assert [p["name"] for p in two["profiles"]] == ["decode_t256", "decode_t256@1"]
    assert two["profiles"][0]["guards"] == two["profiles"][1]["guards"] == one["profiles"][0]["guards"]
    assert two["workspace_bytes"] == one["workspace_bytes"] and two["operations"] == one["operations"]
    validate_engine_directory(tmp_path / "two")
    with pytest.raises(ValidationError):
        compile_engine(MODEL, "decode_t256", tmp_path / "bad", copy_cubin=False, binding_sets=0)


def test_mxfp4_pair_blocks_byte_transform():
    """CPU statement of the pack step: every source byte appears once, rows of a tile pair end up side by side."""
    rng = np.random.default_rng(3)
    codes = rng.integers(0, 256, (512, 256), dtype=np.uint8)         # 512 rows, k = 512
    scales = rng.integers(0, 256, (512, 16), dtype=np.uint8)
    c, s = layouts.mxfp4_pair_blocks(codes, scales, 128)
    assert c.shape == codes.shape and s.shape == scales.shape
    blocks = c.reshape(2, 4, 2, 128, 64)                              # [pair, kb, tile of the pair, r, 64]
    assert np.array_equal(blocks[1, 2, 1], codes[384:512, 128:192])   # pair 1 = tiles 2 and 3; tile 3, K-block 2
    atoms = s.reshape(2, 4, 2, 32, 4, 4)
    assert np.array_equal(atoms[0, 3, 0, 5, 2], scales[2 * 32 + 5, 12:16])     # row 69 of tile 0, K-block 3
    c13, _ = layouts.mxfp4_pair_blocks(np.tile(codes, (4, 1)), np.tile(scales, (4, 1)), 512)      # 2 slabs of 1024 rows
    assert np.array_equal(c13.reshape(2, 4, 4, 2, 128, 64)[1, 3, 0, 1], np.tile(codes, (4, 1))[1024 + 512 + 384:1024 + 1024, 0:64])
    with pytest.raises(ValidationError):
        layouts.mxfp4_pair_blocks(codes, scales, 96)


def _plan(model_path, profile_name, **kw):
    model = frontend.load_model(model_path)
    reg = profiles.load_profile_registry(LIB_ROOT, TARGET, 1)
    profile = next(p for p in reg if p.name == profile_name)
    graph = frontend.routed_moe_layer_graph(model, profile)
    tactics = kw.pop("tactics", None) or catalog.load_fixed_tactic_catalog(LIB_ROOT, TARGET)
    return planner.plan_graph(graph, profile, TARGET, tactics, frontend.dimensions_for(model, profile),
                              frontend.options_for(model), **kw)


def test_planner_selects_by_layout_size_and_never_a_rejected_tactic():
    plan = _plan(MODEL, "decode_t256")
    chosen = {p.operation.name: p.tactic.name for p in plan.operations}
    assert chosen["gate_up"].endswith("tiles128") and chosen["token_sort"] == "token_sort_single_block"
    assert chosen["combine"] == "combine_slot_ordered_fp32" and not plan.requires_fallback
    combine = next(p for p in plan.operations if p.operation.name == "combine")
    rejected = [c for c in combine.explanation if c["tactic"] == "combine_atomic_fp32_experiment"][0]
    assert not rejected["selected"] and "tactic is rejected" in rejected["reasons"]
    big = _plan(MODEL_ZIPF, "prefill_t8192")
    names = [p.operation.name for p in big.operations]
    assert names[2:5] == ["sort_hist", "sort_scan", "sort_scatter"]
    # 8,192 tokens: the token-major GEMM form (row-major weights in this model), with its register contract
    down = next(p for p in big.operations if p.operation.name == "down")
    assert down.tactic.name == "down_projection_umma_tokmajor_row_major"
    assert down.contract.launch.registers_per_thread == 168 and down.contract.launch.block == (384, 1, 1)
    gate = next(p for p in big.operations if p.operation.name == "gate_up")
    assert gate.tactic.name == "gate_up_silu_requant_umma_tokmajor_row_major"
    other = [c for c in gate.explanation if c["tactic"] == "gate_up_silu_requant_umma_swapab_tiles128"][0]
    assert any("semantic layouts mismatch" in r for r in other["reasons"])
    # below 1,024 tokens the token-major tactics are out of their size limits and the swap-AB form is requested
    small_gate = next(p for p in plan.operations if p.operation.name == "gate_up")
    assert small_gate.tactic.name == "gate_up_silu_requant_umma_swapab_tiles128" and "registers_per_thread" not in small_gate.contract.launch.to_dict()


def test_planner_falls_back_and_refuses_ambiguity():
    tactics = catalog.load_fixed_tactic_catalog(LIB_ROOT, TARGET)
    without_sort = tuple(t for t in tactics if t.operation != "token_sort")
    plan = _plan(MODEL, "decode_t256", tactics=without_sort)
    sort = next(p for p in plan.operations if p.operation.name == "token_sort")
    assert sort.execution == "fallback" and plan.requires_fallback and sort.fallback == "framework.token_sort"
    twin = dataclasses.replace(next(t for t in tactics if t.name == "combine_slot_ordered_fp32"), name="combine_twin")
    with pytest.raises(ValidationError, match="ambiguous fixed tactics"):
        _plan(MODEL, "decode_t256", tactics=tactics + (twin,))
    wrong_const = dataclasses.replace(next(t for t in tactics if t.operation == "router_logits"),
                                      constants=(("hidden", 4096), ("routed_experts", 256)))
    reasons = wrong_const.rejection_reasons(planner.fixed_request(plan.graph.operations[0], TARGET, {"m": 256}, {}))
    assert any("hidden mismatch" in r for r in reasons)
    experiment = dataclasses.replace(tactics[0], maturity=Maturity.EXPERIMENT)
    req = planner.fixed_request(plan.graph.operations[0], TARGET, {"m": 256}, {})
    assert "experimental tactic requires --allow-experimental" in experiment.rejection_reasons(req)
    assert experiment.rejection_reasons(req, allow_experimental=True) == ()


# ------------------------------------------------------------------ engine emitter and validator
def test_engine_compile_is_deterministic_and_valid(tmp_path):
    a = compile_engine(MODEL, "decode_t256", tmp_path / "a")
    b = compile_engine(MODEL, "decode_t256", tmp_path / "b")
    assert a["engine_id"] == b["engine_id"] and a["engine_id"].startswith("ne_")
    assert engine.semantic_file_hashes(tmp_path / "a") == engine.semantic_file_hashes(tmp_path / "b")
    assert compile_engine(MODEL, "cpu_t16", tmp_path / "c")["engine_id"] != a["engine_id"]
    validate_engine_directory(tmp_path / "a")
    doc = json.loads((tmp_path / "a" / "engine.json").read_text())
    assert doc["target"] == "sm_100a" and doc["wave_size"] == 32 and doc["required_cuda"]["minimum"] == "12.8"
    assert [o["name"] for o in doc["operations"]] == ["router_logits", "topk_quant", "token_sort", "gather_rows", "gate_up", "down", "combine"]
    assert all(o["execution"] == "kernel" for o in doc["operations"]) and doc["fallbacks"] == {}
    recipe = json.loads((tmp_path / "a" / "graph_recipe.json").read_text())
    assert recipe["operations"][4]["depends_on"] == [2, 3] and recipe["operations"][6]["depends_on"] == [1, 2, 5]
    assert set(recipe["binding_slots"]) == {"hidden", "output", "router_weight", "w13", "w13_scale", "w2", "w2_scale"}
    # optional operands the model lacks become null pointers, workspace offsets land inside the plan
    topk = doc["operations"][1]["arguments"]
    assert [a["source"] for a in topk if a["name"] in ("router_bias", "shared_weight")] == ["null", "null"]
    explain = json.loads((tmp_path / "a" / "explain.json").read_text())
    assert len(explain["operations"]) == 7 and all(any(c["selected"] for c in o["candidates"]) for o in explain["operations"])


def test_engine_with_bias_shared_weight_and_segmented_sort(tmp_path):
    doc = compile_engine(MODEL_ZIPF, "prefill_t8192", tmp_path / "e")
    names = [o["name"] for o in doc["operations"]]
    assert names == ["router_logits", "topk_quant", "sort_hist", "sort_scan", "sort_scatter", "gather_rows", "gate_up", "down", "combine"]
    recipe = json.loads((tmp_path / "e" / "graph_recipe.json").read_text())
    assert {"router_bias", "shared_weight"} <= set(recipe["binding_slots"])
    assert json.loads((tmp_path / "e" / "layout_plan.json").read_text())["steps"] == []
    gate = doc["operations"][6]
    assert gate["arguments"][0]["tensor_map"] == {"rows": 257 * 1024, "row_bytes": 2048, "box_rows": 128, "box_bytes": 128, "swizzle": "128B"}
    assert gate["launch"]["grid"] == [148, 1, 1]


def test_validator_catches_tampering(tmp_path):
    compile_engine(MODEL, "cpu_t16", tmp_path / "e")
    path = tmp_path / "e" / "engine.json"
    good = json.loads(path.read_text())

    def with_change(mutate):
        doc = json.loads(json.dumps(good))
        mutate(doc)
        path.write_text(json.dumps(doc))
        with pytest.raises(ValidationError):
            validate_engine_directory(tmp_path / "e")
        path.write_text(json.dumps(good))

    with_change(lambda d: d.__setitem__("target", "gfx950"))
    with_change(lambda d: d["operations"][0].__setitem__("cubin", "cubin/../x.cubin"))
    with_change(lambda d: d["operations"][0]["arguments"][1].__setitem__("offset", 4))
    with_change(lambda d: d["operations"][4]["arguments"][4].__setitem__("workspace_offset", 1 << 40))
    with_change(lambda d: d["operations"][0].__setitem__("contract_id", "nk_missing"))
    with_change(lambda d: d["artifact_files"].__setitem__("cubin/netra_moe_sm100a.cubin", "0" * 64))
    validate_engine_directory(tmp_path / "e")
    (tmp_path / "e" / "explain.json").unlink()
    with pytest.raises(ValidationError, match="lacks explain.json"):
        validate_engine_directory(tmp_path / "e")


def test_unknown_profile_and_bad_model_are_reported(tmp_path):
    with pytest.raises(ValidationError, match="unknown profile"):
        compile_engine(MODEL, "decode_t255", tmp_path / "x")
    bad = json.loads(MODEL.read_text())
    bad["constants"]["hidden"] = -1
    (tmp_path / "bad.json").write_text(json.dumps(bad))
    with pytest.raises(ValidationError):
        compile_engine(tmp_path / "bad.json", "decode_t256", tmp_path / "y")
    bad = json.loads(MODEL.read_text())
    bad["constants"]["hidden"] = 4096          # valid manifest, but no kernel is built for it
    (tmp_path / "h4096.json").write_text(json.dumps(bad))
    doc = compile_engine(tmp_path / "h4096.json", "decode_t256", tmp_path / "z")
    assert doc["fallbacks"] and any(o["execution"] == "fallback" for o in doc["operations"])


def test_cli_round_trip(tmp_path, capsys):
    from netra_kernel_b200.compiler import cli
    assert cli.main(["compile", "--model", str(MODEL), "--profile", "cpu_t16", "--output", str(tmp_path / "e")]) == 0
    assert cli.main(["validate", str(tmp_path / "e")]) == 0
    assert cli.main(["list-tactics"]) == 0
    out = capsys.readouterr().out
    assert "engine_id ne_" in out and "router_logits_bf16_fp64_mma" in out
    assert cli.main(["compile", "--model", str(MODEL), "--profile", "nope", "--output", str(tmp_path / "f")]) == 2


# ------------------------------------------------------------------ layout plan, dense contract, verify profile
def test_weight_and_scale_layout_plans_and_their_byte_transforms():
    import numpy as np
    from netra_kernel_b200.compiler import layouts as L
    same = L.plan_weight_layout("w2", L.ROW_MAJOR, L.ROW_MAJOR)
    assert same.steps == ()
    tiled = L.plan_weight_layout("w2", L.ROW_MAJOR, L.TILES128, checkpoint_tensors=("w2",))
    assert [s.operation for s in tiled.steps] == ["tile_128x128"] and tiled.steps[0].entry_point == "netra_moe_repack_tiles_launch"
    split = L.plan_weight_layout("w13", L.SPLIT_GATE_UP, L.TILES128, checkpoint_tensors=("gate_proj", "up_proj"))
    assert [s.operation for s in split.steps] == ["concatenate_output_shards", "tile_128x128"]
    with pytest.raises(ValidationError):
        L.plan_weight_layout("w13", L.SPLIT_GATE_UP, L.TILES128, checkpoint_tensors=("gate_proj",))
    with pytest.raises(ValidationError):
        L.plan_weight_layout("w13", "aiter_shuffle_16x16_fp8_block128", L.TILES128)
    scale = L.plan_scale_layout("w13_scale", ("gate_proj_scale_inv", "up_proj_scale_inv"), checkpoint_dtype="bf16", kernel_dtype="fp32",
                                block=(128, 128))
    assert scale.steps == ("concatenate_output_scale_shards_axis0", "widen_bf16_to_fp32_exact")
    with pytest.raises(ValidationError):
        L.plan_scale_layout("s", ("a",), checkpoint_dtype="fp32", kernel_dtype="bf16", block=(128, 128))
    with pytest.raises(ValidationError):
        L.plan_scale_layout("s", (), checkpoint_dtype="fp32", kernel_dtype="fp32", block=(128, 128))
    # byte level: tile (i, j) of the output is rows [128 i, +128) x bytes [128 j, +128) of the input, and the transform inverts
    rng = np.random.default_rng(0)
    data = rng.integers(0, 256, (384, 512), dtype=np.uint8)
    out = L.tile_128x128(data)
    tiles = out.reshape(3, 4, 128, 128)
    for i, j in ((0, 0), (1, 3), (2, 1)):
        assert np.array_equal(tiles[i, j], data[128 * i:128 * i + 128, 128 * j:128 * j + 128])
    assert np.array_equal(L.untile_128x128(out), data) and out.tobytes() != data.tobytes()
    gate, up = rng.integers(0, 256, (2, 128, 256), dtype=np.uint8), rng.integers(0, 256, (2, 128, 256), dtype=np.uint8)
    streamed = L.apply_weight_steps(split, [gate, up])
    assert streamed.shape == (2, 256, 256)
    assert np.array_equal(L.untile_128x128(streamed.reshape(512, 256)).reshape(2, 256, 256), np.concatenate([gate, up], axis=1))
    bits = np.array([0x3F80, 0xBF00, 0x0000, 0x7F7F], np.uint16)
    assert L.widen_bf16_to_fp32(bits).tolist() == [1.0, -0.5, 0.0, float(np.float32(3.3895313892515355e38))]
    with pytest.raises(ValidationError):
        L.tile_128x128(np.zeros((100, 128), np.uint8))


def test_engine_layout_plan_names_the_repack_and_scale_steps(tmp_path):
    compile_engine(MODEL, "decode_t256", tmp_path / "e", copy_cubin=False)
    plan = json.loads((tmp_path / "e" / "layout_plan.json").read_text())
    assert plan["format"] == "netra-layout-plan-2" and [w["tensor"] for w in plan["weights"]] == ["w13", "w2"]
    assert plan["weights"][0]["steps"][0]["entry_point"] == "netra_moe_repack_tiles_launch" and len(plan["steps"]) == 2
    assert all(sc["steps"] == [] for sc in plan["scales"])                         # FP32 scales need no step
    doc = json.loads(MODEL.read_text())
    doc["options"].update({"split_gate_up": True, "checkpoint_scale_dtype": "bf16"})
    (tmp_path / "m.json").write_text(json.dumps(doc))
    compile_engine(tmp_path / "m.json", "decode_t256", tmp_path / "f", copy_cubin=False)
    plan = json.loads((tmp_path / "f" / "layout_plan.json").read_text())
    assert [st["operation"] for st in plan["weights"][0]["steps"]] == ["concatenate_output_shards", "tile_128x128"]
    assert plan["scales"][0]["steps"] == ["concatenate_output_scale_shards_axis0", "widen_bf16_to_fp32_exact"]
    zipf = json.loads((tmp_path / "e" / "layout_plan.json").read_text())
    compile_engine(MODEL_ZIPF, "decode_t256", tmp_path / "g", copy_cubin=False)      # row-major weights: nothing to repack
    assert json.loads((tmp_path / "g" / "layout_plan.json").read_text())["steps"] == [] and zipf["steps"]


def test_dense_block_scale_contract_and_registry():
    from netra_kernel_b200.compiler import dense
    request = dense.dense_request(1, 2048, 4096)
    contract, explanation = dense.plan_dense(request)
    assert isinstance(contract, contracts.FallbackKernelContract) and contract.fallback == "framework.fp8_blockscale_linear"
    assert explanation[0]["selected"] and explanation[0]["reasons"] == []
    contract2, explanation2 = dense.plan_dense(dense.dense_request(16, 2048, 4096, epilogue="silu"))
    assert not any(e["selected"] for e in explanation2) and any("M=16" in r for r in explanation2[0]["reasons"])
    assert any("epilogue" in r for r in explanation2[0]["reasons"]) and contract2.stable_id == contract.stable_id
    launch = contracts.Launch((16, 1, 1), (320, 1, 1), 0, 200000)
    kc = dense.KernelContract(TARGET, 32, "dense", 1, 2048, 4096, "fp8_e4m3", "fp8_e4m3", "fp32", "bf16", "fp8_e4m3_per_token_block128_amax448",
                              "fp8_e4m3_w128x128", 128, (128, 128), "row_major_fp8_block128", "tiles128x128_fp8_block128", "row_major_bf16",
                              "identity", "probe", launch)
    assert kc.stable_id.startswith("nk_") and len(kc.stable_id) == 27 and kc.to_dict()["shape"] == [1, 2048, 4096]
    assert dataclasses.replace(kc, m=2).stable_id != kc.stable_id and dataclasses.replace(kc, evidence_refs=("x",)).stable_id == kc.stable_id
    for bad in (dict(k=4000), dict(n=2000), dict(accumulator_dtype="bf16"), dict(operation="conv"), dict(m=0),
                dict(numerical=dense.NumericalContract(deterministic=False))):
        with pytest.raises(ValidationError):
            dataclasses.replace(kc, **bad)


def test_verify_profile_fixes_the_routed_rows(tmp_path):
    """The reference's exact verify profile (12 draft positions x 64 sequences = 768 routed rows): the graph is sized by
    route_rows, the runtime guards are m and batch."""
    reg = profiles.load_profile_registry(LIB_ROOT, TARGET, tensor_parallel=1)
    verify = next(p for p in reg if p.name == "verify_m12_b64_routes768")
    assert frontend.token_rows(verify) == 768
    hit = profiles.select_profile(reg, {"m": 12, "batch": 64, "sequence": 0, "route_rows": 768}, quantization="fp8_block128", tensor_parallel=1)
    assert hit.supported and hit.profile.name == "verify_m12_b64_routes768"
    engine_doc = compile_engine(MODEL, "verify_m12_b64_routes768", tmp_path / "v", copy_cubin=False)
    guards = engine_doc["profiles"][0]["guards"]
    assert guards["m"] == {"min": 12, "max": 12} and guards["batch"] == {"min": 64, "max": 64}
    router = engine_doc["operations"][0]
    assert router["launch"]["grid"][0] == 768 // 16 and [o["tactic"] for o in engine_doc["operations"]][2] == "token_sort_single_block"
    bad = profiles.ShapeProfile("bad", (("batch", profiles.DimensionGuard(64, 64)), ("m", profiles.DimensionGuard(12, 12)),
                                        ("route_rows", profiles.DimensionGuard(700, 700))))
    with pytest.raises(ValidationError):
        frontend.token_rows(bad)

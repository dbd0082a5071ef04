"""Engine-directory emitter: model manifest + profile + tactic catalog -> a deterministic folder
(``engine.json`` and siblings, plus ``cubin/``) that the runtime loads.  Role of the reference's
``compiler/netra_compiler/engine.py:373-504``; file set and the fields the runtime consumes follow
it, with ``target: sm_100a``, ``wave_size: 32``, ``required_cuda`` and ``cubin`` in place of the
ROCm / HSACO fields."""
from __future__ import annotations

import shutil
from pathlib import Path
from typing import Any

from . import __name__ as _pkg
from .catalog import FixedCudaTactic, load_fixed_tactic_catalog
from .expr import evaluate
from .frontend import dimensions_for, load_model, options_for, routed_moe_layer_graph
from .layouts import moe_layer_layout_plan
from .library import KernelLibrary
from .memory import BufferRequest, plan_buffers
from .planner import Plan, PlannedOperation, plan_graph
from .profiles import load_profile_registry
from .types import TARGET, WARP_SIZE, ValidationError, file_sha256, stable_hash, write_json

ENGINE_FORMAT = "netra-engine-1"
REQUIRED_CUDA_MINIMUM = "12.8"
COMPILER_VERSION = "0.1.0"
# read back by callers after a launch, so their bytes are never shared with another buffer
PINNED_WORKSPACE = ("topk_ids", "topk_weights", "perm", "inv_perm", "counts", "offsets", "status")


def _compiler_source_hash() -> str:
    here = Path(__file__).resolve().parent
    return stable_hash({p.name: file_sha256(p) for p in sorted(here.glob("*.py"))})


def _memory_plan(plan: Plan) -> dict[str, Any]:
    uses: dict[str, list[int]] = {}
    for index, planned in enumerate(plan.operations):
        for name in (*planned.operation.inputs, *planned.operation.outputs):
            uses.setdefault(name, []).append(index)
    requests = []
    for tensor in plan.graph.tensors:
        if tensor.role != "workspace":
            continue
        touched = uses.get(tensor.name)
        if not touched:
            raise ValidationError(f"workspace tensor {tensor.name!r} is never used")
        pinned = tensor.name in PINNED_WORKSPACE
        requests.append(BufferRequest(tensor.name, tensor.bytes, tensor.alignment, min(touched),
                                      len(plan.operations) - 1 if pinned else max(touched), pinned))
    placed, total = plan_buffers(requests, alignment=1024)
    return {"format": "netra-memory-plan-1", "workspace_bytes": total, "workspace_alignment": 1024,
            "buffers": [p.to_dict() for p in placed]}


def _dependencies(plan: Plan) -> list[list[int]]:
    """RAW / WAR / WAW edges between operations, by tensor name, in program order."""
    last_write: dict[str, int] = {}
    readers: dict[str, list[int]] = {}
    out = []
    for index, planned in enumerate(plan.operations):
        deps: set[int] = set()
        for name in planned.operation.inputs:
            if name in last_write:
                deps.add(last_write[name])
        for name in planned.operation.outputs:
            if name in last_write:
                deps.add(last_write[name])
            deps.update(readers.get(name, ()))
        deps.discard(index)
        out.append(sorted(deps))
        for name in planned.operation.inputs:
            readers.setdefault(name, []).append(index)
        for name in planned.operation.outputs:
            last_write[name] = index
            readers[name] = []
    return out


def _argument_records(planned: PlannedOperation, plan: Plan, offsets: dict[str, int], env: dict[str, int]) -> list[dict[str, Any]]:
    tactic: FixedCudaTactic = planned.tactic  # type: ignore[assignment]
    known = {t.name: t for t in plan.graph.tensors}
    records = []
    byte = 0
    for arg in tactic.arguments:
        size = {"pointer": 8, "tensor_map": 128, "u32": 4}[arg.kind]
        align = 64 if arg.kind == "tensor_map" else size
        byte = (byte + align - 1) // align * align
        if arg.kind == "u32":
            records.append({"name": arg.name, "kind": "u32_constant", "offset": byte, "value": evaluate(arg.value, env)})
        else:
            record: dict[str, Any] = {"name": arg.name, "kind": arg.kind, "offset": byte, "access": arg.access, "tensor": arg.tensor}
            tensor = known.get(arg.tensor)
            if tensor is None:
                if not arg.optional:
                    raise ValidationError(f"tactic {tactic.name} needs tensor {arg.tensor!r}, which the graph does not define")
                record["source"] = "null"
            elif tensor.role == "workspace":
                record["source"] = "workspace"
                record["workspace_offset"] = offsets[tensor.name]
            else:
                record["source"] = "binding"
            if arg.kind == "tensor_map":
                if tensor is None:
                    raise ValidationError(f"tensor_map argument {arg.name} cannot be optional")
                record["tensor_map"] = {"rows": evaluate(arg.map["rows"], env), "row_bytes": evaluate(arg.map["row_bytes"], env),
                                        "box_rows": evaluate(arg.map["box_rows"], env), "box_bytes": 128, "swizzle": "128B"}
                if arg.map.get("element", "u8") != "u8":      # "e2m1": four-bit codes, 64 bytes per 128-element row in memory
                    record["tensor_map"]["element"] = str(arg.map["element"])
                span = record["tensor_map"]["rows"] * record["tensor_map"]["row_bytes"]
                if span > tensor.bytes:
                    raise ValidationError(f"tensor map {arg.name} covers {span} bytes but tensor {tensor.name} has {tensor.bytes}")
            records.append(record)
        byte += size
    return records


def compile_engine(model_path: Path | str, profile_name: str, output: Path | str, *, library_root: Path | str | None = None,
                   allow_experimental: bool = False, checkpoint_hash: str = "", copy_cubin: bool = True,
                   binding_sets: int = 1) -> dict[str, Any]:
    """``binding_sets`` > 1 emits the profile that many times (``name``, ``name@1``, ...): every entry is a profile id of its
    own at run time - its own bound pointers and captured graph - over the engine's one workspace and code object.  A
    serving loop that double-buffers its activations binds one input / output pair per set and alternates the profile id."""
    if not 1 <= int(binding_sets) <= 8:
        raise ValidationError("binding_sets must be between 1 and 8")
    library = KernelLibrary.discover(library_root)
    model = load_model(Path(model_path))
    tp = int(model["deployment"]["tensor_parallel"])
    profiles = load_profile_registry(library.root, TARGET, tp)
    profile = next((p for p in profiles if p.name == profile_name), None)
    if profile is None:
        raise ValidationError(f"unknown profile {profile_name!r}; known: {', '.join(p.name for p in profiles)}")
    if profile.quantization != model.get("quantization"):
        raise ValidationError(f"profile {profile.name} is for {profile.quantization}, model is {model.get('quantization')}")
    tactics = load_fixed_tactic_catalog(library.root, TARGET)
    graph = routed_moe_layer_graph(model, profile)
    dims, opts = dimensions_for(model, profile), options_for(model)
    plan = plan_graph(graph, profile, TARGET, tactics, dims, opts, allow_experimental=allow_experimental)
    memory = _memory_plan(plan)
    offsets = {b["name"]: b["offset"] for b in memory["buffers"]}
    deps = _dependencies(plan)

    operations, recipe_ops, contracts, explain, symbols, fallbacks = [], [], {}, [], [], {}
    bindings: dict[str, list[dict[str, int]]] = {}
    cubins: set[str] = set()
    for index, planned in enumerate(plan.operations):
        op = planned.operation
        contracts[planned.contract.stable_id] = planned.contract.to_dict()
        explain.append({"operation": op.name, "candidates": list(planned.explanation)})
        record: dict[str, Any] = {"index": index, "name": op.name, "kind": op.kind, "contract_id": planned.contract.stable_id,
                                  "execution": planned.execution, "fallback": planned.fallback,
                                  "bindings": {"inputs": list(op.inputs), "outputs": list(op.outputs)}}
        if planned.execution == "kernel":
            tactic = planned.tactic
            contract = planned.contract
            env = {**dict(tactic.constants), **dims, **opts}
            args = _argument_records(planned, plan, offsets, env)
            record.update({"tactic": tactic.name, "maturity": tactic.maturity.value, "kernel_symbol": tactic.symbol,
                           "launch": contract.launch.to_dict(), "artifact_kind": "cuda_cubin_kernel",
                           "kernarg_size": contract.kernarg_size, "cubin": f"cubin/{tactic.cubin}", "arguments": args})
            cubins.add(tactic.cubin)
            symbols.append(tactic.symbol)
            for slot, arg in enumerate(args):
                if arg.get("source") == "binding":
                    bindings.setdefault(arg["tensor"], []).append({"operation": index, "argument": slot})
        else:
            fallbacks[op.name] = planned.fallback
        operations.append(record)
        recipe_ops.append({"index": index, "name": op.name, "depends_on": deps[index], "execution": planned.execution,
                           "kernel_symbol": record.get("kernel_symbol"), "launch": record.get("launch"),
                           "bindings": record["bindings"]})

    out = Path(output)
    out.mkdir(parents=True, exist_ok=True)
    artifact_files = {}
    if copy_cubin:
        for name in sorted(cubins):
            source = library.csrc / name
            if not source.is_file():
                raise ValidationError(f"{source} is missing: build it with `python -m netra_kernel_b200.csrc.build`")
            (out / "cubin").mkdir(exist_ok=True)
            shutil.copyfile(source, out / "cubin" / name)
            artifact_files[f"cubin/{name}"] = file_sha256(source)

    # declarative weight / scale layout plan (layouts.py); "steps" keeps the flat list of device repacks the runtime helper runs
    layout_plan = moe_layer_layout_plan(model["options"]["weight_layout"], split_gate_up=bool(model["options"].get("split_gate_up", False)),
                                        scale_dtype=str(model["options"].get("checkpoint_scale_dtype", "fp32")))
    if model["options"]["weight_layout"] == "mxfp4_paired_blocks":
        layout_plan["steps"] = [
            {"tensor": name, "scale_tensor": name + "_scale", "from": "row_major[group,n,k/2] e2m1x2 + [group,n,k/32] ue8m0",
             "to": "blocks128x64B[pair,k/128,2,128,64] + scale_atoms512B[pair,k/128,2]", "kernel": "netra_moe_mxfp4_pack_sm100",
             "entry_point": "netra_moe_mxfp4_pack_launch", "paired_half_rows": half}
            for name, half in (("w13", 512), ("w2", 128))]
    else:
        layout_plan["steps"] = [
            {"tensor": name, "from": "row_major[group,n,k]", "to": "tiles128x128[group,n/128,k/128,128,128]",
             "kernel": "netra_moe_repack_tiles_sm100", "entry_point": "netra_moe_repack_tiles_launch", "scales": "unchanged"}
            for name in ("w13", "w2")] if opts["w_tiled"] else []
    selected = [{"operation": p.operation.name, "tactic": p.tactic.name, "contract_id": p.contract.stable_id}
                for p in plan.operations if p.tactic is not None]
    identity = {
        "format_version": ENGINE_FORMAT, "target": TARGET, "wave_size": WARP_SIZE, "model_configuration_hash": stable_hash(model),
        "profile": profile.to_dict(), "operations": operations, "memory_plan": memory, "layout_plan": layout_plan,
        "compiler": {"name": _pkg, "version": COMPILER_VERSION, "source_hash": _compiler_source_hash()},
        "catalog_sources": sorted({h for t in tactics for h in t.source_hashes}), "checkpoint_hash": checkpoint_hash,
    }
    engine = {
        **identity, "engine_id": "ne_" + stable_hash(identity)[:24],
        "required_cuda": {"minimum": REQUIRED_CUDA_MINIMUM, "cubin_arch": TARGET},
        "workspace_bytes": memory["workspace_bytes"], "tensor_parallel": tp,
        "profiles": [{"name": profile.name if i == 0 else f"{profile.name}@{i}", "guards": {k: g.to_dict() for k, g in profile.guards},
                      "tensor_parallel": profile.tensor_parallel, "quantization": profile.quantization}
                     for i in range(int(binding_sets))],
        "fallbacks": fallbacks, "kernel_symbols": sorted(set(symbols)), "selected_tactics": selected,
        "artifact_files": artifact_files,
        "deployment_guards": {"device": "NVIDIA B200", "compute_capability": "10.0", "sm_count": opts["sm_count"],
                              "data_parallel_workers": int(model["deployment"]["data_parallel_workers"]),
                              "required_environment": {}},
        "validation_status": {"static": "passed", "parity": "see tests", "graph_replay": "see tests", "matched_server_ab": "not_run"},
        "graph_recipe": "graph_recipe.json",
    }
    write_json(out / "engine.json", engine)
    write_json(out / "contracts.json", {"format": "netra-contract-set-1", "contracts": [contracts[k] for k in sorted(contracts)]})
    write_json(out / "graph.json", graph.to_dict())
    write_json(out / "graph_recipe.json", {"format": "netra-graph-recipe-1", "capture_at_initialization": True,
                                           "portable_serialized_cuda_graph": False, "operations": recipe_ops,
                                           "binding_slots": {k: bindings[k] for k in sorted(bindings)},
                                           "workspace_tensors": {b["name"]: {"offset": b["offset"], "bytes": b["bytes"]} for b in memory["buffers"]}})
    write_json(out / "memory_plan.json", memory)
    write_json(out / "layout_plan.json", layout_plan)
    write_json(out / "symbols.json", {"selected": sorted(set(symbols)), "candidates": sorted({t.symbol for t in tactics})})
    write_json(out / "validation_plan.json", {"format": "netra-validation-plan-1", "promotion_eligible": False,
                                              "status": engine["validation_status"],
                                              "candidates": [{"tactic": t.name, "maturity": t.maturity.value,
                                                              "sources": dict(t.source_hashes)} for t in tactics]})
    write_json(out / "explain.json", {"format": "netra-explain-1", "profile": profile.name, "operations": explain})
    return engine


def semantic_file_hashes(directory: Path | str) -> dict[str, str]:
    """sha256 of every JSON file of an engine directory (two compiles must agree byte for byte)."""
    d = Path(directory)
    return {p.name: file_sha256(p) for p in sorted(d.glob("*.json"))}

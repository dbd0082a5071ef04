"""Static re-check of an engine directory without a GPU: required files and fields, artifact
hashes, kernel-parameter offsets (no overlap, inside ``kernarg_size``), workspace ranges, cubin
paths.  Role of the reference's ``compiler/netra_compiler/validation.py:22-144``."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any

from .types import TARGET, WARP_SIZE, ValidationError, file_sha256

ENGINE_FILES = ("engine.json", "contracts.json", "graph.json", "graph_recipe.json", "memory_plan.json",
                "layout_plan.json", "symbols.json", "validation_plan.json", "explain.json")
_ARG_SIZE = {"pointer": 8, "tensor_map": 128, "u32_constant": 4}


def _load(path: Path) -> Any:
    try:
        return json.loads(path.read_text(encoding="utf-8"))
    except (OSError, json.JSONDecodeError) as exc:
        raise ValidationError(f"cannot read {path}: {exc}") from exc


def validate_engine_directory(directory: Path | str, *, require_artifacts: bool = True) -> dict[str, Any]:
    d = Path(directory)
    for name in ENGINE_FILES:
        if not (d / name).is_file():
            raise ValidationError(f"engine directory lacks {name}")
    engine = _load(d / "engine.json")
    if engine.get("format_version") != "netra-engine-1" or engine.get("target") != TARGET or engine.get("wave_size") != WARP_SIZE:
        raise ValidationError("engine target/format/wave contract mismatch")
    for key in ("engine_id", "required_cuda", "workspace_bytes", "profiles", "operations", "tensor_parallel"):
        if key not in engine:
            raise ValidationError(f"engine.json lacks {key}")
    workspace = int(engine["workspace_bytes"])
    contracts = {c["id"] for c in _load(d / "contracts.json").get("contracts", [])}
    for profile in engine["profiles"]:
        for dim in ("m", "batch", "sequence"):
            g = profile.get("guards", {}).get(dim)
            if not isinstance(g, dict) or not 0 <= int(g.get("min", -1)) <= int(g.get("max", -1)):
                raise ValidationError(f"profile {profile.get('name')} lacks a valid {dim} guard")
    for op in engine["operations"]:
        if op.get("contract_id") not in contracts:
            raise ValidationError(f"operation {op.get('name')} names an unknown contract")
        if op.get("execution") != "kernel":
            continue
        cubin = op.get("cubin", "")
        parts = cubin.split("/")
        if len(parts) < 2 or parts[0] != "cubin" or any(p in ("", ".", "..") for p in parts) or "\\" in cubin:
            raise ValidationError(f"operation {op['name']}: cubin must be a normalized engine-relative path")
        if require_artifacts:
            if not (d / cubin).is_file():
                raise ValidationError(f"operation {op['name']}: {cubin} is missing")
            if engine.get("artifact_files", {}).get(cubin) != file_sha256(d / cubin):
                raise ValidationError(f"operation {op['name']}: {cubin} does not match its recorded sha256")
        launch = op.get("launch", {})
        if len(launch.get("grid", [])) != 3 or len(launch.get("block", [])) != 3 or min(*launch["grid"], *launch["block"]) <= 0:
            raise ValidationError(f"operation {op['name']}: launch dimensions must be three positive integers")
        args = op.get("arguments", [])
        if not args or len(args) > 32:
            raise ValidationError(f"operation {op['name']}: needs 1..32 typed arguments")
        end = 0
        for arg in args:
            size = _ARG_SIZE.get(arg.get("kind"))
            if size is None:
                raise ValidationError(f"operation {op['name']}: unsupported argument kind {arg.get('kind')!r}")
            if arg["offset"] < end:
                raise ValidationError(f"operation {op['name']}: kernel parameter {arg['name']} overlaps its predecessor")
            end = arg["offset"] + size
            if arg.get("source") == "workspace" and not 0 <= arg.get("workspace_offset", -1) < workspace:
                raise ValidationError(f"operation {op['name']}: workspace offset of {arg['name']} is out of range")
            if arg["kind"] == "tensor_map" and arg.get("source") == "null":
                raise ValidationError(f"operation {op['name']}: tensor map {arg['name']} cannot be null")
        if end > op.get("kernarg_size", 0):
            raise ValidationError(f"operation {op['name']}: arguments exceed kernarg_size")
    plan = _load(d / "memory_plan.json")
    for b in plan.get("buffers", []):
        if b["offset"] % plan["workspace_alignment"] or b["offset"] + b["bytes"] > plan["workspace_bytes"]:
            raise ValidationError(f"workspace buffer {b['name']} is misplaced")
    if plan["workspace_bytes"] != workspace:
        raise ValidationError("memory_plan.json and engine.json disagree on workspace_bytes")
    return engine

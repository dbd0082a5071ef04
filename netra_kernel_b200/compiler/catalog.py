"""Fixed CUDA tactic catalog for sm_100a: loads ``manifests/sm_100a/tactics/*.json``, checks the
hashes of the kernel sources each tactic was validated against, and turns a planner request into a
``FixedKernelContract`` or a list of rejection reasons.  Role of the reference's
``compiler/netra_compiler/backends/gfx950/catalog.py:22-576`` (there: assembler templates and
``NETRA_REQUIRE_EQ`` guards; here: CUDA sources, a cubin, and declared constants)."""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .contracts import FixedKernelContract, KernelSemantics, Launch, Workspace
from .expr import evaluate
from .types import TARGET, WARP_SIZE, Maturity, ValidationError, file_sha256

CATALOG_FORMAT = "netra-cuda-tactic-catalog-1"
ARGUMENT_KINDS = ("pointer", "tensor_map", "u32")
_ARG_BYTES = {"pointer": 8, "tensor_map": 128, "u32": 4}


@dataclass(frozen=True)
class TacticArgument:
    name: str
    kind: str
    tensor: str | None = None       # logical tensor (pointer / tensor_map)
    access: str = "read"
    optional: bool = False          # absent tensor -> null pointer
    value: Any = None               # u32: integer expression
    map: Mapping[str, Any] | None = None   # tensor_map: rows / row_bytes / box_rows expressions


@dataclass(frozen=True)
class FixedCudaTactic:
    name: str
    family: str
    operation: str
    rank: int
    maturity: Maturity
    symbol: str
    cubin: str
    constants: tuple[tuple[str, int], ...]
    limits: tuple[tuple[str, int, int], ...]      # inclusive ranges over profile dimensions
    semantics: KernelSemantics
    launch: Mapping[str, Any]
    arguments: tuple[TacticArgument, ...]
    fallback: str
    source_refs: tuple[str, ...]
    evidence_refs: tuple[str, ...]
    source_hashes: tuple[tuple[str, str], ...]

    def rejection_reasons(self, request: Mapping[str, Any], *, allow_experimental: bool = False) -> tuple[str, ...]:
        """Empty tuple = this tactic can serve the request."""
        reasons: list[str] = []
        if request["target"] != TARGET:
            reasons.append("target mismatch")
        if request["family"] != self.family:
            reasons.append("tactic-family mismatch")
        if request["operation"] != self.operation:
            reasons.append("operation mismatch")
        if reasons:
            return tuple(reasons)
        wanted: KernelSemantics = request["semantics"]
        for field_name in self.semantics.differences(wanted):
            reasons.append(f"semantic {field_name} mismatch: {getattr(self.semantics, field_name)} != {getattr(wanted, field_name)}")
        declared = dict(self.constants)
        for key, value in sorted(request["constants"].items()):
            if key not in declared:
                reasons.append(f"undeclared compile-time constant {key}")
            elif declared[key] != value:
                reasons.append(f"{key} mismatch: kernel is fixed to {declared[key]}, request has {value}")
        for key in sorted(set(declared) - set(request["constants"])):
            reasons.append(f"request does not pin constant {key}")
        dims = request["dimensions"]
        for key, lo, hi in self.limits:
            if key not in dims:
                reasons.append(f"profile does not fix dimension {key}")
            elif not lo <= dims[key] <= hi:
                reasons.append(f"{key}={dims[key]} outside the kernel's range [{lo}, {hi}]")
        if self.maturity is Maturity.REJECTED:
            reasons.append("tactic is rejected")
        elif self.maturity is Maturity.EXPERIMENT and not allow_experimental:
            reasons.append("experimental tactic requires --allow-experimental")
        return tuple(reasons)

    def kernarg_size(self) -> int:
        offset = 0
        for arg in self.arguments:
            size = _ARG_BYTES[arg.kind]
            align = 64 if arg.kind == "tensor_map" else size
            offset = (offset + align - 1) // align * align + size
        return (offset + 3) // 4 * 4

    def make_contract(self, request: Mapping[str, Any]) -> FixedKernelContract:
        env = {**dict(self.constants), **request["dimensions"], **request.get("options", {})}
        launch = Launch(tuple(evaluate(v, env) for v in self.launch["grid"]),
                        tuple(evaluate(v, env) for v in self.launch["block"]),
                        evaluate(self.launch.get("lds_bytes", 0), env),
                        evaluate(self.launch.get("dynamic_lds_bytes", 0), env),
                        int(self.launch.get("registers_per_thread", 0)))
        return FixedKernelContract(
            target=TARGET, wave_size=WARP_SIZE, operation=self.operation, family=self.family,
            constants=self.constants, specialization=tuple(sorted(request["dimensions"].items())),
            semantics=self.semantics, kernarg_size=self.kernarg_size(), symbol=self.symbol, launch=launch,
            workspace=Workspace(0, 1024), graph_capture=True, deterministic=True, fallback=self.fallback,
            maturity=self.maturity, source_refs=self.source_refs, evidence_refs=self.evidence_refs)


def _argument(raw: Mapping[str, Any], where: str) -> TacticArgument:
    kind = raw.get("kind")
    if kind not in ARGUMENT_KINDS or not raw.get("name"):
        raise ValidationError(f"{where}: argument needs a name and a kind in {ARGUMENT_KINDS}")
    if kind == "u32":
        if "value" not in raw:
            raise ValidationError(f"{where}: u32 argument {raw['name']} needs a value")
        return TacticArgument(raw["name"], kind, value=raw["value"])
    if not raw.get("tensor"):
        raise ValidationError(f"{where}: argument {raw['name']} needs a tensor")
    if kind == "tensor_map" and not all(k in raw.get("map", {}) for k in ("rows", "row_bytes", "box_rows")):
        raise ValidationError(f"{where}: tensor_map argument {raw['name']} needs rows, row_bytes and box_rows")
    return TacticArgument(raw["name"], kind, tensor=raw["tensor"], access=raw.get("access", "read"),
                          optional=bool(raw.get("optional", False)), map=raw.get("map"))


def load_fixed_tactic_catalog(library_root: Path, target: str = TARGET, *, verify_sources: bool = True
                              ) -> tuple[FixedCudaTactic, ...]:
    folder = library_root / "manifests" / target / "tactics"
    if not folder.is_dir():
        raise ValidationError(f"missing tactic catalog for target {target!r}")
    tactics: list[FixedCudaTactic] = []
    for path in sorted(folder.glob("*.json")):
        doc = json.loads(path.read_text(encoding="utf-8"))
        if doc.get("format") != CATALOG_FORMAT or doc.get("target") != target:
            raise ValidationError(f"{path}: not a {CATALOG_FORMAT} catalog for {target}")
        hashes = []
        for rel, digest in sorted(doc.get("source_sha256", {}).items()):
            source = library_root / "csrc" / rel
            if verify_sources:
                if not source.is_file():
                    raise ValidationError(f"{path}: kernel source {rel} is missing")
                if file_sha256(source) != digest:
                    raise ValidationError(f"{path}: kernel source {rel} changed since the catalog was locked "
                                          f"(run `python -m netra_kernel_b200.compiler.cli lock-catalog`)")
            hashes.append((rel, digest))
        for raw in doc.get("tactics", []):
            where = f"{path.name}:{raw.get('name')}"
            try:
                tactic = FixedCudaTactic(
                    name=raw["name"], family=raw["family"], operation=raw["operation"], rank=int(raw["rank"]),
                    maturity=Maturity(raw["maturity"]), symbol=raw["symbol"], cubin=doc["cubin"],
                    constants=tuple(sorted((str(k), int(v)) for k, v in raw.get("constants", {}).items())),
                    limits=tuple(sorted((str(k), int(v[0]), int(v[1])) for k, v in raw.get("limits", {}).items())),
                    semantics=KernelSemantics(**raw["semantics"]), launch=raw["launch"],
                    arguments=tuple(_argument(a, where) for a in raw["arguments"]),
                    fallback=raw.get("fallback", "framework"), source_refs=tuple(raw.get("source_refs", ())),
                    evidence_refs=tuple(raw.get("evidence_refs", ())), source_hashes=tuple(hashes))
            except (KeyError, TypeError, ValueError) as exc:
                raise ValidationError(f"{where}: malformed tactic entry ({exc})") from exc
            if tactic.rank < 0:
                raise ValidationError(f"{where}: rank must be nonnegative")
            if any(word in tactic.name.lower() for word in ("qwen", "gemma", "llama")):
                raise ValidationError(f"{where}: tactic identity must be model-independent")
            if len(tactic.arguments) > 32:
                raise ValidationError(f"{where}: more than 32 kernel arguments")
            tactics.append(tactic)
    names = [t.name for t in tactics]
    if len(names) != len(set(names)):
        raise ValidationError("duplicate tactic name in catalog")
    return tuple(tactics)


def lock_catalog_sources(library_root: Path, target: str = TARGET) -> None:
    """Rewrites the ``source_sha256`` table of every catalog with the current kernel sources."""
    folder = library_root / "manifests" / target / "tactics"
    for path in sorted(folder.glob("*.json")):
        doc = json.loads(path.read_text(encoding="utf-8"))
        doc["source_sha256"] = {rel: file_sha256(library_root / "csrc" / rel) for rel in sorted(doc.get("source_sha256", {}))}
        path.write_text(json.dumps(doc, indent=1) + "\n", encoding="utf-8")

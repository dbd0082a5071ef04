"""Shape profiles: named sets of exact or bounded dimension guards (tokens ``m``, ``batch``,
``sequence`` ...) plus a quantisation tag and a tensor-parallel degree.  An engine is compiled for
exactly one profile; a launch whose shape falls outside the guards is refused, never approximated.
Same public names as the reference's ``compiler/netra_compiler/profiles.py``."""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Mapping

from .types import ValidationError

PROFILE_FORMAT = "netra-profile-1"


@dataclass(frozen=True)
class DimensionGuard:
    """Closed integer interval [minimum, maximum]; ``exact(v)`` is the one-point interval."""
    minimum: int
    maximum: int

    def __post_init__(self) -> None:
        if not (0 <= self.minimum <= self.maximum):
            raise ValidationError(f"guard [{self.minimum}, {self.maximum}] is not a nonnegative interval")

    @staticmethod
    def exact(value: int) -> "DimensionGuard":
        return DimensionGuard(value, value)

    @property
    def is_exact(self) -> bool:
        return self.minimum == self.maximum

    def matches(self, value: int) -> bool:
        return self.minimum <= value <= self.maximum

    def to_dict(self) -> dict[str, int]:
        return {"min": self.minimum, "max": self.maximum}


@dataclass(frozen=True)
class ShapeProfile:
    name: str
    guards: tuple[tuple[str, DimensionGuard], ...]
    quantization: str = "fp8_block128"
    tensor_parallel: int = 1
    priority: int = 0

    def __post_init__(self) -> None:
        if self.tensor_parallel < 1:
            raise ValidationError("tensor parallel degree must be positive")
        seen: set[str] = set()
        for key, _ in self.guards:
            if key in seen:
                raise ValidationError(f"profile {self.name!r} guards dimension {key!r} twice")
            seen.add(key)

    def guard(self, dimension: str) -> DimensionGuard:
        found = dict(self.guards).get(dimension)
        if found is None:
            raise ValidationError(f"profile {self.name!r} does not guard {dimension!r}")
        return found

    def exact_value(self, dimension: str) -> int:
        g = self.guard(dimension)
        if not g.is_exact:
            raise ValidationError(f"profile {self.name!r} does not fix {dimension!r} to one value")
        return g.minimum

    def matches(self, dimensions: Mapping[str, int], *, quantization: str, tensor_parallel: int) -> bool:
        if quantization != self.quantization or tensor_parallel != self.tensor_parallel:
            return False
        for key, g in self.guards:
            if key not in dimensions or not g.matches(dimensions[key]):
                return False
        return True

    def to_dict(self) -> dict[str, object]:
        return {"name": self.name, "guards": {key: g.to_dict() for key, g in self.guards},
                "quantization": self.quantization, "tensor_parallel": self.tensor_parallel, "priority": self.priority}


@dataclass(frozen=True)
class ProfileSelection:
    supported: bool
    profile: ShapeProfile | None
    reason: str


def select_profile(profiles: Iterable[ShapeProfile], dimensions: Mapping[str, int], *, quantization: str,
                   tensor_parallel: int) -> ProfileSelection:
    """Highest priority first, name as tie-break; the first profile whose every guard holds wins."""
    ranked = sorted(profiles, key=lambda p: (-p.priority, p.name))
    hit = next((p for p in ranked
                if p.matches(dimensions, quantization=quantization, tensor_parallel=tensor_parallel)), None)
    if hit is None:
        return ProfileSelection(False, None, "unsupported contract/profile; framework fallback required")
    return ProfileSelection(True, hit, "all exact/bounded guards matched")


def _profile_from_manifest(path: Path, deployment_tp: int) -> ShapeProfile:
    try:
        doc = json.loads(path.read_text(encoding="utf-8"))
    except (OSError, json.JSONDecodeError) as exc:
        raise ValidationError(f"cannot read profile manifest {path}: {exc}") from exc
    if doc.get("format") != PROFILE_FORMAT:
        raise ValidationError(f"invalid profile format in {path}")
    bounds = doc.get("guards")
    if not isinstance(bounds, Mapping) or not bounds:
        raise ValidationError(f"profile {path} must define nonempty guards")
    guards = []
    for dimension in sorted(bounds):
        entry = bounds[dimension]
        if not isinstance(entry, Mapping) or "min" not in entry or "max" not in entry:
            raise ValidationError(f"invalid bounds for guard {dimension!r} in {path}")
        try:
            guards.append((str(dimension), DimensionGuard(int(entry["min"]), int(entry["max"]))))
        except (TypeError, ValueError) as exc:
            raise ValidationError(f"invalid bounds for guard {dimension!r} in {path}") from exc
    tp = doc.get("tensor_parallel", "deployment")
    if tp == "deployment":          # reusable profile bound to the deployment's own degree
        tp = deployment_tp
    elif isinstance(tp, bool) or not isinstance(tp, int):
        raise ValidationError(f"invalid tensor_parallel constraint in {path}")
    return ShapeProfile(name=str(doc.get("name", "")), guards=tuple(guards),
                        quantization=str(doc.get("quantization", "")), tensor_parallel=tp,
                        priority=int(doc.get("priority", 0)))


def load_profile_registry(library_root: Path, target: str, tensor_parallel: int) -> tuple[ShapeProfile, ...]:
    """Every ``manifests/<target>/profiles/*.json`` as a name-sorted tuple."""
    folder = library_root / "manifests" / target / "profiles"
    if not folder.is_dir():
        raise ValidationError(f"missing profile registry for target {target!r}")
    loaded = [_profile_from_manifest(p, tensor_parallel) for p in sorted(folder.glob("*.json"))]
    if not loaded:
        raise ValidationError(f"profile registry for target {target!r} is empty")
    by_name: dict[str, ShapeProfile] = {}
    for profile in loaded:
        if profile.name in by_name:
            raise ValidationError(f"duplicate profile name in target {target!r}")
        by_name[profile.name] = profile
    return tuple(by_name[name] for name in sorted(by_name))

"""Immutable kernel contracts with content-derived ids (``nk_`` + 24 hex digits of the sha256 of the
identity).  Public names and the identity's field set follow the reference's
``compiler/netra_compiler/contracts.py`` (``Launch`` :13, ``Workspace`` :34, ``KernelSemantics`` :55,
``FixedKernelContract`` :93, ``FallbackKernelContract`` :287); the target here is sm_100a / warp 32."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .types import TARGET, WARP_SIZE, Maturity, ValidationError, stable_hash

MAX_BLOCK_SMEM = 232448            # static + dynamic shared memory one B200 block may use
_SEMANTIC_FIELDS = ("abi", "dtypes", "quantization", "layouts", "numerical")
_MODEL_WORDS = ("qwen", "gemma", "llama")


def _contract_id(identity: dict[str, Any]) -> str:
    return "nk_" + stable_hash(identity)[:24]


def _triple(values, what: str) -> tuple[int, int, int]:
    values = tuple(int(v) for v in values)
    if len(values) != 3:
        raise ValidationError(f"launch {what} must have three dimensions")
    if min(values) <= 0:
        raise ValidationError("launch dimensions must be positive")
    return values  # type: ignore[return-value]


@dataclass(frozen=True)
class Launch:
    """Fixed launch shape.  ``lds_bytes`` is the code object's static shared memory and
    ``dynamic_lds_bytes`` the amount passed at launch (the reference's two LDS fields)."""
    grid: tuple[int, int, int]
    block: tuple[int, int, int]
    lds_bytes: int = 0
    dynamic_lds_bytes: int = 0
    registers_per_thread: int = 0      # nonzero: the loaded code object must report exactly this allocation

    def __post_init__(self) -> None:
        object.__setattr__(self, "grid", _triple(self.grid, "grid"))
        object.__setattr__(self, "block", _triple(self.block, "block"))
        threads = self.block[0] * self.block[1] * self.block[2]
        if threads > 1024:
            raise ValidationError("threads per block exceeds 1024")
        if min(self.lds_bytes, self.dynamic_lds_bytes) < 0:
            raise ValidationError("shared-memory bytes must be nonnegative")
        if not 0 <= self.registers_per_thread <= 255:
            raise ValidationError("registers per thread must be 0 (unchecked) or 1..255")
        if self.lds_bytes + self.dynamic_lds_bytes > MAX_BLOCK_SMEM:
            raise ValidationError("shared memory exceeds what one B200 block can use")

    def to_dict(self) -> dict[str, Any]:
        doc = {"grid": list(self.grid), "block": list(self.block), "lds_bytes": self.lds_bytes,
               "dynamic_lds_bytes": self.dynamic_lds_bytes}
        if self.registers_per_thread:      # kernels that re-balance registers between warpgroups (setmaxnreg)
            doc["registers_per_thread"] = self.registers_per_thread
        return doc


@dataclass(frozen=True)
class Workspace:
    bytes: int = 0
    alignment: int = 256

    def __post_init__(self) -> None:
        if not (0 <= self.bytes < 1 << 64):
            raise ValidationError("workspace byte count is outside uint64")
        if self.alignment < 1 or self.alignment & (self.alignment - 1):
            raise ValidationError("workspace alignment must be a power of two")

    def to_dict(self) -> dict[str, int]:
        return {"bytes": self.bytes, "alignment": self.alignment}


@dataclass(frozen=True)
class KernelSemantics:
    """Versioned, model-independent meaning of a kernel's argument list.  Two kernels with equal
    dimensions are interchangeable only if all five identifiers agree."""
    abi: str
    dtypes: str
    quantization: str
    layouts: str
    numerical: str

    def __post_init__(self) -> None:
        for name in _SEMANTIC_FIELDS:
            text = getattr(self, name)
            if not text or text.split() != [text]:
                raise ValidationError(f"kernel semantic identifier {name} must be nonempty and whitespace-free")
            if any(word in text.lower() for word in _MODEL_WORDS):
                raise ValidationError(f"kernel semantic identifier {name} must be model-independent")

    def to_dict(self) -> dict[str, str]:
        return {name: getattr(self, name) for name in _SEMANTIC_FIELDS}

    def differences(self, other: "KernelSemantics") -> list[str]:
        return [name for name in _SEMANTIC_FIELDS if getattr(self, name) != getattr(other, name)]


@dataclass(frozen=True)
class FixedKernelContract:
    """One completely specialised kernel launch.  ``constants`` are invariants of the kernel,
    ``specialization`` the concrete values chosen for this engine (token rows, segment counts ...).
    The symbol name is deliberately not part of the identity."""
    target: str
    wave_size: int
    operation: str
    family: str
    constants: tuple[tuple[str, int], ...]
    specialization: tuple[tuple[str, int], ...]
    semantics: KernelSemantics
    kernarg_size: int
    symbol: str
    launch: Launch
    workspace: Workspace = field(default_factory=Workspace)
    graph_capture: bool = True
    deterministic: bool = True
    fallback: str = "framework"
    maturity: Maturity = Maturity.EXPERIMENT
    source_refs: tuple[str, ...] = ()
    evidence_refs: tuple[str, ...] = ()

    def __post_init__(self) -> None:
        if (self.target, self.wave_size) != (TARGET, WARP_SIZE):
            raise ValidationError("fixed contracts of this compiler require sm_100a / warp 32")
        if not (self.operation and self.family and self.symbol):
            raise ValidationError("fixed kernel operation, family, and symbol are required")
        if self.kernarg_size <= 0 or self.kernarg_size % 4:
            raise ValidationError("fixed kernel parameter size must be positive and dword aligned")
        pairs = (*self.constants, *self.specialization)
        if len({name for name, _ in pairs}) != len(pairs):
            raise ValidationError("duplicate fixed kernel compile-time constant")
        for name, value in pairs:
            if not name or value < 0:
                raise ValidationError("fixed kernel constants require names and nonnegative integers")

    def identity_dict(self) -> dict[str, Any]:
        return {
            "target": self.target, "wave_size": self.wave_size, "operation": self.operation, "family": self.family,
            "constants": dict(self.constants), "specialization": dict(self.specialization),
            "semantics": self.semantics.to_dict(), "kernarg_size": self.kernarg_size,
            "launch": self.launch.to_dict(), "workspace": self.workspace.to_dict(),
            "graph_capture": self.graph_capture, "deterministic": self.deterministic,
        }

    @property
    def stable_id(self) -> str:
        return _contract_id(self.identity_dict())

    def to_dict(self) -> dict[str, Any]:
        return {**self.identity_dict(), "id": self.stable_id, "symbol": self.symbol, "fallback": self.fallback,
                "maturity": self.maturity.value, "artifact_kind": "cuda_cubin_kernel",
                "source_refs": list(self.source_refs), "evidence_refs": list(self.evidence_refs)}


@dataclass(frozen=True)
class FallbackKernelContract:
    """An operation that stays with the framework: no tactic covers it."""
    target: str
    operation: str
    family: str
    fallback: str
    reason: str

    def identity_dict(self) -> dict[str, Any]:
        return {"kind": "fallback", "target": self.target, "operation": self.operation, "family": self.family,
                "fallback": self.fallback}

    @property
    def stable_id(self) -> str:
        return _contract_id(self.identity_dict())

    def to_dict(self) -> dict[str, Any]:
        return {**self.identity_dict(), "id": self.stable_id, "reason": self.reason,
                "artifact_kind": "framework_external"}

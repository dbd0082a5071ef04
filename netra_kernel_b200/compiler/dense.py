"""The dense FP8 block-scale GEMM contract and its tactic registry (role of the reference's ``KernelContract``,
``compiler/netra_compiler/contracts.py:175-284``, and ``gfx950_registry``, ``compiler/netra_compiler/tactics.py:207-220``).
As in the reference, the only registered tactic for the dense projection (M x 2048 x 4096, FP8 x FP8 -> BF16, identity
epilogue) is the framework's own kernel: the contract exists so that a model graph can name the operation, the planner
can explain why no fixed kernel serves it, and the engine records the fallback it requires."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Iterable

from .contracts import FallbackKernelContract, Launch, Workspace
from .types import TARGET, WARP_SIZE, Maturity, ValidationError, stable_hash


@dataclass(frozen=True)
class NumericalContract:
    accumulation_dtype: str = "fp32"
    output_rounding: str = "rne"
    reduction_order: str = "kblock_ascending"
    nan_behavior: str = "propagate"
    deterministic: bool = True


@dataclass(frozen=True)
class KernelContract:
    """One dense block-scaled GEMM: ``out[m, n] = sum_kb a_s[m, kb] * w_s[n/128, kb] * sum_k A[m, k] W[n, k]``."""
    target: str
    wave_size: int
    operation: str
    m: int
    n: int
    k: int
    input_dtype: str
    weight_dtype: str
    accumulator_dtype: str
    output_dtype: str
    activation_quantization: str
    weight_quantization: str
    activation_scale_block: int
    weight_scale_block: tuple[int, int]
    activation_layout: str
    weight_layout: str
    output_layout: str
    epilogue: str
    tactic: str
    launch: Launch
    workspace: Workspace = field(default_factory=lambda: Workspace(0, 1024))
    graph_capture: bool = True
    deterministic: bool = True
    numerical: NumericalContract = field(default_factory=NumericalContract)
    fallback: str = "framework"
    maturity: Maturity = Maturity.EXPERIMENT
    source_refs: tuple[str, ...] = ()
    evidence_refs: tuple[str, ...] = ()

    def __post_init__(self) -> None:
        if self.target != TARGET or self.wave_size != WARP_SIZE:
            raise ValidationError(f"dense contracts are for {TARGET} with {WARP_SIZE}-wide warps")
        if self.operation != "dense":
            raise ValidationError(f"unsupported operation: {self.operation}")
        if min(self.m, self.n, self.k) <= 0:
            raise ValidationError("M, N and K must be positive")
        if self.activation_scale_block <= 0 or min(self.weight_scale_block) <= 0:
            raise ValidationError("scale blocks must be positive")
        if self.k % self.activation_scale_block:
            raise ValidationError("K must be divisible by the activation scale block")
        if self.n % self.weight_scale_block[0] or self.k % self.weight_scale_block[1]:
            raise ValidationError("N and K must be divisible by the weight scale block")
        if self.accumulator_dtype != "fp32":
            raise ValidationError("the dense slice accumulates in FP32")
        if self.deterministic and not self.numerical.deterministic:
            raise ValidationError("a deterministic contract cannot carry nondeterministic numerical rules")

    def identity_dict(self) -> dict[str, Any]:
        """The computation only: no model name, evidence or build path enters the id."""
        return {
            "target": self.target, "wave_size": self.wave_size, "operation": self.operation, "shape": [self.m, self.n, self.k],
            "dtypes": [self.input_dtype, self.weight_dtype, self.accumulator_dtype, self.output_dtype],
            "quantization": {"activation": self.activation_quantization, "weight": self.weight_quantization,
                             "activation_scale_block": self.activation_scale_block, "weight_scale_block": list(self.weight_scale_block)},
            "layouts": [self.activation_layout, self.weight_layout, self.output_layout], "epilogue": self.epilogue, "tactic": self.tactic,
            "launch": {"grid": list(self.launch.grid), "block": list(self.launch.block), "lds_bytes": self.launch.lds_bytes,
                       "dynamic_lds_bytes": self.launch.dynamic_lds_bytes},
            "workspace": {"bytes": self.workspace.bytes, "alignment": self.workspace.alignment},
            "graph_capture": self.graph_capture, "deterministic": self.deterministic,
            "numerical": {"accumulation_dtype": self.numerical.accumulation_dtype, "output_rounding": self.numerical.output_rounding,
                          "reduction_order": self.numerical.reduction_order, "nan_behavior": self.numerical.nan_behavior,
                          "deterministic": self.numerical.deterministic},
        }

    @property
    def stable_id(self) -> str:
        return "nk_" + stable_hash(self.identity_dict())[:24]

    def to_dict(self) -> dict[str, Any]:
        doc = self.identity_dict()
        doc.update({"id": self.stable_id, "fallback": self.fallback, "maturity": self.maturity.value,
                    "source_refs": list(self.source_refs), "evidence_refs": list(self.evidence_refs)})
        return doc


@dataclass(frozen=True)
class DensePredicate:
    """What a dense tactic accepts: allowed M / N / K values, dtypes, scale blocks, layouts and epilogues."""
    m: tuple[int, ...]
    n: tuple[int, ...]
    k: tuple[int, ...]
    input_dtype: str
    weight_dtype: str
    output_dtype: str
    activation_scale_block: int
    weight_scale_block: tuple[int, int]
    activation_layout: str
    weight_layout: str
    output_layout: str
    epilogues: tuple[str, ...]

    def rejection_reasons(self, request: dict[str, Any]) -> list[str]:
        reasons = []
        for key, allowed in (("m", self.m), ("n", self.n), ("k", self.k)):
            if request[key] not in allowed:
                reasons.append(f"{key.upper()}={request[key]} is not one of {list(allowed)}")
        for key in ("input_dtype", "weight_dtype", "output_dtype", "activation_scale_block", "activation_layout", "weight_layout",
                    "output_layout"):
            if request[key] != getattr(self, key):
                reasons.append(f"{key} mismatch: tactic has {getattr(self, key)}, request has {request[key]}")
        if tuple(request["weight_scale_block"]) != tuple(self.weight_scale_block):
            reasons.append("weight_scale_block mismatch")
        if request["epilogue"] not in self.epilogues:
            reasons.append(f"epilogue {request['epilogue']} is not supported")
        return reasons


@dataclass(frozen=True)
class DenseTactic:
    name: str
    predicate: DensePredicate
    maturity: Maturity
    artifact_kind: str          # "framework_external": the serving framework's own kernel runs the operation
    rank: int
    evidence_refs: tuple[str, ...] = ()


def sm100a_dense_registry() -> tuple[DenseTactic, ...]:
    predicate = DensePredicate((1,), (2048,), (4096,), "fp8_e4m3", "fp8_e4m3", "bf16", 128, (128, 128), "row_major_fp8_block128",
                               "row_major_fp8_block128", "row_major_bf16", ("identity",))
    return (DenseTactic("sm100a.framework_blockscale_dense_m1.compat", predicate, Maturity.ACCEPTED, "framework_external", 1000,
                        ("the framework's block-scaled FP8 linear; no fixed sm_100a kernel is registered for the dense projection",)),)


def dense_request(m: int, n: int, k: int, *, epilogue: str = "identity", weight_layout: str = "row_major_fp8_block128") -> dict[str, Any]:
    return {"target": TARGET, "operation": "dense", "m": m, "n": n, "k": k, "input_dtype": "fp8_e4m3", "weight_dtype": "fp8_e4m3",
            "output_dtype": "bf16", "activation_scale_block": 128, "weight_scale_block": (128, 128),
            "activation_layout": "row_major_fp8_block128", "weight_layout": weight_layout, "output_layout": "row_major_bf16",
            "epilogue": epilogue}


def plan_dense(request: dict[str, Any], tactics: Iterable[DenseTactic] | None = None):
    """(contract, explanation): every registered tactic with its rejection reasons; the best accepted one decides.  A
    ``framework_external`` tactic (and no tactic at all) yields a ``FallbackKernelContract``."""
    tactics = tuple(tactics if tactics is not None else sm100a_dense_registry())
    accepted, explanation = [], []
    for t in sorted(tactics, key=lambda t: t.name):
        reasons = t.predicate.rejection_reasons(request)
        if t.maturity is Maturity.REJECTED:
            reasons.append("tactic is rejected")
        explanation.append({"tactic": t.name, "reasons": reasons})
        if not reasons:
            accepted.append(t)
    accepted.sort(key=lambda t: (-t.rank, t.name))
    if accepted and accepted[0].artifact_kind == "framework_external":
        why = f"the accepted tactic {accepted[0].name} is the framework's own kernel"
    elif not accepted:
        why = "no registered tactic accepts this dense request"
    else:
        raise ValidationError("fixed dense kernels are not registered for sm_100a")
    contract = FallbackKernelContract(TARGET, "dense", "dense_fp8_blockscale", "framework.fp8_blockscale_linear", why)
    for entry in explanation:
        entry["selected"] = bool(accepted) and entry["tactic"] == accepted[0].name
    return contract, explanation

"""Per-operation tactic selection with recorded reasons.  For every ``fixed_kernel`` operation:
filter the catalog by family / operation / semantics / constants / dimension limits / maturity,
rank the survivors (lower rank wins), refuse equal-rank ambiguity, otherwise fall back.  Role of
the reference's ``compiler/netra_compiler/planner.py:139-266``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .catalog import FixedCudaTactic
from .contracts import FallbackKernelContract, FixedKernelContract, KernelSemantics
from .ir import Graph, Operation
from .profiles import ShapeProfile
from .types import ValidationError


@dataclass(frozen=True)
class PlannedOperation:
    operation: Operation
    contract: FixedKernelContract | FallbackKernelContract
    tactic: FixedCudaTactic | None
    execution: str                       # "kernel" | "fallback"
    fallback: str
    explanation: tuple[dict[str, Any], ...]


@dataclass(frozen=True)
class Plan:
    graph: Graph
    profile: ShapeProfile
    operations: tuple[PlannedOperation, ...]

    @property
    def requires_fallback(self) -> bool:
        return any(p.execution != "kernel" for p in self.operations)


def fixed_request(op: Operation, target: str, dimensions: Mapping[str, int], options: Mapping[str, int]) -> dict[str, Any]:
    sem = op.attributes.get("semantics")
    if not isinstance(sem, Mapping):
        raise ValidationError(f"operation {op.name!r} does not state its kernel semantics")
    return {"target": target, "family": op.family, "operation": op.operation, "semantics": KernelSemantics(**sem),
            "constants": dict(op.attributes.get("constants", {})), "dimensions": dict(dimensions),
            "options": dict(options), "fallback": str(op.attributes.get("fallback", "framework"))}


def plan_graph(graph: Graph, profile: ShapeProfile, target: str, tactics: tuple[FixedCudaTactic, ...],
               dimensions: Mapping[str, int], options: Mapping[str, int], *, allow_experimental: bool = False) -> Plan:
    planned = []
    for op in graph.operations:
        if op.kind != "fixed_kernel":
            fb = str(op.attributes.get("fallback", "framework"))
            planned.append(PlannedOperation(op, FallbackKernelContract(target, op.operation, op.family, fb,
                                                                        "operation kind is outside this compiler"),
                                            None, "fallback", fb,
                                            ({"tactic": None, "selected": False, "reasons": ["operation kind is outside this compiler"]},)))
            continue
        request = fixed_request(op, target, dimensions, options)
        accepted, refused = [], []
        for tactic in tactics:
            reasons = tactic.rejection_reasons(request, allow_experimental=allow_experimental)
            (refused if reasons else accepted).append((tactic, reasons))
        accepted.sort(key=lambda item: (item[0].rank, item[0].name))
        refused.sort(key=lambda item: item[0].name)
        explanation = [{"tactic": t.name, "selected": i == 0, "reasons": []} for i, (t, _) in enumerate(accepted)]
        explanation += [{"tactic": t.name, "selected": False, "reasons": list(r)} for t, r in refused]
        if not accepted:
            planned.append(PlannedOperation(op, FallbackKernelContract(target, op.operation, op.family, request["fallback"],
                                                                        "no tactic accepts this request"),
                                            None, "fallback", request["fallback"], tuple(explanation)))
            continue
        if len(accepted) > 1 and accepted[0][0].rank == accepted[1][0].rank:
            tied = ", ".join(t.name for t, _ in accepted if t.rank == accepted[0][0].rank)
            raise ValidationError(f"ambiguous fixed tactics at rank {accepted[0][0].rank} for {op.name}: {tied}")
        best = accepted[0][0]
        contract = best.make_contract(request)
        planned.append(PlannedOperation(op, contract, best, "kernel", contract.fallback, tuple(explanation)))
    return Plan(graph, profile, tuple(planned))

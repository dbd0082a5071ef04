"""Typed tensor / operation graph handed from the frontend to the planner (thin counterpart of the
reference's ``compiler/netra_compiler/ir.py:28-249``)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .types import ValidationError

ROLES = ("input", "output", "weight", "workspace")


@dataclass(frozen=True)
class Tensor:
    name: str
    dtype: str
    shape: tuple[int, ...]
    role: str
    bytes: int
    alignment: int = 1024

    def __post_init__(self) -> None:
        if self.role not in ROLES:
            raise ValidationError(f"tensor {self.name!r} has unknown role {self.role!r}")
        if self.bytes <= 0 or any(d <= 0 for d in self.shape):
            raise ValidationError(f"tensor {self.name!r} must have positive extent")
        if self.alignment <= 0 or self.alignment & (self.alignment - 1):
            raise ValidationError(f"tensor {self.name!r} alignment must be a power of two")

    def to_dict(self) -> dict[str, Any]:
        return {"name": self.name, "dtype": self.dtype, "shape": list(self.shape), "role": self.role,
                "bytes": self.bytes, "alignment": self.alignment}


@dataclass(frozen=True)
class Operation:
    name: str
    kind: str                      # "fixed_kernel" | "fallback"
    family: str
    operation: str
    inputs: tuple[str, ...]
    outputs: tuple[str, ...]
    attributes: dict[str, Any] = field(default_factory=dict)

    def to_dict(self) -> dict[str, Any]:
        return {"name": self.name, "kind": self.kind, "family": self.family, "operation": self.operation,
                "inputs": list(self.inputs), "outputs": list(self.outputs), "attributes": dict(self.attributes)}


@dataclass(frozen=True)
class Graph:
    name: str
    tensors: tuple[Tensor, ...]
    operations: tuple[Operation, ...]

    def __post_init__(self) -> None:
        names = [t.name for t in self.tensors]
        if len(names) != len(set(names)):
            raise ValidationError("duplicate tensor name in graph")
        known = set(names)
        produced = {t.name for t in self.tensors if t.role in ("input", "weight")}
        op_names = set()
        for op in self.operations:
            if op.name in op_names:
                raise ValidationError(f"duplicate operation name {op.name!r}")
            op_names.add(op.name)
            for t in (*op.inputs, *op.outputs):
                if t not in known:
                    raise ValidationError(f"operation {op.name!r} references unknown tensor {t!r}")
            for t in op.inputs:
                if t not in produced:
                    raise ValidationError(f"operation {op.name!r} reads {t!r} before any producer")
            produced.update(op.outputs)
        for t in self.tensors:
            if t.role == "output" and t.name not in produced:
                raise ValidationError(f"graph output {t.name!r} is never written")

    def tensor(self, name: str) -> Tensor:
        for t in self.tensors:
            if t.name == name:
                return t
        raise ValidationError(f"unknown tensor {name!r}")

    def to_dict(self) -> dict[str, Any]:
        return {"format": "netra-graph-1", "name": self.name, "tensors": [t.to_dict() for t in self.tensors],
                "operations": [o.to_dict() for o in self.operations]}

"""Locates the kernel library root: the folder holding ``manifests/`` and ``csrc/`` (role of the
reference's ``compiler/netra_compiler/library.py:20-74``)."""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

from .types import ValidationError


@dataclass(frozen=True)
class KernelLibrary:
    root: Path

    @classmethod
    def discover(cls, root: Path | str | None = None) -> "KernelLibrary":
        base = Path(root) if root is not None else Path(__file__).resolve().parents[1]
        if not (base / "manifests").is_dir():
            raise ValidationError(f"{base} is not a kernel library root (no manifests/ folder)")
        return cls(base.resolve())

    @property
    def csrc(self) -> Path:
        return self.root / "csrc"

    def manifest_dir(self, target: str, kind: str) -> Path:
        return self.root / "manifests" / target / kind

"""Canonical JSON and content hashes for the compiler's artefacts, plus its small shared vocabulary.

The serialisation rules are the reference's (``compiler/netra_compiler/types.py:36-61``) because contract and
engine ids are hashes of it and have to be comparable: keys sorted, no insignificant spaces, UTF-8 text, one
trailing newline; enums by value, paths in POSIX form, dataclasses as mappings of their fields, tuples as lists.
``tests/golden/compiler_hash_kat.json`` pins the resulting ids against the reference compiler's own output.
"""
from __future__ import annotations

import dataclasses
import enum
import hashlib
import json
from collections.abc import Mapping
from functools import singledispatch
from pathlib import Path, PurePath
from typing import Any

TARGET = "sm_100a"
WARP_SIZE = 32


class NetraCompilerError(Exception):
    """Base class of actionable compiler errors."""


class ValidationError(NetraCompilerError):
    """An input (manifest, catalog, graph, engine directory) breaks a rule the compiler checks."""


class UnsupportedContract(NetraCompilerError):
    """No tactic and no fallback can serve a requested operation."""


class Maturity(str, enum.Enum):
    """Life-cycle state of a catalog tactic; the planner only ever selects the middle two."""
    EXPERIMENT = "experiment"
    VERIFIED = "verified"
    ACCEPTED = "accepted"
    REJECTED = "rejected"


# ---- reduction of arbitrary compiler values to JSON-ready data, one rule per type -------------------
@singledispatch
def _jsonable(value: Any) -> Any:
    if dataclasses.is_dataclass(value) and not isinstance(value, type):
        return {f.name: _jsonable(getattr(value, f.name)) for f in dataclasses.fields(value)}
    return value


@_jsonable.register
def _(value: enum.Enum) -> Any:
    return value.value


@_jsonable.register
def _(value: PurePath) -> str:
    return value.as_posix()


@_jsonable.register
def _(value: Mapping) -> dict:
    return {str(key): _jsonable(item) for key, item in value.items()}


@_jsonable.register(list)
@_jsonable.register(tuple)
def _(value) -> list:
    return [_jsonable(item) for item in value]


def canonical_json(value: Any) -> str:
    """Byte-stable text of ``value`` across runs and machines."""
    text = json.dumps(_jsonable(value), ensure_ascii=False, sort_keys=True, separators=(",", ":"))
    return text + "\n"


def _sha256_hex(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


def stable_hash(value: Any) -> str:
    """sha256 of the canonical text."""
    return _sha256_hex(canonical_json(value).encode("utf-8"))


def file_sha256(path: Path) -> str:
    return _sha256_hex(Path(path).read_bytes())


def write_json(path: Path, value: Any) -> None:
    """Writes the canonical text, creating parent directories."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(canonical_json(value), encoding="utf-8")

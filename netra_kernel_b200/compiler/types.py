"""Canonical JSON and stable hashing (same definitions as the reference's
``compiler/netra_compiler/types.py:36-61`` so that contract ids are comparable), enums, errors."""
from __future__ import annotations

import hashlib
import json
from collections.abc import Mapping
from dataclasses import asdict, is_dataclass
from enum import Enum
from pathlib import Path
from typing import Any

TARGET = "sm_100a"
WARP_SIZE = 32


class Maturity(str, Enum):
    EXPERIMENT = "experiment"
    VERIFIED = "verified"
    ACCEPTED = "accepted"
    REJECTED = "rejected"


class NetraCompilerError(Exception):
    """Base class of actionable compiler errors."""


class ValidationError(NetraCompilerError):
    pass


class UnsupportedContract(NetraCompilerError):
    pass


def _plain(value: Any) -> Any:
    if isinstance(value, Enum):
        return value.value
    if isinstance(value, Path):
        return value.as_posix()
    if is_dataclass(value):
        return {k: _plain(v) for k, v in asdict(value).items()}
    if isinstance(value, Mapping):
        return {str(k): _plain(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [_plain(v) for v in value]
    return value


def canonical_json(value: Any) -> str:
    """Sorted keys, no spaces, UTF-8, trailing newline: byte-stable across runs and machines."""
    return json.dumps(_plain(value), sort_keys=True, separators=(",", ":"), ensure_ascii=False) + "\n"


def stable_hash(value: Any) -> str:
    return hashlib.sha256(canonical_json(value).encode("utf-8")).hexdigest()


def write_json(path: Path, value: Any) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(canonical_json(value), encoding="utf-8")


def file_sha256(path: Path) -> str:
    return hashlib.sha256(path.read_bytes()).hexdigest()

"""Static workspace plan: every workspace tensor gets a fixed offset in one buffer; tensors whose
lifetimes (first writer .. last reader, in operation order) do not overlap may share bytes.
First-fit over lifetime intervals, as in the reference's ``compiler/netra_compiler/memory.py:56-112``."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable

from .types import ValidationError

_U64_MAX = (1 << 64) - 1


def checked_mul(a: int, b: int) -> int:
    if a < 0 or b < 0:
        raise ValidationError("sizes must be nonnegative")
    if a and b > _U64_MAX // a:
        raise ValidationError("size overflows uint64")
    return a * b


def align_up(value: int, alignment: int) -> int:
    if alignment <= 0 or alignment & (alignment - 1):
        raise ValidationError("alignment must be a power of two")
    out = (value + alignment - 1) & ~(alignment - 1)
    if out > _U64_MAX:
        raise ValidationError("aligned size overflows uint64")
    return out


@dataclass(frozen=True)
class BufferRequest:
    name: str
    bytes: int
    alignment: int
    first_use: int      # operation index of the first access
    last_use: int       # operation index of the last access
    pinned: bool = False  # never shares bytes (read back by the caller after the launch)


@dataclass(frozen=True)
class PlacedBuffer:
    name: str
    offset: int
    bytes: int
    first_use: int
    last_use: int

    def to_dict(self) -> dict[str, int | str]:
        return {"name": self.name, "offset": self.offset, "bytes": self.bytes, "first_use": self.first_use,
                "last_use": self.last_use}


def plan_buffers(requests: Iterable[BufferRequest], alignment: int = 1024) -> tuple[tuple[PlacedBuffer, ...], int]:
    """Returns (placements in request order, total bytes).  Deterministic: requests are placed in
    the order (first_use, name) at the lowest aligned offset free over their whole lifetime."""
    requests = list(requests)
    if len({r.name for r in requests}) != len(requests):
        raise ValidationError("duplicate workspace buffer name")
    done: list[tuple[BufferRequest, PlacedBuffer]] = []
    total = 0
    for r in sorted(requests, key=lambda r: (r.first_use, r.name)):
        if r.bytes <= 0 or r.first_use < 0 or r.last_use < r.first_use:
            raise ValidationError(f"invalid workspace request {r.name!r}")
        step = max(alignment, r.alignment)
        live = sorted((p.offset, p.offset + p.bytes) for q, p in done
                      if q.pinned or r.pinned or not (q.last_use < r.first_use or r.last_use < q.first_use))
        offset = 0
        for lo, hi in live:
            if offset + r.bytes <= lo:
                break
            offset = max(offset, align_up(hi, step))
        done.append((r, PlacedBuffer(r.name, offset, r.bytes, r.first_use, r.last_use)))
        total = max(total, offset + r.bytes)
    by_name = {q.name: p for q, p in done}
    return tuple(by_name[r.name] for r in requests), align_up(total, alignment)

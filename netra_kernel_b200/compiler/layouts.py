"""Declarative weight- and scale-layout plans: which steps turn a checkpoint's tensors into the layout a
kernel streams, recorded in ``layout_plan.json`` and executed once at load.  Role of the reference's
``compiler/netra_compiler/layouts.py:109-206`` (there: AITER's 16x16 shuffle; here: the 128x128-byte tile order the
TMA boxes of the grouped GEMMs read as contiguous 16 KiB blocks).  The byte transforms below are the CPU statement
of each step; the GPU entry points (``netra_moe_repack_tiles_launch``, ``netra_moe_widen_scales_bf16_launch``) are
checked against them byte for byte."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import numpy as np

from .types import ValidationError

ROW_MAJOR = "checkpoint_row_major_fp8_block128"
SPLIT_GATE_UP = "checkpoint_split_gate_up_row_major_fp8_block128"     # gate_proj and up_proj as two tensors
TILES128 = "tiles128x128_fp8_block128"
MXFP4_ROW_MAJOR = "checkpoint_row_major_mxfp4_block32"               # e2m1 codes [n, k/2] + ue8m0 scales [n, k/32]
MXFP4_PAIRED_BLOCKS = "paired_blocks128x64B_mxfp4_block32"           # 8 KiB code blocks + 512-byte scale atoms, tile pairs adjacent
TILE = 128


@dataclass(frozen=True)
class RepackStep:
    source_layout: str
    target_layout: str
    operation: str                       # "concatenate_output_shards" | "tile_128x128"
    parameters: tuple[tuple[str, Any], ...] = ()
    entry_point: str | None = None       # the C-ABI call that performs the step on the device (None: host concatenation)

    def to_dict(self) -> dict[str, Any]:
        doc = {"from": self.source_layout, "to": self.target_layout, "operation": self.operation,
               "parameters": {k: v for k, v in self.parameters}}
        if self.entry_point:
            doc["entry_point"] = self.entry_point
        return doc


@dataclass(frozen=True)
class LayoutBinding:
    tensor: str
    checkpoint_layout: str
    kernel_layout: str
    steps: tuple[RepackStep, ...]
    checkpoint_tensors: tuple[str, ...] = ()

    def to_dict(self) -> dict[str, Any]:
        return {"tensor": self.tensor, "checkpoint_layout": self.checkpoint_layout, "kernel_layout": self.kernel_layout,
                "checkpoint_tensors": list(self.checkpoint_tensors), "steps": [s.to_dict() for s in self.steps]}


@dataclass(frozen=True)
class ScaleBinding:
    tensor: str
    checkpoint_tensors: tuple[str, ...]
    checkpoint_dtype: str
    kernel_dtype: str
    block: tuple[int, int]
    steps: tuple[str, ...]

    def to_dict(self) -> dict[str, Any]:
        return {"tensor": self.tensor, "checkpoint_tensors": list(self.checkpoint_tensors), "checkpoint_dtype": self.checkpoint_dtype,
                "kernel_dtype": self.kernel_dtype, "block": list(self.block), "steps": list(self.steps)}


_TILE_STEP = RepackStep(ROW_MAJOR, TILES128, "tile_128x128", (("tile_rows", TILE), ("tile_bytes", TILE)),
                        "netra_moe_repack_tiles_launch")


def _mxfp4_pack_step(paired_half_rows: int) -> RepackStep:
    return RepackStep(MXFP4_ROW_MAJOR, MXFP4_PAIRED_BLOCKS, "mxfp4_pair_blocks",
                      (("block_rows", TILE), ("block_k", TILE), ("paired_half_rows", paired_half_rows), ("scale_atom_bytes", 512)),
                      "netra_moe_mxfp4_pack_launch")


def plan_weight_layout(tensor: str, checkpoint_layout: str, kernel_layout: str, *,
                       checkpoint_tensors: tuple[str, ...] = ()) -> LayoutBinding:
    """One explicit chain of steps from the checkpoint's layout to the kernel's; unknown pairs are refused."""
    if checkpoint_layout == kernel_layout:
        return LayoutBinding(tensor, checkpoint_layout, kernel_layout, (), checkpoint_tensors)
    steps: list[RepackStep] = []
    current = checkpoint_layout
    if current == SPLIT_GATE_UP:
        if len(checkpoint_tensors) != 2:
            raise ValidationError("the split gate/up checkpoint layout names exactly two source tensors (gate, up)")
        steps.append(RepackStep(SPLIT_GATE_UP, ROW_MAJOR, "concatenate_output_shards", (("axis", 0), ("shards", 2))))
        current = ROW_MAJOR
    if current == ROW_MAJOR and kernel_layout == TILES128:
        steps.append(_TILE_STEP)
        current = TILES128
    if current == MXFP4_ROW_MAJOR and kernel_layout == MXFP4_PAIRED_BLOCKS:
        steps.append(_mxfp4_pack_step(512 if tensor == "w13" else TILE))
        current = MXFP4_PAIRED_BLOCKS
    if current != kernel_layout:
        raise ValidationError(f"unsupported weight layout transform: {checkpoint_layout} -> {kernel_layout}")
    return LayoutBinding(tensor, checkpoint_layout, kernel_layout, tuple(steps), checkpoint_tensors)


def plan_scale_layout(tensor: str, checkpoint_tensors: tuple[str, ...], *, checkpoint_dtype: str, kernel_dtype: str,
                      block: tuple[int, int]) -> ScaleBinding:
    """Scales keep their logical [N/128, K/128] order; shards are concatenated along N and BF16 scales widened (exactly)."""
    if not checkpoint_tensors:
        raise ValidationError("a scale layout needs its checkpoint source tensors")
    if len(block) != 2 or min(block) <= 0:
        raise ValidationError("a scale layout needs a positive two-dimensional block")
    if checkpoint_dtype == kernel_dtype == "ue8m0":
        # MXFP4: one byte per 32 weights along K; the pack step of the weight tensor re-orders the bytes into 512-byte atoms
        return ScaleBinding(tensor, tuple(checkpoint_tensors), "ue8m0", "ue8m0", tuple(block), ("reorder_with_weight_blocks",))
    if checkpoint_dtype not in ("bf16", "fp32") or kernel_dtype not in ("bf16", "fp32"):
        raise ValidationError("unsupported checkpoint or kernel scale dtype")
    steps = []
    if len(checkpoint_tensors) > 1:
        steps.append("concatenate_output_scale_shards_axis0")
    if checkpoint_dtype != kernel_dtype:
        if (checkpoint_dtype, kernel_dtype) != ("bf16", "fp32"):
            raise ValidationError("unsupported scale dtype transform (only bf16 -> fp32 is exact)")
        steps.append("widen_bf16_to_fp32_exact")
    return ScaleBinding(tensor, tuple(checkpoint_tensors), checkpoint_dtype, kernel_dtype, tuple(block), tuple(steps))


# ----------------------------------------------------------------------------- byte transforms (CPU statement)
def tile_128x128(data: np.ndarray) -> np.ndarray:
    """uint8 ``[rows, k_bytes]`` row-major (rows and k_bytes multiples of 128) -> the same bytes in tile order
    ``[rows/128, k_bytes/128, 128, 128]``: tile (i, j) holds rows ``[128 i, +128)`` x bytes ``[128 j, +128)``, row-major."""
    if data.dtype != np.uint8 or data.ndim != 2:
        raise ValidationError("tile_128x128 takes a two-dimensional uint8 array")
    rows, k = data.shape
    if rows % TILE or k % TILE or rows == 0 or k == 0:
        raise ValidationError("rows and row bytes must be positive multiples of 128")
    return np.ascontiguousarray(data.reshape(rows // TILE, TILE, k // TILE, TILE).transpose(0, 2, 1, 3)).reshape(rows, k)


def untile_128x128(data: np.ndarray) -> np.ndarray:
    """Inverse of ``tile_128x128``."""
    rows, k = data.shape
    return np.ascontiguousarray(data.reshape(rows // TILE, k // TILE, TILE, TILE).transpose(0, 2, 1, 3)).reshape(rows, k)


def widen_bf16_to_fp32(bits: np.ndarray) -> np.ndarray:
    """BF16 bit patterns (uint16) -> FP32 values with the same value (exact)."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def mxfp4_pair_blocks(codes: np.ndarray, scales: np.ndarray, paired_half_rows: int) -> tuple[np.ndarray, np.ndarray]:
    """CPU statement of ``netra_moe_mxfp4_pack_launch``: uint8 codes ``[rows, k/2]`` and scale bytes ``[rows, k/32]`` ->
    code blocks and scale atoms in (group, tile within the half, K-block, half) order; inside an atom row r's four
    bytes sit at ``16 (r % 32) + 4 (r / 32)``.  Shapes are kept; only the byte order changes."""
    rows, half_k = codes.shape
    k = 2 * half_k
    h = paired_half_rows // TILE
    if codes.dtype != np.uint8 or scales.dtype != np.uint8 or scales.shape != (rows, k // 32):
        raise ValidationError("mxfp4_pair_blocks takes uint8 codes [rows, k/2] and scales [rows, k/32]")
    if paired_half_rows <= 0 or paired_half_rows % TILE or rows % (2 * paired_half_rows) or k % TILE:
        raise ValidationError("rows must be whole groups of 2 * paired_half_rows and k a multiple of 128")
    groups, kb = rows // (2 * paired_half_rows), k // TILE
    c = codes.reshape(groups, 2, h, TILE, kb, 64).transpose(0, 2, 4, 1, 3, 5)            # [group, tile, kb, half, r, 64]
    s = scales.reshape(groups, 2, h, 4, 32, kb, 4).transpose(0, 2, 5, 1, 4, 3, 6)         # [group, tile, kb, half, r % 32, r / 32, 4]
    return np.ascontiguousarray(c).reshape(rows, half_k), np.ascontiguousarray(s).reshape(rows, k // 32)


def apply_weight_steps(binding: LayoutBinding, sources: list[np.ndarray]) -> np.ndarray:
    """Runs a binding's steps on uint8 ``[slabs, N, K]`` sources (CPU); returns the bytes the kernel will stream."""
    data = sources
    for step in binding.steps:
        if step.operation == "concatenate_output_shards":
            data = [np.concatenate(data, axis=1)]
        elif step.operation == "tile_128x128":
            slabs, n, k = data[0].shape
            data = [tile_128x128(data[0].reshape(slabs * n, k)).reshape(slabs, n, k)]
        else:
            raise ValidationError(f"unknown repack operation {step.operation!r}")
    if len(data) != 1:
        raise ValidationError("the layout steps left more than one tensor")
    return data[0]


def moe_layer_layout_plan(weight_layout: str, *, split_gate_up: bool = False, scale_dtype: str = "fp32") -> dict[str, Any]:
    """The ``layout_plan.json`` document of one routed-MoE layer."""
    if weight_layout == "mxfp4_paired_blocks":
        if split_gate_up:
            raise ValidationError("the MXFP4 plan takes the concatenated gate/up tensor")
        weights = [plan_weight_layout("w13", MXFP4_ROW_MAJOR, MXFP4_PAIRED_BLOCKS, checkpoint_tensors=("w13",)),
                   plan_weight_layout("w2", MXFP4_ROW_MAJOR, MXFP4_PAIRED_BLOCKS, checkpoint_tensors=("w2",))]
        scales = [plan_scale_layout(name + "_scale", (name + "_scale",), checkpoint_dtype="ue8m0", kernel_dtype="ue8m0", block=(1, 32))
                  for name in ("w13", "w2")]
        return {"format": "netra-layout-plan-2", "weights": [w.to_dict() for w in weights], "scales": [s.to_dict() for s in scales]}
    kernel = TILES128 if weight_layout == "tiles128" else ROW_MAJOR
    w13_sources = ("gate_proj", "up_proj") if split_gate_up else ("w13",)
    w13 = plan_weight_layout("w13", SPLIT_GATE_UP if split_gate_up else ROW_MAJOR, kernel, checkpoint_tensors=w13_sources)
    w2 = plan_weight_layout("w2", ROW_MAJOR, kernel, checkpoint_tensors=("w2",))
    scales = [plan_scale_layout("w13_scale", tuple(s + "_scale_inv" for s in w13_sources), checkpoint_dtype=scale_dtype,
                                kernel_dtype="fp32", block=(TILE, TILE)),
              plan_scale_layout("w2_scale", ("w2_scale_inv",), checkpoint_dtype=scale_dtype, kernel_dtype="fp32", block=(TILE, TILE))]
    return {"format": "netra-layout-plan-2", "weights": [w13.to_dict(), w2.to_dict()], "scales": [s.to_dict() for s in scales]}

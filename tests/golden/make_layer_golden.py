"""Generates tests/golden/moe_layer_t16.npz: the CPU checker's results for the T=16 decode case
(hidden seed 0, router seed 1, expert seed 1000) plus digests of the seeded operands, so that
the checker, the operand generator and the GPU path are all pinned to one set of bytes.

Usage: python tests/golden/make_layer_golden.py
"""
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from netra_kernel_b200 import synth  # noqa: E402
from oracle import moe_ref  # noqa: E402


def bits(t):
    return np.ascontiguousarray(t.view(torch.int16).numpy().view(np.uint16))


def u8(t):
    return np.ascontiguousarray(t.view(torch.uint8).numpy())


def digest(a) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main() -> None:
    ops = synth.make_operands(16)
    ref = moe_ref.moe_layer(bits(ops.hidden), bits(ops.router_w), u8(ops.w13), ops.w13_scale.numpy(),
                            u8(ops.w2), ops.w2_scale.numpy())
    out = Path(__file__).resolve().parent / "moe_layer_t16.npz"
    np.savez_compressed(
        out, logits=ref["logits"], topk_ids=ref["topk_ids"], topk_w=ref["topk_w"], perm=ref["perm"],
        counts=ref["counts"], offsets=ref["offsets"], a_fp8=ref["a_fp8"], a_scale=ref["a_scale"],
        h_fp8=ref["h_fp8"], h_scale=ref["h_scale"], out=ref["out"],
        digests=np.array([digest(bits(ops.hidden)), digest(bits(ops.router_w)), digest(u8(ops.w13)),
                          digest(ops.w13_scale.numpy()), digest(u8(ops.w2)), digest(ops.w2_scale.numpy())]))
    print(out, out.stat().st_size)


if __name__ == "__main__":
    main()

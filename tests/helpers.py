"""Shared test helpers: numpy views of torch operands and the ctypes wrapper of the C checker."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = ROOT / "tests" / "golden"

# Parity gates (BF16 output vs the CPU checker on identical operands).
MAX_ABS = 2e-2
REL_L2 = 5e-3


def bits(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16))


def u8(t: torch.Tensor) -> np.ndarray:
    return np.ascontiguousarray(t.detach().cpu().contiguous().view(torch.uint8).numpy())


def load_c_oracle() -> ctypes.CDLL:
    lib = ROOT / "oracle" / "libmoe_ref.so"
    src = ROOT / "oracle" / "moe_ref.c"
    if not lib.exists() or lib.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True, capture_output=True)
    return ctypes.CDLL(str(lib))


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def c_layer(lib, hidden_bits, router_bits, w13, w13_s, w2, w2_s, bias=None, shared_w=None) -> dict:
    """Run the C checker's whole layer; returns the same keys as oracle.moe_ref.moe_layer."""
    t = hidden_bits.shape[0]
    out = {
        "logits": np.zeros((t, 256), np.uint16), "topk_ids": np.zeros((t, 9), np.int32),
        "topk_w": np.zeros((t, 9), np.float32), "perm": np.zeros(t * 8, np.int32),
        "counts": np.zeros(256, np.int32), "offsets": np.zeros(257, np.int32),
        "a_fp8": np.zeros((t, 2048), np.uint8), "a_scale": np.zeros((t, 16), np.float32),
        "h_fp8": np.zeros((t, 9, 512), np.uint8), "h_scale": np.zeros((t, 9, 4), np.float32),
        "out": np.zeros((t, 2048), np.uint16),
    }
    bias = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    shared_w = None if shared_w is None else np.ascontiguousarray(shared_w, dtype=np.float32)
    rc = lib.moe_ref_layer(_p(hidden_bits), _p(router_bits), _p(bias), _p(shared_w), _p(w13), _p(w13_s), _p(w2), _p(w2_s),
                           ctypes.c_int(t), _p(out["logits"]), _p(out["topk_ids"]), _p(out["topk_w"]), _p(out["perm"]),
                           _p(out["counts"]), _p(out["offsets"]), _p(out["a_fp8"]), _p(out["a_scale"]),
                           _p(out["h_fp8"]), _p(out["h_scale"]), _p(out["out"]))
    assert rc == 0
    return out


def np_weights(weights):
    w13, w13_s, w2, w2_s = weights
    return u8(w13), w13_s.numpy(), u8(w2), w2_s.numpy()

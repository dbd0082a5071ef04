"""Generates tests/golden/mxfp4_dequant.npz by importing the reference's own MXFP4 dequantiser
(tests/gfx1151/test_netra_mxfp4_sgl_decode.py:23-31 inside the reference project) and running
it on seeded codes.  Needs the reference checkout; the committed .npz is what the tests read.

Usage: python tests/golden/make_mxfp4_golden.py /path/to/reference
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch


def main() -> None:
    ref_root = Path(sys.argv[1])
    spec = importlib.util.spec_from_file_location(
        "ref_mxfp4_test", ref_root / "tests/gfx1151/test_netra_mxfp4_sgl_decode.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    g = torch.Generator().manual_seed(4)
    packed = torch.randint(0, 256, (8, 64), generator=g, dtype=torch.uint8)     # 8 rows, K = 128
    packed[0, :16] = torch.arange(16, dtype=torch.uint8) * 17                    # every code in both nibbles
    scales = torch.randint(100, 140, (8, 4), generator=g, dtype=torch.uint8)
    scales[1] = torch.tensor([1, 127, 254, 128], dtype=torch.uint8)
    values = mod.dequant(packed, scales)
    out = Path(__file__).resolve().parent / "mxfp4_dequant.npz"
    np.savez_compressed(out, packed=packed.numpy(), scales=scales.numpy(), values=values.numpy())
    print(out, values.shape, values.dtype)


if __name__ == "__main__":
    main()

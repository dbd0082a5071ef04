"""Builds libnetra_sm100.so (kernels + C ABI) for sm_100a with nvcc, in-tree.

Usage: python -m netra_kernel_b200.csrc.build [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "libnetra_sm100.so"
CUBIN = HERE / "netra_moe_sm100a.cubin"
SOURCES = ["api.cu", "engine.cpp"]
DEPENDS = ["api.cu", "engine.cpp", "kernels_cubin.cu", "common.cuh", "route_kernels.cu", "bridge_kernels.cu",
           "umma_kernels.cu", "umma_tokmajor.cu", "router_umma.cu", "ep_kernels.cu", "mxfp4_kernels.cu", "ep_p2p.cu", "static_scratch_sort.cu", "prefill_m768_bridge.cu", "../../include/netra_moe.h", "../../include/netra_engine.h"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-ccbin", "g++"]
NVCC_FLAGS = [*ARCH_FLAGS, "--shared", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def stale() -> bool:
    if not LIB.exists() or not CUBIN.exists():
        return True
    built = min(LIB.stat().st_mtime, CUBIN.stat().st_mtime)
    return any((HERE / d).stat().st_mtime > built for d in DEPENDS)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-o", str(LIB), *[str(HERE / s) for s in SOURCES], "-lcudart"]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=HERE)
    log = proc.stdout + proc.stderr
    (HERE / "build.log").write_text(log)
    if verbose or proc.returncode != 0:
        print(log)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed building libnetra_sm100.so (see csrc/build.log)")
    # the same kernels as a stand-alone code object for the engine runtime (cuModuleLoadData)
    cmd = [nvcc, *ARCH_FLAGS, "-cubin", "-o", str(CUBIN), str(HERE / "kernels_cubin.cu")]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=HERE)
    (HERE / "build_cubin.log").write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        if verbose:
            print(proc.stdout + proc.stderr)
        raise RuntimeError("nvcc failed building netra_moe_sm100a.cubin (see csrc/build_cubin.log)")
    return LIB


if __name__ == "__main__":
    build(force=True, verbose="--verbose" in sys.argv)
    print(LIB)

"""CPU tests of the C-ABI library: it builds for sm_100a, loads, and exports every symbol the
header declares.  No compute call is made (there is no GPU here)."""
import ctypes
import re

from netra_kernel_b200 import abi
from tests import helpers


def _declared_symbols(header: str):
    text = (helpers.ROOT / "include" / header).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(netra_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    from netra_kernel_b200.csrc import build
    path = build.build()
    lib = ctypes.CDLL(str(path))
    names = _declared_symbols("netra_moe.h")
    assert len(names) >= 25
    for name in names:
        assert hasattr(lib, name), name
    assert set(names) == set(abi.SIGNATURES), set(names) ^ set(abi.SIGNATURES)


def test_struct_sizes_and_argument_checks_without_a_device():
    lib = abi.load()
    lay = abi.WorkspaceLayout()
    lay.struct_size = 4                       # wrong size is rejected, as in the reference ABI
    assert lib.netra_moe_workspace_layout_query(16, ctypes.byref(lay)) == -1
    assert b"struct_size" in lib.netra_moe_last_error()
    lay.struct_size = ctypes.sizeof(lay)
    assert lib.netra_moe_workspace_layout_query(0, ctypes.byref(lay)) == -1
    assert lib.netra_moe_workspace_layout_query(256, ctypes.byref(lay)) == 0
    rows = 256 * 9
    assert lay.a_scale - lay.a_fp8 >= rows * 2048 and lay.total_bytes > lay.down_f32 + rows * 2048 * 4
    for field, _ in abi.WorkspaceLayout._fields_[3:]:
        assert getattr(lay, field) % 1024 == 0, field
    # null pointers are refused before any launch
    assert lib.netra_qwen36_router_bf16_launch(None, None, None, 4, None) == -1
    assert lib.netra_qwen36_moe_gate_up_launch(None, None, None, None, None, None, 1, None) == -1
    # load() runs the per-device set-up: without a device it must fail with the runtime's message, never silently succeed
    rc = lib.netra_qwen36_moe_silu_mul_quant_load(None)
    import torch
    if torch.cuda.is_available():
        assert rc == 0
    else:
        assert rc != 0 and b"cudaGetDevice" in lib.netra_qwen36_moe_silu_mul_quant_last_error()

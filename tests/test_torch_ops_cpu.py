"""The torch.library ops register without a GPU, trace through their fake kernels, and refuse CPU tensors."""
import pytest
import torch

from netra_kernel_b200 import torch_ops


def test_ops_are_registered_with_fake_kernels():
    from torch._subclasses.fake_tensor import FakeTensorMode
    assert torch.ops.netra.moe_layer is not None and torch.ops.netra.moe_apply is not None
    with FakeTensorMode():
        h = torch.empty(5, 2048, dtype=torch.bfloat16, device="cuda")
        w = torch.empty(5, 8, dtype=torch.float32, device="cuda")
        i = torch.empty(5, 8, dtype=torch.int32, device="cuda")
        assert torch.ops.netra.moe_layer(h, 1).shape == (5, 2048)
        out = torch.ops.netra.moe_apply(h, w, i, 1)
        assert out.shape == (5, 2048) and out.dtype == torch.bfloat16


def test_handles_and_the_missing_cpu_path():
    handle = torch_ops.register_layer(object())
    assert handle in torch_ops._layers
    torch_ops.release_layer(handle)
    assert handle not in torch_ops._layers
    with pytest.raises(Exception):          # no CPU kernel is registered: the ops exist for CUDA tensors only
        torch.ops.netra.moe_layer(torch.zeros(2, 2048, dtype=torch.bfloat16), handle)


def test_fp16_partial_row_panels_read_back_as_rows():
    """The down projection's FP16 partial rows are stored as sixteen column panels [rows, 128] with the 16-byte chunks
    of a panel row permuted by the row index; the host-side view used by the parity tests undoes exactly that."""
    from netra_kernel_b200.moe import _f16_rows_from_panels
    rows = 37
    logical = torch.arange(rows * 2048, dtype=torch.float32).remainder(2039).view(rows, 2048).to(torch.float16)
    raw = torch.zeros(16, rows, 16, 8, dtype=torch.float16)
    for p in range(rows):
        for j in range(16):
            raw[:, p, j ^ (p & 15)] = logical[p].view(16, 16, 8)[:, j]
    assert torch.equal(_f16_rows_from_panels(raw.reshape(-1), rows), logical)

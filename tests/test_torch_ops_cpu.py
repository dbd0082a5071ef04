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

"""``torch.library`` custom ops over the layer's C ABI, for serving stacks that call operators by name
(the role of the reference's SGLang custom-op registration, ``scripts/rocm/integrations/sglang/netra_gfx1151_sglang.py:1121-1311``).

    handle = register_layer(layer)                       # a RoutedMoELayer
    out = torch.ops.netra.moe_layer(hidden, handle)      # router + top-8 inside
    out = torch.ops.netra.moe_apply(hidden, topk_weights, topk_ids, handle)   # the caller's top-k

A handle is a small integer naming a live layer object of this process; ``release_layer`` drops it.
Both ops run on torch's current stream through ``libnetra_sm100.so`` and have fake (meta) kernels, so
they can sit inside traced graphs; there is no CPU implementation.
"""
from __future__ import annotations

import torch

_layers: dict[int, object] = {}
_next_handle = 1


def register_layer(layer) -> int:
    global _next_handle
    handle = _next_handle
    _next_handle += 1
    _layers[handle] = layer
    return handle


def release_layer(handle: int) -> None:
    _layers.pop(handle, None)


def _lookup(handle: int):
    layer = _layers.get(int(handle))
    if layer is None:
        raise RuntimeError(f"netra: no registered layer with handle {handle}")
    return layer


@torch.library.custom_op("netra::moe_layer", mutates_args=(), device_types="cuda")
def moe_layer(hidden: torch.Tensor, handle: int) -> torch.Tensor:
    return _lookup(handle)(hidden.contiguous())


@moe_layer.register_fake
def _(hidden: torch.Tensor, handle: int) -> torch.Tensor:
    return torch.empty_like(hidden)


@torch.library.custom_op("netra::moe_apply", mutates_args=(), device_types="cuda")
def moe_apply(hidden: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, handle: int) -> torch.Tensor:
    return _lookup(handle).apply(hidden.contiguous(), topk_weights.contiguous(), topk_ids.contiguous())


@moe_apply.register_fake
def _(hidden: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, handle: int) -> torch.Tensor:
    return torch.empty_like(hidden)

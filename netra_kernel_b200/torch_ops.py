"""``torch.library`` custom ops over the layer's C ABI, for serving stacks that call operators by name
(the role of the reference's SGLang custom-op registration, ``scripts/rocm/integrations/sglang/netra_gfx1151_sglang.py:1121-1311``).

    handle = register_layer(layer)                       # a RoutedMoELayer
    out = torch.ops.netra.moe_layer(hidden, handle)      # router + top-8 inside
    out = torch.ops.netra.moe_apply(hidden, topk_weights, topk_ids, handle)   # the caller's top-k

A handle is a small integer naming a live layer object of this process; ``release_layer`` drops it.
Both ops run on torch's current stream through ``libnetra_sm100.so`` and have fake (meta) kernels, so
they can sit inside traced graphs; there is no CPU implementation.

Bring-up modes (the role of the reference's ``SGLANG_NETRA_ENGINE_MODE`` shadow / compare modes,
``docs/compiler/validation.md:187-193``), chosen by the environment variable ``NETRA_ENGINE_MODE`` when a layer is
registered with its row-major weights (``register_layer(layer, shadow_weights=...)``):
``engine`` (default) runs the fused layer only; ``shadow`` also runs the slot-order per-kernel bridges on the layer's
own routing and records the comparison in ``last_comparison(handle)``; ``compare`` raises when the two disagree
beyond the layer tolerances.  Both extra modes synchronise and are meant for bring-up, not for serving.
"""
from __future__ import annotations

import torch

import os

_layers: dict[int, object] = {}
_shadow: dict[int, tuple] = {}
_comparisons: dict[int, dict] = {}
_next_handle = 1
MAX_ABS, REL_L2 = 2e-2, 5e-3          # BF16 output tolerances of the layer


def register_layer(layer, shadow_weights=None) -> int:
    """``shadow_weights`` = (w13, w13_scale, w2, w2_scale) in the checkpoint's row-major layout, on the GPU; needed only
    for the shadow / compare modes."""
    global _next_handle
    handle = _next_handle
    _next_handle += 1
    _layers[handle] = layer
    if shadow_weights is not None:
        _shadow[handle] = tuple(shadow_weights)
    return handle


def release_layer(handle: int) -> None:
    _layers.pop(handle, None)
    _shadow.pop(handle, None)
    _comparisons.pop(handle, None)


def last_comparison(handle: int):
    """{"max_abs", "rel_l2"} of the most recent shadow / compare call of this layer, or None."""
    return _comparisons.get(int(handle))


def _mode() -> str:
    mode = os.environ.get("NETRA_ENGINE_MODE", "engine")
    if mode not in ("engine", "shadow", "compare"):
        raise RuntimeError(f"NETRA_ENGINE_MODE must be engine, shadow or compare, not {mode!r}")
    return mode


def _check_against_bridges(handle: int, hidden: torch.Tensor, out: torch.Tensor) -> None:
    """Recompute the expert part with the slot-order bridge kernels from the layer's own routing and quantised rows."""
    from . import moe
    mode = _mode()
    if mode == "engine":
        return
    if handle not in _shadow:
        raise RuntimeError("netra: shadow / compare mode needs register_layer(layer, shadow_weights=...)")
    layer = _layers[handle]
    w13, w13_s, w2, w2_s = _shadow[handle]
    tokens = hidden.shape[0]
    torch.cuda.current_stream().synchronize()
    inter = layer.intermediates(tokens)
    pairs = tokens * 8
    a_fp8 = inter["a_fp8"][pairs:pairs + tokens].contiguous()
    a_scale = inter["a_scale"][pairs:pairs + tokens].contiguous()
    ids9, w9 = inter["topk_ids"].contiguous(), inter["topk_w"].contiguous()
    gate_up = moe.bridge_gate_up(a_fp8, a_scale, w13, w13_s, ids9)
    act, act_s = moe.bridge_silu_mul_quant(gate_up)
    ref = moe.bridge_down_reduce(act, act_s, w2, w2_s, w9, ids9)
    torch.cuda.current_stream().synchronize()
    d = out.float() - ref.float()
    result = {"max_abs": float(d.abs().max()), "rel_l2": float(d.norm() / ref.float().norm().clamp_min(1e-30))}
    _comparisons[handle] = result
    if mode == "compare" and (result["max_abs"] > MAX_ABS or result["rel_l2"] > REL_L2):
        raise RuntimeError(f"netra: fused layer and bridge path disagree: {result}")


def _lookup(handle: int):
    layer = _layers.get(int(handle))
    if layer is None:
        raise RuntimeError(f"netra: no registered layer with handle {handle}")
    return layer


@torch.library.custom_op("netra::moe_layer", mutates_args=(), device_types="cuda")
def moe_layer(hidden: torch.Tensor, handle: int) -> torch.Tensor:
    hidden = hidden.contiguous()
    out = _lookup(handle)(hidden)
    _check_against_bridges(int(handle), hidden, out)
    return out


@moe_layer.register_fake
def _(hidden: torch.Tensor, handle: int) -> torch.Tensor:
    return torch.empty_like(hidden)


@torch.library.custom_op("netra::moe_apply", mutates_args=(), device_types="cuda")
def moe_apply(hidden: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, handle: int) -> torch.Tensor:
    hidden = hidden.contiguous()
    out = _lookup(handle).apply(hidden, topk_weights.contiguous(), topk_ids.contiguous())
    _check_against_bridges(int(handle), hidden, out)
    return out


@moe_apply.register_fake
def _(hidden: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor, handle: int) -> torch.Tensor:
    return torch.empty_like(hidden)

"""Seeded synthetic operands for the routed-MoE layer (Qwen3.6-35B-A3B shapes).

The reference replays captured serving operands that are not shipped with it
(``harness/gfx950/fp8/moe/decode/qwen36_moe_gate_up_fp8_mfma_gfx950.hip:72-88``),
so every operand here is drawn from a seeded CPU generator with the shapes of
``manifests/gfx950/models/qwen36-moe-m1-golden.json:47-49,101-102``:

* hidden BF16 ``[T, 2048]`` ~ N(0, 1), seed 0
* router weight BF16 ``[256, 2048]`` ~ N(0, 0.02), seed 1
* expert slabs (256 routed + slab 256 = shared expert), FP32 ~ N(0, 0.02),
  seed ``1000 + layer``: W13 ``[257, 1024, 2048]`` (rows 0..511 gate, 512..1023
  up) and W2 ``[257, 2048, 512]``, quantised to FP8 E4M3 with one FP32 scale
  per 128x128 block (``scale = max(amax, 1e-10) / 448``).

All draws happen on the CPU so that the CPU checker and the GPU path see the
same bytes on every machine with the same torch build.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional

import torch

HIDDEN = 2048
INTER = 512
N_ROUTED = 256
TOPK = 8
SLOTS = TOPK + 1          # slot 8 is the shared expert (expert id 256)
N_SLABS = N_ROUTED + 1
BLOCK = 128
FP8_MAX = 448.0
ZIPF_S = 1.1
# Bias strength found by bisect_zipf_alpha() for T=8192 with seeds 0/1: the
# hottest expert then receives 10x the mean load (2,560 of 65,536 pairs).
ZIPF_ALPHA_T8192 = 0.2664


def quantize_fp8_block128(w: torch.Tensor):
    """FP32 ``[N, K]`` -> (FP8 E4M3 ``[N, K]``, FP32 scales ``[N/128, K/128]``).

    ``scale = max(amax_block, 1e-10) / 448`` in FP32, ``q = sat_rne(w / scale)``.
    torch's CPU cast to ``float8_e4m3fn`` rounds to nearest even but does not
    saturate (465 -> NaN), hence the clamp.
    """
    n, k = w.shape
    b = w.view(n // BLOCK, BLOCK, k // BLOCK, BLOCK)
    amax = b.abs().amax(dim=(1, 3)).clamp_min(1e-10)
    scale = (amax / FP8_MAX).to(torch.float32)
    q = (b / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX)
    return q.to(torch.float8_e4m3fn).view(n, k).contiguous(), scale.contiguous()


_E2M1_THRESHOLDS = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])


def quantize_mxfp4(w: torch.Tensor):
    """FP32 ``[N, K]`` -> (packed E2M1 ``[N, K/2]`` u8, E8M0 ``[N, K/32]`` u8).

    Same arithmetic as ``tools/checkpoint/quantize_qwen36_lm_head_mxfp4.py:58-67``:
    ``e = ceil(log2(max(amax/6, 2^-126)))``, scale byte ``clamp(e+127, 1, 254)``,
    magnitude code = bucketize(|x| / 2^e) over the E2M1 midpoints, sign in bit 3,
    byte = ``code[k even] | code[k odd] << 4``.  The physical layout here keeps
    K contiguous per output row (the reference stores K-major for its GPU).
    """
    n, k = w.shape
    x = w.reshape(n, k // 32, 32)
    max_abs = x.abs().amax(dim=2)
    exponent = torch.ceil(torch.log2(torch.clamp(max_abs / 6.0, min=2.0 ** -126))).to(torch.int32)
    scale_byte = torch.clamp(exponent + 127, 1, 254).to(torch.uint8)
    scale = torch.exp2(exponent.to(torch.float32))
    normalized = x.abs() / scale.unsqueeze(2)
    magnitude = torch.bucketize(normalized, _E2M1_THRESHOLDS.to(w.device)).to(torch.uint8)
    sign = torch.signbit(x).to(torch.uint8) << 3
    code = (magnitude | sign).reshape(n, k)
    packed = code[:, 0::2] | (code[:, 1::2] << 4)
    return packed.contiguous(), scale_byte.contiguous()


def zipf_bias(alpha: float, n: int = N_ROUTED, s: float = ZIPF_S) -> torch.Tensor:
    """Per-expert FP32 logit bias ``alpha * log(zipf_pmf(e + 1; s, n))``."""
    ranks = torch.arange(1, n + 1, dtype=torch.float64)
    pmf = ranks.pow(-s)
    pmf = pmf / pmf.sum()
    return (alpha * pmf.log()).to(torch.float32)


def _bf16_from_f64(x: torch.Tensor) -> torch.Tensor:
    """Round FP64 to BF16 once (no intermediate FP32 rounding)."""
    bits = x.contiguous().view(torch.int64)
    sign = bits < 0
    mag = bits & 0x7FFFFFFFFFFFFFFF
    rounded = (mag + ((1 << 44) - 1) + ((mag >> 45) & 1)) >> 45
    rounded = rounded - (896 << 7)           # exponent bias 1023 -> 127
    rounded = torch.where(rounded < (1 << 7), torch.zeros_like(rounded), rounded)
    rounded = torch.clamp(rounded, max=0x7F80)                                   # overflow and infinity
    rounded = torch.where(mag > 0x7FF0000000000000, torch.full_like(rounded, 0x7FC0), rounded)   # NaN
    out = rounded | torch.where(sign, 0x8000, 0)
    return torch.where(out >= 0x8000, out - 0x10000, out).to(torch.int16).view(torch.bfloat16)   # bit pattern as is


def routed_load(hidden: torch.Tensor, router_w: torch.Tensor, bias: Optional[torch.Tensor]):
    """Pairs per expert under (logit desc, expert id asc) top-8 selection."""
    logits = _bf16_from_f64(hidden.double() @ router_w.double().T).float()
    if bias is not None:
        logits = logits + bias
    order = torch.sort(-logits, dim=1, stable=True).indices[:, :TOPK]
    return torch.bincount(order.reshape(-1), minlength=N_ROUTED)


def bisect_zipf_alpha(hidden, router_w, target: float = 10.0, iters: int = 24) -> float:
    """Bias strength for which the hottest expert gets ``target`` x the mean load."""
    lo, hi = 0.0, 2.0
    for _ in range(iters):
        mid = 0.5 * (lo + hi)
        load = routed_load(hidden, router_w, zipf_bias(mid)).double()
        if (load.max() / load.mean()).item() < target:
            lo = mid
        else:
            hi = mid
    return 0.5 * (lo + hi)


@dataclass
class MoEOperands:
    """Operands of one routed-MoE layer, all on the CPU."""
    hidden: torch.Tensor                 # bf16 [T, 2048]
    router_w: torch.Tensor               # bf16 [256, 2048]
    router_bias: Optional[torch.Tensor]  # f32 [256] or None
    shared_w: torch.Tensor               # f32 [T] weight of the shared slot (1.0 = always on)
    w13: torch.Tensor                    # fp8 [E', 1024, 2048]
    w13_scale: torch.Tensor              # f32 [E', 8, 16]
    w2: torch.Tensor                     # fp8 [E', 2048, 512]
    w2_scale: torch.Tensor               # f32 [E', 16, 4]
    meta: dict = field(default_factory=dict)

    @property
    def tokens(self) -> int:
        return self.hidden.shape[0]


def make_activations(tokens: int, zipf_alpha: Optional[float] = None, seed: int = 0):
    hidden = torch.randn(tokens, HIDDEN, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)
    router_w = (0.02 * torch.randn(N_ROUTED, HIDDEN, generator=torch.Generator().manual_seed(1))).to(torch.bfloat16)
    bias = zipf_bias(zipf_alpha) if zipf_alpha else None
    return hidden, router_w, bias


def make_expert_weights(layer: int = 0, n_slabs: int = N_SLABS, keep_fp32: bool = False):
    """Quantised expert slabs for one layer, generated slab by slab (12 MiB FP32 each)."""
    g = torch.Generator().manual_seed(1000 + layer)
    w13 = torch.empty(n_slabs, 2 * INTER, HIDDEN, dtype=torch.float8_e4m3fn)
    w13_s = torch.empty(n_slabs, 2 * INTER // BLOCK, HIDDEN // BLOCK, dtype=torch.float32)
    w2 = torch.empty(n_slabs, HIDDEN, INTER, dtype=torch.float8_e4m3fn)
    w2_s = torch.empty(n_slabs, HIDDEN // BLOCK, INTER // BLOCK, dtype=torch.float32)
    fp32 = []
    for e in range(n_slabs):
        a = 0.02 * torch.randn(2 * INTER, HIDDEN, generator=g)
        b = 0.02 * torch.randn(HIDDEN, INTER, generator=g)
        w13[e], w13_s[e] = quantize_fp8_block128(a)
        w2[e], w2_s[e] = quantize_fp8_block128(b)
        if keep_fp32:
            fp32.append((a, b))
    return (w13, w13_s, w2, w2_s, fp32) if keep_fp32 else (w13, w13_s, w2, w2_s)


def make_expert_weights_device(layer: int, device, n_slabs: int = N_SLABS, slabs_per_chunk: int = 32, mxfp4: bool = False):
    """The same distributions drawn and quantised ON THE DEVICE (seed ``1000 + layer`` of that device's generator), for
    workloads whose weights would take minutes to draw on the host (a 40-layer stack is 32 GB of FP8).  The values differ
    from ``make_expert_weights`` (another generator) but every rank of a job that calls this with the same layer index on
    the same GPU model gets the same bytes.  Returns (W13, W13 scales, W2, W2 scales); with ``mxfp4`` the FP32 slabs are
    quantised to MXFP4 instead: (W13 packed, W13 E8M0 scales, W2 packed, W2 scales) as in ``make_expert_weights_mxfp4``."""
    g = torch.Generator(device=device).manual_seed(1000 + layer)
    out13, out13s, out2, out2s = [], [], [], []
    for first in range(0, n_slabs, slabs_per_chunk):
        n = min(slabs_per_chunk, n_slabs - first)
        a = 0.02 * torch.randn(n * 2 * INTER, HIDDEN, generator=g, device=device)
        b = 0.02 * torch.randn(n * HIDDEN, INTER, generator=g, device=device)
        qa, sa = (quantize_mxfp4 if mxfp4 else quantize_fp8_block128)(a)
        qb, sb = (quantize_mxfp4 if mxfp4 else quantize_fp8_block128)(b)
        out13.append(qa.view(n, 2 * INTER, -1)); out13s.append(sa.view(n, -1, sa.shape[-1]) if mxfp4 else sa.view(n, 2 * INTER // BLOCK, -1))
        out2.append(qb.view(n, HIDDEN, -1)); out2s.append(sb.view(n, -1, sb.shape[-1]) if mxfp4 else sb.view(n, HIDDEN // BLOCK, -1))
        del a, b
    return torch.cat(out13), torch.cat(out13s), torch.cat(out2), torch.cat(out2s)


def make_expert_weights_mxfp4(layer: int = 0, n_slabs: int = N_SLABS):
    """The same FP32 slabs as ``make_expert_weights`` (same seeds, same draw order), quantised to MXFP4 instead:
    (W13 packed ``[n, 1024, 1024]`` u8, W13 E8M0 scales ``[n, 1024, 64]`` u8, W2 packed ``[n, 2048, 256]``,
    W2 scales ``[n, 2048, 16]``)."""
    g = torch.Generator().manual_seed(1000 + layer)
    p13 = torch.empty(n_slabs, 2 * INTER, HIDDEN // 2, dtype=torch.uint8)
    s13 = torch.empty(n_slabs, 2 * INTER, HIDDEN // 32, dtype=torch.uint8)
    p2 = torch.empty(n_slabs, HIDDEN, INTER // 2, dtype=torch.uint8)
    s2 = torch.empty(n_slabs, HIDDEN, INTER // 32, dtype=torch.uint8)
    for e in range(n_slabs):
        a = 0.02 * torch.randn(2 * INTER, HIDDEN, generator=g)
        b = 0.02 * torch.randn(HIDDEN, INTER, generator=g)
        p13[e], s13[e] = quantize_mxfp4(a)
        p2[e], s2[e] = quantize_mxfp4(b)
    return p13, s13, p2, s2


def make_operands(tokens: int, layer: int = 0, zipf_alpha: Optional[float] = None,
                  n_slabs: int = N_SLABS) -> MoEOperands:
    """One layer's operands.  ``n_slabs < 257`` is for small CPU tests only: routing
    still ranges over 256 experts, so such operands suit the routing functions
    and GEMM cases whose expert ids are remapped by the caller."""
    hidden, router_w, bias = make_activations(tokens, zipf_alpha)
    w13, w13_s, w2, w2_s = make_expert_weights(layer, n_slabs)
    return MoEOperands(hidden, router_w, bias, torch.ones(tokens, dtype=torch.float32),
                       w13, w13_s, w2, w2_s,
                       {"tokens": tokens, "layer": layer, "zipf_alpha": zipf_alpha,
                        "seeds": {"hidden": 0, "router": 1, "experts": 1000 + layer}})


def workload_bytes_decode(tokens: int, experts_hit: int = N_ROUTED, mxfp4: bool = False) -> int:
    """Algorithmic HBM bytes of one layer call: every hit expert slab and its scales
    once, the shared slab, the router weight, BF16 hidden in and BF16 out.  ``mxfp4``: the slabs are
    E2M1 codes (half a byte per weight) with one E8M0 byte per 32 weights."""
    weights = 2 * INTER * HIDDEN + HIDDEN * INTER
    slab = weights // 2 + weights // 32 if mxfp4 else weights + 4 * (8 * 16 + 16 * 4)
    return (experts_hit + 1) * slab + N_ROUTED * HIDDEN * 2 + 2 * tokens * HIDDEN * 2


def workload_flops(tokens: int) -> int:
    """FP8 GEMM flops of one layer call (8 routed rows + 1 shared row per token)."""
    return tokens * SLOTS * (2 * HIDDEN * 2 * INTER + 2 * INTER * HIDDEN)

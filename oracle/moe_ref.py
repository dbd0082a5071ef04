"""CPU checker for the FP8 block-scaled routed-MoE layer.  TEST INFRASTRUCTURE ONLY.

Nothing that ships may import this module: only ``tests/``, the smoke check and
the ``cpu_baseline`` / ``--impl reference`` legs of the benchmark use it, and
only to check or to time the CPU restatement, never to produce a product result.

What it restates (paths are inside the reference project):

* router logits  - ``tools/benchmark/export_qwen36_router_bf16_capture.py:78``
  (BF16 ``F.linear`` -> BF16).  The FP32 accumulation order of that call is
  unspecified, so the checker defines the logit as the exact dot product
  rounded ONCE to BF16 (FP64 accumulation, direct FP64->BF16 rounding).
* softmax / top-8 / renormalise - not in the reference: it calls SGLang's
  ``fused_topk`` (sgl-project/sglang @ 1eee8fbdcc25b44e13bc097d5ff6ac24e8c24af4,
  call site ``scripts/rocm/integrations/sglang/sglang-gfx1151-bf16-router.patch:64``).
  Restated as FP32 softmax, selection by (logit desc, expert id asc), FP32
  renormalisation over the 8 selected probabilities summed in slot order.
* shared slot - ``runtime/gfx950/routing/decode/qwen36_shared_gate_append_bridge.h:10-23``
  (ids/weights [T,8] -> [T,9], slot 8 = expert 256).
* token sort - ``scripts/rocm/integrations/sglang/netra_gfx1151_sglang.py:1186-1209``
  (stable sort of flat pair ids by expert).
* per-128 FP8 quantiser - ``harness/gfx950/fp8/moe/decode/qwen36_moe_silu_mul_quant_fp8_gfx950.hip:57-94``
  (``scale = max(amax, 1e-10) * fl32(1/448)``, ``q = sat_rne(x * (1/scale))``).
* gate_up / down - ``tools/benchmark/export_qwen36_moe_stage1_capture.py:80-97``
  and ``export_qwen36_moe_stage2_capture.py:90-110`` (dequantise activation and
  weight block in FP32, FP32 matvec, add K-blocks ascending; slot-ascending
  weighted sum; one BF16 rounding).
* SiLU*up - ``kernels/gfx950/templates/moe/decode/silu_quant.inc:54-131``
  (FP32 SiLU, BF16 rounding BEFORE the per-128 amax).
* MXFP4 - ``tests/gfx1151/test_netra_mxfp4_sgl_decode.py:23-31`` (dequantiser)
  and ``tools/checkpoint/quantize_qwen36_lm_head_mxfp4.py:58-67`` (quantiser).

PARITY UNPINNED for the numeric path: the reference ships no golden vectors for
it (its harnesses replay captures that are not in the tree) and top-k, sorting
and input quantisation are third-party.  What IS pinned, in
``tests/test_oracle_pins.py``: the constants ``fl32(1/448) = 0x3b124925`` and
``1e-10f = 0x2edbe6ff`` (``silu_quant.inc:40-41``), the FP8 E4M3 codec against
torch's ``float8_e4m3fn``, and the MXFP4 dequantiser against vectors produced by
importing the reference's own ``dequant`` (``tests/golden/make_mxfp4_golden.py``).
"""
from __future__ import annotations

import numpy as np

HIDDEN = 2048
INTER = 512
N_ROUTED = 256
TOPK = 8
SLOTS = 9
BLOCK = 128
INV_448 = np.frombuffer(np.uint32(0x3B124925).tobytes(), dtype=np.float32)[0]
AMAX_FLOOR = np.frombuffer(np.uint32(0x2EDBE6FF).tobytes(), dtype=np.float32)[0]


# ----------------------------------------------------------------------------- scalar formats
def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even FP32 -> BF16 bit patterns (finite inputs)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))
    return (r >> 16).astype(np.uint16)


def bf16_round(x: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


def f64_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round FP64 to BF16 once (no intermediate FP32 rounding); |x| < 2^-126 -> signed zero,
    |x| >= 2^128 and infinity -> infinity, NaN -> quiet NaN with the sign kept."""
    bits = np.ascontiguousarray(x, dtype=np.float64).view(np.int64)
    sign = bits < 0
    mag = bits & np.int64(0x7FFFFFFFFFFFFFFF)
    r = (mag + np.int64((1 << 44) - 1) + ((mag >> 45) & 1)) >> 45
    r = r - np.int64(896 << 7)
    r = np.where(r < (1 << 7), 0, r)
    r = np.minimum(r, 0x7F80)
    r = np.where(mag > np.int64(0x7FF0000000000000), 0x7FC0, r)
    return (r | np.where(sign, 0x8000, 0)).astype(np.uint16)


def _e4m3_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for c in range(256):
        e, m = (c >> 3) & 15, c & 7
        v = (m / 8.0) * 2.0 ** -6 if e == 0 else (1 + m / 8.0) * 2.0 ** (e - 7)
        if (c & 0x7F) == 0x7F:
            v = np.nan
        t[c] = -v if c & 0x80 else v
    return t


E4M3_TABLE = _e4m3_table()


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
    return E4M3_TABLE[codes]


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """FP32 -> OCP E4M3 (e4m3fn) codes, round-to-nearest-even, saturating at 448."""
    x = np.asarray(x, dtype=np.float32)
    a = np.minimum(np.abs(x), np.float32(448.0)).astype(np.float64)
    _, ex = np.frexp(a)
    e = np.maximum(ex - 1, -6)
    step = np.ldexp(1.0, e - 3)
    q = np.rint(a / step)                      # half-to-even, exact scaling
    v = q * step
    _, ex2 = np.frexp(v)
    e2 = ex2 - 1
    normal = v >= 2.0 ** -6
    mant = np.where(normal, (v / np.ldexp(1.0, e2) - 1.0) * 8.0, v * 512.0)
    code = np.where(normal, ((e2 + 7) << 3), 0).astype(np.int64) + mant.astype(np.int64)
    code = np.where(np.isnan(x), 0x7F, code)
    return (code | np.where(np.signbit(x), 0x80, 0)).astype(np.uint8)


# ----------------------------------------------------------------------------- routing
def router_logits(hidden_bits: np.ndarray, router_bits: np.ndarray) -> np.ndarray:
    """BF16 bit patterns [T,H] x [E,H] -> BF16 bit patterns [T,E] (exact dot, one rounding)."""
    h = bf16_bits_to_f32(hidden_bits).astype(np.float64)
    w = bf16_bits_to_f32(router_bits).astype(np.float64)
    return f64_to_bf16_bits(h @ w.T)


def shared_gate(hidden_bits: np.ndarray, gate_bits: np.ndarray) -> np.ndarray:
    """Shared-expert gate of ``runtime/gfx950/routing/decode/qwen36_shared_gate_append_bridge.h:10-23``: BF16 bit
    patterns of sigmoid(hidden . gate_w) per row.  Defined exactly: the logit is the exact dot product rounded once to
    BF16, the gate is the sigmoid of that BF16 logit evaluated in FP64 and rounded once to BF16."""
    h = bf16_bits_to_f32(hidden_bits).astype(np.float64)
    g = bf16_bits_to_f32(gate_bits).astype(np.float64)
    logit = bf16_bits_to_f32(f64_to_bf16_bits(h @ g)).astype(np.float64)
    return f64_to_bf16_bits(1.0 / (1.0 + np.exp(-logit)))


def route_topk(logit_bits: np.ndarray, bias: np.ndarray | None = None):
    """-> ids int32 [T,8] (logit desc, id asc), weights f32 [T,8] renormalised softmax."""
    z = bf16_bits_to_f32(logit_bits)
    if bias is not None:
        z = (z + bias.astype(np.float32)[None, :]).astype(np.float32)
    order = np.argsort(-z, axis=1, kind="stable")[:, :TOPK]
    zmax = z.max(axis=1, keepdims=True)
    p = np.exp((z - zmax).astype(np.float32)).astype(np.float32)
    denom = np.zeros(z.shape[0], dtype=np.float32)
    for e in range(z.shape[1]):                # ascending-id FP32 sum
        denom = (denom + p[:, e]).astype(np.float32)
    prob = (p / denom[:, None]).astype(np.float32)
    sel = np.take_along_axis(prob, order, axis=1)
    s = np.zeros(z.shape[0], dtype=np.float32)
    for k in range(TOPK):                      # slot-order FP32 sum
        s = (s + sel[:, k]).astype(np.float32)
    return order.astype(np.int32), (sel / s[:, None]).astype(np.float32)


def append_shared(ids: np.ndarray, w: np.ndarray, shared_w: np.ndarray):
    t = ids.shape[0]
    ids9 = np.concatenate([ids, np.full((t, 1), N_ROUTED, np.int32)], axis=1)
    w9 = np.concatenate([w, shared_w.astype(np.float32).reshape(t, 1)], axis=1)
    return ids9, w9


def sort_pairs(ids: np.ndarray, n_experts: int = N_ROUTED):
    """Routed ids [T,8] -> perm[P] (pair index t*8+s, expert-major, stable),
    counts[E], offsets[E+1] (exclusive prefix sum)."""
    flat = ids.reshape(-1)
    perm = np.argsort(flat, kind="stable").astype(np.int32)
    counts = np.bincount(flat, minlength=n_experts).astype(np.int32)
    offsets = np.zeros(n_experts + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts)
    return perm, counts, offsets


# ----------------------------------------------------------------------------- quantisers
def quant_fp8_group128(x: np.ndarray):
    """FP32 [R,C] -> (E4M3 codes [R,C], FP32 scales [R,C/128])."""
    r, c = x.shape
    g = np.ascontiguousarray(x, dtype=np.float32).reshape(r, c // BLOCK, BLOCK)
    amax = np.maximum(np.abs(g).max(axis=2), AMAX_FLOOR).astype(np.float32)
    scale = (amax * INV_448).astype(np.float32)
    inv = (np.float32(1.0) / scale).astype(np.float32)
    q = e4m3_encode((g * inv[:, :, None]).astype(np.float32))
    return q.reshape(r, c), scale


def add_rmsnorm_group_quant(input_bits: np.ndarray, residual_bits: np.ndarray, weight: np.ndarray, epsilon: float = 1e-6):
    """Residual add + RMSNorm + per-128 FP8 quantisation, numerical id ``residual_add_fp32_rms_bf16_round_then_fp8_rne_fixed``
    of ``manifests/gfx950/tactics/fixed_assembly.json:754-786`` (ABI ``runtime/gfx950/group_quant/verify/group_quant_assembly_bridge.h:21-31``).
    The kernel is AMD assembly and its framework fallback (AITER ``add_rmsnorm_quant``) is third-party, so the order of the
    FP32 operations is restated here as: FP32 add, mean of squares rounded once to FP32 (the squares are summed exactly),
    ``inv = 1 / sqrt(var + eps)``, ``y = bf16((x * inv) * w)``, then the per-128 quantiser.  PARITY UNPINNED.
    Returns (output BF16 bits, residual_out BF16 bits, FP8 codes, scales [rows, C/128])."""
    x = (bf16_bits_to_f32(input_bits) + bf16_bits_to_f32(residual_bits)).astype(np.float32)
    var = ((x.astype(np.float64) ** 2).sum(axis=1) / x.shape[1]).astype(np.float32)
    inv = (np.float32(1.0) / np.sqrt((var + np.float32(epsilon)).astype(np.float32))).astype(np.float32)
    y_bits = f32_to_bf16_bits(((x * inv[:, None]).astype(np.float32) * weight.astype(np.float32)[None, :]).astype(np.float32))
    q, s = quant_fp8_group128(bf16_bits_to_f32(y_bits))
    return y_bits, f32_to_bf16_bits(x), q, s


def silu_mul_quant(gate_up: np.ndarray):
    """FP32 [R,1024] (gate | up) -> BF16-rounded silu(gate)*up -> per-128 FP8."""
    g = gate_up[:, :INTER].astype(np.float32)
    u = gate_up[:, INTER:].astype(np.float32)
    sig = (np.float32(1.0) / (np.float32(1.0) + np.exp(-g).astype(np.float32))).astype(np.float32)
    h = bf16_round(((g * sig).astype(np.float32) * u).astype(np.float32))
    q, s = quant_fp8_group128(h)
    return q, s, h


# ----------------------------------------------------------------------------- block-scaled GEMM
def blockscale_matmul(aq: np.ndarray, a_s: np.ndarray, wq: np.ndarray, w_s: np.ndarray) -> np.ndarray:
    """``out[r,n] = sum_kb (A_deq[r,kb] . W_deq[n,kb])``, K-blocks ascending, FP32.

    aq codes [R,K], a_s [R,K/128]; wq codes [N,K], w_s [N/128,K/128].
    """
    r, k = aq.shape
    n = wq.shape[0]
    a = (e4m3_decode(aq).reshape(r, k // BLOCK, BLOCK) * a_s[:, :, None]).astype(np.float32)
    w = e4m3_decode(wq).reshape(n // BLOCK, BLOCK, k // BLOCK, BLOCK)
    w = (w * w_s[:, None, :, None]).astype(np.float32).reshape(n, k // BLOCK, BLOCK)
    out = np.zeros((r, n), dtype=np.float32)
    for kb in range(k // BLOCK):
        out += a[:, kb, :] @ w[:, kb, :].T
    return out


def expert_mlp(aq, a_s, w13q, w13_s, w2q, w2_s):
    """One expert over its rows: gate_up -> SiLU*up requant -> down.  Returns
    (down FP32 [R,2048], intermediate codes [R,512], intermediate scales [R,4])."""
    g = blockscale_matmul(aq, a_s, w13q, w13_s)
    hq, h_s, _ = silu_mul_quant(g)
    return blockscale_matmul(hq, h_s, w2q, w2_s), hq, h_s


def combine(down: np.ndarray, w9: np.ndarray, partials: str = "f32") -> np.ndarray:
    """down FP32 [T,9,H], weights [T,9] -> BF16 bits [T,H]; slot-ascending FP32 sum.

    ``partials="f16"`` is the reference's prefill contract: each row is rounded to FP16 when it
    leaves the down projection (``kernels/gfx950/templates/moe/prefill/fused_splitk2/down_partial.inc:435-458``)
    and the reducer computes ``f32(partial) * weight`` slot ascending with one BF16 rounding
    (``kernels/gfx950/templates/moe/prefill/route_reduce_splitk2_f16.inc:107-118``)."""
    if partials == "f16":
        down = down.astype(np.float16).astype(np.float32)
    elif partials != "f32":
        raise ValueError("partials must be 'f32' or 'f16'")
    acc = np.zeros((down.shape[0], down.shape[2]), dtype=np.float32)
    for s in range(down.shape[1]):
        acc = (acc + (down[:, s, :] * w9[:, s, None]).astype(np.float32)).astype(np.float32)
    return f32_to_bf16_bits(acc)


def moe_layer(hidden_bits, router_bits, w13q, w13_s, w2q, w2_s, bias=None, shared_w=None,
              token_subset=None, external_topk=None, partials: str = "f32"):
    """Whole layer.  ``w13q`` etc. hold ``E'+1`` slabs, the last one the shared expert.
    With ``token_subset`` the GEMMs and the output cover only those tokens (routing,
    sort and quantisation are always complete).  Returns a dict of every tensor the
    GPU path exposes."""
    t = hidden_bits.shape[0]
    shared_slab = w13q.shape[0] - 1
    logits = router_logits(hidden_bits, router_bits)
    ids, w = external_topk if external_topk is not None else route_topk(logits, bias)
    shared_w = np.ones(t, np.float32) if shared_w is None else shared_w
    ids9, w9 = append_shared(ids, w, shared_w)
    perm, counts, offsets = sort_pairs(ids)
    aq, a_s = quant_fp8_group128(bf16_bits_to_f32(hidden_bits))
    toks = np.arange(t) if token_subset is None else np.asarray(token_subset)
    pos = -np.ones(t, dtype=np.int64)
    pos[toks] = np.arange(len(toks))
    down = np.zeros((len(toks), SLOTS, HIDDEN), dtype=np.float32)
    hq_all = np.zeros((len(toks), SLOTS, INTER), dtype=np.uint8)
    hs_all = np.zeros((len(toks), SLOTS, INTER // BLOCK), dtype=np.float32)
    for e in range(shared_slab):
        pairs = perm[offsets[e]:offsets[e + 1]]
        pt, ps = pairs // TOPK, pairs % TOPK
        keep = pos[pt] >= 0
        if not keep.any():
            continue
        pt, ps = pt[keep], ps[keep]
        d, hq, h_s = expert_mlp(aq[pt], a_s[pt], w13q[e], w13_s[e], w2q[e], w2_s[e])
        down[pos[pt], ps], hq_all[pos[pt], ps], hs_all[pos[pt], ps] = d, hq, h_s
    d, hq, h_s = expert_mlp(aq[toks], a_s[toks], w13q[shared_slab], w13_s[shared_slab],
                            w2q[shared_slab], w2_s[shared_slab])
    down[:, TOPK], hq_all[:, TOPK], hs_all[:, TOPK] = d, hq, h_s
    return {
        "logits": logits, "topk_ids": ids9, "topk_w": w9, "perm": perm, "counts": counts,
        "offsets": offsets, "a_fp8": aq, "a_scale": a_s, "h_fp8": hq_all, "h_scale": hs_all,
        "tokens": toks, "out": combine(down, w9[toks], partials), "down": down,
    }


# ----------------------------------------------------------------------------- MXFP4
E2M1_LUT = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], dtype=np.float64)
E2M1_THRESHOLDS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)


def mxfp4_dequant(packed: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """packed u8 [..., K/2] (low nibble = even k), E8M0 scales u8 [..., K/32] -> FP64 [..., K]."""
    low, high = packed & 15, packed >> 4
    lv = E2M1_LUT[low & 7] * np.where(low & 8, -1.0, 1.0)
    hv = E2M1_LUT[high & 7] * np.where(high & 8, -1.0, 1.0)
    vals = np.stack([lv, hv], axis=-1).reshape(*packed.shape[:-1], -1)
    scale = np.exp2(scales.astype(np.float64) - 127.0)
    return vals * np.repeat(scale, 32, axis=-1)


def mxfp4_quantize(w: np.ndarray):
    """FP32 [N,K] -> (packed u8 [N,K/2], E8M0 u8 [N,K/32])."""
    n, k = w.shape
    x = np.ascontiguousarray(w, dtype=np.float32).reshape(n, k // 32, 32)
    amax = np.abs(x).max(axis=2)
    exponent = np.ceil(np.log2(np.maximum(amax / np.float32(6.0), np.float32(2.0 ** -126)))).astype(np.int32)
    scale_byte = np.clip(exponent + 127, 1, 254).astype(np.uint8)
    scale = np.exp2(exponent.astype(np.float32)).astype(np.float32)
    norm = (np.abs(x) / scale[:, :, None]).astype(np.float32)
    mag = np.searchsorted(E2M1_THRESHOLDS, norm, side="left").astype(np.uint8)
    code = (mag | (np.signbit(x).astype(np.uint8) << 3)).reshape(n, k)
    return (code[:, 0::2] | (code[:, 1::2] << 4)).astype(np.uint8), scale_byte


def mxfp4_expand(packed: np.ndarray, scales: np.ndarray):
    """MXFP4 rows -> the FP8 operand format of the grouped GEMMs: E4M3 codes [rows, K] and one
    power-of-two FP32 scale per 128 x 128 tile [rows/128, K/128], plus the number of nonzero elements
    that E4M3 cannot hold exactly (scales inside a tile more than 15 binades apart).
    Per tile s_ref = max(scale byte) - 6, tile scale 2^(s_ref - 127), element = lut * 2^(s - s_ref)."""
    rows, k = packed.shape[0], packed.shape[1] * 2
    s = scales.astype(np.int32).reshape(rows // 128, 128, k // 128, 4)
    s_ref = s.max(axis=(1, 3)) - 6                                        # [rows/128, K/128]
    j = s - s_ref[:, None, :, None]                                       # <= 6
    low, high = packed & 15, packed >> 4
    code = np.stack([low, high], axis=-1).reshape(rows, k)
    mag = E2M1_LUT[code & 7] * np.where(code & 8, -1.0, 1.0)
    jj = np.repeat(j.reshape(rows, k // 32), 32, axis=1)
    vals = (mag * np.exp2(np.maximum(jj, -30).astype(np.float64))).astype(np.float32)
    inexact = int(np.count_nonzero(((code & 7) != 0) & (jj < -8)))
    return e4m3_encode(vals), np.exp2((s_ref - 127).astype(np.float64)).astype(np.float32), inexact


def parity_metrics(got_bits: np.ndarray, ref_bits: np.ndarray) -> dict:
    """Metric definitions of ``tests/gfx1151/test_netra_mxfp4_sgl_decode.py:137-152``."""
    g = bf16_bits_to_f32(got_bits).astype(np.float64)
    r = bf16_bits_to_f32(ref_bits).astype(np.float64)
    d = g - r
    return {"max_abs": float(np.abs(d).max()) if d.size else 0.0,
            "rel_l2": float(np.linalg.norm(d) / max(np.linalg.norm(r), 1e-30)),
            "exact_fraction": float((got_bits == ref_bits).mean()) if d.size else 1.0}

"""CPU tests: the checker against every pin that exists for this path, and the C restatement
against the numpy one."""
import numpy as np
import pytest
import torch

from netra_kernel_b200 import synth
from oracle import moe_ref as R
from tests import helpers


def test_constants_match_reference_assembly():
    # kernels/gfx950/templates/moe/decode/silu_quant.inc:40-41
    assert R.INV_448.view(np.uint32) == 0x3B124925
    assert R.AMAX_FLOOR.view(np.uint32) == 0x2EDBE6FF
    assert R.INV_448 == np.float32(1.0) / np.float32(448.0)
    assert R.AMAX_FLOOR == np.float32(1e-10)


def test_e4m3_codec_matches_torch_float8():
    g = torch.Generator().manual_seed(7)
    x = (torch.randn(400000, generator=g) * torch.exp(4 * torch.randn(400000, generator=g))).clamp(-448, 448)
    x[:12] = torch.tensor([0.0, -0.0, 448.0, -448.0, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -9, 2.0 ** -6,
                           0.0146484375, 447.0, 464.0, 3.0 * 2.0 ** -10]).clamp(-448, 448)
    want = x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(R.e4m3_encode(x.numpy()), want)
    codes = torch.arange(256, dtype=torch.uint8)
    dec = codes.view(torch.float8_e4m3fn).float().numpy()
    assert np.array_equal(np.nan_to_num(dec, nan=12345.0), np.nan_to_num(R.E4M3_TABLE, nan=12345.0))
    # saturation (the hardware conversion saturates, torch's CPU cast does not)
    assert R.e4m3_encode(np.array([1e9, -1e9, 465.0], np.float32)).tolist() == [0x7E, 0xFE, 0x7E]


def test_c_e4m3_encoder_matches_numpy(c_oracle):
    import ctypes
    c_oracle.moe_ref_e4m3_encode.restype = ctypes.c_uint8
    c_oracle.moe_ref_e4m3_encode.argtypes = [ctypes.c_float]
    g = np.random.default_rng(3)
    x = (g.standard_normal(20000) * np.exp(4 * g.standard_normal(20000))).astype(np.float32)
    got = np.array([c_oracle.moe_ref_e4m3_encode(float(v)) for v in x], np.uint8)
    assert np.array_equal(got, R.e4m3_encode(x))


def test_bf16_roundings_match_torch():
    g = torch.Generator().manual_seed(5)
    y = torch.randn(200000, generator=g)
    assert np.array_equal(R.f32_to_bf16_bits(y.numpy()), helpers.bits(y.to(torch.bfloat16)))
    # single rounding from FP64: a value that double rounding (via FP32) gets wrong
    x = np.array([1.0 + 2.0 ** -8 + 2.0 ** -30, 1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -8, -0.0, 0.0])
    assert R.f64_to_bf16_bits(x).tolist() == [0x3F81, 0x3F80, 0x3F82, 0x8000, 0x0000]
    yd = torch.randn(200000, generator=g, dtype=torch.float64)
    assert np.array_equal(R.f64_to_bf16_bits(yd.numpy()), helpers.bits(synth._bf16_from_f64(yd)))
    # non-finite and out-of-range sums keep their meaning instead of wrapping into finite patterns
    z = np.array([np.inf, -np.inf, 2.0 ** 128, -1e300, np.nan, 2.0 ** -127, -2.0 ** -130])
    want = [0x7F80, 0xFF80, 0x7F80, 0xFF80, 0x7FC0, 0x0000, 0x8000]
    assert R.f64_to_bf16_bits(z).tolist() == want
    assert helpers.bits(synth._bf16_from_f64(torch.from_numpy(z))).tolist() == want


def _stage_pins():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_stage_golden", helpers.GOLDEN / "make_stage_golden.py")
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    return gen, np.load(helpers.GOLDEN / "reference_stage_pins.npz")


def test_gemm_and_combine_arithmetic_matches_the_reference_exporters():
    """The fixture holds what the reference's own stage-1 / stage-2 exporters computed (run unmodified, see
    tests/golden/make_stage_golden.py) on operands this test regenerates from the same seeds.  The checker's block-scaled
    GEMM and combine follow the same arithmetic (dequantise both blocks, FP32 dot per K-block, K-blocks ascending; slot
    ascending weighted sum; one BF16 rounding): they may differ only by the summation order inside a 128-long FP32 dot,
    bounded here by 1e-5 of the row's magnitude."""
    gen, pins = _stage_pins()
    for case in range(gen.CASES):
        ops = gen.operands(case)
        assert bytes(pins[f"case{case}_operands_sha256"]).hex() == gen.operands_sha256(ops), "operands differ from the generator's"
        aq, a_s = R.quant_fp8_group128(R.bf16_bits_to_f32(helpers.bits(ops["hidden"])))
        w1, w1_s = helpers.u8(ops["w1"]), ops["w1_scale"].numpy()
        w2, w2_s = helpers.u8(ops["w2"]), ops["w2_scale"].numpy()
        # stage 1: slot s uses the slab of its expert (w1[s] here is the slab of slot s)
        got1 = np.stack([R.blockscale_matmul(aq, a_s, w1[s], w1_s[s])[0] for s in range(9)])
        want1 = pins[f"case{case}_stage1_f32"]
        scale1 = np.abs(want1).max(axis=1, keepdims=True)
        assert np.abs(got1 - want1).max() <= 1e-5 * scale1.max(), np.abs(got1 - want1).max()
        assert np.all(np.abs(got1 - want1) <= 1e-5 * scale1)
        # SiLU * up requantisation of the reference's stage-1 values reproduces the activation fed to its stage 2
        hq, h_s, _ = R.silu_mul_quant(want1)
        assert np.array_equal(hq, pins[f"case{case}_act_fp8"]) and np.array_equal(h_s, pins[f"case{case}_act_scale"])
        # stage 2 + combine
        down = np.stack([R.blockscale_matmul(hq[s:s + 1], h_s[s:s + 1], w2[s], w2_s[s])[0] for s in range(9)])[None]
        want2 = pins[f"case{case}_stage2_f32"]
        acc = np.zeros((1, 2048), np.float32)
        for s in range(9):
            acc = (acc + (down[:, s] * ops["topk_w"].numpy()[:, s, None]).astype(np.float32)).astype(np.float32)
        assert np.abs(acc - want2).max() <= 1e-5 * np.abs(want2).max()
        got_bits = R.combine(down, ops["topk_w"].numpy())
        m = R.parity_metrics(got_bits, pins[f"case{case}_stage2_bf16"])
        # BF16 results agree except where the FP32 sums straddle a rounding boundary
        assert m["exact_fraction"] >= 0.995 and m["max_abs"] <= 2.0 ** -8 * np.abs(want2).max() * 2, m


def test_router_logits_against_the_reference_exporter():
    """The reference's router semantic is torch's BF16 ``F.linear`` (unspecified FP32 order); the checker defines the logit
    as the exact dot product rounded once.  On the reference's own output for 96 x 256 logits the two agree except for a
    few values that sit on a rounding boundary, where they differ by exactly one BF16 step."""
    gen, pins = _stage_pins()
    hidden, weight = gen.router_operands()
    digest = __import__("hashlib").sha256(hidden.view(torch.uint8).numpy().tobytes() + weight.view(torch.uint8).numpy().tobytes()).digest()
    assert bytes(pins["router_operands_sha256"]) == digest
    want = pins["router_logits_bf16"]
    got = R.router_logits(helpers.bits(hidden), helpers.bits(weight))
    differ = got != want
    assert differ.mean() <= 1e-3, differ.mean()
    step = np.abs(got.astype(np.int32) - want.astype(np.int32))[differ]
    assert np.all(step == 1)


def test_mxfp4_dequant_matches_reference_vectors():
    data = np.load(helpers.GOLDEN / "mxfp4_dequant.npz")
    got = R.mxfp4_dequant(data["packed"], data["scales"])
    assert np.array_equal(got, data["values"])


def test_mxfp4_quantiser_round_trip_and_generator_agreement():
    g = torch.Generator().manual_seed(11)
    w = 0.02 * torch.randn(64, 256, generator=g)
    p_t, s_t = synth.quantize_mxfp4(w)
    p_n, s_n = R.mxfp4_quantize(w.numpy())
    assert np.array_equal(p_t.numpy(), p_n) and np.array_equal(s_t.numpy(), s_n)
    deq = R.mxfp4_dequant(p_n, s_n)
    # E2M1 with a power-of-two scale >= amax/6: error at most half the largest code gap (1.0) x scale
    scale = np.repeat(np.exp2(s_n.astype(np.float64) - 127.0), 32, axis=1)
    assert np.all(np.abs(deq - w.numpy()) <= 1.0 * scale + 1e-12)
    # representable values survive exactly
    exact = (R.E2M1_LUT[None, :] * np.array([[1.0], [-1.0]])).reshape(1, 16).repeat(2, axis=1).astype(np.float32)
    p, s = R.mxfp4_quantize(exact * 0.25)
    assert np.array_equal(R.mxfp4_dequant(p, s), (exact * 0.25).astype(np.float64))


def test_mxfp4_expansion_to_fp8_tiles_is_exact_within_fifteen_binades():
    """The load-time expansion (E4M3 codes x one power-of-two scale per 128 x 128 tile) must reproduce the
    reference dequantiser exactly, and must count what it cannot hold."""
    g = torch.Generator().manual_seed(12)
    w = 0.02 * torch.randn(256, 512, generator=g)
    w[:, 130:160] *= 2.0 ** -9                       # one scale group far below its neighbours, still inside 15 binades
    packed, scales = R.mxfp4_quantize(w.numpy())
    codes, tile_scale, inexact = R.mxfp4_expand(packed, scales)
    assert inexact == 0 and codes.shape == (256, 512) and tile_scale.shape == (2, 4)
    got = R.e4m3_decode(codes).astype(np.float64) * np.repeat(np.repeat(tile_scale.astype(np.float64), 128, axis=0), 128, axis=1)
    assert np.array_equal(got, R.mxfp4_dequant(packed, scales))
    assert np.all(np.log2(tile_scale) == np.round(np.log2(tile_scale)))      # powers of two
    scales2 = scales.copy()
    scales2[5, 1] = scales2[5, 0] - 20               # 20 binades below its tile: rounded away and counted
    _, _, inexact2 = R.mxfp4_expand(packed, scales2)
    assert inexact2 == np.count_nonzero(np.stack([packed[5, 16:32] & 7, (packed[5, 16:32] >> 4) & 7]))


def test_topk_tie_break_and_renormalisation():
    logits = np.zeros((2, 256), np.float32)
    logits[0, [5, 9, 200]] = 2.0             # three-way tie for the top: ids ascending
    logits[0, 100] = 3.0
    logits[1, :] = -1.0                      # everything ties: first eight ids
    ids, w = R.route_topk(R.f32_to_bf16_bits(logits))
    assert ids[0].tolist() == [100, 5, 9, 200, 0, 1, 2, 3]
    assert ids[1].tolist() == list(range(8))
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-6)
    assert np.allclose(w[1], 0.125)
    # bias is added in FP32 before selection
    bias = np.zeros(256, np.float32); bias[77] = 10.0
    ids_b, _ = R.route_topk(R.f32_to_bf16_bits(logits), bias)
    assert ids_b[0, 0] == 77 and ids_b[1, 0] == 77


def test_sort_is_stable_and_consistent():
    g = np.random.default_rng(0)
    ids = g.integers(0, 256, size=(300, 8)).astype(np.int32)
    ids[:, 0] = 3                             # a heavy expert
    perm, counts, offsets = R.sort_pairs(ids)
    flat = ids.reshape(-1)
    assert np.array_equal(np.sort(perm), np.arange(2400))
    assert np.all(np.diff(flat[perm]) >= 0)
    for e in (3, 17, 255):
        seg = perm[offsets[e]:offsets[e + 1]]
        assert np.all(np.diff(seg) > 0) and np.all(flat[seg] == e)
    assert offsets[-1] == 2400 and counts.sum() == 2400
    # empty input segment / single token
    perm1, counts1, _ = R.sort_pairs(np.arange(8, dtype=np.int32)[None, :])
    assert perm1.tolist() == list(range(8)) and counts1[:8].tolist() == [1] * 8


def test_quantiser_edge_cases():
    x = np.zeros((2, 256), np.float32)
    x[1, :128] = 448.0 * 3
    x[1, 128] = -1e-12
    q, s = R.quant_fp8_group128(x)
    assert np.all(q[0] == 0) and np.all(s[0] == R.AMAX_FLOOR * R.INV_448)
    assert np.all(q[1, :128] == 0x7E)          # amax maps to 448 exactly
    assert s[1, 0] == np.float32(1344.0) * R.INV_448


def test_python_checker_reproduces_golden_layer(expert_weights):
    data = np.load(helpers.GOLDEN / "moe_layer_t16.npz")
    hidden, router_w, _ = synth.make_activations(16)
    w13, w13_s, w2, w2_s = helpers.np_weights(expert_weights)
    ref = R.moe_layer(helpers.bits(hidden), helpers.bits(router_w), w13, w13_s, w2, w2_s)
    for key in ("logits", "topk_ids", "perm", "counts", "offsets", "a_fp8", "h_fp8", "out"):
        assert np.array_equal(ref[key], data[key]), key
    assert np.array_equal(ref["topk_w"], data["topk_w"])


def test_c_checker_matches_python_checker(expert_weights, c_oracle):
    data = np.load(helpers.GOLDEN / "moe_layer_t16.npz")
    hidden, router_w, _ = synth.make_activations(16)
    w13, w13_s, w2, w2_s = helpers.np_weights(expert_weights)
    got = helpers.c_layer(c_oracle, helpers.bits(hidden), helpers.bits(router_w), w13, w13_s, w2, w2_s)
    for key in ("logits", "topk_ids", "perm", "counts", "a_fp8"):
        assert np.array_equal(got[key], data[key]), key
    assert np.array_equal(got["offsets"], data["offsets"])
    assert np.allclose(got["topk_w"], data["topk_w"], rtol=2e-6, atol=1e-7)
    assert np.array_equal(got["a_scale"], data["a_scale"])
    # the two restatements differ only in FP32 summation order inside a K-block
    assert (got["h_fp8"] != data["h_fp8"]).mean() < 1e-3
    m = R.parity_metrics(got["out"], data["out"])
    assert m["max_abs"] <= 4e-3 and m["rel_l2"] <= 5e-4, m


def test_c_checker_with_bias_and_shared_weight(expert_weights, c_oracle):
    hidden, router_w, _ = synth.make_activations(24)
    bias = synth.zipf_bias(1.5).numpy()
    shared_w = np.linspace(0.0, 1.0, 24).astype(np.float32)
    w13, w13_s, w2, w2_s = helpers.np_weights(expert_weights)
    ref = R.moe_layer(helpers.bits(hidden), helpers.bits(router_w), w13, w13_s, w2, w2_s, bias=bias, shared_w=shared_w)
    got = helpers.c_layer(c_oracle, helpers.bits(hidden), helpers.bits(router_w), w13, w13_s, w2, w2_s, bias, shared_w)
    assert np.array_equal(got["topk_ids"], ref["topk_ids"]) and np.array_equal(got["perm"], ref["perm"])
    assert ref["counts"].max() >= 10             # the bias really skews the load
    m = R.parity_metrics(got["out"], ref["out"])
    assert m["max_abs"] <= 4e-3 and m["rel_l2"] <= 5e-4, m


def test_zipf_bias_reaches_ten_times_mean_load():
    hidden, router_w, _ = synth.make_activations(8192)
    load = synth.routed_load(hidden, router_w, synth.zipf_bias(synth.ZIPF_ALPHA_T8192)).double()
    ratio = (load.max() / load.mean()).item()
    assert 9.5 <= ratio <= 10.5, ratio
    assert int(load.argmax()) == 0 and int(load.sum()) == 8192 * 8

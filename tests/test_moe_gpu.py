"""GPU parity tests: the sm_100a path through the C ABI against the CPU checker on identical
seeded operands.  Integer results (logits bits, ids, permutation, counts, offsets, input FP8
codes) must be bit-exact; the BF16 output must be within max-abs 2e-2 and relative-L2 5e-3."""
import os

import numpy as np
import pytest
import torch

from netra_kernel_b200 import synth
from oracle import moe_ref as R
from tests import helpers

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu_weights(expert_weights):
    return tuple(t.cuda() for t in expert_weights)


def make_layer(gpu_weights, router_w, max_tokens, bias=None, tiled=True):
    from netra_kernel_b200.moe import RoutedMoELayer
    w13, w13_s, w2, w2_s = gpu_weights
    return RoutedMoELayer(router_w.cuda(), w13, w13_s, w2, w2_s, max_tokens,
                          None if bias is None else bias.cuda(), tiled=tiled)


def run_layer(layer, hidden, shared_w=None):
    sw = None if shared_w is None else torch.from_numpy(shared_w).cuda()
    out = layer(hidden.cuda(), sw)
    torch.cuda.synchronize()
    layer.check_status()
    inter = {k: v.cpu() for k, v in layer.intermediates(hidden.shape[0]).items()}
    return out.cpu(), inter


def f32_of(bits: np.ndarray) -> np.ndarray:
    return R.bf16_bits_to_f32(bits).astype(np.float64)


def check_logits(inter, ref, tokens, bound=2.5e-4):
    """Up to 1,024 rows (and in router modes 1 and 2) every logit is the exactly rounded dot product.  Above, the default
    router guarantees that for every logit that can reach the top 8 - checked here on the selected ones - while the rest
    keep the rounded tensor-core value: within the accumulation bound (2^-18 |h| |w|, about 1.6e-4 for the benchmark
    distributions) plus one BF16 spacing of the exact rounding."""
    got, want = helpers.bits(inter["logits"]), ref["logits"]
    if tokens <= 1024:
        assert np.array_equal(got, want), "router logits must be bit-exact"
        return
    g, w = f32_of(got), f32_of(want)
    assert np.all(np.abs(g - w) <= bound + np.abs(w) * 2.0 ** -7), "a router logit is outside the documented bound"
    ids = ref["topk_ids"][:, :8]
    assert np.array_equal(np.take_along_axis(got, ids, 1), np.take_along_axis(want, ids, 1)), "selected logits must be bit-exact"


def check_against(ref, out, inter, tokens, *, subset=None):
    pairs = tokens * 8
    check_logits(inter, ref, tokens)
    assert np.array_equal(inter["topk_ids"].numpy(), ref["topk_ids"]), "top-k ids must be bit-exact"
    assert np.array_equal(inter["perm"].numpy(), ref["perm"]), "permutation must be bit-exact"
    assert np.array_equal(inter["counts"].numpy(), ref["counts"])
    assert np.array_equal(inter["offsets"].numpy()[:257], ref["offsets"][:257])
    assert inter["offsets"][257].item() == pairs + tokens
    inv = inter["inv_perm"].numpy()
    assert np.array_equal(inv[ref["perm"]], np.arange(pairs))
    np.testing.assert_allclose(inter["topk_w"].numpy(), ref["topk_w"], rtol=2e-6, atol=1e-7)
    # input quantisation: rows [pairs, pairs+tokens) are token order, rows [0, pairs) the gather
    a = inter["a_fp8"].numpy()
    assert np.array_equal(a[pairs:], ref["a_fp8"]), "input FP8 codes must be bit-exact"
    assert np.array_equal(inter["a_scale"].numpy()[pairs:], ref["a_scale"])
    assert np.array_equal(a[:pairs], ref["a_fp8"][ref["perm"] // 8])
    toks = np.arange(tokens) if subset is None else np.asarray(subset)
    # intermediate FP8 codes: slot order in the checker, sorted rows on the GPU
    h = inter["h_fp8"].numpy()
    pos = np.concatenate([inv.reshape(tokens, 8), (pairs + np.arange(tokens))[:, None]], axis=1)[toks]
    got_h = h[pos]
    mism = (got_h != ref["h_fp8"]).mean()
    assert mism < 2e-3, f"intermediate FP8 code mismatch fraction {mism}"
    m = R.parity_metrics(helpers.bits(out)[toks], ref["out"])
    assert m["max_abs"] <= helpers.MAX_ABS and m["rel_l2"] <= helpers.REL_L2, m
    return m


def test_layer_t16_matches_golden_fixture(gpu_weights):
    data = dict(np.load(helpers.GOLDEN / "moe_layer_t16.npz"))
    hidden, router_w, _ = synth.make_activations(16)
    layer = make_layer(gpu_weights, router_w, 16)
    assert layer.launches_per_call(16) == 7 and layer.launches_per_call(2048) == 9
    out, inter = run_layer(layer, hidden)
    m = check_against(data, out, inter, 16)
    assert m["rel_l2"] < 1e-3


@pytest.mark.parametrize("tiled", [True, False])
def test_layer_t256_decode_matches_c_checker(gpu_weights, expert_weights, c_oracle, tiled):
    hidden, router_w, _ = synth.make_activations(256)
    ref = helpers.c_layer(c_oracle, helpers.bits(hidden), helpers.bits(router_w), *helpers.np_weights(expert_weights))
    layer = make_layer(gpu_weights, router_w, 256, tiled=tiled)
    out, inter = run_layer(layer, hidden)
    check_against(ref, out, inter, 256)
    assert int((ref["counts"] > 0).sum()) == 256      # every expert is hit at T=256


@pytest.mark.parametrize("tokens", [1, 7, 129])
def test_ragged_token_counts(gpu_weights, expert_weights, c_oracle, tokens):
    hidden, router_w, _ = synth.make_activations(tokens, seed=20 + tokens)
    shared_w = np.linspace(0.25, 1.0, tokens).astype(np.float32)
    ref = helpers.c_layer(c_oracle, helpers.bits(hidden), helpers.bits(router_w), *helpers.np_weights(expert_weights),
                          shared_w=shared_w)
    layer = make_layer(gpu_weights, router_w, 256)        # capacity above the call size
    out, inter = run_layer(layer, hidden, shared_w)
    check_against(ref, out, inter, tokens)


def test_skewed_routing_with_empty_and_overfull_experts(gpu_weights, expert_weights):
    """Strong Zipf bias: most experts empty, the hottest far above 128 rows (several work items)."""
    tokens = 1024
    hidden, router_w, _ = synth.make_activations(tokens, seed=5)
    bias = synth.zipf_bias(3.0)
    subset = np.arange(0, tokens, 37)
    ref = R.moe_layer(helpers.bits(hidden), helpers.bits(router_w), *helpers.np_weights(expert_weights),
                      bias=bias.numpy(), token_subset=subset)
    assert (ref["counts"] == 0).sum() > 50 and ref["counts"].max() > 512
    layer = make_layer(gpu_weights, router_w, tokens, bias)
    out, inter = run_layer(layer, hidden)
    check_against(ref, out, inter, tokens, subset=subset)


def test_prefill_t8192_zipf_sampled_tokens(gpu_weights, expert_weights):
    tokens = 8192
    hidden, router_w, bias = synth.make_activations(tokens, synth.ZIPF_ALPHA_T8192)
    subset = np.arange(5, tokens, 257)
    ref = R.moe_layer(helpers.bits(hidden), helpers.bits(router_w), *helpers.np_weights(expert_weights),
                      bias=bias.numpy(), token_subset=subset)
    layer = make_layer(gpu_weights, router_w, tokens, bias)
    out, inter = run_layer(layer, hidden)
    check_against(ref, out, inter, tokens, subset=subset)
    # size-independent properties at full size: permutation is a bijection, expert-major, stable
    perm = inter["perm"].numpy()
    flat = inter["topk_ids"].numpy()[:, :8].reshape(-1)
    assert np.array_equal(np.sort(perm), np.arange(tokens * 8))
    keys = flat[perm].astype(np.int64) * (tokens * 8) + perm
    assert np.all(np.diff(keys) > 0)
    assert np.array_equal(np.bincount(flat, minlength=256), inter["counts"].numpy())


@pytest.mark.parametrize("tokens,alpha", [(1024, 0.0), (1031, 0.5), (2048, 0.0), (3000, 1.2), (1500, 3.0), (4096, 0.0)])
def test_token_major_and_swap_ab_gemms_agree_bitwise(gpu_weights, tokens, alpha):
    """From 1,024 tokens the layer runs the token-major GEMMs (128 token rows x 256 weight rows per MMA); the
    swap-AB kernels computing the same rows must give the same intermediate codes, scales, FP32 rows and output."""
    hidden, router_w, bias = synth.make_activations(tokens, alpha or None, seed=9)
    layer = make_layer(gpu_weights, router_w, tokens, bias)
    out_tm, inter_tm = run_layer(layer, hidden)
    layer.set_gemm_mode(1)
    out_sw, inter_sw = run_layer(layer, hidden)
    rows = tokens * 9
    for key in ("h_fp8", "h_scale", "down"):
        assert torch.equal(inter_tm[key][:rows], inter_sw[key][:rows]), key
    assert torch.equal(out_tm.view(torch.int16), out_sw.view(torch.int16))
    counts = inter_tm["counts"].numpy()
    if alpha >= 1.0:
        assert counts.max() > 256 and counts.min() < 16      # several 128-row tiles for the hottest, ragged tails elsewhere
    if alpha >= 3.0:
        assert (counts == 0).sum() > 50                      # most experts empty: groups without any work item


def _router_case(kind: str, tokens: int, seed: int):
    """Hidden rows and router weights for the router comparison: the benchmark distributions, and rows built to stress the
    error bound (a wide dynamic range across and inside rows, zero rows, exact cancellation, BF16 subnormals)."""
    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(tokens, 2048, generator=g)
    w = 0.02 * torch.randn(256, 2048, generator=g)
    if kind == "wide":
        hidden *= torch.exp2(torch.randint(-20, 21, (tokens, 1), generator=g).float())      # rows from 1e-6 to 1e6
        hidden[:, ::17] *= 64.0                                                                # outlier channels
        w *= torch.exp2(torch.randint(-6, 7, (256, 1), generator=g).float())
        hidden[3] = 0.0
        hidden[5, 1:] = 0.0                                                                    # one product decides the logit
        hidden[7, :1024] = hidden[7, 1024:]                                                    # exact cancellation against ...
        w[9, :1024] = -w[9, 1024:]                                                             # ... this router row: logit 0
        hidden[11] = 1e-39                                                                     # BF16 subnormals
    return hidden.to(torch.bfloat16), w.to(torch.bfloat16)


@pytest.mark.parametrize("kind,tokens,seed", [("bench", 8192, 0), ("bench", 1025, 1), ("bench", 16384, 2), ("wide", 4096, 3),
                                               ("wide", 1300, 4)])
def test_tensor_core_router_against_the_fp64_router(gpu_weights, kind, tokens, seed):
    """Above 1,024 rows the router runs as a BF16 tensor-core pass plus FP64 recomputation of logits whose rounding the
    FP32 value cannot decide.  Mode 2 recomputes every such logit: all logits must equal the FP64 router's (mode 1), i.e.
    the correctly rounded exact dot products.  Mode 0 (default) recomputes only those that can reach the top 8: ids,
    weights, permutation and quantised rows must still be identical, the selected logits exact, every other logit within
    the bound plus one BF16 spacing.  The measured accumulation error must stay well inside the bound the recomputation test assumes
    (kRouterErrScale = 2^-18 of |h| |w|)."""
    hidden, router_w = _router_case(kind, tokens, seed)
    bias = synth.zipf_bias(0.5).cuda() if seed % 2 else None
    layer = make_layer(gpu_weights, router_w, tokens, None if bias is None else bias.cpu())
    h = hidden.cuda()
    out = torch.empty_like(h)
    results = {}
    for mode in (1, 2, 0):
        layer.set_router_mode(mode)
        before = layer.router_stats()[0]
        for stage in range(5):
            layer.launch_stage(stage, h, out)
        torch.cuda.synchronize()
        layer.check_status()
        inter = layer.intermediates(tokens)
        results[mode] = {k: inter[k].clone() for k in ("logits", "topk_ids", "topk_w", "perm", "counts", "a_fp8", "a_scale",
                                                       "logits_f32", "wnorm")}
        results[mode]["fixed"] = layer.router_stats()[0] - before
    ref, full, fast = results[1], results[2], results[0]
    assert torch.equal(full["logits"].view(torch.int16), ref["logits"].view(torch.int16)), "mode 2 logits differ from the FP64 router"
    for key in ("topk_ids", "topk_w", "perm", "counts", "a_fp8", "a_scale"):
        assert torch.equal(full[key], ref[key]), ("mode 2", key)
        assert torch.equal(fast[key], ref[key]), ("mode 0", key)
    assert ref["fixed"] == 0 and 0 < fast["fixed"] < full["fixed"]
    ids = ref["topk_ids"][:, :8].long()
    assert torch.equal(torch.gather(fast["logits"].view(torch.int16), 1, ids), torch.gather(ref["logits"].view(torch.int16), 1, ids))
    # the FP64 router against the CPU checker on a sample of rows (all rows are covered by the equalities above)
    rows = np.arange(0, tokens, max(1, tokens // 64))
    want = R.router_logits(helpers.bits(hidden)[rows], helpers.bits(router_w))
    assert np.array_equal(helpers.bits(ref["logits"].cpu())[rows], want)
    # measured error of the tensor-core pass relative to the product of the norms (rows whose bound underflows FP32 are
    # always recomputed and are left out of the measurement)
    exact = h.double() @ router_w.cuda().double().T
    hn = h.double().norm(dim=1, keepdim=True)
    wn = router_w.cuda().double().norm(dim=1)[None, :]
    scale = hn * wn
    err = torch.where(scale > 1e-30, (fast["logits_f32"].double() - exact).abs() / scale.clamp_min(1e-30), torch.zeros_like(scale))
    worst = float(err.max())
    # mode 0 leaves the logits that cannot be selected at the rounded tensor-core value: inside bound + one BF16 spacing
    gap = (fast["logits"].double() - ref["logits"].double()).abs()
    allowed = 1.01 * 2.0 ** -18 * scale + ref["logits"].double().abs() * 2.0 ** -7 + 1e-37
    assert bool(torch.all(gap <= allowed))
    off = int((fast["logits"].view(torch.int16) != ref["logits"].view(torch.int16)).sum())
    print(f"router[{kind},{tokens}]: max |f32 - exact| / (|h||w|) = {worst:.3e} (bound 2^-18 = {2.0 ** -18:.3e}); recomputed "
          f"{fast['fixed']} (mode 0) / {full['fixed']} (mode 2) of {tokens * 256} logits; "
          f"{off} logits differ from the exact rounding in mode 0 (none of them selectable)")
    assert worst <= 2.0 ** -20, "the tensor-core accumulation error is within a factor 4 of the bound: widen kRouterErrScale"
    assert torch.all(full["wnorm"].double() >= wn[0])


def test_prefill_fp16_partial_rows_tactic(gpu_weights, expert_weights):
    """The prefill contract of the reference: FP16 partial rows out of the down projection, reduced as f32(p) * w in slot
    order.  Against the checker run with the same rounding point, and against the FP32-row tactic of the same layer."""
    tokens = 8192
    hidden, router_w, bias = synth.make_activations(tokens, synth.ZIPF_ALPHA_T8192)
    subset = np.arange(3, tokens, 311)
    ref = R.moe_layer(helpers.bits(hidden), helpers.bits(router_w), *helpers.np_weights(expert_weights),
                      bias=bias.numpy(), token_subset=subset, partials="f16")
    layer = make_layer(gpu_weights, router_w, tokens, bias)
    out32, inter32 = run_layer(layer, hidden)
    down32 = inter32["down"][: tokens * 9].clone()
    layer.set_partial_format(1)
    out16, inter16 = run_layer(layer, hidden)
    m = check_against(ref, out16, inter16, tokens, subset=subset)
    assert m["rel_l2"] < 2e-3
    # every FP16 row is the FP32 row of the other tactic rounded once
    assert torch.equal(inter16["down_f16"][: tokens * 9], down32.to(torch.float16))
    m2 = R.parity_metrics(helpers.bits(out16), helpers.bits(out32))
    assert m2["max_abs"] <= 8e-3 and m2["rel_l2"] <= 1e-3, m2
    # a call below the token-major threshold keeps FP32 rows under the same setting
    small, _, _ = synth.make_activations(64, seed=3)
    ref_small = layer(small.cuda()).clone()
    layer.set_partial_format(0)
    assert torch.equal(layer(small.cuda()).view(torch.int16), ref_small.view(torch.int16))


@pytest.mark.parametrize("tokens,alpha", [(1, 0.0), (15, 0.0), (256, 0.0), (700, 3.0), (1024, 0.5)])
def test_routing_front_end_in_one_launch_equals_the_three_launches(gpu_weights, tokens, alpha):
    """The recorded tactic that runs router, top-8 + quantisation and sort as one launch whose blocks hand over by
    last-arriver counters.  Logits, ids, weights, quantised rows, permutation, counts and offsets must equal the three-launch form bit
    for bit, call after call (the counters return to zero), with a shared-expert weight and a bias in play."""
    hidden, router_w, bias = synth.make_activations(tokens, alpha or None, seed=41)
    shared_w = np.linspace(0.5, 1.5, tokens).astype(np.float32)
    layer = make_layer(gpu_weights, router_w, 1024, bias)
    three = layer.launches_per_call(tokens)
    out_b, inter_b = run_layer(layer, hidden, shared_w)
    layer.set_front_mode(1)
    assert layer.launches_per_call(tokens) == three - 2
    fused = [run_layer(layer, hidden, shared_w) for _ in range(3)]
    pairs = tokens * 8
    for out_a, inter_a in fused:
        for key in ("logits", "topk_ids", "topk_w", "perm", "inv_perm", "counts"):
            assert torch.equal(inter_a[key], inter_b[key]), key
        assert torch.equal(inter_a["offsets"][:258], inter_b["offsets"][:258])
        assert torch.equal(inter_a["a_fp8"][pairs:pairs + tokens], inter_b["a_fp8"][pairs:pairs + tokens])
        assert torch.equal(inter_a["a_scale"][pairs:pairs + tokens], inter_b["a_scale"][pairs:pairs + tokens])
        assert torch.equal(out_a.view(torch.int16), out_b.view(torch.int16))


@pytest.mark.parametrize("tokens,alpha", [(1, 0.0), (16, 0.0), (256, 0.0), (700, 3.0), (1000, 0.0)])
def test_both_projections_in_one_launch_equal_the_two_launch_form(gpu_weights, tokens, alpha):
    """The recorded tactic that runs gate_up and down in one launch (the down half waits per expert chunk for the gate_up
    half's rows): every intermediate and the output must equal the two-launch form bit for bit, call after call (the
    arrival counters are zeroed by the gather launch each time), also with most experts empty and one far above a chunk."""
    hidden, router_w, bias = synth.make_activations(tokens, alpha or None, seed=31)
    layer = make_layer(gpu_weights, router_w, 1024, bias)
    two = layer.launches_per_call(tokens)
    out_b, inter_b = run_layer(layer, hidden)
    layer.set_gemm_mode(2)
    assert layer.launches_per_call(tokens) == two - 1
    outs = []
    for _ in range(3):
        out_a, inter_a = run_layer(layer, hidden)
        outs.append(out_a)
    rows = tokens * 9
    for key in ("h_fp8", "h_scale", "down"):
        assert torch.equal(inter_a[key][:rows], inter_b[key][:rows]), key
    for out_a in outs:
        assert torch.equal(out_a.view(torch.int16), out_b.view(torch.int16))


def test_token_rows_gathered_inside_the_gemm_give_the_same_bytes(gpu_weights):
    """The recorded tactic that skips the expert-sorted copy: gate_up (token-major form, and swap-AB form at decode sizes)
    fetches its rows from token order with four-row TMA gathers.  Intermediates and output must equal the default form's
    bit for bit; one launch fewer."""
    for tokens, alpha in ((2048, 0.0), (1500, 3.0), (256, 0.0), (37, 2.0), (1, 0.0)):
        hidden, router_w, bias = synth.make_activations(tokens, alpha or None, seed=12)
        layer = make_layer(gpu_weights, router_w, tokens, bias)
        out_a, inter_a = run_layer(layer, hidden)
        launches = layer.launches_per_call(tokens)
        layer.set_row_gather(True)
        assert layer.launches_per_call(tokens) == launches - 1
        layer.intermediates(tokens)["a_fp8"][: tokens * 8].zero_()          # nothing may read the sorted copy now
        out_b, inter_b = run_layer(layer, hidden)
        rows = tokens * 9
        for key in ("h_fp8", "h_scale", "down"):
            assert torch.equal(inter_a[key][:rows], inter_b[key][:rows]), key
        assert torch.equal(out_a.view(torch.int16), out_b.view(torch.int16))
        assert not inter_b["a_fp8"][: tokens * 8].any()


def test_mxfp4_expansion_kernel_and_layer(expert_weights):
    """MXFP4 expert weights (the reference's quantiser) expanded on the GPU into FP8 tiles: the kernel must equal
    the CPU restatement bit for bit, the expansion must be exact, and the layer on the expanded weights must
    match the checker run on the same operands."""
    from netra_kernel_b200.moe import RoutedMoELayer, expand_mxfp4
    g = torch.Generator().manual_seed(21)
    slabs, tokens = 257, 64
    # a handful of distinct FP32 slabs reused cyclically keeps the host-side quantisation cheap
    base13 = [0.02 * torch.randn(1024, 2048, generator=g) for _ in range(3)]
    base2 = [0.02 * torch.randn(2048, 512, generator=g) for _ in range(3)]
    q13 = [synth.quantize_mxfp4(w) for w in base13]
    q2 = [synth.quantize_mxfp4(w) for w in base2]
    p13 = torch.stack([q13[e % 3][0] for e in range(slabs)]).cuda()
    s13 = torch.stack([q13[e % 3][1] for e in range(slabs)]).cuda()
    p2 = torch.stack([q2[e % 3][0] for e in range(slabs)]).cuda()
    s2 = torch.stack([q2[e % 3][1] for e in range(slabs)]).cuda()
    w13, w13_s, bad13 = expand_mxfp4(p13, s13)
    w2, w2_s, bad2 = expand_mxfp4(p2, s2)
    torch.cuda.synchronize()
    assert bad13 == 0 and bad2 == 0
    for e in range(3):                                  # kernel == CPU restatement, and exact against the reference dequantiser
        codes, tile_scale, _ = R.mxfp4_expand(q13[e][0].numpy(), q13[e][1].numpy())
        assert np.array_equal(w13[e].view(torch.uint8).cpu().numpy(), codes)
        assert np.array_equal(w13_s[e].cpu().numpy(), tile_scale)
        deq = R.e4m3_decode(codes).astype(np.float64) * np.repeat(np.repeat(tile_scale.astype(np.float64), 128, 0), 128, 1)
        assert np.array_equal(deq, R.mxfp4_dequant(q13[e][0].numpy(), q13[e][1].numpy()))
    codes2, tile2, _ = R.mxfp4_expand(q2[1][0].numpy(), q2[1][1].numpy())
    assert np.array_equal(w2[1].view(torch.uint8).cpu().numpy(), codes2) and np.array_equal(w2_s[1].cpu().numpy(), tile2)
    hidden, router_w, _ = synth.make_activations(tokens, seed=6)
    layer = RoutedMoELayer(router_w.cuda(), w13, w13_s, w2, w2_s, tokens)
    out, inter = run_layer(layer, hidden)
    ref = R.moe_layer(helpers.bits(hidden), helpers.bits(router_w), w13.view(torch.uint8).cpu().numpy(), w13_s.cpu().numpy(),
                      w2.view(torch.uint8).cpu().numpy(), w2_s.cpu().numpy())
    check_against(ref, out, inter, tokens)


def test_native_mxfp4_layer_streams_four_bit_weights(expert_weights):
    """The native MXFP4 tactic: the packed E2M1 slabs and E8M0 scales are only re-ordered at load (checked byte for byte
    against the layout rule) and multiplied on the block-scaled tensor-core path.  The layer must match the checker run on
    the exactly expanded weights within the output gates, route identically, and agree with the expansion path on nearly
    every intermediate FP8 code (both sum the same exact products; only the FP32 summation order differs)."""
    from netra_kernel_b200.moe import RoutedMoELayer, expand_mxfp4, pack_mxfp4
    g = torch.Generator().manual_seed(22)
    slabs = 257
    base13 = [0.02 * torch.randn(1024, 2048, generator=g) for _ in range(3)]
    base2 = [0.02 * torch.randn(2048, 512, generator=g) for _ in range(3)]
    base13[1][:, 512:1024] *= 2.0 ** -9            # scale bytes that differ widely inside one tile
    q13 = [synth.quantize_mxfp4(w) for w in base13]
    q2 = [synth.quantize_mxfp4(w) for w in base2]
    p13 = torch.stack([q13[e % 3][0] for e in range(slabs)]).cuda()
    s13 = torch.stack([q13[e % 3][1] for e in range(slabs)]).cuda()
    p2 = torch.stack([q2[e % 3][0] for e in range(slabs)]).cuda()
    s2 = torch.stack([q2[e % 3][1] for e in range(slabs)]).cuda()
    # the load-time re-ordering, against its definition: W13 blocks in (slab, channel tile, K-block, gate | up) order,
    # W2 blocks in (tile pair, K-block, tile of the pair) order; inside a scale atom row r sits at 16 * (r % 32) + 4 * (r / 32)
    codes, atoms = pack_mxfp4(p13[:2], s13[:2], paired_half_rows=512)
    codes2, atoms2 = pack_mxfp4(p2[:1], s2[:1], paired_half_rows=128)
    torch.cuda.synchronize()
    src_c = p13[:2].cpu().numpy().reshape(2, 2, 4, 128, 16, 64)                    # [slab, half, tile, r, kb, 64]
    assert np.array_equal(codes.cpu().numpy().reshape(2, 4, 16, 2, 128, 64), src_c.transpose(0, 2, 4, 1, 3, 5))
    src_s = s13[:2].cpu().numpy().reshape(2, 2, 4, 4, 32, 16, 4)                   # [slab, half, tile, r / 32, r % 32, kb, 4]
    assert np.array_equal(atoms.cpu().numpy().reshape(2, 4, 16, 2, 32, 4, 4), src_s.transpose(0, 2, 5, 1, 4, 3, 6))
    src_c2 = p2[:1].cpu().numpy().reshape(8, 2, 128, 4, 64)                        # [tile pair, tile of the pair, r, kb, 64]
    assert np.array_equal(codes2.cpu().numpy().reshape(8, 4, 2, 128, 64), src_c2.transpose(0, 3, 1, 2, 4))
    src_s2 = s2[:1].cpu().numpy().reshape(8, 2, 4, 32, 4, 4)                       # [pair, tile, r / 32, r % 32, kb, 4]
    assert np.array_equal(atoms2.cpu().numpy().reshape(8, 4, 2, 32, 4, 4), src_s2.transpose(0, 4, 1, 3, 2, 5))
    w13, w13_s, bad13 = expand_mxfp4(p13, s13)
    w2, w2_s, bad2 = expand_mxfp4(p2, s2)
    assert bad13 == 0 and bad2 == 0
    np_w = (w13.view(torch.uint8).cpu().numpy(), w13_s.cpu().numpy(), w2.view(torch.uint8).cpu().numpy(), w2_s.cpu().numpy())
    for tokens, alpha in ((64, None), (300, None), (1500, 3.0)):
        hidden, router_w, bias = synth.make_activations(tokens, alpha, seed=9)
        b = None if bias is None else bias.cuda()
        native = RoutedMoELayer(router_w.cuda(), p13, s13, p2, s2, tokens, b, mxfp4=True)
        out, inter = run_layer(native, hidden)
        expanded = RoutedMoELayer(router_w.cuda(), w13, w13_s, w2, w2_s, tokens, b)
        expanded.set_gemm_mode(1)
        out_e, inter_e = run_layer(expanded, hidden)
        rows = tokens * 9
        assert torch.equal(inter["perm"], inter_e["perm"]) and torch.equal(inter["topk_ids"], inter_e["topk_ids"])
        differ = (inter["h_fp8"][:rows] != inter_e["h_fp8"][:rows]).float().mean().item()
        assert differ < 2e-3, f"native and expanded MXFP4 paths differ in {differ:.2%} of the intermediate codes"
        d, de = inter["down"][:rows].double(), inter_e["down"][:rows].double()
        assert ((d - de).norm() / de.norm()).item() < 2e-3
        if tokens <= 300:
            ref = R.moe_layer(helpers.bits(hidden), helpers.bits(router_w), *np_w)
            check_against(ref, out, inter, tokens)
        else:
            m = R.parity_metrics(helpers.bits(out), helpers.bits(out_e))
            assert m["max_abs"] <= helpers.MAX_ABS and m["rel_l2"] <= helpers.REL_L2, m
        native.close(); expanded.close()


def test_external_topk_entry_and_custom_ops(gpu_weights):
    """A caller that keeps its own top-k: feeding the layer's own ids and weights back through apply() (and through
    the registered torch ops) must reproduce the fused call bit for bit; a different top-k changes the result."""
    from netra_kernel_b200 import torch_ops
    tokens = 96
    hidden, router_w, _ = synth.make_activations(tokens, seed=8)
    layer = make_layer(gpu_weights, router_w, tokens)
    h = hidden.cuda()
    want = layer(h).clone()
    torch.cuda.synchronize()
    inter = layer.intermediates(tokens)
    ids = inter["topk_ids"][:, :8].contiguous().clone()
    w = inter["topk_w"][:, :8].contiguous().clone()
    got = layer.apply(h, w, ids)
    torch.cuda.synchronize()
    layer.check_status()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    handle = torch_ops.register_layer(layer)
    assert torch.equal(torch.ops.netra.moe_layer(h, handle).view(torch.int16), want.view(torch.int16))
    assert torch.equal(torch.ops.netra.moe_apply(h, w, ids, handle).view(torch.int16), want.view(torch.int16))
    # a top-k from plain torch ops on the exact logits selects the same experts (ties aside) with FP32 weights close by
    logits = inter["logits"].float()
    p = torch.softmax(logits, dim=1)
    tw, ti = torch.topk(p, 8, dim=1)
    tw = (tw / tw.sum(1, keepdim=True)).contiguous()
    other = layer.apply(h, tw, ti.to(torch.int32).contiguous())
    torch.cuda.synchronize()
    m = R.parity_metrics(helpers.bits(other.cpu()), helpers.bits(want.cpu()))
    assert m["max_abs"] <= helpers.MAX_ABS and m["rel_l2"] <= helpers.REL_L2, m
    # uniform weights over the same experts is a different layer: the entry point really uses what it is given
    flat = layer.apply(h, torch.full_like(w, 0.125), ids)
    torch.cuda.synchronize()
    assert not torch.equal(flat.view(torch.int16), want.view(torch.int16))
    with pytest.raises(ValueError, match="topk_ids"):
        layer.apply(h, w, ids.long())
    torch_ops.release_layer(handle)
    with pytest.raises(RuntimeError, match="no registered layer"):
        torch.ops.netra.moe_layer(h, handle)
    # bring-up modes: the slot-order bridge kernels recompute the expert part from the layer's own routing
    shadow = torch_ops.register_layer(layer, shadow_weights=gpu_weights)
    try:
        os.environ["NETRA_ENGINE_MODE"] = "compare"
        assert torch.equal(torch.ops.netra.moe_layer(h, shadow).view(torch.int16), want.view(torch.int16))
        cmp = torch_ops.last_comparison(shadow)
        assert cmp["max_abs"] <= helpers.MAX_ABS and cmp["rel_l2"] <= helpers.REL_L2, cmp
        broken = (gpu_weights[0], gpu_weights[1] * 1.5, gpu_weights[2], gpu_weights[3])     # a wrong checkpoint on the shadow side
        bad = torch_ops.register_layer(layer, shadow_weights=broken)
        with pytest.raises(RuntimeError, match="disagree"):
            torch.ops.netra.moe_layer(h, bad)
        os.environ["NETRA_ENGINE_MODE"] = "shadow"                                         # reports, does not raise
        torch.ops.netra.moe_layer(h, bad)
        assert torch_ops.last_comparison(bad)["rel_l2"] > helpers.REL_L2
    finally:
        os.environ.pop("NETRA_ENGINE_MODE", None)


def test_bridge_kernels_against_checker(gpu_weights, expert_weights):
    """The three-launch slot-order boundary of the reference's decode bridges."""
    from netra_kernel_b200 import moe
    tokens = 16
    data = dict(np.load(helpers.GOLDEN / "moe_layer_t16.npz"))
    hidden, router_w, _ = synth.make_activations(tokens)
    w13, w13_s, w2, w2_s = gpu_weights
    logits = moe.bridge_router_bf16(hidden.cuda(), router_w.cuda())
    assert np.array_equal(helpers.bits(logits), data["logits"])
    a_fp8 = torch.from_numpy(data["a_fp8"]).cuda()
    a_scale = torch.from_numpy(data["a_scale"]).cuda()
    ids9 = torch.from_numpy(data["topk_ids"]).cuda()
    w9 = torch.from_numpy(data["topk_w"]).cuda()
    gu = moe.bridge_gate_up(a_fp8, a_scale, w13, w13_s, ids9)
    cw13, cw13_s, cw2, cw2_s = helpers.np_weights(expert_weights)
    want = np.stack([R.blockscale_matmul(data["a_fp8"][t:t + 1], data["a_scale"][t:t + 1], cw13[e], cw13_s[e])[0]
                     for t in range(tokens) for e in data["topk_ids"][t]])
    np.testing.assert_allclose(gu.cpu().numpy(), want, rtol=1e-4, atol=2e-5)
    # SiLU*up + requant on the SAME FP32 input: codes and scales as the checker computes them
    q, s = moe.bridge_silu_mul_quant(gu)
    want_q, want_s, _ = R.silu_mul_quant(gu.cpu().numpy())
    assert (q.cpu().numpy() != want_q).mean() < 5e-4
    np.testing.assert_allclose(s.cpu().numpy(), want_s, rtol=1e-6)
    out = moe.bridge_down_reduce(q, s, w2, w2_s, w9, ids9)
    torch.cuda.synchronize()
    m = R.parity_metrics(helpers.bits(out), data["out"])
    assert m["max_abs"] <= helpers.MAX_ABS and m["rel_l2"] <= helpers.REL_L2, m


def test_shared_gate_append_bridge():
    from netra_kernel_b200 import moe
    g = torch.Generator().manual_seed(9)
    hidden = torch.randn(5, 2048, generator=g).to(torch.bfloat16)
    gate_w = (0.02 * torch.randn(2048, generator=g)).to(torch.bfloat16)
    ids8 = torch.randint(0, 256, (5, 8), generator=g, dtype=torch.int32)
    w8 = torch.rand(5, 8, generator=g)
    ids9, w9 = moe.bridge_shared_gate_append(hidden.cuda(), gate_w.cuda(), ids8.cuda(), w8.cuda())
    assert torch.equal(ids9[:, :8].cpu(), ids8) and torch.equal(w9[:, :8].cpu(), w8)
    assert ids9[:, 8].cpu().tolist() == [256] * 5
    # bit for bit against the checker's restatement (exact BF16 logit, FP64 sigmoid, one BF16 rounding)
    want = R.shared_gate(helpers.bits(hidden), helpers.bits(gate_w))
    got = helpers.bits(w9[:, 8].cpu().to(torch.bfloat16))
    assert torch.equal(w9[:, 8].cpu().to(torch.bfloat16).float(), w9[:, 8].cpu()), "the gate must be a BF16 value"
    assert np.array_equal(got, want)


def _aiter_sorted_ids(ids9: np.ndarray, rows: int = 768, capacity_blocks: int = 365):
    """The routing of one call in the sorted-id format the reference's 768-row producer reads
    (kernels/gfx950/templates/moe/prefill/fused_splitk2/entry_routing.inc:67-111): per expert (ascending id, 256 = shared) the
    words token | slot << 24 in token order, each expert padded to whole 64-entry blocks with words whose token is >= rows."""
    words, block_experts = [], []
    for e in range(257):
        tok, slot = np.nonzero(ids9 == e)
        if tok.size == 0:
            continue
        w = (tok.astype(np.int64) | (slot.astype(np.int64) << 24)).tolist()
        w += [rows | (9 << 24)] * ((-len(w)) % 64)
        words += w
        block_experts += [e] * (len(w) // 64)
    assert len(block_experts) <= capacity_blocks
    num_valid = len(words)
    words += [rows | (9 << 24)] * (capacity_blocks * 64 - len(words))
    block_experts += [0] * (capacity_blocks - len(block_experts))
    return (np.array(words, np.int64).astype(np.uint32).view(np.int32), np.array(block_experts, np.int32),
            np.array([num_valid], np.int32))


def test_prefill_m768_bridge_matches_the_checker(expert_weights):
    """netra_moe_prefill_m768_launch with the reference's argument list: quantised rows, row-major slabs, sorted ids of
    64-entry expert blocks.  The output must match the checker run with the same top-k, and a second call with other
    tokens must not see anything of the first."""
    import ctypes
    from netra_kernel_b200 import abi
    lib = abi.load()
    w13, w13_s, w2, w2_s = (t.cuda() for t in expert_weights)
    assert lib.netra_moe_prefill_m768_launch(*([None] * 15)) == -1            # not loaded
    abi.check(lib.netra_moe_prefill_m768_load(None, None), "prefill_m768_load")
    abi.check(lib.netra_moe_prefill_m768_load(b"ignored", b"ignored"), "prefill_m768_load")   # idempotent
    for seed in (11, 12):
        hidden, router_w, _ = synth.make_activations(768, seed=seed)
        hb, rb = helpers.bits(hidden), helpers.bits(router_w)
        ids, w = R.route_topk(R.router_logits(hb, rb))
        shared_w = np.linspace(0.5, 1.0, 768).astype(np.float32)
        subset = np.arange(seed % 7, 768, 23)
        ref = R.moe_layer(hb, rb, *helpers.np_weights(expert_weights), shared_w=shared_w, token_subset=subset, external_topk=(ids, w))
        aq, a_s = R.quant_fp8_group128(R.bf16_bits_to_f32(hb))
        sorted_ids, block_experts, num_valid = _aiter_sorted_ids(ref["topk_ids"])
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        t_aq, t_as, t_sorted, t_blocks, t_valid = dev(aq), dev(a_s), dev(sorted_ids), dev(block_experts), dev(num_valid)
        t_w9 = dev(ref["topk_w"])
        t_sw = torch.zeros(365 * 64, device="cuda")
        scratch = torch.zeros(1024, device="cuda")
        out = torch.zeros(768, 2048, dtype=torch.bfloat16, device="cuda")
        rc = lib.netra_moe_prefill_m768_launch(t_aq.data_ptr(), t_as.data_ptr(), w13.data_ptr(), w13_s.data_ptr(), w2.data_ptr(),
                                               w2_s.data_ptr(), t_sorted.data_ptr(), t_sw.data_ptr(), t_blocks.data_ptr(),
                                               t_valid.data_ptr(), t_w9.data_ptr(), scratch.data_ptr(), scratch.data_ptr(),
                                               out.data_ptr(), torch.cuda.current_stream().cuda_stream)
        abi.check(rc, "prefill_m768_launch")
        torch.cuda.synchronize()
        words = (ctypes.c_uint32 * 4)()
        abi.check(lib.netra_moe_prefill_m768_status(ctypes.byref(words)), "prefill_m768_status")
        assert list(words) == [0, 0, 0, 0]
        m = R.parity_metrics(helpers.bits(out.cpu())[subset], ref["out"])
        assert m["max_abs"] <= helpers.MAX_ABS and m["rel_l2"] <= helpers.REL_L2, m
    assert lib.netra_moe_prefill_m768_unload() == 0


def test_grouped_tensor_core_path_agrees_with_bridge_path(gpu_weights):
    """Independent GPU cross-check at a size the CPU checker does not cover in full."""
    from netra_kernel_b200 import moe
    tokens = 512
    hidden, router_w, bias = synth.make_activations(tokens, 1.0, seed=3)
    layer = make_layer(gpu_weights, router_w, tokens, bias)
    out, inter = run_layer(layer, hidden)
    w13, w13_s, w2, w2_s = gpu_weights
    pairs = tokens * 8
    a_fp8 = inter["a_fp8"][pairs:].cuda()
    a_scale = inter["a_scale"][pairs:].cuda()
    ids9, w9 = inter["topk_ids"].cuda(), inter["topk_w"].cuda()
    q, s = moe.bridge_silu_mul_quant(moe.bridge_gate_up(a_fp8, a_scale, w13, w13_s, ids9))
    ref = moe.bridge_down_reduce(q, s, w2, w2_s, w9, ids9)
    torch.cuda.synchronize()
    m = R.parity_metrics(helpers.bits(out), helpers.bits(ref))
    assert m["max_abs"] <= helpers.MAX_ABS and m["rel_l2"] <= 1e-3, m


def test_repeat_launch_and_graph_replay_are_bitwise_identical(gpu_weights):
    tokens = 256
    hidden, router_w, _ = synth.make_activations(tokens)
    layer = make_layer(gpu_weights, router_w, tokens)
    h = hidden.cuda()
    first = layer(h).clone()
    for _ in range(5):
        assert torch.equal(layer(h), first)
    stream = torch.cuda.Stream()
    static_out = torch.empty_like(h)
    with torch.cuda.stream(stream):
        layer(h, out=static_out)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            layer(h, out=static_out)
    for _ in range(20):
        static_out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(static_out, first)
    layer.check_status()


def test_outputs_stay_inside_their_buffers(gpu_weights):
    """Guard words around the output catch out-of-bounds stores (no sanitizer on this pool)."""
    tokens = 33
    hidden, router_w, _ = synth.make_activations(tokens, seed=8)
    layer = make_layer(gpu_weights, router_w, 64)
    guard = 4096
    buf = torch.full((guard + tokens * 2048 + guard,), -7.0, dtype=torch.bfloat16, device="cuda")
    out = buf[guard:guard + tokens * 2048].view(tokens, 2048)
    layer(hidden.cuda(), out=out)
    torch.cuda.synchronize()
    layer.check_status()
    assert torch.all(buf[:guard] == -7.0) and torch.all(buf[-guard:] == -7.0)
    assert torch.isfinite(out.float()).all()


def test_argument_errors_are_reported(gpu_weights):
    from netra_kernel_b200 import abi
    hidden, router_w, _ = synth.make_activations(8)
    layer = make_layer(gpu_weights, router_w, 8)
    with pytest.raises(abi.NetraError, match="capacity"):
        layer(torch.zeros(9, 2048, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError):
        layer(torch.zeros(8, 1024, dtype=torch.bfloat16, device="cuda"))


def test_add_rmsnorm_group_quant_bridge_and_fused_layer_entry(gpu_weights):
    """The upstream fusion at width 2048: every output of the bridge bit for bit against the checker's restatement (ragged
    row counts, a zero row, large and tiny rows), and the layer entry that takes the un-normalised input must equal the
    plain layer call on the normalised rows bit for bit."""
    from netra_kernel_b200 import moe
    g = torch.Generator().manual_seed(31)
    for rows in (1, 5, 260):
        x = torch.randn(rows, 2048, generator=g)
        res = torch.randn(rows, 2048, generator=g)
        if rows > 4:
            x[1] = 0.0; res[1] = 0.0
            x[2] *= 1e4
            x[3] *= 1e-6; res[3] *= 1e-6
        x, res = x.to(torch.bfloat16), res.to(torch.bfloat16)
        w = 1.0 + 0.1 * torch.randn(2048, generator=g)
        y, r, q, s = moe.bridge_add_rmsnorm_group_quant(x.cuda(), res.cuda(), w.cuda(), 1e-6)
        torch.cuda.synchronize()
        wy, wr, wq, ws = R.add_rmsnorm_group_quant(helpers.bits(x), helpers.bits(res), w.numpy(), 1e-6)
        assert np.array_equal(helpers.bits(r), wr), rows
        assert np.array_equal(helpers.bits(y), wy), rows
        assert np.array_equal(q.cpu().numpy(), wq) and np.array_equal(s.cpu().numpy(), ws), rows
    tokens = 200
    hidden, router_w, _ = synth.make_activations(tokens, seed=14)
    layer = make_layer(gpu_weights, router_w, 256)
    res = torch.randn(tokens, 2048, generator=g).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(2048, generator=g)).cuda()
    out, res_out, normed = layer.forward_with_norm(hidden.cuda(), res.cuda(), w, 1e-6)
    torch.cuda.synchronize()
    layer.check_status()
    a_rows = layer.intermediates(tokens)["a_fp8"][tokens * 8:].clone()
    want = layer(normed)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), want.view(torch.int16))
    assert torch.equal(layer.intermediates(tokens)["a_fp8"][tokens * 8:], a_rows)
    wy, wr, wq, _ = R.add_rmsnorm_group_quant(helpers.bits(hidden), helpers.bits(res), w.cpu().numpy(), 1e-6)
    assert np.array_equal(helpers.bits(normed), wy) and np.array_equal(helpers.bits(res_out), wr) and np.array_equal(a_rows.cpu().numpy(), wq)


def test_weight_repack_and_scale_widening_match_the_layout_plan_byte_for_byte():
    """The device steps of the layout plan against their CPU statement (compiler/layouts.py): the 128 x 128 tile repack of
    random bytes for both slab shapes, and the exact BF16 -> FP32 widening of block scales."""
    from netra_kernel_b200 import abi
    from netra_kernel_b200.compiler import layouts as L
    lib = abi.load()
    g = torch.Generator().manual_seed(17)
    for slabs, n, k in ((3, 1024, 2048), (2, 2048, 512), (1, 128, 128)):
        src = torch.randint(0, 256, (slabs * n, k), generator=g, dtype=torch.uint8)
        dst = torch.zeros_like(src).cuda()
        abi.check(lib.netra_moe_repack_tiles_launch(dst.data_ptr(), src.cuda().data_ptr(), slabs * n, k, None), "repack_tiles_launch")
        torch.cuda.synchronize()
        assert np.array_equal(dst.cpu().numpy(), L.tile_128x128(src.numpy())), (slabs, n, k)
    bits = torch.randint(0, 1 << 16, (257 * 8 * 16,), generator=g, dtype=torch.int32).to(torch.uint16)
    bits = bits[(bits & 0x7F80) != 0x7F80]            # finite values
    out = torch.zeros(bits.numel(), dtype=torch.float32, device="cuda")
    abi.check(lib.netra_moe_widen_scales_bf16_launch(out.data_ptr(), bits.cuda().data_ptr(), bits.numel(), None), "widen_scales_launch")
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), L.widen_bf16_to_fp32(bits.numpy()).view(np.uint32))
    assert lib.netra_moe_widen_scales_bf16_launch(None, None, 4, None) == -1
    assert lib.netra_moe_repack_tiles_launch(dst.data_ptr(), dst.data_ptr(), 128, 128, None) == -1      # aliased

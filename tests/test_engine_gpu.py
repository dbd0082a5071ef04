"""GPU tests of the compiler -> engine directory -> runtime ABI path: the layer launched through
netra_engine_launch must match the CPU checker, replay identically from a captured CUDA graph,
and answer the reference's status codes for guard misses and call-order errors."""
import ctypes

import numpy as np
import pytest
import torch

from netra_kernel_b200 import engine_runtime as er
from netra_kernel_b200 import synth
from netra_kernel_b200.compiler import compile_engine
from netra_kernel_b200.compiler.library import KernelLibrary
from oracle import moe_ref as R
from tests import helpers

pytestmark = pytest.mark.gpu

MANIFESTS = KernelLibrary.discover().root / "manifests" / "sm_100a" / "models"
MODEL = MANIFESTS / "routed-moe-layer-fp8.json"
MODEL_ZIPF = MANIFESTS / "routed-moe-layer-fp8-zipf.json"


@pytest.fixture(autouse=True)
def side_stream():
    """Stream capture is not allowed on the legacy default stream: every test runs on its own stream."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        yield stream
    torch.cuda.synchronize()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _session(tmp_path, model, profile, tensors, graph=True):
    compile_engine(model, profile, tmp_path / profile)
    session = er.EngineSession(tmp_path / profile, device_id=0, enable_graph_capture=graph)
    bound = session.prepare_weights(tensors)
    torch.cuda.synchronize()
    session.bind(bound)
    session.finalize()
    return session


def _tensors(expert_weights, tokens, zipf_alpha=None, shared=False, seed=0):
    hidden, router_w, bias = synth.make_activations(tokens, zipf_alpha, seed=seed)
    w13, w13_s, w2, w2_s = (t.cuda() for t in expert_weights)
    t = {"hidden": hidden.cuda(), "output": torch.zeros(tokens, 2048, dtype=torch.bfloat16, device="cuda"),
         "router_weight": router_w.cuda(), "w13": w13, "w13_scale": w13_s, "w2": w2, "w2_scale": w2_s}
    if bias is not None:
        t["router_bias"] = bias.cuda()
    if shared:
        t["shared_weight"] = torch.linspace(0.5, 1.0, tokens).cuda()
    return t, hidden, router_w, bias


def _status_words(session):
    words = session.workspace_view("status", torch.int32, "cuda").cpu()
    return words.tolist()


def test_engine_t16_matches_golden_fixture_direct_and_graph(tmp_path, expert_weights):
    data = dict(np.load(helpers.GOLDEN / "moe_layer_t16.npz"))
    tensors, *_ = _tensors(expert_weights, 16)
    session = _session(tmp_path, MODEL, "cpu_t16", tensors)
    info = session.profile()
    assert (info.min_m, info.max_m, info.requires_fallback, info.tensor_parallel) == (16, 16, 0, 1)
    assert info.workspace_bytes == session.manifest["workspace_bytes"] and er.load().netra_engine_profile_count(session.handle) == 1
    session.launch(_stream())                       # direct launches
    torch.cuda.synchronize()
    assert _status_words(session) == [0, 0, 0, 0]
    direct = tensors["output"].clone()
    assert np.array_equal(session.workspace_view("topk_ids", torch.int32, "cuda").cpu().numpy().reshape(16, 9), data["topk_ids"])
    assert np.array_equal(session.workspace_view("perm", torch.int32, "cuda").cpu().numpy(), data["perm"])
    assert np.array_equal(session.workspace_view("counts", torch.int32, "cuda").cpu().numpy(), data["counts"])
    m = R.parity_metrics(helpers.bits(direct), data["out"])
    assert m["max_abs"] <= helpers.MAX_ABS and m["rel_l2"] <= helpers.REL_L2, m
    session.prepare(_stream())                      # capture, then replay 20 times
    for _ in range(20):
        tensors["output"].zero_()
        session.launch(_stream())
        torch.cuda.synchronize()
        assert torch.equal(tensors["output"], direct)
    assert session.close() == 0


def test_engine_t256_matches_c_checker(tmp_path, expert_weights, c_oracle):
    tensors, hidden, router_w, _ = _tensors(expert_weights, 256)
    ref = helpers.c_layer(c_oracle, helpers.bits(hidden), helpers.bits(router_w), *helpers.np_weights(expert_weights))
    session = _session(tmp_path, MODEL, "decode_t256", tensors)
    session.prepare(_stream())
    session.launch(_stream())
    torch.cuda.synchronize()
    assert _status_words(session) == [0, 0, 0, 0]
    assert np.array_equal(session.workspace_view("topk_ids", torch.int32, "cuda").cpu().numpy().reshape(256, 9), ref["topk_ids"])
    assert np.array_equal(session.workspace_view("perm", torch.int32, "cuda").cpu().numpy(), ref["perm"])
    assert np.array_equal(session.workspace_view("offsets", torch.int32, "cuda").cpu().numpy()[:257], ref["offsets"])
    m = R.parity_metrics(helpers.bits(tensors["output"]), ref["out"])
    assert m["max_abs"] <= helpers.MAX_ABS and m["rel_l2"] <= helpers.REL_L2, m


def test_engine_with_bias_shared_weight_row_major_and_segmented_sort(tmp_path, expert_weights):
    """Second model manifest: router bias + shared-weight column bound, row-major weights, 2048
    tokens (above the single-block sort limit)."""
    tokens = 2048
    tensors, hidden, router_w, bias = _tensors(expert_weights, tokens, zipf_alpha=0.8, shared=True, seed=4)
    subset = np.arange(3, tokens, 131)
    ref = R.moe_layer(helpers.bits(hidden), helpers.bits(router_w), *helpers.np_weights(expert_weights), bias=bias.numpy(),
                      shared_w=tensors["shared_weight"].cpu().numpy(), token_subset=subset)
    session = _session(tmp_path, MODEL_ZIPF, "ep8_local_t2048", tensors)
    assert [o["name"] for o in session.manifest["operations"]][2:5] == ["sort_hist", "sort_scan", "sort_scatter"]
    # 2,048 tokens select the token-major GEMMs, whose register contract the runtime checks against the loaded cubin
    gate = next(o for o in session.manifest["operations"] if o["name"] == "gate_up")
    assert gate["kernel_symbol"] == "netra_moe_gate_up_tokmajor_sm100" and gate["launch"]["registers_per_thread"] == 168
    session.launch(_stream())
    torch.cuda.synchronize()
    assert _status_words(session) == [0, 0, 0, 0]
    assert np.array_equal(session.workspace_view("perm", torch.int32, "cuda").cpu().numpy(), ref["perm"])
    m = R.parity_metrics(helpers.bits(tensors["output"])[subset], ref["out"])
    assert m["max_abs"] <= helpers.MAX_ABS and m["rel_l2"] <= helpers.REL_L2, m


def test_engine_prefill_manifest_runs_the_fp16_partial_row_tactics(tmp_path, expert_weights):
    """The prefill model manifest (router bias, FP16 partial rows) at 2,048 tokens through the engine ABI: the tensor-core
    router pair, the token-major GEMMs, the FP16-row down projection and its reducer, against the checker run with the same
    rounding point."""
    tokens = 2048
    tensors, hidden, router_w, bias = _tensors(expert_weights, tokens, zipf_alpha=0.8, seed=4)
    subset = np.arange(1, tokens, 97)
    ref = R.moe_layer(helpers.bits(hidden), helpers.bits(router_w), *helpers.np_weights(expert_weights), bias=bias.numpy(),
                      token_subset=subset, partials="f16")
    session = _session(tmp_path, MANIFESTS / "routed-moe-layer-fp8-prefill.json", "ep8_local_t2048", tensors)
    symbols = [o["kernel_symbol"] for o in session.manifest["operations"]]
    assert symbols[:2] == ["netra_router_logits_f32_umma_sm100", "netra_moe_topk_quant_fix_sm100"]
    assert symbols[-2:] == ["netra_moe_down_tokmajor_f16_sm100", "netra_moe_combine_f16_sm100"]
    session.prepare(_stream())
    session.launch(_stream())
    torch.cuda.synchronize()
    assert _status_words(session) == [0, 0, 0, 0]
    assert np.array_equal(session.workspace_view("topk_ids", torch.int32, "cuda").cpu().numpy().reshape(tokens, 9), ref["topk_ids"])
    assert np.array_equal(session.workspace_view("perm", torch.int32, "cuda").cpu().numpy(), ref["perm"])
    m = R.parity_metrics(helpers.bits(tensors["output"])[subset], ref["out"])
    assert m["max_abs"] <= helpers.MAX_ABS and m["rel_l2"] <= helpers.REL_L2, m


def test_engine_on_mxfp4_weights_equals_the_fused_layer_call(tmp_path):
    """The MXFP4 model manifest through the engine ABI at both profile sizes: the layout plan's pack step, four-bit tensor
    maps encoded by the runtime, the block-scaled kernels launched from the cubin - bit for bit the fused-layer call."""
    from netra_kernel_b200.moe import RoutedMoELayer
    p13, s13, p2, s2 = synth.make_expert_weights_device(0, torch.device("cuda", 0), mxfp4=True)
    for profile, tokens, symbol in (("decode_t256_mxfp4", 256, "netra_moe_gate_up_mxfp4_umma_sm100"),
                                    ("prefill_t8192_mxfp4", 8192, "netra_moe_gate_up_mxfp4_tokmajor_sm100")):
        hidden, router_w, _ = synth.make_activations(tokens, None, seed=3)
        tensors = {"hidden": hidden.cuda(), "output": torch.zeros(tokens, 2048, dtype=torch.bfloat16, device="cuda"),
                   "router_weight": router_w.cuda(), "w13": p13, "w13_scale": s13, "w2": p2, "w2_scale": s2}
        session = _session(tmp_path, MANIFESTS / "routed-moe-layer-mxfp4.json", profile, tensors)
        assert symbol in [o["kernel_symbol"] for o in session.manifest["operations"]]
        session.prepare(_stream())
        session.launch(_stream())
        torch.cuda.synchronize()
        assert _status_words(session) == [0, 0, 0, 0]
        layer = RoutedMoELayer(tensors["router_weight"], p13, s13, p2, s2, tokens, mxfp4=True)
        want = layer(tensors["hidden"])
        torch.cuda.synchronize()
        layer.check_status()
        assert torch.equal(tensors["output"].view(torch.int16), want.view(torch.int16))
        assert tensors["output"].float().abs().max().item() > 0
        layer.close()
        session.close()


def test_two_binding_sets_share_one_engine(tmp_path, expert_weights):
    """An engine compiled with two binding sets: profile ids 0 and 1 are bound to different input / output buffers, captured
    separately and launched alternately over the one workspace; each reproduces the result of its own input."""
    tokens = 256
    tensors, hidden, router_w, _ = _tensors(expert_weights, tokens)
    other, _, _ = synth.make_activations(tokens, None, seed=11)
    compile_engine(MODEL, "decode_t256", tmp_path / "e", binding_sets=2)
    session = er.EngineSession(tmp_path / "e", device_id=0, enable_graph_capture=True)
    bound = session.prepare_weights(tensors)
    second = {**bound, "hidden": other.cuda(), "output": torch.zeros(tokens, 2048, dtype=torch.bfloat16, device="cuda")}
    torch.cuda.synchronize()
    session.bind(bound, profile_id=0)
    session.bind(second, profile_id=1)
    session.finalize()
    session.prepare(_stream(), profile_id=0)
    session.prepare(_stream(), profile_id=1)
    for _ in range(3):
        session.launch(_stream(), profile_id=0)
        session.launch(_stream(), profile_id=1)
    torch.cuda.synchronize()
    assert _status_words(session) == [0, 0, 0, 0]
    from netra_kernel_b200.moe import RoutedMoELayer
    layer = RoutedMoELayer(tensors["router_weight"], *(t.cuda() for t in expert_weights), tokens)
    for io in (bound, second):
        want = layer(io["hidden"]).clone()
        torch.cuda.synchronize()
        assert torch.equal(io["output"].view(torch.int16), want.view(torch.int16))
    assert not torch.equal(bound["output"], second["output"])
    session.close()


def test_status_codes_for_guards_and_call_order(tmp_path, expert_weights):
    lib = er.load()
    tensors, *_ = _tensors(expert_weights, 16)
    compile_engine(MODEL, "cpu_t16", tmp_path / "e")
    session = er.EngineSession(tmp_path / "e", 0, True)
    shape = er.LaunchShape(16, 1, 0, 1)
    stream = _stream()
    # launch before bindings are finalised
    assert lib.netra_engine_launch(session.handle, 0, ctypes.byref(shape), stream) == 6          # BINDING
    assert lib.netra_engine_finalize_bindings(session.handle) == 6                                # unbound pointers
    assert b"must be bound" in lib.netra_engine_last_error(session.handle)
    slot = session.recipe["binding_slots"]["hidden"][0]
    assert lib.netra_engine_bind(session.handle, 0, slot["operation"], 31, tensors["hidden"].data_ptr()) == 6
    assert lib.netra_engine_bind(session.handle, 0, 99, 0, tensors["hidden"].data_ptr()) == 6
    assert lib.netra_engine_bind(session.handle, 0, 0, 3, tensors["hidden"].data_ptr()) == 6     # a u32 constant slot
    assert lib.netra_engine_bind(session.handle, 0, 0, 0, tensors["hidden"].data_ptr()) == 6     # a workspace slot
    assert lib.netra_engine_bind(session.handle, 0, slot["operation"], slot["argument"], None) == 1
    bound = session.prepare_weights(tensors)
    session.bind(bound)
    session.finalize()
    assert lib.netra_engine_bind(session.handle, 0, slot["operation"], slot["argument"], tensors["hidden"].data_ptr()) == 8  # BUSY
    for bad in (er.LaunchShape(17, 1, 0, 1), er.LaunchShape(16, 0, 0, 1), er.LaunchShape(16, 1, 0, 2), er.LaunchShape(16, 1, 1 << 30, 1)):
        assert lib.netra_engine_launch(session.handle, 0, ctypes.byref(bad), stream) == 5       # UNSUPPORTED_PROFILE
    assert lib.netra_engine_launch(session.handle, 7, ctypes.byref(shape), stream) == 1
    assert lib.netra_engine_launch(session.handle, 0, None, stream) == 1
    info = er.ProfileInfo()
    info.struct_size = 8
    assert lib.netra_engine_query_profile(session.handle, 0, ctypes.byref(info)) == 1
    info.struct_size = ctypes.sizeof(info)
    assert lib.netra_engine_query_profile(session.handle, 3, ctypes.byref(info)) == 5
    # one operation at a time, then with caller-local pointers
    for index in range(len(session.manifest["operations"])):
        session.launch_operation(index, stream)
    torch.cuda.synchronize()
    first = tensors["output"].clone()
    other = torch.zeros_like(first)
    last = len(session.manifest["operations"]) - 1
    binding = (er.PointerBinding * 1)(er.PointerBinding(0, 0, other.data_ptr()))
    assert lib.netra_engine_launch_operation_bound(session.handle, 0, last, ctypes.byref(shape), binding, 1, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(other, first) and first.float().abs().sum() > 0
    assert lib.netra_engine_launch_operation_bound(session.handle, 0, last, ctypes.byref(shape), binding, 0, stream) == 6
    dup = (er.PointerBinding * 1)(er.PointerBinding(0, 1, other.data_ptr()))
    assert lib.netra_engine_launch_operation_bound(session.handle, 0, last, ctypes.byref(shape), dup, 1, stream) == 6
    assert lib.netra_engine_launch_operation_bound(session.handle, 0, last, ctypes.byref(shape), binding, 17, stream) == 1
    session.prepare(stream)
    assert lib.netra_engine_launch_operation(session.handle, 0, 0, ctypes.byref(shape), stream) == 8   # BUSY after capture
    assert lib.netra_engine_launch_operation_bound(session.handle, 0, last, ctypes.byref(shape), binding, 1, stream) == 8
    session.launch(stream)
    torch.cuda.synchronize()
    assert torch.equal(tensors["output"], first)
    assert session.close() == 0


def test_engine_with_fallback_operation_refuses_to_launch(tmp_path, expert_weights):
    import json
    doc = json.loads(MODEL.read_text())
    doc["constants"]["hidden"] = 4096                      # no kernel is built for this width
    (tmp_path / "m.json").write_text(json.dumps(doc))
    compile_engine(tmp_path / "m.json", "cpu_t16", tmp_path / "e")
    session = er.EngineSession(tmp_path / "e", 0, True)
    assert session.profile().requires_fallback == 1
    lib = er.load()
    shape = er.LaunchShape(16, 1, 0, 1)
    assert lib.netra_engine_finalize_bindings(session.handle) == 0      # nothing to bind
    assert lib.netra_engine_launch(session.handle, 0, ctypes.byref(shape), _stream()) == 9        # FALLBACK_REQUIRED
    assert lib.netra_engine_prepare_profile(session.handle, 0, _stream()) == 9
    assert lib.netra_engine_launch_operation(session.handle, 0, 0, ctypes.byref(shape), _stream()) == 9


def test_create_names_the_cause_of_a_failure(tmp_path):
    """A missing code object is an IO failure, a driver older than the engine requires an unsupported target, a code
    object that is not one a CUDA failure, a damaged engine.json a manifest failure - each with its text kept for the
    calling thread, and the caller's current device left as it was."""
    import json
    lib = er.load()
    before = torch.cuda.current_device()
    compile_engine(MODEL, "cpu_t16", tmp_path / "e")
    (tmp_path / "e" / "cubin" / "netra_moe_sm100a.cubin").unlink()
    with pytest.raises(er.EngineError) as err:
        er.EngineSession(tmp_path / "e")
    assert err.value.status == 2 and b"cannot open" in lib.netra_engine_create_error()
    compile_engine(MODEL, "cpu_t16", tmp_path / "f")
    doc = json.loads((tmp_path / "f" / "engine.json").read_text())
    doc["required_cuda"]["minimum"] = "99.0"
    (tmp_path / "f" / "engine.json").write_text(json.dumps(doc))
    with pytest.raises(er.EngineError) as err:
        er.EngineSession(tmp_path / "f")
    assert err.value.status == 4 and b"requires 99.0" in lib.netra_engine_create_error()
    compile_engine(MODEL, "cpu_t16", tmp_path / "g")
    (tmp_path / "g" / "cubin" / "netra_moe_sm100a.cubin").write_bytes(b"not a code object" * 64)
    with pytest.raises(er.EngineError) as err:
        er.EngineSession(tmp_path / "g")
    assert err.value.status == 7 and b"cuModuleLoadData" in lib.netra_engine_create_error()
    compile_engine(MODEL, "cpu_t16", tmp_path / "h")
    (tmp_path / "h" / "engine.json").write_text("{")
    options = er.EngineOptions(ctypes.sizeof(er.EngineOptions), 0, 1)
    handle = ctypes.c_void_p()
    assert lib.netra_engine_create(str(tmp_path / "h").encode(), ctypes.byref(options), ctypes.byref(handle)) == 3
    assert lib.netra_engine_create_error() != b"" and not handle.value
    assert torch.cuda.current_device() == before
    # a successful create clears the text
    compile_engine(MODEL, "cpu_t16", tmp_path / "ok")
    session = er.EngineSession(tmp_path / "ok")
    assert lib.netra_engine_create_error() == b""
    assert session.close() == 0


def test_c_caller_runs_the_documented_sequence(tmp_path):
    """tests/engine_abi_example.c (the sequence INTEGRATION.md documents) compiled with gcc and run on a compiled engine
    directory: create, query_profile, bind per slot, finalize, prepare (graph capture), three launches, destroy."""
    import json
    import subprocess
    from netra_kernel_b200 import abi
    exe = tmp_path / "engine_abi_example"
    cmd = ["gcc", "-std=c11", "-I", str(helpers.ROOT / "include"), "-I", "/usr/local/cuda/include",
           str(helpers.ROOT / "tests" / "engine_abi_example.c"), "-o", str(exe), "-L", str(abi.LIB_PATH.parent),
           "-l:" + abi.LIB_PATH.name, "-L", "/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath," + str(abi.LIB_PATH.parent)]
    subprocess.run(cmd, check=True, capture_output=True)
    for profile, m in (("cpu_t16", 16), ("decode_t256", 256)):
        directory = tmp_path / profile
        compile_engine(MODEL, profile, directory)
        recipe = json.loads((directory / "graph_recipe.json").read_text())
        sizes = {t["name"]: t["bytes"] for t in json.loads((directory / "graph.json").read_text())["tensors"]}
        lines = [f"{name} {slot['operation']} {slot['argument']} {sizes[name]}"
                 for name, places in sorted(recipe["binding_slots"].items()) for slot in places]
        (directory / "slots.txt").write_text("\n".join(lines) + "\n")
        done = subprocess.run([str(exe), str(directory), str(directory / "slots.txt"), str(m)], capture_output=True, text=True, timeout=120)
        assert done.returncode == 0 and done.stdout.strip() == "ok", (done.returncode, done.stdout, done.stderr)
    # a shape outside the guards is refused by the example before it binds anything
    done = subprocess.run([str(exe), str(tmp_path / "cpu_t16"), str(tmp_path / "cpu_t16" / "slots.txt"), "17"], capture_output=True, text=True)
    assert done.returncode == 1


def test_verify_profile_engine_runs_768_routed_rows(tmp_path, expert_weights):
    """The exact verify profile (m = 12 draft positions, batch = 64 -> 768 routed rows): launch shape (12, 64), parity of
    the routing and of sampled outputs against the checker, and the m / batch guards."""
    tokens = 768
    tensors, hidden, router_w, _ = _tensors(expert_weights, tokens, seed=6)
    subset = np.arange(2, tokens, 53)
    ref = R.moe_layer(helpers.bits(hidden), helpers.bits(router_w), *helpers.np_weights(expert_weights), token_subset=subset)
    session = _session(tmp_path, MODEL, "verify_m12_b64_routes768", tensors)
    assert (session.shape.m, session.shape.batch) == (12, 64)
    session.prepare(_stream())
    session.launch(_stream())
    torch.cuda.synchronize()
    assert _status_words(session) == [0, 0, 0, 0]
    assert np.array_equal(session.workspace_view("topk_ids", torch.int32, "cuda").cpu().numpy().reshape(tokens, 9), ref["topk_ids"])
    assert np.array_equal(session.workspace_view("perm", torch.int32, "cuda").cpu().numpy(), ref["perm"])
    m = R.parity_metrics(helpers.bits(tensors["output"])[subset], ref["out"])
    assert m["max_abs"] <= helpers.MAX_ABS and m["rel_l2"] <= helpers.REL_L2, m
    lib = er.load()
    for bad in (er.LaunchShape(768, 1, 0, 1), er.LaunchShape(12, 63, 0, 1)):
        assert lib.netra_engine_launch(session.handle, 0, ctypes.byref(bad), _stream()) == 5

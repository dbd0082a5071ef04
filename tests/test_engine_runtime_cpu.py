"""CPU tests of the engine runtime: manifest failures injected on the host (no GPU is touched),
exported symbols, and the hot-path source rules of the reference
(tests/compiler/test_runtime_hotpath.py:17-72): launch functions do not allocate, synchronise,
open files, read the environment or use string/map lookups."""
import ctypes
import json
import re

import pytest

from netra_kernel_b200 import abi
from netra_kernel_b200 import engine_runtime as er
from netra_kernel_b200.compiler import compile_engine
from netra_kernel_b200.compiler.library import KernelLibrary
from tests import helpers

MODEL = KernelLibrary.discover().root / "manifests" / "sm_100a" / "models" / "routed-moe-layer-fp8.json"


@pytest.fixture()
def engine_dir(tmp_path):
    compile_engine(MODEL, "cpu_t16", tmp_path / "e")
    return tmp_path / "e"


def _mutate(engine_dir, fn):
    path = engine_dir / "engine.json"
    doc = json.loads(path.read_text())
    fn(doc)
    path.write_text(json.dumps(doc))


def test_library_exports_the_engine_abi():
    lib = er.load()
    text = (helpers.ROOT / "include" / "netra_engine.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = sorted(set(re.findall(r"\b(netra_engine_[a-z_]+)\s*\(", text)))
    assert len(declared) == 14 and set(declared) == set(er.ENGINE_SIGNATURES)
    for name in declared:
        assert hasattr(lib, name), name
    # struct layouts of runtime/gfx950/engine/netra_engine.h:27-58
    assert ctypes.sizeof(er.EngineOptions) == 12 and ctypes.sizeof(er.LaunchShape) == 24
    assert ctypes.sizeof(er.ProfileInfo) == 64 and ctypes.sizeof(er.PointerBinding) == 16


def test_compiled_manifest_is_accepted(engine_dir):
    assert er.check_manifest(engine_dir) == (0, "")


@pytest.mark.parametrize("mutate, message", [
    (lambda d: d.__setitem__("target", "gfx950"), "contract mismatch"),
    (lambda d: d.__setitem__("wave_size", 64), "contract mismatch"),
    (lambda d: d.__setitem__("format_version", "netra-engine-2"), "contract mismatch"),
    (lambda d: d["required_cuda"].__setitem__("minimum", "12"), "MAJOR.MINOR"),
    (lambda d: d.pop("workspace_bytes"), "workspace_bytes"),
    (lambda d: d.__setitem__("profiles", []), "no profile"),
    (lambda d: d["profiles"][0]["guards"].pop("batch"), "batch"),
    (lambda d: d["operations"][0].__setitem__("cubin", "cubin/../../etc/passwd"), "traversal"),
    (lambda d: d["operations"][0].__setitem__("cubin", "/abs/k.cubin"), "normalized"),
    (lambda d: d["operations"][0]["launch"].__setitem__("grid", [0, 1, 1]), "nonzero"),
    (lambda d: d["operations"][0]["launch"].__setitem__("block", [256, 1]), "three dimensions"),
    (lambda d: d["operations"][0].__setitem__("arguments", []), "typed arguments"),
    (lambda d: d["operations"][0].__setitem__("arguments", d["operations"][0]["arguments"] * 9), "more than 32"),
    (lambda d: d["operations"][0]["arguments"][0].__setitem__("workspace_offset", 1 << 40), "out of range"),
    (lambda d: d["operations"][0]["arguments"][0].__setitem__("kind", "f64_constant"), "unsupported kernel argument kind"),
    (lambda d: d["operations"][0]["arguments"][1].__setitem__("source", "heap"), "unsupported pointer argument source"),
    (lambda d: d["operations"][4]["arguments"][0]["tensor_map"].__setitem__("swizzle", "64B"), "unsupported tensor_map"),
    (lambda d: d["operations"][3]["arguments"][3].__setitem__("value", -1), "uint32"),
])
def test_manifest_failures_are_reported_with_manifest_status(engine_dir, mutate, message):
    _mutate(engine_dir, mutate)
    rc, text = er.check_manifest(engine_dir)
    assert rc == 3 and message in text, (rc, text)


def test_corrupt_and_missing_manifest(engine_dir, tmp_path):
    (engine_dir / "engine.json").write_text('{"format_version": "netra-engine-1", ')
    rc, text = er.check_manifest(engine_dir)
    assert rc == 3 and "engine.json" in text
    rc, text = er.check_manifest(tmp_path / "nowhere")
    assert rc == 3 and "cannot open" in text
    assert er.load().netra_engine_check_manifest(None, None, 0) == 1


def test_argument_checks_that_need_no_device():
    lib = er.load()
    handle = ctypes.c_void_p()
    options = er.EngineOptions(4, 0, 1)      # wrong struct_size
    assert lib.netra_engine_create(b"/tmp", ctypes.byref(options), ctypes.byref(handle)) == 1
    assert lib.netra_engine_create(None, ctypes.byref(options), ctypes.byref(handle)) == 1
    assert lib.netra_engine_profile_count(None) == 0
    assert lib.netra_engine_destroy(None) == 0
    assert lib.netra_engine_last_error(None) == b"netra_engine is null"
    info = er.ProfileInfo()
    assert lib.netra_engine_query_profile(None, 0, ctypes.byref(info)) == 1
    assert lib.netra_engine_bind(None, 0, 0, 0, None) == 1
    assert lib.netra_engine_finalize_bindings(None) == 1


# ------------------------------------------------------------------ hot-path source scan
def _function_body(source: str, name: str) -> str:
    start = source.index(f"extern \"C\" netra_status_t {name}(")
    depth, i = 0, source.index("{", start)
    begin = i
    while True:
        depth += source[i] == "{"
        depth -= source[i] == "}"
        if depth == 0:
            return source[begin:i + 1]
        i += 1


FORBIDDEN = ("cudaMalloc", "cudaFree", "cudaMemcpy", "cudaMemset", "Synchronize", "ifstream", "getenv", "fopen",
             "ModuleLoad", "ModuleGetFunction", "std::map", "std::string", "std::vector<", "new ", "parse_manifest",
             "read_file", "JsonReader")


@pytest.mark.parametrize("name", ["netra_engine_launch", "netra_engine_launch_operation", "netra_engine_launch_operation_bound"])
def test_launch_functions_contain_no_control_plane_work(name):
    source = (helpers.ROOT / "netra_kernel_b200" / "csrc" / "engine.cpp").read_text()
    body = _function_body(source, name)
    for token in FORBIDDEN:
        assert token not in body, f"{name} contains {token}"
    for helper in ("launch_record", "launch_one", "direct_launch"):
        start = source.index(f"netra_status_t {helper}(")
        helper_body = source[start:source.index("\n}\n", start)]
        for token in FORBIDDEN:
            assert token not in helper_body, f"{helper} contains {token}"


def test_fused_layer_launch_path_does_not_allocate_or_synchronise():
    source = (helpers.ROOT / "netra_kernel_b200" / "csrc" / "api.cu").read_text()
    start = source.index("int launch_stage(")
    body = source[start:source.index("int netra_moe_repack_tiles_launch", start)]
    for token in ("cudaMalloc", "cudaFree", "cudaMemcpy", "Synchronize", "getenv", "fopen"):
        assert token not in body, token
    # the one descriptor encoded per call is the caller's token buffer for the tensor-core router: host arithmetic
    # only (no driver state, no allocation), and it happens exactly once in the sequence
    assert body.count("encode_u8_2d(") == 1
    scratch = (helpers.ROOT / "netra_kernel_b200" / "csrc" / "static_scratch_sort.cu").read_text()
    code = re.sub(r"//.*", "", scratch)
    assert "cudaMalloc" not in code and "cudaFree" not in code


# ------------------------------------------------------------------ the documented C caller
def _c_example_snippet() -> str:
    import textwrap
    c = (helpers.ROOT / "tests" / "engine_abi_example.c").read_text()
    begin, end = "/* [integration-snippet-begin] */\n", "  /* [integration-snippet-end] */"
    return textwrap.dedent(c[c.index(begin) + len(begin):c.index(end)])


def test_integration_page_quotes_the_c_example_verbatim():
    page = (helpers.ROOT / "INTEGRATION.md").read_text()
    assert "```c\n" + _c_example_snippet() + "```" in page, "INTEGRATION.md section 5 and tests/engine_abi_example.c have drifted apart"


def test_c_example_compiles_and_links_against_the_header(tmp_path):
    """gcc (C11) against include/netra_engine.h and the built library: every call of the documented sequence exists with
    the documented argument list."""
    import subprocess
    out = tmp_path / "engine_abi_example"
    cmd = ["gcc", "-std=c11", "-Wall", "-Werror=implicit-function-declaration", "-Werror=incompatible-pointer-types",
           "-I", str(helpers.ROOT / "include"), "-I", "/usr/local/cuda/include", str(helpers.ROOT / "tests" / "engine_abi_example.c"),
           "-o", str(out), "-L", str(abi.LIB_PATH.parent), "-l:" + abi.LIB_PATH.name, "-L", "/usr/local/cuda/lib64", "-lcudart",
           "-Wl,-rpath," + str(abi.LIB_PATH.parent)]
    done = subprocess.run(cmd, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
    assert out.exists()

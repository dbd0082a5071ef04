"""Generates tests/golden/reference_stage_pins.npz by running the reference's own CPU exporters,
UNMODIFIED, on seeded synthetic operands, and keeping what they compute:

* ``tools/benchmark/export_qwen36_moe_stage1_capture.py``  -> ``reference_stage1_f32`` [9, 1024]
  (block-scaled FP8 gate_up: per K-block dequantise activation and weight, FP32 ``mv``, K-blocks ascending)
* ``tools/benchmark/export_qwen36_moe_stage2_capture.py``  -> ``reference_output_f32`` / ``_bf16`` [1, 2048]
  (block-scaled FP8 down + slot-ascending weighted sum, one BF16 rounding)
* ``tools/benchmark/export_qwen36_router_bf16_capture.py`` -> ``expected_logits_bf16`` [1, 256]
  (BF16 ``F.linear``)

Each exporter reads the small ``.pt`` / safetensors files a serving capture would hold; this script writes
those files from ``operands(case)`` below (the test regenerates the same operands from the same seeds and
checks their hash), runs the exporter's ``main()`` as it stands in the reference checkout, and reads the
binaries it wrote.  Needs the reference checkout; the committed .npz is what the tests read.

Usage: python tests/golden/make_stage_golden.py /path/to/reference
"""
import hashlib
import importlib.util
import json
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from netra_kernel_b200 import synth  # noqa: E402
from oracle import moe_ref as R      # noqa: E402

CASES = 4            # independent M=1 cases (the exporters accept exactly one token and nine slots)
ROUTER_ROWS = 96     # M=1 router calls


def operands(case: int) -> dict:
    """Seeded operands of one M=1 call: a BF16 token, nine distinct experts (eight routed + id 256 as the shared
    slot), their FP8 block-scaled W13 / W2 slabs, routing weights.  Everything a test needs to regenerate."""
    g = torch.Generator().manual_seed(7000 + case)
    hidden = torch.randn(1, 2048, generator=g).to(torch.bfloat16)
    routed = torch.randperm(256, generator=g)[:8].to(torch.int32)
    topk_ids = torch.cat([routed, torch.tensor([256], dtype=torch.int32)]).view(1, 9)      # slot order
    selected = torch.sort(topk_ids.view(-1)).values.to(torch.int32)                        # the capture keeps slabs by ascending id
    w1, w1_s, w2, w2_s = [], [], [], []
    for _ in range(9):
        q, s = synth.quantize_fp8_block128(0.02 * torch.randn(1024, 2048, generator=g))
        w1.append(q); w1_s.append(s)
        q, s = synth.quantize_fp8_block128(0.02 * torch.randn(2048, 512, generator=g))
        w2.append(q); w2_s.append(s)
    weights = torch.softmax(torch.randn(8, generator=g), 0)
    topk_w = torch.cat([weights, torch.tensor([1.0])]).to(torch.float32).view(1, 9)
    return {"hidden": hidden, "topk_ids": topk_ids, "selected": selected, "w1": torch.stack(w1), "w1_scale": torch.stack(w1_s),
            "w2": torch.stack(w2), "w2_scale": torch.stack(w2_s), "topk_w": topk_w}


def operands_sha256(ops: dict) -> str:
    h = hashlib.sha256()
    for key in sorted(ops):
        h.update(ops[key].contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def router_operands():
    g = torch.Generator().manual_seed(7100)
    hidden = torch.randn(ROUTER_ROWS, 2048, generator=g).to(torch.bfloat16)
    weight = (0.02 * torch.randn(256, 2048, generator=g)).to(torch.bfloat16)
    return hidden, weight


def load_exporter(ref_root: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, ref_root / "tools" / "benchmark" / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def run_main(mod, argv):
    old = sys.argv
    sys.argv = [mod.__name__] + [str(a) for a in argv]
    try:
        mod.main()
    finally:
        sys.argv = old


def read_bin(path: Path, dtype, shape):
    return np.frombuffer(path.read_bytes(), dtype=dtype).reshape(shape).copy()


def main() -> None:
    ref_root = Path(sys.argv[1])
    stage1 = load_exporter(ref_root, "export_qwen36_moe_stage1_capture")
    stage2 = load_exporter(ref_root, "export_qwen36_moe_stage2_capture")
    router = load_exporter(ref_root, "export_qwen36_router_bf16_capture")
    out = {}
    import contextlib
    import io
    for case in range(CASES):
        ops = operands(case)
        out[f"case{case}_operands_sha256"] = np.frombuffer(bytes.fromhex(operands_sha256(ops)), dtype=np.uint8)
        aq, a_s = R.quant_fp8_group128(R.bf16_bits_to_f32(ops["hidden"].view(torch.int16).numpy().view(np.uint16)))
        compact = {int(e): i for i, e in enumerate(ops["selected"].tolist())}
        order = [compact[int(e)] for e in ops["topk_ids"].view(-1).tolist()]
        with tempfile.TemporaryDirectory() as tmp:
            cap, dst1, dst2 = Path(tmp) / "capture", Path(tmp) / "stage1", Path(tmp) / "stage2"
            cap.mkdir()
            # the capture stores the nine selected slabs by ascending expert id
            inv = [ops["topk_ids"].view(-1).tolist().index(int(e)) for e in ops["selected"].tolist()]
            sel_w1, sel_w1_s = ops["w1"][inv].contiguous(), ops["w1_scale"][inv].contiguous()
            sel_w2, sel_w2_s = ops["w2"][inv].contiguous(), ops["w2_scale"][inv].contiguous()
            torch.save({"hidden_states_fp8": torch.from_numpy(aq).view(torch.float8_e4m3fn), "hidden_states_scale": torch.from_numpy(a_s)},
                       cap / "aiter_moe_input_quant_000.pt")
            torch.save({"stage1_fp32": torch.zeros(9, 1024)}, cap / "aiter_moe_activation_000.pt")   # only compared, never used
            call = {"selected_expert_ids_i32": ops["selected"], "topk_ids_i32": ops["topk_ids"], "selected_w1_fp8": sel_w1,
                    "selected_w1_scale": sel_w1_s, "selected_w2_fp8": sel_w2, "selected_w2_scale": sel_w2_s,
                    "topk_weights_fp32": ops["topk_w"], "output_bf16": torch.zeros(1, 2048, dtype=torch.bfloat16)}
            torch.save(call, cap / "aiter_moe_call_000.pt")
            with contextlib.redirect_stdout(io.StringIO()):
                run_main(stage1, ["--capture-dir", cap, "--output-dir", dst1])
            ref1 = read_bin(dst1 / "reference_stage1_f32.bin", np.float32, (9, 1024))
            assert json.loads((dst1 / "manifest.json").read_text())["compact_topk_ids"] == order
            # stage 2 consumes the requantised SiLU(gate) * up of the reference's own stage-1 result
            hq, h_s, _ = R.silu_mul_quant(ref1)
            torch.save({"activation_fp8": torch.from_numpy(hq).view(torch.float8_e4m3fn).view(1, 9, 512),
                        "activation_scale": torch.from_numpy(h_s).view(1, 9, 4)}, cap / "aiter_moe_quant_000.pt")
            with contextlib.redirect_stdout(io.StringIO()):
                run_main(stage2, ["--capture-dir", cap, "--output-dir", dst2])
            out[f"case{case}_stage1_f32"] = ref1
            out[f"case{case}_act_fp8"] = hq
            out[f"case{case}_act_scale"] = h_s
            out[f"case{case}_stage2_f32"] = read_bin(dst2 / "reference_output_f32.bin", np.float32, (1, 2048))
            out[f"case{case}_stage2_bf16"] = read_bin(dst2 / "reference_output_bf16.bin", np.uint16, (1, 2048))

    # router: one exporter run per row (the exporter accepts exactly one row); a tiny safetensors "checkpoint" holds the weight
    from safetensors.torch import save_file
    hidden, weight = router_operands()
    logits = np.zeros((ROUTER_ROWS, 256), np.uint16)
    with tempfile.TemporaryDirectory() as tmp:
        model = Path(tmp) / "model"
        model.mkdir()
        key = "model.language_model.layers.0.mlp.gate.weight"
        save_file({key: weight}, str(model / "model-00001.safetensors"))
        (model / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {key: "model-00001.safetensors"}}))
        for r in range(ROUTER_ROWS):
            call = Path(tmp) / f"call{r}.pt"
            torch.save({"hidden_states_bf16": hidden[r:r + 1].clone()}, call)
            dst = Path(tmp) / f"out{r}"
            run_main(router, ["--aiter-call", call, "--model-dir", model, "--layer-id", 0, "--output-dir", dst])
            logits[r] = read_bin(dst / "expected_logits_bf16.bin", np.uint16, (256,))
    out["router_logits_bf16"] = logits
    out["router_operands_sha256"] = np.frombuffer(
        hashlib.sha256(hidden.view(torch.uint8).numpy().tobytes() + weight.view(torch.uint8).numpy().tobytes()).digest(), dtype=np.uint8)
    path = Path(__file__).resolve().parent / "reference_stage_pins.npz"
    np.savez_compressed(path, **out)
    print(path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()

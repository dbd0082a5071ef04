"""Generates tests/golden/compiler_hash_kat.json by importing the REFERENCE compiler
(compiler/netra_compiler/types.py:49-56 canonical_json / stable_hash, contracts.py stable ids) and
hashing a few fixed values, so that this repository's hashing can be checked against it.

Usage: python tests/golden/make_compiler_kat.py /path/to/reference
"""
import json
import sys
from pathlib import Path


def main() -> None:
    ref = Path(sys.argv[1])
    sys.path.insert(0, str(ref / "compiler"))
    from netra_compiler.types import canonical_json, stable_hash  # type: ignore
    from netra_compiler.contracts import FixedKernelContract, KernelSemantics, Launch, Workspace  # type: ignore
    values = [
        {"b": 1, "a": [1, 2, {"z": None, "y": True}], "c": "text/é"},
        [3, 2, 1],
        {"launch": {"grid": [16, 768, 1], "block": [64, 1, 1]}, "name": "route_reduce", "rows": 768},
        "plain",
        {"nested": {"k": {"deep": [0.5, -1, "x"]}}},
    ]
    contract = FixedKernelContract(
        target="gfx950", wave_size=64, operation="moe_route_reduce", family="moe_prefill",
        constants=(("NETRA_ROWS", 768), ("NETRA_TOPK", 9)), specialization=(("NETRA_HIDDEN_SIZE", 2048),),
        semantics=KernelSemantics("abi.v1", "f16_f32_bf16", "none", "row_major", "slot_ascending.v1"),
        kernarg_size=32, symbol="sym", launch=Launch((16, 768, 1), (64, 1, 1), 0, 0), workspace=Workspace(0, 256))
    out = {
        "values": values,
        "canonical": [canonical_json(v) for v in values],
        "sha256": [stable_hash(v) for v in values],
        "contract_identity": contract.identity_dict(),
        "contract_id": contract.stable_id,
    }
    path = Path(__file__).resolve().parent / "compiler_hash_kat.json"
    path.write_text(json.dumps(out, indent=1, ensure_ascii=False) + "\n", encoding="utf-8")
    print(path, contract.stable_id)


if __name__ == "__main__":
    main()

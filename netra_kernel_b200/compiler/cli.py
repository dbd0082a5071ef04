"""``python -m netra_kernel_b200.compiler.cli {list-tactics,compile,inspect,explain,validate,lock-catalog}``
(role of the reference's ``compiler/netra_compiler/cli.py:17-69``)."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from .catalog import load_fixed_tactic_catalog, lock_catalog_sources
from .engine import compile_engine
from .library import KernelLibrary
from .types import TARGET, NetraCompilerError
from .validation import validate_engine_directory


def _parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="netra-compile")
    p.add_argument("--library-root", default=None)
    sub = p.add_subparsers(dest="command", required=True)
    sub.add_parser("list-tactics")
    sub.add_parser("lock-catalog")
    c = sub.add_parser("compile")
    c.add_argument("--model", required=True)
    c.add_argument("--profile", required=True)
    c.add_argument("--output", required=True)
    c.add_argument("--target", default=TARGET)
    c.add_argument("--allow-experimental", action="store_true")
    c.add_argument("--checkpoint-hash", default="")
    c.add_argument("--binding-sets", type=int, default=1,
                   help="emit the profile this many times: one set of bound pointers and one captured graph each, one workspace")
    for name in ("inspect", "explain", "validate"):
        s = sub.add_parser(name)
        s.add_argument("engine")
    return p


def main(argv=None) -> int:
    args = _parser().parse_args(argv)
    try:
        root = KernelLibrary.discover(args.library_root).root
        if args.command == "list-tactics":
            for t in load_fixed_tactic_catalog(root, TARGET):
                print(f"{t.name}\t{t.family}/{t.operation}\trank {t.rank}\t{t.maturity.value}\t{t.symbol}")
        elif args.command == "lock-catalog":
            lock_catalog_sources(root, TARGET)
        elif args.command == "compile":
            if args.target != TARGET:
                raise NetraCompilerError(f"this compiler emits {TARGET} engines only")
            engine = compile_engine(args.model, args.profile, args.output, library_root=root,
                                    allow_experimental=args.allow_experimental, checkpoint_hash=args.checkpoint_hash,
                                    binding_sets=args.binding_sets)
            print("engine_id", engine["engine_id"])
        elif args.command == "validate":
            engine = validate_engine_directory(args.engine)
            print("valid", engine["engine_id"])
        elif args.command == "inspect":
            engine = json.loads((Path(args.engine) / "engine.json").read_text())
            print(json.dumps({k: engine[k] for k in ("engine_id", "target", "workspace_bytes", "selected_tactics", "fallbacks")}, indent=1))
        elif args.command == "explain":
            print((Path(args.engine) / "explain.json").read_text())
    except NetraCompilerError as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 2
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

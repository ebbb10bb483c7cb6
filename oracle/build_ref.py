"""Builds ``oracle/_ref/``: the reference's own Python modules for the hot path, byte-compiled
(TEST / BENCHMARK INFRASTRUCTURE, never imported by the product).

    python -m oracle.build_ref [--reference /path/to/TAAC_2026]

The reference is Python, so its "build" is CPython's compiler: every module of ``src/taac2026`` and of
``experiments/onetrans`` is compiled from the source where it lies in the checkout into a code object,
and all of them go into ONE archive, ``oracle/_ref/reference_modules.bin`` (a marshalled table
``module name -> (is package, code)``), next to a small ``BUILD_INFO.json``.  No source file is copied;
``oracle/_ref/`` is git-ignored.  ``oracle/ref_runtime.py`` imports the modules from the archive where no
checkout is available, so that the benchmark's CPU arm and the GPU tests can run the reference's own
``PCVROneTrans`` (experiments/onetrans/model.py) and its operator dispatchers instead of a port.  Code
objects are tied to the interpreter version that wrote them; ``BUILD_INFO.json`` records it and the runtime
refuses a mismatch.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import marshal
import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
ARCHIVE = OUT / "reference_modules.bin"
PACKAGES = ("src/taac2026", "experiments/__init__.py", "experiments/onetrans")


def find_reference(explicit: str | None = None) -> Path | None:
    """The checkout named explicitly, by TAAC2026_REFERENCE, or a sibling ``reference/`` directory."""
    sibling = HERE.parent.parent / "reference"
    for candidate in (explicit, os.environ.get("TAAC2026_REFERENCE"), str(sibling)):
        if candidate and (Path(candidate) / "src" / "taac2026").is_dir():
            return Path(candidate)
    return None


def build(reference: Path | None = None, *, quiet: bool = True) -> Path | None:
    """Compile the reference's modules into ``oracle/_ref``; returns the folder, or None without a checkout."""
    root = reference or find_reference()
    if root is None:
        return None
    if OUT.exists():
        shutil.rmtree(OUT)
    OUT.mkdir(parents=True)
    table: dict[str, tuple[bool, bytes]] = {}
    for rel in PACKAGES:
        base = root / rel
        files = [base] if base.is_file() else sorted(base.rglob("*.py"))
        for src in files:
            module_path = src.relative_to(root)
            if module_path.parts[0] == "src":
                module_path = Path(*module_path.parts[1:])
            is_package = module_path.name == "__init__.py"
            parts = module_path.parts[:-1] if is_package else (*module_path.parts[:-1], module_path.stem)
            code = compile(src.read_bytes(), str(module_path), "exec", dont_inherit=True, optimize=0)
            table[".".join(parts)] = (is_package, marshal.dumps(code))
    ARCHIVE.write_bytes(marshal.dumps(table))
    info = {"modules": len(table), "python": list(sys.version_info[:3]), "magic": importlib.util.MAGIC_NUMBER.hex(),
            "packages": list(PACKAGES), "archive": ARCHIVE.name}
    (OUT / "BUILD_INFO.json").write_text(json.dumps(info, indent=1))
    if not quiet:
        print(f"compiled {len(table)} modules into {ARCHIVE}")
    return OUT


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    parser.add_argument("--reference", default=None, help="root of the reference checkout")
    args = parser.parse_args()
    if build(find_reference(args.reference), quiet=False) is None:
        raise SystemExit("no reference checkout found (pass --reference or set TAAC2026_REFERENCE)")


if __name__ == "__main__":
    main()

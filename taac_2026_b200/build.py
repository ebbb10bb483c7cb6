"""Builds ``libtb200.so`` (the C-ABI library of sm_100a kernels) in-tree with nvcc.

Run ``python -m taac_2026_b200.build`` after editing anything under ``csrc/``.  nvcc
cross-compiles for sm_100a, so this works on a machine without a GPU.  Object files are
cached under ``csrc/build/`` and rebuilt only when a source or header is newer.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD = CSRC / "build"
LIB_PATH = PKG_DIR / "libtb200.so"
INCLUDE = PKG_DIR.parent / "include"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; the tb200 kernels cannot be built")
    return nvcc


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(src: Path, verbose: bool, ptxas_info: bool) -> Path:
    obj = BUILD / (src.stem + ".o")
    if not _stale(obj, [src, *_headers(), Path(__file__)]):
        return obj
    cmd = [_nvcc(), *ARCH_FLAGS, *COMMON_FLAGS, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
    if ptxas_info:
        cmd += ["-Xptxas", "-v"]
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    if ptxas_info:
        print(proc.stderr, flush=True)
    return obj


def build(*, verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libtb200.so``.  Returns its path."""
    BUILD.mkdir(parents=True, exist_ok=True)
    if force:
        for obj in BUILD.glob("*.o"):
            obj.unlink()
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose, ptxas_info), srcs))
    if force or _stale(LIB_PATH, objs):
        cmd = [_nvcc(), *ARCH_FLAGS, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-lcudart"]
        if verbose:
            print(" ".join(cmd), flush=True)
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)

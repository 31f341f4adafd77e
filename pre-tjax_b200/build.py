"""Builds csrc/*.cu into one shared library next to this file, for sm_100a only.

Usage: ``python pre-tjax_b200/build.py [--force] [--verbose]``. The library (``libptj_b200.so``) exports the C ABI
declared in ``include/ptj_b200.h`` and is what the Python operators load with ctypes. Object files are rebuilt only
when a source or header is newer.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libptj_b200.so"
INCLUDE_DIR = PKG_DIR.parent / "include"

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler", "-fPIC",  # no --use_fast_math: the parity tolerances are tight
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build the sm_100a kernels")
    return exe


def _newest_header_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE_DIR.glob("*.h"))
    return max(h.stat().st_mtime for h in hdrs)


def _compile_one(src: Path, verbose: bool, ptxas_info: bool) -> str:
    obj = OBJ_DIR / (src.stem + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(INCLUDE_DIR), "-c", str(src), "-o", str(obj)]
    if ptxas_info:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose or ptxas_info:
        return f"== {src.name}\n{res.stderr}"
    return ""


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    OBJ_DIR.mkdir(exist_ok=True)
    hdr_m = _newest_header_mtime()
    stale = []
    for s in sources:
        obj = OBJ_DIR / (s.stem + ".o")
        if force or ptxas_info or not obj.exists() or obj.stat().st_mtime < max(s.stat().st_mtime, hdr_m):
            stale.append(s)
    logs = []
    if stale:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(stale))) as pool:
            logs = list(pool.map(lambda s: _compile_one(s, verbose, ptxas_info), stale))
    objs = [OBJ_DIR / (s.stem + ".o") for s in sources]
    if stale or not LIB_PATH.exists():
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB_PATH), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    for l in logs:
        if l:
            print(l)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)

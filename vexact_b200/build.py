"""Builds libvexact_b200.so (sm_100a only) in-tree with nvcc.

The library is one translation unit (csrc/lib.cu).  It links the CUDA runtime
statically and does not link libcuda, so it can be loaded, and its symbols
listed, on a machine without a GPU.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OUT_DIR = PKG_DIR / "_C"
LIB_PATH = OUT_DIR / "libvexact_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
    "-cudart", "static",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else "nvcc"


def _source_hash() -> str:
    h = hashlib.sha256()
    for p in sorted(CSRC.iterdir()):
        if p.suffix in (".cu", ".cuh"):
            h.update(p.name.encode())
            h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def built_hash() -> str | None:
    """Source hash compiled into the library on disk (b200_source_hash), None when there is none."""
    if not LIB_PATH.exists():
        return None
    try:
        import ctypes

        lib = ctypes.CDLL(str(LIB_PATH))
        fn = lib.b200_source_hash
        fn.restype = ctypes.c_char_p
        return fn().decode()
    except (OSError, AttributeError):
        return None


def sources_present() -> bool:
    return (CSRC / "lib.cu").exists()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library unless the one on disk was built from exactly these sources; return its path.

    The hash of the sources and flags is compiled into the library itself, so a stale library (sources
    updated by a checkout, library left over from before) is recognised whatever files sit beside it."""
    OUT_DIR.mkdir(exist_ok=True)
    want = _source_hash()
    if not force and built_hash() == want:
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, f'-DB200_SOURCE_HASH="{want}"', "-I", str(CSRC), str(CSRC / "lib.cu"), "-o",
           str(LIB_PATH)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
        print(" ".join(cmd), file=sys.stderr)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(res.stderr, file=sys.stderr)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

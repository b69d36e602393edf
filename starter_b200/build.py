"""Builds libqdecode.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

The library is plain C ABI: no torch headers, so it compiles in seconds and can
be loaded with ctypes from any host language.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = Path(os.environ.get("QDECODE_LIB", ROOT / "libqdecode.so"))
SOURCES = ["capi.cu", "gemm_streamk.cu", "gemm_tc.cu", "fused_ops.cu", "attention.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-DQDECODE_BUILD",
    "-Xcompiler", "-fPIC,-O2,-Wall",
    "-shared",
]


def _stale() -> bool:
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [ROOT.parent / "include" / "qdecode.h"]
    return any(p.stat().st_mtime > built for p in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if any source is newer than it. Returns its path."""
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS, *os.environ.get("QDECODE_NVCC_EXTRA", "").split()]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(CSRC / s) for s in SOURCES] + ["-o", str(LIB)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

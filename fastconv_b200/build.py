"""In-tree build of libfastconv_b200.so (hand-written CUDA for sm_100a behind a C ABI).

nvcc cross-compiles without a GPU, so this runs on a CPU-only machine as well.  The shared
object is written next to this file; it links the CUDA runtime statically and resolves the
driver API at run time, so it loads (and its symbols can be listed) on a machine with no GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libfastconv_b200.so"

SOURCES = [
    "fc_capi.cu",
    "fc_wino_transforms.cu",
    "fc_wino_gemm_ffma.cu",
    "fc_igemm_ffma.cu",
    "fc_gemm_tc.cu",
    "fc_igemm_tc.cu",
    "fc_direct_tc.cu",
    "fc_static_scratch.cu",
    "fc_peer.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-O2,-Wall,-Wno-unused-function",
    "-shared", "-cudart", "static",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: cannot build libfastconv_b200.so")
    return cand


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    lib_mtime = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh"))
    deps.append(PKG_DIR.parent / "include" / "fastconv_b200.h")
    return any(p.stat().st_mtime > lib_mtime for p in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source into libfastconv_b200.so; returns its path."""
    if not force and not needs_build():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, "-o", str(LIB_PATH), *[str(CSRC / s) for s in SOURCES]]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd), file=sys.stderr)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stderr, file=sys.stderr)
    return LIB_PATH


if __name__ == "__main__":
    build_library(force=True, verbose="-v" in sys.argv)
    print(LIB_PATH)

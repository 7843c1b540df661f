"""In-tree build of libfastconv_b200.so (hand-written CUDA for sm_100a behind a C ABI).

nvcc cross-compiles without a GPU, so this runs on a CPU-only machine as well.  The shared
object is written next to this file; it links the CUDA runtime statically and resolves the
driver API at run time, so it loads (and its symbols can be listed) on a machine with no GPU.
"""
from __future__ import annotations

import fcntl
import hashlib
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
    "fc_comm.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-O2,-Wall,-Wno-unused-function",
    "-shared", "-cudart", "static", "-ldl",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: cannot build libfastconv_b200.so")
    return cand


HASH_PATH = PKG_DIR / "libfastconv_b200.srchash"  # digest of the sources the library was built from


def _dependencies():
    deps = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))
    deps.append(PKG_DIR.parent / "include" / "fastconv_b200.h")
    return deps


def source_digest() -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for p in _dependencies():
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def needs_build() -> bool:
    """True when the library is missing or was built from other sources than those on disk.  Decided by content, not
    by modification time: a copy of the tree to another machine keeps the contents but not necessarily the times."""
    if not LIB_PATH.exists() or not HASH_PATH.exists():
        return True
    return HASH_PATH.read_text().strip() != source_digest()


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source into libfastconv_b200.so; returns its path.  Processes that race here (one per GPU
    under a launcher) take turns on a lock file, and all but the first find the work done."""
    if not force and not needs_build():
        return LIB_PATH
    with open(PKG_DIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not needs_build():
            return LIB_PATH
        tmp = LIB_PATH.with_suffix(".so.tmp%d" % os.getpid())
        cmd = [_nvcc(), *NVCC_FLAGS, "-o", str(tmp), *[str(CSRC / s) for s in SOURCES]]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), file=sys.stderr)
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            if tmp.exists():
                tmp.unlink()
            raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
        if verbose:
            print(proc.stderr, file=sys.stderr)
        os.replace(tmp, LIB_PATH)
        HASH_PATH.write_text(source_digest() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    build_library(force=True, verbose="-v" in sys.argv)
    print(LIB_PATH)

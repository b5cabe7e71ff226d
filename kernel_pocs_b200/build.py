"""Builds the native library in-tree with nvcc for sm_100a.

    python -m kernel_pocs_b200.build [--force] [--verbose]

Output: kernel_pocs_b200/libswiglu_b200.so, a plain C-ABI shared library (it links the CUDA
runtime statically and knows nothing about PyTorch).  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
INCLUDE = ROOT / "include"
LIB_PATH = PKG / "libswiglu_b200.so"
STAMP_PATH = PKG / "libswiglu_b200.so.stamp"  # digest of the sources the library was built from

SOURCES = [CSRC / "swiglu_capi.cu", CSRC / "swiglu_host.cu", CSRC / "swiglu_gemm.cu", CSRC / "swiglu_gemm_bwd.cu", CSRC / "swiglu_lora.cu",
           CSRC / "swiglu_selftest.cu"]
HEADERS = [CSRC / "swiglu_kernels.cuh", CSRC / "tcgen05_common.cuh", INCLUDE / "swiglu_b200.h"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-shared",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: the swiglu_b200 library cannot be built")
    return exe


def source_digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for p in SOURCES + HEADERS:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def is_stale() -> bool:
    """True when the library is missing or was built from other sources (compared by content,
    because file times do not survive a copy of the tree to another machine)."""
    if not (LIB_PATH.exists() and STAMP_PATH.exists()):
        return True
    return STAMP_PATH.read_text().strip() != source_digest()


def build(force: bool = False, verbose: bool = False, extra_flags: list[str] | None = None) -> Path:
    """Compiles the library if it is missing or older than its sources; returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, f"-I{INCLUDE}", f"-I{CSRC}"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += list(extra_flags or [])
    tmp = LIB_PATH.with_suffix(f".so.tmp{os.getpid()}")
    cmd += [*map(str, SOURCES), "-o", str(tmp)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, LIB_PATH)
    stamp_tmp = STAMP_PATH.with_suffix(f".stamp.tmp{os.getpid()}")
    stamp_tmp.write_text(source_digest() + "\n")
    os.replace(stamp_tmp, STAMP_PATH)
    if verbose:
        sys.stderr.write(proc.stderr)
    return LIB_PATH


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="pass -Xptxas -v and print registers/spills")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose))


if __name__ == "__main__":
    main()

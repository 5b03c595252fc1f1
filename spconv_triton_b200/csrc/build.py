"""Builds libspconv_b200.so in place with nvcc for sm_100a.

    python -m spconv_triton_b200.csrc.build [--force] [--verbose]

The shared library is a plain C-ABI CUDA library (no Python, no torch
headers); it is loaded with ctypes by ``spconv_triton_b200._lib``.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
SOURCES = ["capi.cu", "rulebook.cu", "gemm_simt.cu", "gemm_tc.cu", "gemm_tma.cu", "gemm_wgrad_tc.cu", "gemm.cu", "pool.cu", "voxelize.cu", "dense.cu", "hash.cu", "global_pool.cu", "from_dense.cu", "tf32_prep.cu", "sequence.cu"]
LIB = HERE / "libspconv_b200.so"
STAMP = HERE / "build" / "sources.sha256"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build libspconv_b200.so")
    return exe


def _sources():
    return [s for s in SOURCES if (HERE / s).exists()]


def _digest() -> str:
    h = hashlib.sha256()
    files = sorted(HERE.glob("*.cu")) + sorted(HERE.glob("*.cuh")) + [HERE.parent.parent / "include" / "spconv_b200.h"]
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    digest = _digest()
    if not force and LIB.exists() and STAMP.exists() and STAMP.read_text() == digest:
        return LIB
    nvcc = _nvcc()
    objdir = HERE / "build"
    objdir.mkdir(exist_ok=True)

    def compile_one(src: str) -> Path:
        obj = objdir / (Path(src).stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(HERE / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose and res.stderr:
            print(res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, _sources()))
    cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    STAMP.write_text(digest)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)

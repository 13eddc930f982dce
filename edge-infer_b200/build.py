"""Builds the sm_100a shared library in-tree with nvcc (cross-compiles without a GPU).

    python edge-infer_b200/build.py            # incremental
    python edge-infer_b200/build.py --force

Output: edge-infer_b200/libedge_infer_b200.so (git-ignored; it travels with the tree).
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
LIB = HERE / "libedge_infer_b200.so"
SOURCES = ["abi_ops.cu", "smallm_gemm.cu", "prompt_gemm.cu", "elementwise.cu", "attention.cu", "sampling.cu", "runtime.cu"]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
]


def _newest_dependency() -> float:
    paths = list(CSRC.glob("*")) + [HERE.parent / "include" / "edge_infer_b200.h", Path(__file__)]
    return max(p.stat().st_mtime for p in paths)


def _compile(source: str, verbose: bool) -> None:
    out = OBJ / (source + ".o")
    cmd = [NVCC, *FLAGS, "-c", str(CSRC / source), "-o", str(out)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    result = subprocess.run(cmd, capture_output=True, text=True)
    if verbose and result.stderr:
        (OBJ / (source + ".ptxas.txt")).write_text(result.stderr)
    if result.returncode:
        raise RuntimeError(f"nvcc failed for {source}:\n{result.stdout}\n{result.stderr}")


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every CUDA source for sm_100a and links the shared library."""
    if not force and LIB.exists() and LIB.stat().st_mtime >= _newest_dependency():
        return LIB
    OBJ.mkdir(exist_ok=True)
    stale = [s for s in SOURCES
             if force or not (OBJ / (s + ".o")).exists() or (OBJ / (s + ".o")).stat().st_mtime < _newest_dependency()]
    with ThreadPoolExecutor(max_workers=min(8, len(stale) or 1)) as pool:
        list(pool.map(lambda s: _compile(s, verbose), stale))
    objects = [str(OBJ / (s + ".o")) for s in SOURCES]
    link = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB), *objects,
            "-lcudart"]
    result = subprocess.run(link, capture_output=True, text=True)
    if result.returncode:
        raise RuntimeError(f"link failed:\n{result.stdout}\n{result.stderr}")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)

"""Builds libcamel_tensor_b200.so in-tree with nvcc for sm_100a.

    python -m camel_b200.build [--force] [--verbose]

The library is plain CUDA runtime code: no torch, no cuBLAS/cuDNN, no libcuda at link time.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
INCLUDE = ROOT.parent / "include"
OBJ_DIR = ROOT / "build"
LIB = ROOT / "libcamel_tensor_b200.so"

SOURCES = ["runtime.cu", "elementwise.cu", "reduce.cu", "gemm_simt.cu", "gemm_tc.cu", "contract.cu",
           "graph.cu", "peak.cu", "conv_tmem.cu", "conv_halo.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--fmad=false",            # the reference computes a*b then +: never contract
    "-I", str(INCLUDE), "-I", str(CSRC),
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(d).stat().st_mtime <= t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    headers = list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    OBJ_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    for src in SOURCES:
        s = CSRC / src
        o = OBJ_DIR / (s.stem + ".o")
        if force or not _newer(o, [s, *headers]):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(s), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    with ThreadPoolExecutor(max_workers=max(1, min(8, len(jobs) or 1))) as ex:
        for log in ex.map(run, jobs):
            if verbose and log:
                print(log)
    objs = [str(OBJ_DIR / (Path(s).stem + ".o")) for s in SOURCES]
    if force or jobs or not LIB.exists():
        run([nvcc, "-shared", "-o", str(LIB), *objs, "-lcudart_static", "-lpthread", "-ldl", "-lrt"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

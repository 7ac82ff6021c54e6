"""Build libpiper_b200.so in-tree with nvcc for sm_100a.

Usage: ``python -m piper_kernels_b200.csrc.build [--force] [--verbose]``.  The shared library
is written next to the package (``piper_kernels_b200/libpiper_b200.so``); it links only the
CUDA runtime (the driver's tensor-map encoder is resolved at run time).
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
LIB = PKG / "libpiper_b200.so"
SOURCES = ["cabi.cu", "prepass.cu", "fused_attention.cu"]
HEADERS = ["pk_internal.h", "pk_ptx.cuh", "../../include/piper_b200.h"]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC")
    return cand


def stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = [CSRC / s for s in SOURCES + HEADERS] + [Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not stale():
        return LIB
    objs = []
    common = [
        "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
        "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    ]
    if verbose:
        common += ["-Xptxas", "-v"]
    procs = []
    for src in SOURCES:
        obj = CSRC / (Path(src).stem + ".o")
        cmd = [nvcc_path(), *common, "-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        if out.strip() and (verbose or pr.returncode):
            print(f"--- {src}\n{out}", file=sys.stderr)
        failed |= pr.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    link = [nvcc_path(), "-shared", "-o", str(LIB), *objs, "-cudart", "shared"]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))

"""Builds libgranite_cuda.so in-tree with nvcc for sm_100a (the only target).

Usage: ``python -m granite_b200.build [--force] [--verbose]``.  Each ``csrc/*.cu`` is compiled to
an object next to it and the objects are linked into ``granite_b200/libgranite_cuda.so``.
A file is recompiled when it, or any header in ``csrc/`` or ``include/``, is newer than its object.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
LIB = PKG / "libgranite_cuda.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
    "-Xptxas", "-v",
    f"-I{INCLUDE}",
] + os.environ.get("GB_EXTRA_NVCC_FLAGS", "").split()


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    return cand if Path(cand).exists() else "nvcc"


def _newest_header() -> float:
    hdrs = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")) + list(INCLUDE.glob("*.h"))
    return max((h.stat().st_mtime for h in hdrs), default=0.0)


def build(force: bool = False, verbose: bool = False) -> Path:
    sources = sorted(CSRC.glob("*.cu")) + sorted((CSRC / "host").glob("*.cpp") if (CSRC / "host").exists() else [])
    hdr_time = _newest_header()
    jobs = []
    objs = []
    for src in sources:
        obj = src.with_suffix(".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [_nvcc(), *NVCC_FLAGS, "-x", "cu", "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        return src, res

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            for src, res in pool.map(compile_one, jobs):
                if verbose or res.returncode != 0:
                    sys.stderr.write(f"--- {src.name}\n{res.stdout}{res.stderr}\n")
                if res.returncode != 0:
                    raise RuntimeError(f"nvcc failed on {src}")
    if jobs or force or not LIB.exists():
        cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            sys.stderr.write(res.stdout + res.stderr)
            raise RuntimeError("link of libgranite_cuda.so failed")
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))

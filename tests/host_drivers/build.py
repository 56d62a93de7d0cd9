"""Builds and loads the extern "C" test drivers of the C++ host faces (host_capi.cpp).

TEST CODE.  Two libraries come out of the same driver source:

  libgranite_host_drivers.so   (here) the drivers over the host classes that ship inside
                               granite_b200/libgranite_cuda.so, whose vocabulary (Error, Tensor,
                               IComputeBackend, OperatorRegistry ...) is the restatement in granite_host.h
  oracle/_ref/libgranite_dropin.so
                               (only where the Granite checkout is present; built by oracle/Makefile)
                               the SAME class bodies and drivers compiled against Granite's real headers,
                               -DGRANITE_WITH_REFERENCE_HEADERS, and linked with Granite's own
                               src/core/{tensor,error,operator_registry}.cpp: CudaBackend derives from the
                               real IComputeBackend, CudaAttentionOp from the real IOperator, and the
                               operator is created through the real OperatorRegistry.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
SRC = HERE / "host_capi.cpp"
LIB = HERE / "libgranite_host_drivers.so"
DROPIN = ROOT / "oracle" / "_ref" / "libgranite_dropin.so"
PRODUCT = ROOT / "granite_b200" / "libgranite_cuda.so"


def build(force: bool = False) -> Path:
    newest = max(p.stat().st_mtime for p in [SRC, ROOT / "granite_b200/csrc/host/granite_host.h", PRODUCT])
    if force or not LIB.exists() or LIB.stat().st_mtime < newest:
        cmd = ["g++", "-O1", "-std=c++20", "-fPIC", "-shared", "-Wall", f"-I{ROOT / 'granite_b200/csrc/host'}",
               "-I/usr/local/cuda/include", "-o", str(LIB), str(SRC), f"-L{PRODUCT.parent}", "-lgranite_cuda",
               "-Wl,-rpath,$ORIGIN/../../granite_b200"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("host test drivers failed to build:\n" + res.stdout + res.stderr)
    return LIB


def dropin_available() -> bool:
    return DROPIN.exists()


def load(variant: str = "standin") -> C.CDLL:
    """variant "standin": the drivers over the product library's classes; "reference_headers": the
    library built against Granite's real headers (raises FileNotFoundError where it was not built)."""
    import granite_b200  # noqa: F401  (loads the product library first; both variants call its C ABI)
    if variant == "standin":
        return C.CDLL(str(build()))
    if not DROPIN.exists():
        raise FileNotFoundError(f"{DROPIN} was not built (needs the Granite checkout)")
    return C.CDLL(str(DROPIN))


if __name__ == "__main__":
    print(build(force=True))

"""B200-native attention backend for Granite: hand-written sm_100a kernels behind a C ABI.

The product is ``libgranite_cuda.so`` (built from ``csrc/`` by ``granite_b200.build``) and the
header ``include/granite_cuda.h``.  This package is the thin ctypes binding used by the tests and
the benchmark; importing it never falls back to a CPU implementation - if the library is missing
the import fails.
"""
from .capi import (  # noqa: F401
    ErrorCode,
    GraniteCudaError,
    CudaCompute,
    lib,
    library_path,
)

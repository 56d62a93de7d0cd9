"""B200-native attention backend for Granite: hand-written sm_100a kernels behind a C ABI.

The product is ``libgranite_cuda.so`` (built from ``csrc/`` by ``python -m granite_b200.build``)
and the header ``include/granite_cuda.h``.  This package is the thin ctypes binding used by the
tests and the benchmark.  The binding is loaded on first use of any public name; if the library
is missing that use raises ImportError - there is no CPU or Python implementation to fall back to.
"""
_PUBLIC = ("ErrorCode", "GraniteCudaError", "CudaCompute", "lib", "library_path", "last_error", "check")


def __getattr__(name):
    if name in _PUBLIC:
        from . import capi
        return getattr(capi, name)
    raise AttributeError(f"module 'granite_b200' has no attribute {name!r}")


def __dir__():
    return sorted(list(globals()) + list(_PUBLIC))

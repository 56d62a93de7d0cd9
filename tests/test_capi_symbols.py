"""The C-ABI library loads without a GPU and exports every function include/*.h declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    names = []
    for hdr in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", hdr.read_text(), flags=re.S)
        names += re.findall(r"\b(granite_cuda_\w+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_expected_surface():
    names = declared_functions()
    assert "granite_cuda_batched_paged_attention_decode" in names
    assert "granite_cuda_multihead_attention" in names
    assert len(names) >= 15


def test_library_exports_every_declared_symbol():
    import granite_b200 as g
    lib = ctypes.CDLL(str(g.library_path()))
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, missing


def test_no_cpu_fallback_without_a_device():
    import granite_b200 as g
    if g.lib.granite_cuda_device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(g.GraniteCudaError) as ei:
        g.CudaCompute(0)
    assert ei.value.code == g.ErrorCode.BackendNotInitialized
    assert "no CPU fallback" in str(ei.value)


def test_error_codes_follow_the_reference_enum_order():
    import granite_b200 as g
    # include/granite/error.h:16-57
    assert [g.ErrorCode.Success, g.ErrorCode.OutOfMemory, g.ErrorCode.Timeout, g.ErrorCode.InvalidArgument,
            g.ErrorCode.NotImplemented] == [0, 4, 12, 16, 25]

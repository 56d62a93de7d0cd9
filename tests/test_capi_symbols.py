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


def test_ctypes_structures_match_the_header(tmp_path):
    """Every argument struct of the C ABI, as the header lays it out (compiled with the host C
    compiler), against the ctypes mirror the tests and the benchmark pass: same size, same field
    offsets."""
    import shutil
    import subprocess
    import granite_b200.capi as capi
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    pairs = {"GraniteCudaPagedDecodeArgs": capi.PagedDecodeArgs, "GraniteCudaAttentionArgs": capi.AttentionArgs,
             "GraniteCudaTreeAttentionArgs": capi.TreeAttentionArgs, "GraniteCudaKvAppendArgs": capi.KvAppendArgs,
             "GraniteCudaPagedKvAppendArgs": capi.PagedKvAppendArgs, "GraniteCudaRopeAppendArgs": capi.RopeAppendArgs,
             "GraniteCudaTreeCommitArgs": capi.TreeCommitArgs, "GraniteCudaPagedPrefillArgs": capi.PagedPrefillArgs,
             "GraniteCudaKernelTiming": capi.KernelTiming}
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "granite_cuda.h"', "int main(void) {"]
    for cname, cls in pairs.items():
        lines.append(f'  printf("{cname} %zu\\n", sizeof({cname}));')
        for fname, _ in cls._fields_:
            lines.append(f'  printf("{cname}.{fname} %zu\\n", offsetof({cname}, {fname}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([cc, "-std=c11", f"-I{ROOT / 'include'}", str(src), "-o", str(exe)], check=True)
    out = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for cname, cls in pairs.items():
        assert int(out[cname]) == ctypes.sizeof(cls), cname
        for fname, _ in cls._fields_:
            assert int(out[f"{cname}.{fname}"]) == getattr(cls, fname).offset, f"{cname}.{fname}"


def test_product_library_carries_no_test_drivers():
    """The extern "C" drivers of the C++ host faces are test code: they live in their own library beside the
    tests, and the product library exports none of them."""
    import subprocess
    import granite_b200 as g
    from granite_b200 import capi
    names = subprocess.run(["nm", "-D", "--defined-only", str(capi.library_path())], capture_output=True, text=True).stdout
    assert "granite_cuda_compute_create" in names
    assert "granite_host_" not in names

"""The allocation-free paged decode entry point.

It serves hosts that cannot let this library allocate device memory - a serving process whose own
arena already owns the GPU's memory, or a loop that cannot afford the device-wide synchronisation
inside cudaMalloc/cudaFree - by keeping its scratch in a fixed array inside the library.  The
test calls it through the C ABI twice in a row (a large batch, then a smaller one, so the second
call runs over the first call's leftovers in the shared array) and compares each output with the
regular entry point's output on the same inputs, within the path's tolerance.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test.
"""
import numpy as np
import pytest

from conftest import assert_attention_close
from granite_b200 import synth


def _device_case(case):
    import torch
    dev = "cuda:0"
    return dict(
        q=torch.from_numpy(case.q).to(dev), k=torch.from_numpy(case.k_pool).to(dev),
        v=torch.from_numpy(case.v_pool).to(dev), tables=torch.from_numpy(case.tables).to(dev),
        lens=torch.from_numpy(case.seq_lens).to(dev))


@pytest.mark.gpu
def test_static_scratch_decode_matches_regular_entry_point_twice(compute):
    import torch
    from granite_b200 import capi
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1.0 / np.sqrt(128.0)
    cases = [
        synth.paged_case(seed=41, batch=9, len_lo=1, len_hi=6000, num_heads=32, num_kv_heads=8),
        synth.paged_case(seed=42, batch=3, len_lo=1, len_hi=300, num_heads=64, num_kv_heads=8),
    ]
    for case in cases:
        d = _device_case(case)
        shape = (case.batch, case.num_heads, case.head_dim)
        want = torch.zeros(shape, device="cuda:0")
        compute.batched_paged_attention_decode(d["q"], d["k"], d["v"], d["tables"], d["lens"], want, case.batch,
                                               case.num_heads, case.num_kv_heads, case.head_dim, synth.PAGE,
                                               case.max_blocks, scale, num_blocks=case.num_blocks)
        compute.sync()
        got = torch.full(shape, float("nan"), device="cuda:0")
        status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        capi.batched_paged_attention_decode_static(d["q"], d["k"], d["v"], d["tables"], d["lens"], got, case.batch,
                                                   case.num_heads, case.num_kv_heads, case.head_dim, synth.PAGE,
                                                   case.max_blocks, scale, num_blocks=case.num_blocks,
                                                   stream=stream, device_status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert_attention_close(got.cpu().numpy(), want.cpu().numpy(), f"static scratch, batch {case.batch}")


def test_static_scratch_decode_rejects_sizes_beyond_its_fixed_array():
    """The limits are checked before anything touches a device, so this runs anywhere."""
    import granite_b200 as g
    from granite_b200 import capi
    dummy = 256  # never dereferenced: the call is refused first
    for kw, word in ((dict(batch_size=4097), "batch_size"), (dict(num_heads=128, num_kv_heads=8), "num_heads")):
        a = dict(batch_size=4, num_heads=32, num_kv_heads=8)
        a.update(kw)
        with pytest.raises(g.GraniteCudaError) as ei:
            capi.batched_paged_attention_decode_static(dummy, dummy, dummy, dummy, dummy, dummy, a["batch_size"],
                                                       a["num_heads"], a["num_kv_heads"], 128, 16, 8, 0.1, num_blocks=8)
        assert ei.value.code == g.ErrorCode.BufferTooSmall
        assert word in str(ei.value) and "max" in str(ei.value)

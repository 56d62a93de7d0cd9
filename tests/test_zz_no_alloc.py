"""The allocation-free paged decode entry point.

It serves hosts that cannot let this library allocate device memory - a serving process whose own
arena already owns the GPU's memory, or a loop that cannot afford the device-wide synchronisation
inside cudaMalloc/cudaFree - by keeping its scratch in a fixed array inside the library.  The
tests call it through the C ABI several times in a row, ordered so that every call runs over the
leftovers of a different kind of call in the shared array (a large batch whose cut sequences are
merged inside the decode kernel, the same batch again, a skewed batch with empty sequences, two
small batches that use the separate merge pass), and compare each output with the regular entry
point's output on the same inputs and with the CPU checker, within the path's tolerance.

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


def _free_bytes() -> int:
    """Free device memory as the driver reports it (cudaMemGetInfo): memory that torch's caching
    allocator already holds counts as used, so only a real allocation or release moves it."""
    import torch
    return int(torch.cuda.mem_get_info(0)[0])


def _oracle(case):
    from oracle import pyoracle
    ref, bad = pyoracle.paged_decode_batch(case.q, case.k_pool.view(np.uint16), case.v_pool.view(np.uint16),
                                           np.where(case.tables < 0, 0, case.tables), case.seq_lens, synth.PAGE)
    assert bad == 0
    return ref


def _cases():
    rng = np.random.default_rng(77)
    skewed = rng.integers(0, 120, size=44).astype(np.int32)
    skewed[5] = 9000   # cut by most CTAs: tens of partials for one sequence
    skewed[0] = 0
    skewed[31] = 0
    return [
        # >= 37 sequences (batch * head tiles * 4 >= 148): cut sequences are merged inside the decode
        # kernel, which counts finished pages in the shared array
        ("sixty mid-sized", synth.paged_case(seed=43, batch=60, len_lo=200, len_hi=1500)),
        ("forty, after a larger batch", synth.paged_case(seed=44, batch=40, len_lo=100, len_hi=900)),
        ("forty again", synth.paged_case(seed=44, batch=40, len_lo=100, len_hi=900)),
        ("skewed with empty sequences", synth.paged_case(seed=45, batch=len(skewed), len_lo=0, len_hi=0,
                                                         seq_lens=skewed)),
        # small batches take the separate merge pass
        ("nine", synth.paged_case(seed=41, batch=9, len_lo=1, len_hi=6000, num_heads=32, num_kv_heads=8)),
        ("three, 64 heads", synth.paged_case(seed=42, batch=3, len_lo=1, len_hi=300, num_heads=64, num_kv_heads=8)),
        ("forty once more", synth.paged_case(seed=44, batch=40, len_lo=100, len_hi=900)),
        # two and one KV heads: the warps of a head share its pages and exchange their state in shared memory
        ("fifty, two KV heads", synth.paged_case(seed=48, batch=50, len_lo=0, len_hi=700, num_heads=16, num_kv_heads=2)),
        ("five, one KV head", synth.paged_case(seed=49, batch=5, len_lo=1, len_hi=3000, num_heads=8, num_kv_heads=1)),
    ]


@pytest.mark.gpu
def test_static_scratch_decode_matches_regular_entry_point_and_cpu_checker(compute):
    import torch
    from granite_b200 import capi
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1.0 / np.sqrt(128.0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    for i, (name, case) in enumerate(_cases()):
        d = _device_case(case)
        shape = (case.batch, case.num_heads, case.head_dim)
        want = torch.zeros(shape, device="cuda:0")
        compute.batched_paged_attention_decode(d["q"], d["k"], d["v"], d["tables"], d["lens"], want, case.batch,
                                               case.num_heads, case.num_kv_heads, case.head_dim, synth.PAGE,
                                               case.max_blocks, scale, num_blocks=case.num_blocks)
        compute.sync()
        got = torch.full(shape, float("nan"), device="cuda:0")
        status.zero_()
        torch.cuda.synchronize()
        before = _free_bytes()
        capi.batched_paged_attention_decode_static(d["q"], d["k"], d["v"], d["tables"], d["lens"], got, case.batch,
                                                   case.num_heads, case.num_kv_heads, case.head_dim, synth.PAGE,
                                                   case.max_blocks, scale, num_blocks=case.num_blocks,
                                                   stream=stream, device_status=status)
        torch.cuda.synchronize()
        after = _free_bytes()
        if i > 0:
            # the first call on a device may load the kernels' module; no later call moves free memory
            assert after == before, f"{name}: free device memory moved by {before - after} bytes"
        assert int(status.item()) == 0
        got_np = got.cpu().numpy()
        assert_attention_close(got_np, want.cpu().numpy(), f"static scratch vs regular entry, {name}")
        assert_attention_close(got_np, _oracle(case), f"static scratch vs CPU checker, {name}")
        for b, n in enumerate(case.seq_lens):
            if n == 0:
                assert not got_np[b].any()


@pytest.mark.gpu
def test_static_scratch_decode_after_a_regular_call_with_a_smaller_window(compute):
    """A regular call with one KV head uses small page slots; the allocation-free call that follows
    needs the kernels' full shared-memory window and must still launch."""
    import torch
    from granite_b200 import capi
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    scale = 1.0 / np.sqrt(128.0)
    big = synth.paged_case(seed=46, batch=12, len_lo=50, len_hi=2000)
    small = synth.paged_case(seed=47, batch=4, len_lo=1, len_hi=500, num_heads=8, num_kv_heads=1)
    ref = _oracle(big)
    for _ in range(2):
        d = _device_case(small)
        out = torch.zeros((small.batch, small.num_heads, small.head_dim), device="cuda:0")
        compute.batched_paged_attention_decode(d["q"], d["k"], d["v"], d["tables"], d["lens"], out, small.batch,
                                               small.num_heads, small.num_kv_heads, small.head_dim, synth.PAGE,
                                               small.max_blocks, scale, num_blocks=small.num_blocks)
        compute.sync()
        assert_attention_close(out.cpu().numpy(), _oracle(small), "regular entry, one KV head")
        d = _device_case(big)
        got = torch.full((big.batch, big.num_heads, big.head_dim), float("nan"), device="cuda:0")
        status = torch.zeros(1, dtype=torch.int32, device="cuda:0")
        capi.batched_paged_attention_decode_static(d["q"], d["k"], d["v"], d["tables"], d["lens"], got, big.batch,
                                                   big.num_heads, big.num_kv_heads, big.head_dim, synth.PAGE,
                                                   big.max_blocks, scale, num_blocks=big.num_blocks,
                                                   stream=stream, device_status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert_attention_close(got.cpu().numpy(), ref, "static scratch after a one-KV-head call")


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


def test_static_scratch_decode_rejects_shapes_outside_its_kernels():
    """head_dim 64, other page sizes and odd KV-head counts are served by the regular entry point only."""
    import granite_b200 as g
    from granite_b200 import capi
    dummy = 256
    for kw in (dict(head_dim=64), dict(block_size=32), dict(num_heads=12, num_kv_heads=3)):
        a = dict(num_heads=32, num_kv_heads=8, head_dim=128, block_size=16)
        a.update(kw)
        with pytest.raises(g.GraniteCudaError) as ei:
            capi.batched_paged_attention_decode_static(dummy, dummy, dummy, dummy, dummy, dummy, 4, a["num_heads"],
                                                       a["num_kv_heads"], a["head_dim"], a["block_size"], 8, 0.1,
                                                       num_blocks=8)
        assert ei.value.code == g.ErrorCode.InvalidArgument

"""After one warm-up call the attention entry points are pure kernel launches on the compute object's
stream, so a serving loop can capture them into a CUDA graph and replay it: the replay must give the
direct call's result."""
import numpy as np
import pytest

from conftest import assert_attention_close
from granite_b200 import synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_decode_prefill_and_tree_calls_replay_from_a_graph():
    import torch
    import granite_b200 as g
    from test_tree_verify import _tree_inputs
    side = torch.cuda.Stream(device=DEV)
    compute = g.CudaCompute(0, side.cuda_stream)
    hq, hkv, d = 32, 8, 128
    # paged decode, 5 ragged sequences
    case = synth.paged_case(3, 5, 1, 3000, hq, hkv, d, device=DEV)
    tables = torch.from_numpy(case.tables).to(DEV)
    lens = torch.from_numpy(case.seq_lens).to(DEV)
    out_dec = torch.zeros((case.batch, hq, d), device=DEV)
    # causal prefill, 300 tokens, fp16
    gen = torch.Generator(device=DEV)
    gen.manual_seed(1)
    seq = 300
    q = torch.randn((seq, hq, d), device=DEV, generator=gen).half()
    k = torch.randn((hkv, seq, d), device=DEV, generator=gen).half()
    v = torch.randn((hkv, seq, d), device=DEV, generator=gen).half()
    out_pre = torch.zeros((seq, hq, d), device=DEV, dtype=torch.float16)
    # tree verification over the paged prefix of the first two sequences
    n = 64
    qt, kt, vt, parents = _tree_inputs(5, 2, n, hq, hkv)
    qt_d = torch.from_numpy(qt.astype(np.float16)).to(DEV)
    kt_d, vt_d, par_d = torch.from_numpy(kt).to(DEV), torch.from_numpy(vt).to(DEV), torch.from_numpy(parents).to(DEV)
    out_tree = torch.zeros((2, hq, n, d), device=DEV)

    def calls():
        compute.batched_paged_attention_decode(case.q, case.k_pool, case.v_pool, tables, lens, out_dec, case.batch, hq,
                                               hkv, d, synth.PAGE, case.max_blocks, 1.0 / np.sqrt(d),
                                               num_blocks=case.num_blocks)
        compute.multihead_attention(q, k, v, out_pre, hq, hkv, seq, seq, d, 1.0 / np.sqrt(d), seq, q_dtype=1, out_dtype=1)
        compute.attention_tree(qt_d, case.k_pool, case.v_pool, kt_d, vt_d, par_d, out_tree, hq, hkv, n, 0, d,
                               1.0 / np.sqrt(d), batch_size=2, block_tables=tables, max_blocks_per_seq=case.max_blocks,
                               num_blocks=case.num_blocks, cache_lens=lens, q_dtype=1)

    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        calls()  # warm-up: scratch and tensor maps exist afterwards
    compute.sync()
    direct = [t.clone() for t in (out_dec, out_pre, out_tree)]
    for t in (out_dec, out_pre, out_tree):
        t.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        calls()
    torch.cuda.synchronize()
    assert not out_dec.any()  # capture ran nothing
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    compute.sync()  # the status word is clean
    assert torch.equal(out_dec, direct[0])
    # the tensor-core kernels add the hi and lo halves of P.V from two issuing threads in whatever
    # order the pipe takes them: equal within the path's tolerance, not bit for bit
    for got, want, what in ((out_pre, direct[1], "prefill replay"), (out_tree, direct[2], "tree replay")):
        assert_attention_close(got.float().cpu().numpy(), want.float().cpu().numpy(), what)
    compute.shutdown()


def test_two_compute_objects_on_two_streams():
    """One compute object per stream (the reference's one-object-one-queue model, per GPU thread): calls
    enqueued from two objects interleave on the device without sharing scratch or status."""
    import torch
    import granite_b200 as g
    from oracle import pyoracle
    hq, hkv, d = 32, 8, 128
    streams = [torch.cuda.Stream(device=DEV) for _ in range(2)]
    objs = [g.CudaCompute(0, s.cuda_stream) for s in streams]
    cases = [synth.paged_case(70 + i, 7, 1, 4000, hq, hkv, d, device=DEV) for i in range(2)]
    outs = [torch.zeros((c.batch, hq, d), device=DEV) for c in cases]
    tabs = [torch.from_numpy(c.tables).to(DEV) for c in cases]
    lens = [torch.from_numpy(c.seq_lens).to(DEV) for c in cases]
    torch.cuda.synchronize()
    for _ in range(5):
        for o, c, out, t, l in zip(objs, cases, outs, tabs, lens):
            o.batched_paged_attention_decode(c.q, c.k_pool, c.v_pool, t, l, out, c.batch, hq, hkv, d, synth.PAGE, c.max_blocks,
                                             1.0 / np.sqrt(d), num_blocks=c.num_blocks)
    for o in objs:
        o.sync()
    for c, out in zip(cases, outs):
        ref, bad = pyoracle.paged_decode_batch(c.q.cpu().numpy(), c.k_pool.cpu().numpy().view(np.uint16),
                                               c.v_pool.cpu().numpy().view(np.uint16), np.where(c.tables < 0, 0, c.tables),
                                               c.seq_lens, synth.PAGE)
        assert bad == 0
        assert_attention_close(out.cpu().numpy(), ref, "two objects")
    for o in objs:
        o.shutdown()

"""Host-side C++ faces that need no GPU: page-manager block numbering, block tables and the
speculation tree, each replayed against golden outputs of the reference's own compiled classes
(tests/golden/make_golden.py; PagedKVPool / SpeculationTree of src/llm)."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

GOLD = Path(__file__).resolve().parent / "golden"
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")


@pytest.fixture(scope="module", params=["standin", "reference_headers"])
def host_lib(request):
    """The test drivers of the C++ host faces: over the product library's classes, and - where it was
    built from the Granite checkout - the same class bodies compiled against Granite's real headers."""
    from host_drivers import build as drivers
    if request.param == "reference_headers" and not drivers.dropin_available():
        pytest.skip("oracle/_ref/libgranite_dropin.so not built (needs the Granite checkout)")
    lib = drivers.load(request.param)
    lib.granite_host_paged_pool_script.restype = C.c_int
    lib.granite_host_paged_pool_script.argtypes = [C.c_int, C.c_int, C.c_int, _i32p, C.c_int, _i32p, _i32p, _i32p,
                                                   _i32p, C.c_int, _i32p, _i32p]
    lib.granite_host_speculation_tree.argtypes = [_i32p, C.c_int, _i32p, _i32p, _i32p, _i32p, _i32p]
    lib.granite_host_find_accepted_path.argtypes = [_i32p, _i32p, C.c_int, _i32p, C.c_int, _i32p, _i32p]
    lib.granite_host_find_accepted_nodes.argtypes = [_i32p, _i32p, C.c_int, _i32p, C.c_int, _i32p, _i32p]
    lib.granite_host_rope_table.argtypes = [C.c_int, C.c_int, C.c_float, _f32p, _f32p]
    return lib


def _run_script(lib, ms, mt, bs, ops, mb):
    ops = np.ascontiguousarray(ops, np.int32)
    res = np.zeros(len(ops), np.int32)
    seq_lens = np.zeros(ms, np.int32)
    tlens = np.zeros(ms, np.int32)
    tables = np.zeros((ms, mb), np.int32)
    nfree, ntot = np.zeros(1, np.int32), np.zeros(1, np.int32)
    rc = lib.granite_host_paged_pool_script(ms, mt, bs, ops.reshape(-1), len(ops), res, seq_lens, tlens,
                                            tables.reshape(-1), mb, nfree, ntot)
    assert rc == 0
    return res, seq_lens, tlens, tables, int(nfree[0]), int(ntot[0])


def test_page_manager_replays_reference_scripts_bit_for_bit(host_lib):
    lib = host_lib
    g = np.load(GOLD / "ref_paged_pool.npz")
    for i in range(3):
        ms, mt, bs, mb = (int(x) for x in g[f"cfg{i}"])
        res, seq_lens, tlens, tables, nfree, ntot = _run_script(lib, ms, mt, bs, g[f"ops{i}"], mb)
        assert np.array_equal(res, g[f"results{i}"]), f"script {i}: per-operation results differ"
        assert np.array_equal(seq_lens, g[f"seq_lens{i}"])
        assert np.array_equal(tlens, g[f"table_lens{i}"])
        assert np.array_equal(tables, g[f"tables{i}"])
        assert [nfree, ntot] == list(g[f"free{i}"])


def test_block_manager_invariants(host_lib):
    """LIFO free list: first blocks handed out are the highest indices; exhaustion returns -1 and
    keeps what was taken; truncate frees tail blocks; double / out-of-range frees are ignored
    (src/llm/paged_kv_cache.cpp:73-98, :120-145, :169-187)."""
    lib = host_lib
    ops = [(0, 0, 0),            # acquire slot 0
           (1, 0, 33),           # 33 tokens -> 3 blocks: 7, 6, 5
           (6, 0, 0), (6, 0, 16), (6, 0, 32), (7, 0, 35), (6, 0, 48),
           (0, 0, 0),            # slot 1
           (1, 1, 16 * 6),       # wants 6 blocks, only 5 left -> fails, keeps the 5 it took
           (2, 0, 16),           # truncate slot 0 to one block -> frees 5 then 6
           (4, 0, 0),            # next allocation reuses the last freed: 6
           (5, 99, 0), (5, 6, 0), (5, 6, 0),  # bad index ignored; free 6; double free ignored
           (3, 1, 0), (3, 7, 0)]
    res, seq_lens, tlens, tables, nfree, ntot = _run_script(lib, 2, 128, 16, np.array(ops, np.int32), 8)
    assert ntot == 8
    assert list(res[:7]) == [0, 1, 7, 6, 5, 3, -1]
    assert res[7] == 1 and res[8] == 0
    assert res[9] == 16 and res[10] == 6
    assert res[11] == res[10 + 1] and res[12] == res[11] + 1 and res[13] == res[12]
    assert list(seq_lens) == [16, 0] and list(tlens) == [1, 0]
    assert tables[0, 0] == 7 and nfree == 7


def test_speculation_tree_matches_reference(host_lib):
    lib = host_lib
    g = np.load(GOLD / "ref_spec_tree.npz")
    for i in range(4):
        parents = np.ascontiguousarray(g[f"parents{i}"], np.int32)
        n = len(parents)
        po, dep, bfs = np.zeros(n, np.int32), np.zeros(n, np.int32), np.zeros(n, np.int32)
        nb, md = np.zeros(1, np.int32), np.zeros(1, np.int32)
        lib.granite_host_speculation_tree(parents, n, po, dep, bfs, nb, md)
        assert np.array_equal(po, g[f"parents_out{i}"])
        assert np.array_equal(dep, g[f"depths{i}"])
        assert np.array_equal(bfs[: int(nb[0])], g[f"bfs{i}"])
        assert int(md[0]) == int(g[f"max_depth{i}"][0])
    for i in range(6):
        parents = np.ascontiguousarray(g[f"ap_parents{i}"], np.int32)
        tokens = np.ascontiguousarray(g[f"ap_tokens{i}"], np.int32)
        targets = np.ascontiguousarray(g[f"ap_targets{i}"], np.int32)
        out, n_out = np.zeros(len(targets) + 1, np.int32), np.zeros(1, np.int32)
        lib.granite_host_find_accepted_path(parents, tokens, len(parents), targets, len(targets), out, n_out)
        assert np.array_equal(out[: int(n_out[0])], g[f"ap_path{i}"])


def test_accepted_nodes_are_the_nodes_behind_the_reference_path(host_lib):
    """find_accepted_nodes must name the nodes whose tokens open the reference's accepted path: the
    path is those tokens, optionally closed by the target's own choice at the first mismatch."""
    lib = host_lib
    g = np.load(GOLD / "ref_spec_tree.npz")
    for i in range(6):
        parents = np.ascontiguousarray(g[f"ap_parents{i}"], np.int32)
        tokens = np.ascontiguousarray(g[f"ap_tokens{i}"], np.int32)
        targets = np.ascontiguousarray(g[f"ap_targets{i}"], np.int32)
        path = g[f"ap_path{i}"]
        nodes, n_nodes = np.zeros(len(parents) + 1, np.int32), np.zeros(1, np.int32)
        lib.granite_host_find_accepted_nodes(parents, tokens, len(parents), targets, len(targets), nodes, n_nodes)
        nodes = nodes[: int(n_nodes[0])]
        assert len(path) - 1 <= len(nodes) <= len(path)
        assert np.array_equal(tokens[nodes], path[: len(nodes)])
        if len(nodes):
            assert nodes[0] == 0 and all(parents[nodes[j]] == nodes[j - 1] for j in range(1, len(nodes)))
        if len(nodes) < len(path):  # closed by the target's choice where the tree disagreed
            assert path[-1] == targets[len(nodes)]


def test_rope_tables_of_the_host_mirror_match_reference(host_lib):
    lib = host_lib
    g = np.load(GOLD / "ref_rope.npz")
    for i in range(3):
        max_seq, d = (int(x) for x in g[f"t{i}_cfg"])
        cos = np.zeros((max_seq, d // 2), np.float32)
        sin = np.zeros_like(cos)
        assert lib.granite_host_rope_table(max_seq, d, float(g[f"t{i}_theta"][0]), cos.reshape(-1), sin.reshape(-1)) == 0
        rows = g[f"t{i}_rows"] if f"t{i}_rows" in g else np.arange(max_seq)
        assert np.array_equal(cos[rows].view(np.uint32), g[f"t{i}_cos"])
        assert np.array_equal(sin[rows].view(np.uint32), g[f"t{i}_sin"])

"""Multi-GPU host logic on CPU: the sharding plan and the output gather, with world_size-2 gloo ranks."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np

from granite_b200 import sharding, synth

ROOT = Path(__file__).resolve().parent.parent


def test_lpt_plan_is_a_balanced_partition():
    cfg = synth.CONFIGS["paged_decode_long_b256"]
    lens = synth.draw_lengths(np.random.default_rng(cfg["seed"]), cfg["batch"], cfg["len_lo"], cfg["len_hi"], cfg["dist"])
    for n in (1, 2, 4, 8):
        plan = sharding.lpt_assign(lens, n)
        allidx = np.concatenate(plan)
        assert sorted(allidx.tolist()) == list(range(len(lens)))  # each sequence exactly once
        assert sharding.imbalance(lens, plan) < 1.02
    assert sharding.lpt_assign([], 4)[0].size == 0
    plan = sharding.lpt_assign([5, 5, 5], 2)
    assert [p.tolist() for p in plan] == [[0, 2], [1]]  # ties by index, lowest rank first


def test_head_split_and_choice_of_split():
    assert sharding.head_split(64, 8, 8) == [(r, 1, 8 * r, 8) for r in range(8)]
    assert sharding.head_split(32, 8, 2) == [(0, 4, 0, 16), (4, 4, 16, 16)]
    assert sharding.head_split(32, 8, 3) is None and sharding.head_split(12, 3, 2) is None
    pool = np.arange(6 * 4 * 2).reshape(6, 4, 2)
    for r in range(2):
        shard = sharding.shard_pool_by_head(pool, r, 2)
        assert shard.flags.c_contiguous and np.array_equal(shard, pool[:, 2 * r:2 * r + 2])
    q = np.arange(3 * 8 * 2).reshape(3, 8, 2)
    parts = np.stack([sharding.shard_queries_by_head(q, r, 4) for r in range(4)])
    assert np.array_equal(sharding.unshard_heads(parts), q)
    # one very long sequence among short ones: no deal of whole sequences balances, the head split does
    skewed = [100000] + [100] * 15
    assert sharding.choose_split(skewed, 8, 8) == "kv_head"
    assert sharding.choose_split(skewed, 8, 3) == "sequence"   # heads do not divide
    assert sharding.choose_split(skewed, 8, 1) == "sequence"
    assert sharding.predicted_cost(skewed, 8, 8, "kv_head") == sum(skewed) / sharding.HEADS_PER_BOX_EFFICIENCY[1]
    # balanced batches keep whole KV heads together: the decode kernel is slower on one-head pages
    cfg = synth.CONFIGS["paged_decode_long_b256"]
    lens = synth.draw_lengths(np.random.default_rng(cfg["seed"]), cfg["batch"], cfg["len_lo"], cfg["len_hi"], cfg["dist"])
    assert sharding.choose_split(lens, 8, 8) == "sequence"
    assert sharding.predicted_cost(skewed, 8, 8, "sequence") == 100000 * 8 / sharding.HEADS_PER_BOX_EFFICIENCY[8]


def test_head_sharded_gather_with_two_gloo_ranks(tmp_path):
    script = tmp_path / "rank_heads.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {str(ROOT)!r})
        import numpy as np, torch, torch.distributed as dist
        from granite_b200 import sharding
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        b, hq, hkv, d = 5, 8, 4, 6
        split = sharding.head_split(hq, hkv, world)
        kv0, n_kv, q0, n_q = split[rank]
        q = np.random.default_rng(9).standard_normal((b, hq, d)).astype(np.float32)   # same on every rank
        pool = np.random.default_rng(10).standard_normal((32, hkv, d)).astype(np.float32)
        mine_q = sharding.shard_queries_by_head(q, rank, world)
        mine_pool = sharding.shard_pool_by_head(pool, rank, world)
        assert mine_pool.shape == (32, n_kv, d) and mine_q.shape == (b, n_q, d)
        # stand-in for attention: each query head's output is a function of its own KV head's pool slice
        group = hq // hkv
        local = np.stack([mine_q[:, h] * mine_pool[:, h // group].sum() for h in range(n_q)], axis=1)
        gathered = torch.empty((world, b, n_q, d))
        dist.all_gather_into_tensor(gathered.view(world * b, n_q, d), torch.from_numpy(local))
        full = sharding.unshard_heads(gathered.numpy())
        want = np.stack([q[:, h] * pool[:, h // group].sum() for h in range(hq)], axis=1)
        assert np.allclose(full, want), "head slices were not put back in head order"
        dist.barrier()
        dist.destroy_process_group()
        print("rank", rank, "ok")
    """))
    env = dict(os.environ, OMP_NUM_THREADS="1")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29534", str(script)],
                         capture_output=True, text=True, env=env, timeout=240)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.count("ok") == 2


def test_gather_and_unshard_with_two_gloo_ranks(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {str(ROOT)!r})
        import numpy as np, torch, torch.distributed as dist
        from granite_b200 import sharding
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        lens = np.random.default_rng(3).integers(1, 5000, size=37)
        plan = sharding.lpt_assign(lens, world)          # same plan on every rank, no communication
        rows = sharding.padded_rows(plan)
        mine = plan[rank]
        local = torch.zeros((rows, 4, 8))
        # stand-in for this rank's attention outputs: a function of the global sequence index
        local[: len(mine)] = torch.from_numpy(mine.astype(np.float32))[:, None, None] * 10 + torch.arange(8)[None, None, :]
        gathered = torch.empty((world * rows, 4, 8))
        dist.all_gather_into_tensor(gathered, local)
        full = sharding.unshard(gathered.numpy().reshape(world, rows, 4, 8), plan, len(lens))
        want = np.arange(len(lens), dtype=np.float32)[:, None, None] * 10 + np.arange(8, dtype=np.float32)[None, None, :]
        assert np.array_equal(full, np.broadcast_to(want, full.shape)), "gather did not restore sequence order"
        dist.barrier()
        dist.destroy_process_group()
        print("rank", rank, "ok")
    """))
    env = dict(os.environ, OMP_NUM_THREADS="1")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                         capture_output=True, text=True, env=env, timeout=240)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.count("ok") == 2

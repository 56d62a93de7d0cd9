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

"""Host-side logic of the multi-GPU fill on CPU: two gloo ranks agree on who owns which family,
and the per-group broadcast schedule rebuilds the whole table on every rank."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import morello_b200 as m
    from morello_b200 import sharded
    db = m.SynthesisDatabase(device=-1)  # planning only: no GPU here
    db.set_shard(rank, world)
    db.set_lattice_caps([8, 2, 5, 0])
    db.plan_precompute(2)
    fams = db.families()
    n_rows = db.stats()["n_rows"]
    sharded.check_partition(fams, world, n_rows)
    sched = sharded.exchange_schedule(fams, db.num_groups())
    # every rank must have computed the same ownership
    mine = torch.tensor([o for _, o, _, _ in fams], dtype=torch.int64)
    ref = mine.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(mine, ref)
    # stand-in for the fill: a rank "computes" f(row) for the rows it owns, group by group,
    # then the schedule's broadcasts run; children are always in earlier groups.
    table = torch.full((n_rows,), -1, dtype=torch.int64)
    for g, ranges in enumerate(sched):
        for owner, lo, hi in ranges:
            if owner == rank:
                table[lo:hi] = torch.arange(lo, hi) * 7 + 3
        for owner, lo, hi in ranges:
            dist.broadcast(table[lo:hi], src=owner)
    assert torch.equal(table, torch.arange(n_rows) * 7 + 3)
    loads = [0] * world
    for _, o, lo, hi in fams:
        loads[o] += hi - lo
    np.save(os.path.join(out_dir, f"loads_{rank}.npy"), np.array(loads))
    db.close()
    dist.destroy_process_group()


def test_two_rank_ownership_and_exchange_schedule(built_extension, tmp_path):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    loads = np.load(tmp_path / "loads_0.npy")
    assert (loads == np.load(tmp_path / "loads_1.npy")).all()
    assert loads.sum() > 0 and loads.min() > 0.25 * loads.max()  # both ranks get real work


def test_exchange_schedule_merges_neighbours():
    from morello_b200 import sharded
    fams = [(0, 0, 0, 10), (0, 0, 10, 20), (0, 1, 20, 25), (1, 1, 25, 40), (1, 1, 40, 40), (1, 0, 40, 50)]
    assert sharded.exchange_schedule(fams, 2) == [[(0, 0, 20), (1, 20, 25)], [(1, 25, 40), (0, 40, 50)]]
    sharded.check_partition(fams, 2, 50)
    with pytest.raises(ValueError):
        sharded.check_partition(fams, 2, 51)

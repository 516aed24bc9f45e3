"""Host-side logic of the multi-GPU fill on CPU: two gloo ranks agree on who owns which family,
and the per-stage sum over ranks rebuilds every Spec's words on every rank."""
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
    # rank 0 plans; the plan travels to rank 1 as flat byte ranges (over gloo here)
    sharded.plan_on_one_rank(db, lambda: db.plan_precompute(2), dist, torch, device="cpu", chunk_bytes=1 << 20)
    fams = db.families()
    stages = db.stages()
    n_specs = db.stats()["n_specs"]
    assert len(stages) == db.num_stages() == db.stats()["n_stages"]
    owners = db.spec_owners()
    sharded.check_partition(fams, stages, owners, world, n_specs)
    # every rank must have computed the same ownership
    mine = torch.tensor(list(owners), dtype=torch.int64)
    ref = mine.clone()
    dist.broadcast(ref, src=0)
    assert torch.equal(mine, ref)
    # stand-in for the fill: per stage a rank "computes" four mask words for each Spec of the
    # families it owns and leaves the others zero; the sum over ranks is the exchange.
    owner_of = mine
    want = (torch.arange(n_specs * 4, dtype=torch.int32) * 7 + 3).reshape(n_specs, 4)
    table = torch.zeros((n_specs, 4), dtype=torch.int32)
    for lo, hi, _flo, _fhi in stages:
        own = owner_of[lo:hi] == rank
        table[lo:hi][own] = want[lo:hi][own]
        dist.all_reduce(table[lo:hi], op=dist.ReduceOp.SUM)
    assert torch.equal(table, want)
    # the adopted plan is the planned one: same Specs in the same order, same lookups
    own = m.SynthesisDatabase(device=-1)
    own.set_shard(rank, world)
    own.plan_precompute(2)
    assert own.families() == fams and own.stages() == stages and own.spec_owners() == owners
    for i in range(0, n_specs, 97):
        assert own.spec_blob(i) == db.spec_blob(i)
    # headers, candidate records, stages, families, goal ids: byte for byte (Specs are compared
    # through their canonical blobs above: unused tail bytes of a Spec may differ; the id lookup
    # table is built by racing threads)
    for (pa, na), (pb, nb) in zip(own.plan_share()[2:7], db.plan_share()[2:7]):
        assert na == nb
        if na:
            import ctypes
            assert ctypes.string_at(pa, na) == ctypes.string_at(pb, nb)
    own.close()
    np.save(os.path.join(out_dir, f"loads_{rank}.npy"), np.array(sharded.rank_loads(owners, world)))
    db.close()
    dist.destroy_process_group()


def test_two_rank_ownership_and_exchange_schedule(built_extension, tmp_path):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    loads = np.load(tmp_path / "loads_0.npy")
    assert (loads == np.load(tmp_path / "loads_1.npy")).all()
    assert loads.sum() > 0 and loads.min() > 0.25 * loads.max()  # both ranks get real work


def test_check_partition_rejects_gaps_and_bad_owners():
    from morello_b200 import sharded
    stages = [(0, 20, 0, 2), (20, 50, 2, 4)]
    fams = [(0, 0, 0, 10), (0, 1, 10, 20), (1, 1, 20, 40), (1, 0, 40, 50)]
    owners = bytes([0] * 10 + [1] * 10 + [1] * 20 + [0] * 10)
    sharded.check_partition(fams, stages, owners, 2, 50)
    assert sharded.rank_loads(owners, 2) == [20, 30]
    with pytest.raises(ValueError):
        sharded.check_partition(fams, stages, owners, 2, 51)
    with pytest.raises(ValueError):
        sharded.check_partition(fams, stages, owners, 1, 50)  # owner 1 does not exist
    with pytest.raises(ValueError):
        sharded.check_partition([(0, 0, 0, 10), (0, 1, 11, 20)] + fams[2:], stages, owners, 2, 50)

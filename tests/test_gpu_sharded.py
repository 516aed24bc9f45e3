"""Two GPUs, one process each: the sharded fill must produce the same table, byte for byte,
as the single-GPU fill."""
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import morello_b200 as m
    from morello_b200 import sharded
    db = m.SynthesisDatabase(device=rank)
    sharded.precompute_sharded(db, 2, dist, torch)
    ptr, n = db.device_rows()
    got = torch.as_tensor(sharded._DeviceBytes(ptr, n * sharded.row_bytes()), device="cuda").clone()
    # the unsharded fill on this rank's GPU
    solo = m.SynthesisDatabase(device=rank)
    solo.precompute(2)
    sptr, sn = solo.device_rows()
    assert sn == n
    want = torch.as_tensor(sharded._DeviceBytes(sptr, sn * sharded.row_bytes()), device="cuda")
    assert torch.equal(got, want), "sharded table differs from the single-GPU table"
    # and lookups work on every rank
    goal = m.simple_spec(m.KIND_MATMUL, m.DTYPE_U32, [1, 2, 2, 2], m.GL)
    d = db.get(goal)
    assert (d.found, d.action, d.main_cost, d.depth, d.peaks) == (1, 1, 127, 7, (8, 0, 4, 0))
    db.close()
    solo.close()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_fill_equals_single_gpu_fill(built_extension):
    import torch.multiprocessing as mp
    port = 29700 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port), nprocs=2, join=True)

"""One database fill sharded over several GPUs (one process per GPU, torch.distributed).

Every rank plans the same job and keeps the whole table in its own HBM. The plan orders the
Specs into stages; inside a stage the families - Specs that share dtype and shape - do not
depend on each other, so each is computed by one rank. Per stage two small device buffers
cross NVLink / NVSwitch, each with one NCCL all-reduce (sum of int32, in place): first the
limits-grid breakpoint masks of the stage's Specs, which every rank needs to give the stage's
rows the same place in its table, then the stage's finished rows. A Spec's words are zero on
every rank but its owner, so the sum is a gather. Kernels only ever read local HBM.

The reference has no counterpart: its workers are threads sharing one in-process database
(precompute/src/main.rs:229-240,339).
"""
import ctypes
import time
from typing import Callable, List, Sequence, Tuple


def row_bytes() -> int:
    from . import _lib
    return int(_lib.load().mrl_row_bytes())


def check_partition(families: Sequence[Tuple[int, int, int, int]], stages: Sequence[Tuple[int, int, int, int]],
                    owners: bytes, world: int, n_specs: int):
    """families: (stage, owner of the first Spec, first Spec id, end Spec id); stages: (first Spec
    id, end Spec id, first family, end family); owners: one byte per Spec id. Families tile the Spec
    ids in order, stage by stage, and every Spec's owner is a valid rank."""
    pos = 0
    fam = 0
    for s, (lo, hi, flo, fhi) in enumerate(stages):
        if lo != pos or flo != fam or fhi < flo:
            raise ValueError(f"stage {s} starts at Spec {lo} / family {flo}, expected {pos} / {fam}")
        for f in range(flo, fhi):
            stage, _owner, a, b = families[f]
            if stage != s or a != pos or b <= a:
                raise ValueError(f"bad family {f}: stage {stage}, Specs {a}..{b} (expected start {pos})")
            pos = b
        if pos != hi:
            raise ValueError(f"families of stage {s} end at Spec {pos}, the stage at {hi}")
        fam = fhi
    if pos != n_specs or fam != len(families):
        raise ValueError(f"stages cover {pos} Specs of {n_specs}")
    if len(owners) != n_specs or (n_specs and max(owners) >= world):
        raise ValueError("an owner is not a rank of this world")


def rank_loads(owners: bytes, world: int) -> List[int]:
    """Specs per rank (the planner balances candidate records, which track this closely)."""
    loads = [0] * world
    for o in owners:
        loads[o] += 1
    return loads


class _DeviceBytes:
    """Exposes a raw device range to torch through the CUDA array interface (no copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def _sum_over_ranks(ptr, nbytes, dist, torch, process_group):
    if nbytes == 0:
        return
    words = torch.as_tensor(_DeviceBytes(ptr, nbytes), device="cuda").view(torch.int32)
    dist.all_reduce(words, op=dist.ReduceOp.SUM, group=process_group)


def fill_sharded(db, dist, torch, process_group=None):
    """One sharded fill of an uploaded plan, on torch's current CUDA stream."""
    db.set_stream(torch.cuda.current_stream().cuda_stream)
    db.fill_begin()
    for s in range(db.num_stages()):
        ptr, nbytes = db.fill_stage_solve(s)
        _sum_over_ranks(ptr, nbytes, dist, torch, process_group)
        ptr, nbytes = db.fill_stage_place(s)
        _sum_over_ranks(ptr, nbytes, dist, torch, process_group)
    db.fill_end()


def plan_on_one_rank(db, plan_fn: Callable[[], None], dist, torch, process_group=None, device="cuda",
                     chunk_bytes=256 << 20, cands_on_device_only=False):
    """Plans on the first rank only and hands the plan to the others. The ranks of one node share
    its host cores, so planning once with all of them beats every rank planning on a share.
    The plan's eight byte ranges travel by broadcast, staged through `device` memory in chunks
    ("cuda" for NCCL, "cpu" for gloo). cands_on_device_only: the candidate records (most of the
    bytes) are left out here; after upload() call broadcast_device_cands()."""
    rank, world = dist.get_rank(process_group), dist.get_world_size(process_group)
    src = dist.get_global_rank(process_group, 0) if process_group is not None else 0
    db.set_shard(rank, world)
    t0 = time.perf_counter()
    if world == 1:
        plan_fn()
        return
    sizes = torch.zeros(8, dtype=torch.int64, device=device)
    if rank == 0:
        plan_fn()
        blobs = db.plan_share()
        sizes.copy_(torch.tensor([n for _, n in blobs], dtype=torch.int64))
    dist.broadcast(sizes, src=src, group=process_group)
    if rank != 0:
        want = [int(x) for x in sizes.tolist()]
        blobs = list(zip(db.plan_adopt(want, cands_on_device_only), want))
    if cands_on_device_only:
        blobs = [b for k, b in enumerate(blobs) if k != 3]
    chunk = max(1, min(chunk_bytes, max(n for _, n in blobs)))
    host = torch.empty(chunk, dtype=torch.uint8, pin_memory=(device == "cuda"))
    stage = torch.empty(chunk, dtype=torch.uint8, device=device) if device == "cuda" else host
    for ptr, nbytes in blobs:
        for off in range(0, nbytes, chunk):
            n = min(chunk, nbytes - off)
            if rank == 0:
                ctypes.memmove(host.data_ptr(), ptr + off, n)
                if stage is not host:
                    stage[:n].copy_(host[:n])
            dist.broadcast(stage[:n], src=src, group=process_group)
            if rank != 0:
                if stage is not host:
                    host[:n].copy_(stage[:n])
                ctypes.memmove(ptr + off, host.data_ptr(), n)
    if rank != 0:
        db.plan_adopt_done(time.perf_counter() - t0)


def broadcast_device_cands(db, dist, torch, process_group=None):
    """Copies the planning rank's uploaded candidate records into the other ranks' device buffers."""
    ptr, nbytes = db.device_cands()
    if nbytes == 0 or dist.get_world_size(process_group) == 1:
        db.cands_arrived()
        return
    src = dist.get_global_rank(process_group, 0) if process_group is not None else 0
    buf = torch.as_tensor(_DeviceBytes(ptr, nbytes), device="cuda")
    step = 1 << 30
    for off in range(0, nbytes, step):
        dist.broadcast(buf[off:off + step], src=src, group=process_group)
    db.cands_arrived()


def precompute_sharded(db, size, dist, torch, through=2, dtypes=(4, 6), process_group=None):
    """`precompute` on all ranks of the process group."""
    plan_on_one_rank(db, lambda: db.plan_precompute(size, through, dtypes), dist, torch, process_group,
                     cands_on_device_only=True)
    db.upload()
    broadcast_device_cands(db, dist, torch, process_group)
    fill_sharded(db, dist, torch, process_group)

"""One database fill sharded over several GPUs (one process per GPU, torch.distributed).

Every rank plans the same job and keeps the whole row table in its own HBM. Inside a group
(Specs of one kind with one log-shape sum) the families - Specs that also share dtype and
shape - do not depend on each other, so each is computed by one rank. After a group every
family's rows travel from its owner to all ranks (NCCL broadcast over NVLink / NVSwitch, in
place in the replicated table) before the next group starts. Rows only ever cross between
processes through the collective; kernels read local HBM.

The reference has no counterpart: its workers are threads sharing one in-process database
(precompute/src/main.rs:229-240,339).
"""
from typing import List, Sequence, Tuple

def row_bytes() -> int:
    from . import _lib
    return int(_lib.load().mrl_row_bytes())


def exchange_schedule(families: Sequence[Tuple[int, int, int, int]], n_groups: int) -> List[List[Tuple[int, int, int]]]:
    """Per group, the row ranges to broadcast as (owner, first row, end row). Neighbouring
    families of one owner are merged into one range."""
    sched: List[List[Tuple[int, int, int]]] = [[] for _ in range(n_groups)]
    for group, owner, lo, hi in families:
        if hi <= lo:
            continue
        cur = sched[group]
        if cur and cur[-1][0] == owner and cur[-1][2] == lo:
            cur[-1] = (owner, cur[-1][1], hi)
        else:
            cur.append((owner, lo, hi))
    return sched


def check_partition(families: Sequence[Tuple[int, int, int, int]], world: int, n_rows: int):
    """Families tile the table in order and every owner is a valid rank."""
    pos = 0
    for group, owner, lo, hi in families:
        if lo != pos or hi < lo or not (0 <= owner < world):
            raise ValueError(f"bad family partition at row {lo} (expected {pos}), owner {owner}")
        pos = hi
    if pos != n_rows:
        raise ValueError(f"families cover {pos} rows of {n_rows}")


class _DeviceBytes:
    """Exposes a raw device range to torch through the CUDA array interface (no copy)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def fill_sharded(db, dist, torch, process_group=None):
    """One sharded fill of an uploaded plan. Returns (status, caps) like fill_end, agreed over
    all ranks (status 1: refill with the returned caps)."""
    ptr, n_rows = db.device_rows()
    fams = db.families()
    world = dist.get_world_size(process_group)
    check_partition(fams, world, n_rows)
    sched = exchange_schedule(fams, db.num_groups())
    ROW_BYTES = row_bytes()
    rows = torch.as_tensor(_DeviceBytes(ptr, max(n_rows, 1) * ROW_BYTES), device="cuda")
    db.set_stream(torch.cuda.current_stream().cuda_stream)
    db.fill_begin()
    for g, ranges in enumerate(sched):
        db.fill_group(g)
        for owner, lo, hi in ranges:
            dist.broadcast(rows[lo * ROW_BYTES:hi * ROW_BYTES], src=dist.get_global_rank(process_group, owner)
                           if process_group is not None else owner, group=process_group)
    rc, caps = db.fill_end()
    agreed = torch.tensor(caps + [rc], dtype=torch.int32, device="cuda")
    dist.all_reduce(agreed, op=dist.ReduceOp.MAX, group=process_group)
    agreed = [int(x) for x in agreed.tolist()]
    return agreed[4], agreed[:4]


def precompute_sharded(db, size, dist, torch, through=2, dtypes=(4, 6), process_group=None, max_attempts=16):
    """`precompute` on all ranks of the process group; returns the number of fill attempts."""
    rank, world = dist.get_rank(process_group), dist.get_world_size(process_group)
    db.set_shard(rank, world)
    db.plan_precompute(size, through, dtypes)
    for attempt in range(1, max_attempts + 1):
        db.upload()
        rc, caps = fill_sharded(db, dist, torch, process_group)
        if rc == 0:
            return attempt
        db.set_lattice_caps(caps)
    raise RuntimeError("lattice caps did not converge")

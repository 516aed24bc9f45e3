"""Host planner checks that need no GPU (planning-only contexts)."""
import ctypes
import os

import pytest


@pytest.fixture()
def m(built_extension):
    import morello_b200
    return morello_b200


def _same_plan(a, b, size):
    """Headers, candidate records, stages and families byte for byte; the goal ids as a set (their
    order follows how the goals were handed in); Specs by their blobs. (The id lookup table is
    built by racing threads: equal as a map, not as bytes.)"""
    import numpy as np
    ra, rb = a.plan_share(), b.plan_share()
    assert ra[7][1] == rb[7][1]
    for k in (2, 3, 4, 5):
        (pa, na), (pb, nb) = ra[k], rb[k]
        assert na == nb and ctypes.string_at(pa, na) == ctypes.string_at(pb, nb), k
    ga = np.sort(np.frombuffer(ctypes.string_at(*ra[6]), dtype=np.uint32))
    gb = np.sort(np.frombuffer(ctypes.string_at(*rb[6]), dtype=np.uint32))
    assert (ga == gb).all()
    for i in range(0, a.num_specs(), 7 if size < 4 else 101):
        assert a.spec_blob(i) == b.spec_blob(i)


@pytest.mark.parametrize("size", [1, 2, 4])
def test_dtype_twin_plan_equals_direct_plan(m, size):
    """u32 and f32 goals: the planner tabulates u32 only and derives the f32 records. The result
    must be the plan it builds when both dtypes are tabulated - headers, candidate records,
    stages, families, goal ids and the id lookup table byte for byte, Specs by their blobs."""
    a = m.SynthesisDatabase(device=-1)
    a.plan_precompute(size)
    b = m.SynthesisDatabase(device=-1)
    b.set_plan_flags(no_twins=True)
    b.plan_precompute(size)
    keys = ("n_specs", "n_goal_specs", "n_candidates", "n_stages")
    sa, sb = a.stats(), b.stats()
    assert {k: sa[k] for k in keys} == {k: sb[k] for k in keys}
    _same_plan(a, b, size)
    a.close()
    b.close()


@pytest.mark.parametrize("size", [2, 4])
def test_memoised_tabulation_equals_tabulation_from_scratch(m, size):
    """The planner reuses, per operand, its Moves and what tiling does to it. The plan must be the
    one built with every Spec tabulated from scratch."""
    a = m.SynthesisDatabase(device=-1)
    a.set_plan_flags(no_twins=True)
    a.plan_precompute(size)
    b = m.SynthesisDatabase(device=-1)
    b.set_plan_flags(no_twins=True, no_memo=True)
    b.plan_precompute(size)
    _same_plan(a, b, size)
    a.close()
    b.close()


def test_single_dtype_and_uneven_goal_sets_are_planned_directly(m):
    """Twins are only used when the two goal sets mirror each other."""
    db = m.SynthesisDatabase(device=-1)
    db.plan_precompute(2, dtypes=(m.DTYPE_F32,))
    n_f32 = db.stats()["n_specs"]
    db.plan_precompute(2)
    assert db.stats()["n_specs"] == 2 * n_f32
    goals = [m.simple_spec(m.KIND_MATMUL, m.DTYPE_U32, [1, 2, 2, 2], m.GL),
             m.simple_spec(m.KIND_MATMUL, m.DTYPE_F32, [1, 2, 2, 1], m.GL)]
    db.plan_goals(goals)       # different shapes per dtype: no twin derivation, still a valid plan
    assert db.stats()["n_goal_specs"] == 2
    db.close()


def test_mirrored_goal_lists_are_detected(m):
    """top_down_many-style goal lists that contain every goal in both dtypes take the twin path
    too (detected from the goals themselves) and give the direct plan."""
    shapes = ([1, 2, 2, 2], [1, 2, 4, 2], [1, 1, 2, 4])
    goals = [m.simple_spec(m.KIND_MATMUL, dt, sh, m.GL) for dt in (m.DTYPE_F32, m.DTYPE_U32) for sh in shapes]
    a = m.SynthesisDatabase(device=-1)
    a.plan_goals(goals)
    b = m.SynthesisDatabase(device=-1)
    b.set_plan_flags(no_twins=True)
    b.plan_goals(goals)
    assert a.stats()["n_goal_specs"] == b.stats()["n_goal_specs"] == 6
    _same_plan(a, b, 2)
    import numpy as np
    ga = np.frombuffer(ctypes.string_at(*a.plan_share()[6]), dtype=np.uint32)
    gb = np.frombuffer(ctypes.string_at(*b.plan_share()[6]), dtype=np.uint32)
    assert (ga == gb).all()      # here the goal order is the callers' in both
    a.close()
    b.close()


def test_calls_out_of_order_fail_cleanly(m):
    """Status codes, not crashes: lookups before a fill, shard ranks out of range, a shared plan
    whose sizes do not describe a plan."""
    db = m.SynthesisDatabase(device=-1)
    goal = m.simple_spec(m.KIND_MATMUL, m.DTYPE_U32, [1, 2, 2, 2], m.GL)
    with pytest.raises(RuntimeError, match="not filled"):
        db.get(goal)
    with pytest.raises(RuntimeError, match="not filled"):
        db.get_impl(goal)
    with pytest.raises(RuntimeError, match="not filled"):
        db.verify(10)
    with pytest.raises(RuntimeError, match="rank"):
        db.set_shard(2, 2)
    with pytest.raises(RuntimeError, match="nothing planned"):
        db.plan_share()
    with pytest.raises(RuntimeError, match="sizes"):
        db.plan_adopt([1, 2, 3, 4, 5, 6, 7, 8])
    db.plan_goals([goal])
    with pytest.raises(RuntimeError, match="no device"):
        db.upload()          # planning-only context
    assert db.spec_owners() == bytes(db.num_specs())   # not sharded: everything belongs to rank 0
    db.close()


def _adopt_copy(m, src, corrupt=None, cands_on_device_only=False):
    """A second planning context that adopts src's plan byte for byte; corrupt(k, bytearray) may
    change range k on the way."""
    blobs = src.plan_share()
    dst = m.SynthesisDatabase(device=-1)
    ptrs = dst.plan_adopt([n for _, n in blobs], cands_on_device_only)
    for k, ((p, n), q) in enumerate(zip(blobs, ptrs)):
        if q == 0 or n == 0:
            continue
        data = bytearray(ctypes.string_at(p, n))
        if corrupt:
            corrupt(k, data)
        ctypes.memmove(q, bytes(data), n)
    return dst


def test_adopted_plan_is_checked_before_use(m):
    """A plan that arrives as bytes from another process is validated: stage and family ranges,
    candidate ranges, child ids, record fields, the id table. Anything off is refused with a status
    instead of reaching a kernel."""
    import struct
    src = m.SynthesisDatabase(device=-1)
    src.plan_precompute(2)
    ok = _adopt_copy(m, src)
    ok.plan_adopt_done()
    assert ok.stats()["n_specs"] == src.stats()["n_specs"] and ok.stages() == src.stages()
    ok.close()
    n_specs = src.num_specs()

    def child_out_of_range(k, data):
        if k == 3:   # candidate records: 32 bytes each, child ids at offset 16; find one with children
            for off in range(0, len(data), 32):
                if data[off + 3] > 0:
                    struct.pack_into("<I", data, off + 16, n_specs + 7)
                    return

    def bad_kind(k, data):
        if k == 3:
            data[2] = 9

    def cand_range_beyond_records(k, data):
        if k == 2:   # headers: 32 bytes each, cand_off at 24, ncand at 28
            struct.pack_into("<I", data, 32 * (n_specs - 1) + 28, 1 << 30)

    def stage_gap(k, data):
        if k == 4:   # stages: spec_lo, spec_hi, fam_lo, fam_hi, ...
            lo, hi = struct.unpack_from("<II", data, 20)
            struct.pack_into("<II", data, 20, lo + 1, hi)

    def bad_goal(k, data):
        if k == 6:
            struct.pack_into("<I", data, 0, n_specs)

    def bad_id_table(k, data):
        if k == 7:
            struct.pack_into("<I", data, 0, n_specs + 1)

    for corrupt in (child_out_of_range, bad_kind, cand_range_beyond_records, stage_gap, bad_goal, bad_id_table):
        bad = _adopt_copy(m, src, corrupt)
        with pytest.raises(RuntimeError, match="shared plan"):
            bad.plan_adopt_done()
        bad.close()
    # without the candidate records on the host (they travel device to device) the rest is still checked
    partial = _adopt_copy(m, src, cand_range_beyond_records, cands_on_device_only=True)
    with pytest.raises(RuntimeError, match="shared plan"):
        partial.plan_adopt_done()
    partial.close()
    src.close()


def test_saved_database_files_are_validated_on_the_host(m, tmp_path):
    """mrl_load reads and checks a file completely before it touches a device: garbage, a
    truncated file and inconsistent sizes come back as status codes (-7 / -8)."""
    import os
    golden = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "precompute_1.mrldb")
    data = open(golden, "rb").read()
    db = m.SynthesisDatabase(device=-1)

    def status_of(blob):
        path = tmp_path / "x.mrldb"
        path.write_bytes(blob)
        try:
            db.load(str(path))
        except RuntimeError as e:
            return e.status, str(e)
        return 0, ""

    assert status_of(data)[0] == -2 and "no device" in status_of(data)[1]   # a good file gets as far as the device
    assert status_of(b"not a database")[0] == -7
    assert status_of(b"MRLB200\0" + bytes(200))[0] == -7                    # version 0
    assert status_of(data[:len(data) // 2])[0] == -8                         # truncated
    assert status_of(data + b"\0" * 16)[0] == -8                             # trailing bytes
    other_target = bytearray(data)
    other_target[12] = 2                                                      # TARGET tag
    assert status_of(bytes(other_target))[0] == -7
    huge = bytearray(data)
    huge[40:48] = (1 << 60).to_bytes(8, "little")                             # n_specs
    assert status_of(bytes(huge))[0] == -8
    with pytest.raises(RuntimeError, match="cannot open"):
        db.load(str(tmp_path / "missing.mrldb"))
    db.close()

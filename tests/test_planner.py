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

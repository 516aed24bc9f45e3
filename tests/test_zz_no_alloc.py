"""The no-allocation entry point (mrl_top_down_many_noalloc) against mrl_top_down_many.

Collected last on purpose: it exercises a fixed device array shared by every call in the
process, so a failure here cannot hide a failure of any other test.
"""
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def m(built_extension):
    import morello_b200
    return morello_b200


def _goals(m):
    goals, limits = [], []
    for dtype in (m.DTYPE_U32, m.DTYPE_F32):
        for kind, shape in ((m.KIND_MATMUL, [1, 1, 1, 1]), (m.KIND_MATMUL_ACCUM, [1, 1, 1, 1]),
                            (m.KIND_MOVE, [1, 1, 1]), (m.KIND_FILL_ZERO, [1, 1, 1])):
            for mem in (m.GL, m.L1, m.RF):
                goals.append(m.simple_spec(kind, dtype, shape, mem))
                limits.append(m.MAX_MEM)
                goals.append(m.simple_spec(kind, dtype, shape, mem))
                limits.append((1, 0, 2, 0))  # tight limits: some of these are unsatisfiable
    return goals, limits


def test_noalloc_matches_allocating_entry_point_twice_in_a_row(m):
    import torch
    goals, limits = _goals(m)
    db = m.SynthesisDatabase()
    want = db.top_down_many(goals, limits)
    assert any(w.found == 1 for w in want) and any(w.found == 0 for w in want)
    stats_before = db.stats()
    rows_before = db.device_rows()
    first = db.top_down_many_noalloc(goals, limits)   # also the call that resolves the array's address
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    second = db.top_down_many_noalloc(goals, limits)
    assert first == want      # integer results: exact equality is the tolerance
    assert second == want     # the array still holds the first call's contents
    # A different, smaller goal set right after: stale contents must not leak into it.
    sub = goals[5:9]
    got_sub = db.top_down_many_noalloc(sub, limits[5:9])
    # What the entry point is for: not a byte of device memory is taken or given back, and the
    # context's own tables stay as they were.
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert db.stats() == stats_before and db.device_rows() == rows_before
    assert got_sub == db.top_down_many(sub, limits[5:9])
    db.close()


def test_noalloc_refuses_a_fill_beyond_its_fixed_size(m):
    db = m.SynthesisDatabase()
    # the closure of an 8x8x8 Matmul: its plan arrays alone (hundreds of MB) exceed the fixed array
    import torch
    big = m.simple_spec(m.KIND_MATMUL, m.DTYPE_U32, [1, 8, 8, 8], m.GL)
    small = m.simple_spec(m.KIND_MATMUL, m.DTYPE_U32, [1, 1, 1, 1], m.GL)
    db.top_down_many_noalloc([small])
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    with pytest.raises(RuntimeError, match="no-allocation entry point has") as e:
        db.top_down_many_noalloc([big])
    assert e.value.status == -5          # its own code: a goal that cannot be canonicalised is -4
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before   # the refusal allocated nothing either
    # the context is still usable, and the allocating entry point takes the same goal
    assert db.top_down(big).found == 1
    db.close()

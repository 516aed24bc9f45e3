"""GPU parity: the CUDA fill against the CPU oracle, through the C ABI, bit-exact."""
import numpy as np
import pytest

import parity_util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def m(built_extension):
    import morello_b200
    return morello_b200


def test_precompute_size1_matches_oracle_everywhere(m, oracle):
    o = oracle.new()
    o.precompute(1)
    keys, off, rect, dec = o.dump()
    assert o.dominance_conflicts() == 0
    db = m.SynthesisDatabase()
    st = db.precompute(1)
    assert st["n_specs"] == 180
    bad = parity_util.compare_puts(db, keys, off, rect, dec)
    assert not bad, "\n".join(bad)
    db.close()
    o.close()


@pytest.mark.parametrize("dtype_name", ["u32", "f32"])
def test_matmul2_top_down_closure_matches_oracle(m, oracle, dtype_name):
    """BASELINE config 1: `morello matmul 2` (frontend/src/main.rs:192-204) and its f32 twin."""
    dtype = m.DTYPE_U32 if dtype_name == "u32" else m.DTYPE_F32
    goal = m.simple_spec(m.KIND_MATMUL, dtype, [1, 2, 2, 2], m.GL)
    o = oracle.new()
    want = o.top_down(goal, m.MAX_MEM)
    db = m.SynthesisDatabase()
    got = db.top_down(goal)
    assert got.found == 1 and want.found == 1
    assert (got.action, got.main_cost, got.depth, tuple(got.peaks)) == \
        (want.action, want.main, want.depth, tuple(want.peaks))
    keys, off, rect, dec = o.dump()
    bad = parity_util.compare_puts(db, keys, off, rect, dec)
    assert not bad, "\n".join(bad)
    db.close()
    o.close()


def test_precompute_size2_matches_oracle_everywhere(m, oracle):
    """The bench workload at full size: every put of the oracle's size-2 precompute (u32 + f32),
    checked at both corners of its rectangle."""
    o = oracle.new()
    rep = o.precompute(2)
    assert rep["finished"] and o.dominance_conflicts() == 0
    keys, off, rect, dec = o.dump()
    db = m.SynthesisDatabase()
    st = db.precompute(2)
    assert st["n_specs"] == rep["logical_specs"] == 10454
    bad = parity_util.compare_puts(db, keys, off, rect, dec)
    assert not bad, "\n".join(bad)
    db.close()
    o.close()

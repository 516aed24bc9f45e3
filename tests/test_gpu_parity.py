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


@pytest.mark.parametrize("name", ["precompute_1", "matmul2_u32", "matmul2_f32"])
def test_gpu_tables_match_committed_golden_fixtures(m, name):
    """Same checks without the oracle in the loop: the committed fixtures of tests/golden."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name + ".npz"))
    db = m.SynthesisDatabase()
    if name == "precompute_1":
        db.precompute(1)
    else:
        got = db.top_down(g["goal"].tobytes())
        assert [got.found, got.action, got.main_cost, got.depth] + list(got.peaks) == list(g["goal_decision"])
    bad = parity_util.compare_puts(db, g["keys"], g["key_off"], g["rect"], g["dec"])
    assert not bad, "\n".join(bad)
    db.close()


@pytest.mark.parametrize("dtype_name", ["u32", "f32"])
def test_reconstructed_implementation_matches_oracle_and_golden(m, oracle, dtype_name):
    """get_impl (morello/src/db/mod.rs:505-516): the tree reconstructed from the GPU tables is the
    oracle's, line for line - also at lower limits and for a Move goal."""
    import os
    dtype = m.DTYPE_U32 if dtype_name == "u32" else m.DTYPE_F32
    goal = m.simple_spec(m.KIND_MATMUL, dtype, [1, 2, 2, 2], m.GL)
    move = m.simple_spec(m.KIND_MOVE, dtype, [2, 2], m.GL)
    db = m.SynthesisDatabase()
    db.top_down_many([goal, move])
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", f"impl_matmul2_{dtype_name}.txt")) as f:
        assert db.get_impl(goal) == f.read()
    o = oracle.new()
    for spec, limits in ((goal, m.MAX_MEM), (goal, (6, 0, 64, 1024)), (move, m.MAX_MEM), (move, (3, 16, 8, 4096))):
        assert db.get_impl(spec, limits) == o.get_impl(spec, limits)
    with pytest.raises(RuntimeError, match="no implementation"):
        db.get_impl(goal, (2, 0, 0, 0))
    o.close()
    db.close()


def test_edge_cases(m):
    db = m.SynthesisDatabase()
    # empty goal list
    assert db.top_down_many([]) == []
    # zero limits: nothing fits except what needs no memory
    rf_mm = m.simple_spec(m.KIND_MATMUL_ACCUM, m.DTYPE_U32, [1, 1, 1, 1], m.RF)
    gl_mm = m.simple_spec(m.KIND_MATMUL, m.DTYPE_U32, [1, 2, 2, 2], m.GL)
    got = db.top_down_many([rf_mm, gl_mm], [(0, 0, 0, 0), (0, 0, 0, 0)])
    assert got[0].found == 1 and got[0].main_cost == 2 and got[0].peaks == (0, 0, 0, 0)
    assert got[1].found == 0
    # lookups: a Spec outside the tables is a miss, limits above the planned top are a miss
    other = m.simple_spec(m.KIND_MATMUL, m.DTYPE_F32, [1, 2, 2, 2], m.GL)
    assert db.get(other).found == -1
    assert db.get(gl_mm, (17, 16, 1024, 33554432)).found == -1
    # limits between lattice entries read the entry below
    a = db.get(gl_mm, (16, 16, 1024, 33554432))
    b = db.get(gl_mm, (16, 16, 1024, 1 << 20))
    assert a == b and a.found == 1
    # monotone in memory: fewer registers never cost less
    prev = None
    for rf in range(0, 17):
        d = db.get(gl_mm, (rf, 16, 1024, 33554432))
        if d.found == 1:
            if prev is not None:
                assert d.main_cost <= prev
            prev = d.main_cost
    db.close()


def test_precompute_size4_matches_a_bounded_oracle_run(m, oracle):
    """Size 4 (642 k logical Specs with the closure): the oracle cannot finish it in test time, so
    it runs its faithful stage order under a time budget and every put it made so far is checked
    against the full GPU tables."""
    import os
    o = oracle.new()
    rep = o.precompute(4, threads=os.cpu_count() or 1, budget_s=25.0)
    assert o.dominance_conflicts() == 0
    keys, off, rect, dec = o.dump()
    assert len(dec) > 10000
    db = m.SynthesisDatabase()
    st = db.precompute(4)
    assert st["n_goal_specs"] == 410954
    bad = parity_util.compare_puts(db, keys, off, rect, dec)
    assert not bad, "\n".join(bad)
    db.close()
    o.close()


@pytest.mark.parametrize("dtype_name,shape", [("u32", [1, 2, 2, 4]), ("f32", [1, 2, 2, 4]), ("u32", [1, 4, 2, 2]),
                                              ("f32", [1, 2, 4, 4])])
def test_mid_size_matmul_goals_match_oracle(m, oracle, dtype_name, shape):
    """Goals beyond size 2 that the oracle's top-down search still finishes in seconds: dimensions
    of 4, vector registers and packed layouts in the closure. Every put of the oracle (up to
    0.8 M per goal) is checked against the GPU tables at both corners of its rectangle."""
    dtype = m.DTYPE_U32 if dtype_name == "u32" else m.DTYPE_F32
    goal = m.simple_spec(m.KIND_MATMUL, dtype, shape, m.GL)
    o = oracle.new()
    want = o.top_down(goal, m.MAX_MEM)
    db = m.SynthesisDatabase()
    got = db.top_down(goal)
    assert (got.found, got.action, got.main_cost, got.depth, tuple(got.peaks)) == \
        (want.found, want.action, want.main, want.depth, tuple(want.peaks))
    assert o.dominance_conflicts() == 0
    keys, off, rect, dec = o.dump()
    bad = parity_util.compare_puts(db, keys, off, rect, dec)
    assert not bad, "\n".join(bad)
    assert db.get_impl(goal) == o.get_impl(goal, m.MAX_MEM)
    db.close()
    o.close()


def test_size2_tables_satisfy_the_recurrence_at_every_lattice_point(m):
    """Property over the whole table, independent of the oracle: at every one of the 93 636
    limits of every Spec, re-deriving the decision from the children's tables gives the stored
    decision. By induction over the lattice this pins the table to the direct solve everywhere,
    including inside the cells of the compacted grids."""
    db = m.SynthesisDatabase()
    st = db.precompute(2)
    checked, bad = db.verify(0)
    assert checked == st["n_specs"] * 17 * 17 * 12 * 27 and bad == 0
    db.close()


def test_refills_are_identical_and_the_statistics_add_up(m):
    """The relaxation sweeps update cells in place while other warps read them, so how often a
    Spec is looked at differs from run to run; the table must not. Two fills of one plan give the
    same rows (checksum) and the same grids; what the kernel reports about itself is consistent."""
    db = m.SynthesisDatabase()
    db.plan_precompute(4)
    db.upload()
    db.fill()
    first, st1 = db.checksum(), db.stats()
    db.fill()
    second, st2 = db.checksum(), db.stats()
    assert first == second == 0x2C30E967E6CC225F   # the size-4 tables (pinned against the oracle by the tests above)
    for st in (st1, st2):
        assert st["n_rows"] == 3573174
        assert 0 < st["n_cells_unordered"] < st["n_cells_solved"]
        assert st["n_sweeps"] >= st["n_passes"] > 0     # every pass ends with a sweep that changes nothing
        assert 0 < st["n_candidates_swept"] < st["n_candidates_evaluated"]
        assert 0 < sum(st["phase_ms"]) <= st["fill_ms"] * 1.001
    assert st2["n_buffer_growths"] == 0 and st2["n_launches"] == st2["n_stages"]   # the buffers fit by now: one launch per stage
    assert st1["n_rows"] == st2["n_rows"] and st1["n_cells_solved"] == st2["n_cells_solved"] and st1["n_passes"] == st2["n_passes"]
    assert db.verify(5_000_000, seed=9)[1] == 0
    db.close()


def test_verify_notices_a_corrupted_row(m):
    import torch
    from morello_b200 import sharded
    db = m.SynthesisDatabase()
    db.precompute(1)
    assert db.verify(0)[1] == 0
    ptr, n = db.device_rows()
    rows = torch.as_tensor(sharded._DeviceBytes(ptr, n * sharded.row_bytes()), device="cuda").view(torch.int32)
    rows[4 * (n // 2)] += 1      # main cost of one row in the middle of the table
    torch.cuda.synchronize()
    assert db.verify(0)[1] > 0
    db.close()


def test_size8_full_workload_against_oracle_and_recurrence(m, oracle):
    """BASELINE config 2 at full size (10.6 M goal Specs), the configuration the benchmark times.
    The oracle cannot finish it, so every phase (Move, Zero, Matmul) runs its faithful stage order
    under a time budget and every put it made is checked against the GPU table at both corners of
    its rectangle; the recurrence is checked at 500 M random (Spec, limits) points; and a second
    fill reproduces the table bit for bit."""
    import os
    import torch
    from morello_b200 import sharded
    o = oracle.new()
    rep = o.precompute_phases(8, [8.0, 8.0, 8.0], threads=os.cpu_count() or 1)
    assert o.dominance_conflicts() == 0
    assert all(p["goal_specs_completed"] > 0 for p in rep["phases"])   # the sample reaches every phase
    keys, off, rect, dec = o.dump()
    assert len(dec) > 100000
    db = m.SynthesisDatabase()
    st = db.precompute(8)
    assert st["n_goal_specs"] == 10613126
    bad = parity_util.compare_puts(db, keys, off, rect, dec)
    assert not bad, "\n".join(bad)
    o.close()
    checked, bad = db.verify(500_000_000, seed=7)
    assert checked == 500_000_000 and bad == 0
    ptr, n = db.device_rows()
    before = torch.as_tensor(sharded._DeviceBytes(ptr, n * sharded.row_bytes()), device="cuda").clone()
    sum_before = db.checksum()
    db.fill()
    ptr2, n2 = db.device_rows()
    assert n2 == n
    after = torch.as_tensor(sharded._DeviceBytes(ptr2, n2 * sharded.row_bytes()), device="cuda")
    assert torch.equal(before, after) and db.checksum() == sum_before
    # known answers of the small goals still hold inside the big database
    goal = m.simple_spec(m.KIND_MATMUL, m.DTYPE_U32, [1, 2, 2, 2], m.GL)
    d = db.get(goal)
    assert (d.found, d.action, d.main_cost, d.depth, d.peaks) == (1, 1, 127, 7, (8, 0, 4, 0))
    db.close()


def test_save_load_export_and_put(m, tmp_path):
    """Persistence and bulk export: a saved database reloads into a fresh context (lookups only) and
    into a context that holds the job's plan (verify works too) with byte-identical answers; the
    bulk export, the per-Spec export and the rectangle export agree; put accepts what the tables
    hold and refuses anything else."""
    import numpy as np
    db = m.SynthesisDatabase()
    st = db.precompute(2)
    n = db.num_specs()
    path = str(tmp_path / "p2.mrldb")
    db.save(path)
    blobs = [db.spec_blob(i) for i in range(0, n, 7)]
    limits = [(16 - (i % 5), 16, 1024 >> (i % 4), 33554432) for i in range(len(blobs))]
    want = db.get_many(blobs, limits)
    want_sum = db.checksum()

    fresh = m.SynthesisDatabase()
    fresh.load(path)                      # no plan in this context: lookups only
    assert fresh.get_many(blobs, limits) == want and fresh.checksum() == want_sum
    goal = m.simple_spec(m.KIND_MATMUL, m.DTYPE_U32, [1, 2, 2, 2], m.GL)
    assert fresh.get_impl(goal) == db.get_impl(goal)
    with pytest.raises(RuntimeError, match="without their plan"):
        fresh.verify(10)
    with pytest.raises(RuntimeError):
        fresh.fill()
    fresh.close()

    planned = m.SynthesisDatabase()
    planned.plan_precompute(2)
    planned.load(path)                    # same job: the plan's candidate records stay usable
    assert planned.get_many(blobs, limits) == want
    assert planned.verify(5_000_000)[1] == 0
    planned.fill()
    assert planned.checksum() == want_sum
    planned.close()

    other = m.SynthesisDatabase()
    other.plan_precompute(1)              # another job's plan: the file brings its own Specs
    other.load(path)
    assert other.num_specs() == n and other.get_many(blobs, limits) == want
    other.close()

    # a file whose contents were altered after saving fails its checksum
    raw = bytearray(open(path, "rb").read())
    raw[-8] ^= 1
    bad_path = str(tmp_path / "bad.mrldb")
    open(bad_path, "wb").write(bytes(raw))
    broken = m.SynthesisDatabase()
    with pytest.raises(RuntimeError, match="checksum") as e:
        broken.load(bad_path)
    assert e.value.status == -8
    broken.close()

    # bulk export against the per-Spec export and the lookups
    masks, first, rows = db.export_all()
    assert masks.shape == (n, 4) and len(rows) == st["n_rows"] == int(first[n])
    for i in range(0, n, 97):
        grid_masks, cells = db.spec_grid(i)
        assert list(masks[i]) == grid_masks and int(first[i + 1] - first[i]) == cells or int(first[i]) + cells <= len(rows)
        per_spec = db.export_rows(i)
        for j, dcn in enumerate(per_spec):
            r = rows[int(first[i]) + j]
            if dcn.found:
                assert (int(r[0]), int(r[2]) & 0xFFFF, int(r[2]) >> 16) == (dcn.main_cost, dcn.action, dcn.depth)
            else:
                assert int(r[2]) == 0xFFFFFFFF
        # rectangles: they tile the whole lattice box, and every corner reads back its own decision
        rects = db.export_rects(i)
        assert 1 <= len(rects) <= cells
        volume = 0
        for lo, hi, dcn in rects:
            volume += int(np.prod([h - l + 1 for l, h in zip(lo, hi)]))
        assert volume == 17 * 17 * 12 * 27
        blob = db.spec_blob(i)
        for lo, hi, dcn in rects[:6]:
            for corner in (lo, hi):
                lim = (corner[0], corner[1], 0 if corner[2] == 0 else 1 << (corner[2] - 1),
                       0 if corner[3] == 0 else 1 << (corner[3] - 1))
                assert db.get(blob, lim) == dcn
    # put: what the tables hold is accepted, anything else refused
    d = db.get(goal)
    db.put(goal, m.MAX_MEM, d)
    wrong = m.Decision(1, d.action, d.main_cost + 1, d.depth, d.peaks)
    with pytest.raises(RuntimeError, match="another decision") as e:
        db.put(goal, m.MAX_MEM, wrong)
    assert e.value.status == -9
    outside = m.simple_spec(m.KIND_MATMUL, m.DTYPE_U32, [1, 8, 8, 8], m.GL)
    with pytest.raises(RuntimeError, match="not in the tables"):
        db.put(outside, m.MAX_MEM, d)
    db.close()


def test_fill_waits_for_device_candidate_records(m):
    """A plan adopted without its candidate records cannot be filled until they have arrived on
    the device and passed the device-side check; records that name Specs outside the plan are
    refused there."""
    import ctypes
    import torch
    from morello_b200 import sharded
    src = m.SynthesisDatabase()
    src.set_shard(0, 1)
    src.precompute(2)
    blobs = src.plan_share()
    dst = m.SynthesisDatabase()
    dst.set_shard(0, 1)
    ptrs = dst.plan_adopt([nb for _, nb in blobs], cands_on_device_only=True)
    assert ptrs[3] == 0
    for k, ((p, nb), q) in enumerate(zip(blobs, ptrs)):
        if q and nb:
            ctypes.memmove(q, p, nb)
    dst.plan_adopt_done()
    dst.upload()
    with pytest.raises(RuntimeError, match="candidate records are not on the device") as e:
        dst.fill()
    assert e.value.status == -3
    sptr, sbytes = src.device_cands()
    dptr, dbytes = dst.device_cands()
    assert sbytes == dbytes
    s_t = torch.as_tensor(sharded._DeviceBytes(sptr, sbytes), device="cuda")
    d_t = torch.as_tensor(sharded._DeviceBytes(dptr, dbytes), device="cuda")
    d_t.copy_(s_t)
    d_t.view(torch.int32)[0] |= 9 << 16      # record 0: a combine kind that does not exist
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="do not describe this plan"):
        dst.cands_arrived()
    with pytest.raises(RuntimeError, match="candidate records are not on the device"):
        dst.fill()
    d_t.copy_(s_t)
    torch.cuda.synchronize()
    dst.cands_arrived()
    dst.fill()
    assert dst.checksum() == src.checksum()
    dst.close()
    src.close()

"""The planner's action tabulation (morello_b200/csrc/model/) against an independent restatement of
the reference's enumeration (oracle/enumeration.py, written from the Rust sources alone): for every
Spec, the same applicable actions with the same ActionNums, combine kinds, immediates, consumed
memory and sub-Specs, byte for byte. GPU-versus-oracle parity cannot see an error in the tabulation,
because the C++ oracle includes the planner's model headers; this test can."""
import random

import pytest

import enumeration as en


@pytest.fixture(scope="module")
def m(built_extension):
    import morello_b200
    return morello_b200


def _same(m, blob):
    spec = en.parse_blob(blob)
    mine = [(a.number, a.kind, a.imm, a.level if a.kind in (en.MOVE_KIND, en.LEAF) else 0,
             a.units if a.kind in (en.MOVE_KIND, en.LEAF) else 0, a.children) for a in en.enumerate_actions(spec)]
    theirs = [(n, k, imm, lvl if k in (en.MOVE_KIND, en.LEAF) else 0, u if k in (en.MOVE_KIND, en.LEAF) else 0, ch)
              for n, k, imm, lvl, u, ch in m.tabulate(blob)]
    assert mine == theirs, (m.describe_spec(blob), [x for x in mine if x not in theirs][:3],
                            [x for x in theirs if x not in mine][:3])
    return mine


def test_every_size2_spec_is_tabulated_like_the_reference(m):
    """All 10 454 Specs of the size-2 precompute and its closure (u32 and f32)."""
    db = m.SynthesisDatabase(device=-1)
    db.plan_precompute(2)
    n = db.num_specs()
    assert n == 10454
    n_actions = 0
    for i in range(n):
        n_actions += len(_same(m, db.spec_blob(i)))
    assert n_actions == db.stats()["n_candidates"]   # top limits: every applicable action became a candidate record
    db.close()


def test_sampled_larger_specs_are_tabulated_like_the_reference(m):
    """Dimensions of 4, 8 and 16, vector registers, Packed and OddEven layouts: 6 000 random Specs of
    the size-4 precompute, and the closure of 8x8x8 and 16x16x16 Matmul goals walked breadth-first
    through the independent enumeration's own sub-Specs (3 000 Specs each)."""
    rng = random.Random(0x5EED)
    db = m.SynthesisDatabase(device=-1)
    db.plan_precompute(4)
    ids = rng.sample(range(db.num_specs()), 6000)
    seen_kinds, cover = set(), {"packed": 0, "oddeven": 0, "vrf": 0}

    def note(blob):
        spec = en.parse_blob(blob)
        seen_kinds.add(spec.kind)
        for mem, _vs, lay in spec.auxes:
            cover["vrf"] += mem == en.VRF
            cover["packed"] += any(k == en.PACKED for _, k, _ in lay.dims)
            cover["oddeven"] += any(k == en.ODDEVEN for _, k, _ in lay.dims)

    for i in ids:
        blob = db.spec_blob(i)
        _same(m, blob)
        note(blob)
    db.close()
    for size, dtype in ((8, m.DTYPE_U32), (16, m.DTYPE_F32)):
        goal = m.simple_spec(m.KIND_MATMUL, dtype, [1, size, size, size], m.GL)
        seen, frontier, done = {goal}, [goal], 0
        while frontier and done < 3000:
            nxt = []
            rng.shuffle(frontier)
            for blob in frontier:
                if done >= 3000:
                    break
                note(blob)
                for _n, _k, _imm, _lvl, _u, children in _same(m, blob):
                    for c in children:
                        if c not in seen:
                            seen.add(c)
                            nxt.append(c)
                done += 1
            frontier = nxt
        assert done == 3000
    # what the sample covered (4-byte dtypes: OddEven strips start at 8 values, so only the 8 / 16 goals reach them)
    assert seen_kinds == {en.MOVE, en.FILL_ZERO, en.MATMUL_ACCUM, en.MATMUL}
    assert cover["packed"] > 1000 and cover["oddeven"] > 50 and cover["vrf"] > 1000, cover


def test_hand_derived_action_lists(m):
    """ActionNum -> action for a few small Specs, derived by hand from common_actions.rs and cpu.rs."""
    # FillZero([1], u32, L1): 0 Move->L1 (cache-miss self-move, rejected), 1 Move->RF, 2-3 Move->VRF (vector
    # sizes 4 and 8 do not divide one value), 4 TileOut (matches the original), 5 MemsetZero, 6 ValueZero
    blob = m.simple_spec(m.KIND_FILL_ZERO, m.DTYPE_U32, [1], m.L1)
    got = en.enumerate_actions(en.parse_blob(blob))
    assert [(a.number, a.kind, a.what) for a in got] == [(1, en.MOVE_KIND, "move operand 0 to memory 0"),
                                                         (5, en.LEAF, "MemsetZero"), (6, en.LEAF, "ValueZero")]
    assert got[0].imm == 2 and got[0].units == 1 and got[1].imm == 1 and got[2].imm == 3
    _same(m, blob)
    # MatmulAccum([1,1,1,1], u32, RF x3): 0-2 self-Moves, 3-5 TileOuts of size 1 (match), 6 MultAdd; no Split
    blob = m.simple_spec(m.KIND_MATMUL_ACCUM, m.DTYPE_U32, [1, 1, 1, 1], m.RF)
    got = en.enumerate_actions(en.parse_blob(blob))
    assert [(a.number, a.kind, a.imm) for a in got] == [(6, en.LEAF, 2)]
    _same(m, blob)
    # Matmul([1,1,1,1], u32, RF x3): 0-5 as above, no kernel, 6 ToAccum -> FillZero([1,1,1]) then MatmulAccum
    blob = m.simple_spec(m.KIND_MATMUL, m.DTYPE_U32, [1, 1, 1, 1], m.RF)
    got = en.enumerate_actions(en.parse_blob(blob))
    assert [(a.number, a.kind, len(a.children)) for a in got] == [(6, en.BLOCK, 2)]
    assert en.parse_blob(got[0].children[0]).kind == en.FILL_ZERO and en.parse_blob(got[0].children[1]).kind == en.MATMUL_ACCUM
    _same(m, blob)
    # Move([1] u32, RF -> L1): 0 Move src (self), 1 Move dst->L1 (self), 2 dst->RF, 3-4 dst->VRF (rejected),
    # 5 TileOut (matches), 6 Assign = move costs (0 + 2) + 1
    rf = en.Spec(en.MOVE, en.U32, True, (1,), [(en.RF, 0, en.Layout()), (en.L1, 0, en.Layout())])
    got = en.enumerate_actions(rf)
    assert [(a.number, a.kind) for a in got] == [(2, en.MOVE_KIND), (6, en.LEAF)] and got[1].imm == 3
    _same(m, rf.blob())
    # MatmulAccum([1,2,8], u32): lhs in L1 packed by 4 along k, rhs a column of 8 in VRF (vector size 8),
    # out 1x2x1 in RF. A VRF operand, a Packed layout and a dimension of 8 in one Spec.
    lhs = en.layout_new([(1, en.DYNAMIC, 0), (2, en.DYNAMIC, 0), (2, en.PACKED, 4)])
    spec = en.Spec(en.MATMUL_ACCUM, en.U32, True, (1, 2, 8, 1),
                   [(en.L1, 0, lhs), (en.VRF, 8, en.row_major((1, 8, 1))), (en.RF, 0, en.Layout())])
    assert en.canonicalize_spec(spec)
    got = _same(m, spec.blob())
    numbers = [n for n, *_ in got]
    assert numbers == sorted(numbers) and len(set(numbers)) == len(numbers)
    kinds = [k for _, k, *_ in got]
    assert en.MOVE_KIND in kinds and en.LOOP in kinds      # moves of each operand, tile-outs of m, splits of k
    splits = [(n, imm) for n, k, imm, *_ in got if k == en.LOOP and n > max(x for x, kk, *_ in got if kk == en.MOVE_KIND)]
    assert splits, got

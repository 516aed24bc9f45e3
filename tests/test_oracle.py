"""CPU tests of the oracle: the reference's known-answer vectors and the golden fixtures."""
import os
import subprocess

import numpy as np
import pytest

import oracle_lib

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
MAX_MEM = (16, 16, 1024, 33554432)


def _sorted_puts(keys, off, rect, dec):
    kb = keys.tobytes()
    items = []
    for i in range(len(dec)):
        items.append((kb[int(off[i]):int(off[i + 1])], rect[i].tobytes(), dec[i].tobytes()))
    return sorted(items)


def test_known_answer_vectors_of_the_reference(oracle):
    """oracle/kat.cpp replays every deterministic vector the reference's in-tree tests hold for
    this path (layouts, cache lines, loop costs, MemVec rules, reducer ties, kernel costs, ...)."""
    res = subprocess.run([oracle.kat_path], capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "failures: 0" in res.stdout


def test_precompute_size1_matches_golden(oracle):
    o = oracle.new()
    rep = o.precompute(1)
    assert rep["finished"] and rep["logical_specs"] == 180 and o.dominance_conflicts() == 0
    g = np.load(os.path.join(GOLDEN, "precompute_1.npz"))
    assert _sorted_puts(*o.dump()) == _sorted_puts(g["keys"], g["key_off"], g["rect"], g["dec"])
    o.close()


def test_matmul2_top_down_matches_golden(oracle):
    for name in ("u32", "f32"):
        g = np.load(os.path.join(GOLDEN, f"matmul2_{name}.npz"))
        o = oracle.new()
        d = o.top_down(g["goal"].tobytes(), MAX_MEM)
        assert [d.found, d.action, d.main, d.depth] + list(d.peaks) == list(g["goal_decision"])
        assert _sorted_puts(*o.dump()) == _sorted_puts(g["keys"], g["key_off"], g["rect"], g["dec"])
        o.close()


@pytest.mark.parametrize("dtype_name", ["u32", "f32"])
def test_reconstructed_implementation_matches_golden(oracle, dtype_name):
    """get_impl: re-applying the stored actions from the goal down gives the committed tree."""
    g = np.load(os.path.join(GOLDEN, f"matmul2_{dtype_name}.npz"))
    with open(os.path.join(GOLDEN, f"impl_matmul2_{dtype_name}.txt")) as f:
        want = f.read()
    o = oracle.new()
    got = o.get_impl(g["goal"].tobytes(), (16, 16, 1024, 33554432))
    o.close()
    assert got == want
    lines = want.splitlines()
    cost = {"u32": 127, "f32": 119}[dtype_name]   # MultAdd costs 2 on integers, 1 on f32 (cpu.rs:2315-2340): 8 kernels
    assert len(lines) == 17 and lines[0].startswith("Matmul(1x2x2x2") and f" cost {cost} " in lines[0]
    assert lines[-1].lstrip().startswith("MatmulAccum(1x1x1x1") and "Kernel(MultAdd)" in lines[-1]


def test_hand_derived_matmul1_cost(oracle):
    """Matmul 1x1x1 u32 in GL: three cache-miss Moves into L1 (20 + 2 each), MemsetZero (1) and
    MultAdd on L1 scalars (2 + 3 * 2): 75; three L1 lines round up to 4."""
    from golden.make_golden import matmul_goal_blob
    o = oracle.new()
    d = o.top_down(matmul_goal_blob(1, 4), MAX_MEM)
    assert (d.found, d.main, d.depth, list(d.peaks)) == (1, 75, 5, [0, 0, 4, 0])
    d = o.top_down(matmul_goal_blob(1, 6), MAX_MEM)
    assert (d.found, d.main) == (1, 74)  # f32 MultAdd costs 1 instead of 2
    o.close()


def test_more_memory_never_worsens_and_peak_limits_reproduce(oracle):
    """The two relations the reference checks by proptest (morello/src/search/mod.rs:152-199):
    a solve at the result's own peaks gives the same decision, and lower limits never cost less."""
    g = np.load(os.path.join(GOLDEN, "matmul2_u32.npz"))
    keys, off, rect, dec = g["keys"], g["key_off"], g["rect"], g["dec"]
    kb = keys.tobytes()
    rng = np.random.default_rng(0x5EED)
    o = oracle.new()
    o.top_down(g["goal"].tobytes(), MAX_MEM)
    for i in rng.choice(len(dec), size=300, replace=False):
        if dec[i]["found"] != 1:
            continue
        key = kb[int(off[i]):int(off[i + 1])]
        peaks = [int(x) for x in dec[i]["peaks"]]
        again = o.top_down(key, peaks)
        assert (again.found, again.action, again.main, again.depth, list(again.peaks)) == \
            (1, int(dec[i]["action"]), int(dec[i]["main"]), int(dec[i]["depth"]), peaks)
        lower = list(oracle_lib.codes_to_limits(rect[i][4:]))
        k = int(rng.integers(0, 4))
        if lower[k] > 0:
            lower[k] = int(lower[k]) // 2
            lo = o.top_down(key, [int(x) for x in lower])
            assert lo.found == 0 or lo.main >= int(dec[i]["main"])
    assert o.dominance_conflicts() == 0
    o.close()

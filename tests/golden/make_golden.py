"""Regenerates the golden fixtures from the CPU oracle.

    python tests/golden/make_golden.py

The reference (Rust) cannot be built or run where this was written and ships no fixture of
filled-database contents, so these vectors come from the C++ oracle under oracle/, which is
itself pinned by the reference's in-tree known-answer tests (oracle/kat.cpp). Each .npz holds
every `put` of one oracle run: Spec blobs, the rectangle [lo..hi] of the limits lattice the put
fills (lattice codes: registers raw, caches bit length) and the decision stored there.

    python tests/golden/make_golden.py --saved-database      # on a machine with a GPU

writes precompute_1.mrldb: the size-1 precompute filled by the CUDA path and saved with mrl_save
(after its contents were checked against the oracle's puts). The CPU tests use it to exercise the
loader's file validation.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, ROOT)
import oracle_lib  # noqa: E402

MAX_MEM = (16, 16, 1024, 33554432)


def matmul_goal_blob(size, dtype_code):
    """Blob of Matmul([1,s,s,s], dtype, GL row-major x3, serial): frontend/src/main.rs:192-204."""
    def aux(shape):
        dims = [d for d in range(len(shape)) if shape[d] != 1]
        out = bytes([3, 0, len(dims), len(dims)])
        for d in dims:
            out += bytes([d, 0, 0, 0])
        return out
    blob = bytes([3, dtype_code, 1, 4]) + b"".join(int(x).to_bytes(2, "little") for x in (1, size, size, size))
    for shape in ((1, size, size), (1, size, size), (1, size, size)):
        blob += aux(shape)
    return blob


def save(name, oracle, extra=None):
    keys, off, rect, dec = oracle.dump()
    path = os.path.join(HERE, name)
    np.savez_compressed(path, keys=keys, key_off=off, rect=rect, dec=dec, **(extra or {}))
    print(name, len(dec), "puts", os.path.getsize(path), "bytes")


def main():
    fac = oracle_lib.load()
    o = fac.new()
    o.precompute(1)
    save("precompute_1.npz", o)
    o.close()
    for dtype_name, code in (("u32", 4), ("f32", 6)):
        o = fac.new()
        goal = matmul_goal_blob(2, code)
        d = o.top_down(goal, MAX_MEM)
        save(f"matmul2_{dtype_name}.npz", o, {"goal": np.frombuffer(goal, dtype=np.uint8),
                                              "goal_decision": np.array([d.found, d.action, d.main, d.depth] + list(d.peaks))})
        # the optimal implementation reconstructed from the stored actions, one line per node
        with open(os.path.join(HERE, f"impl_matmul2_{dtype_name}.txt"), "w") as f:
            f.write(o.get_impl(goal, MAX_MEM))
        o.close()


def saved_database():
    import morello_b200 as m
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import parity_util
    o = oracle_lib.load().new()
    o.precompute(1)
    db = m.SynthesisDatabase(device=0)
    db.precompute(1)
    bad = parity_util.compare_puts(db, *o.dump())
    assert not bad, bad
    path = os.path.join(HERE, "precompute_1.mrldb")
    db.save(path)
    print("precompute_1.mrldb", os.path.getsize(path), "bytes, checksum %016x" % db.checksum())
    db.close()
    o.close()


if __name__ == "__main__":
    if "--saved-database" in sys.argv:
        saved_database()
    else:
        main()

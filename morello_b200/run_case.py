"""Runs one named fill on cuda:0 and prints its statistics as JSON.

    python -m morello_b200.run_case matmul2 [--fills N]      # closure of `morello matmul 2` (u32)
    python -m morello_b200.run_case precompute1|precompute2  # the precompute of that size
    python -m morello_b200.run_case precompute2_u32          # size 2, u32 tables only (2.8 GB)

Small, fixed cases for profilers (the commands quoted in profiles/ use this module).
"""
import argparse
import json

import morello_b200 as m


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["matmul1", "matmul2", "matmul2_f32", "precompute1", "precompute2", "precompute2_u32",
                                     "precompute4", "precompute4_u32"])
    ap.add_argument("--fills", type=int, default=1, help="fills of the final plan (>= 1)")
    ap.add_argument("--caps", type=str, default=None, help="lattice caps RF,VRF,L1,GL (codes; -1 = all)")
    ap.add_argument("--no-verify", action="store_true",
                    help="keep the given caps even if an optimal peak exceeds them (profiling a smaller table)")
    args = ap.parse_args()
    db = m.SynthesisDatabase(device=0)
    if args.caps:
        db.set_lattice_caps([int(x) for x in args.caps.split(",")], auto_raise=not args.no_verify)
    if args.case.startswith("matmul"):
        size = int(args.case[6])
        dtype = m.DTYPE_F32 if args.case.endswith("f32") else m.DTYPE_U32
        goal = m.simple_spec(m.KIND_MATMUL, dtype, [1, size, size, size], m.GL)
        db.plan_goals([goal])
    else:
        dtypes = (m.DTYPE_U32,) if args.case.endswith("_u32") else (m.DTYPE_U32, m.DTYPE_F32)
        db.plan_precompute(int(args.case[10]), dtypes=dtypes)
    db.upload()
    try:
        db.fill()
    except RuntimeError:
        if args.no_verify:
            pass
        # the first fill found the starting lattice caps too small: let the library raise them
        elif args.case.startswith("matmul"):
            db.top_down(goal)
        else:
            db.precompute(int(args.case[10]), dtypes=dtypes)
    for _ in range(args.fills - 1):
        try:
            db.fill()
        except RuntimeError:
            if not args.no_verify:
                raise
    st = db.stats()
    st["achieved_GBps"] = st["algorithmic_bytes"] / (st["fill_ms"] * 1e-3) / 1e9 if st["fill_ms"] else None
    print(json.dumps(st))
    db.close()


if __name__ == "__main__":
    main()

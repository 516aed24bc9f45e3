"""Runs one named fill on cuda:0 and prints its statistics as JSON.

    python -m morello_b200.run_case matmul2 [--fills N]      # closure of `morello matmul 2` (u32)
    python -m morello_b200.run_case matmul8                  # closure of one 8x8x8 Matmul (473 k Specs, < 1 GB on the device)
    python -m morello_b200.run_case precompute1|precompute2  # the precompute of that size
    python -m morello_b200.run_case precompute4_u32          # size 4, u32 tables only

Small, fixed cases for profilers (the commands quoted in profiles/ use this module).
"""
import argparse
import json

import morello_b200 as m


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["matmul1", "matmul2", "matmul2_f32", "matmul8", "precompute1", "precompute2", "precompute2_u32",
                                     "precompute4", "precompute4_u32", "precompute8", "precompute8_u32"])
    ap.add_argument("--fills", type=int, default=1, help="fills of the final plan (>= 1)")
    ap.add_argument("--through", choices=["move", "zero", "matmul"], default="matmul",
                    help="last phase of a precompute case (move: Move Specs only)")
    args = ap.parse_args()
    db = m.SynthesisDatabase(device=0)
    if args.case.startswith("matmul"):
        size = int(args.case[6])
        dtype = m.DTYPE_F32 if args.case.endswith("f32") else m.DTYPE_U32
        goal = m.simple_spec(m.KIND_MATMUL, dtype, [1, size, size, size], m.GL)
        db.plan_goals([goal])
    else:
        dtypes = (m.DTYPE_U32,) if args.case.endswith("_u32") else (m.DTYPE_U32, m.DTYPE_F32)
        db.plan_precompute(int(args.case[10]), through={"move": m.THROUGH_MOVE, "zero": m.THROUGH_ZERO,
                                                        "matmul": m.THROUGH_MATMUL}[args.through], dtypes=dtypes)
    db.upload()
    for _ in range(args.fills):
        db.fill()
    st = db.stats()
    st["achieved_GBps"] = st["algorithmic_bytes"] / (st["fill_ms"] * 1e-3) / 1e9 if st["fill_ms"] else None
    st["combine_GBps"] = st["algorithmic_bytes"] / (st["combine_ms"] * 1e-3) / 1e9 if st["combine_ms"] else None
    print(json.dumps(st))
    db.close()


if __name__ == "__main__":
    main()

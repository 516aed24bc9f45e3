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
    ap.add_argument("case", choices=["matmul1", "matmul2", "matmul2_f32", "precompute1", "precompute2", "precompute2_u32"])
    ap.add_argument("--fills", type=int, default=1)
    args = ap.parse_args()
    db = m.SynthesisDatabase(device=0)
    if args.case.startswith("matmul"):
        size = int(args.case[6])
        dtype = m.DTYPE_F32 if args.case.endswith("f32") else m.DTYPE_U32
        db.plan_goals([m.simple_spec(m.KIND_MATMUL, dtype, [1, size, size, size], m.GL)])
    else:
        if args.case.endswith("_u32"):
            db.plan_precompute(int(args.case[10]), dtypes=(m.DTYPE_U32,))
        else:
            db.plan_precompute(int(args.case[-1]))
    db.upload()
    for _ in range(args.fills):
        db.fill()
    st = db.stats()
    st["achieved_GBps"] = st["algorithmic_bytes"] / (st["fill_ms"] * 1e-3) / 1e9 if st["fill_ms"] else None
    print(json.dumps(st))
    db.close()


if __name__ == "__main__":
    main()

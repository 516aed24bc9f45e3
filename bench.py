#!/usr/bin/env python
"""Benchmark of the synthesis-database fill.

  python bench.py --gpus N --steps K --warmup W            # the CUDA path
  python bench.py --impl reference --gpus N --steps K ...  # the reference algorithm on host cores

One step = one complete fill of the workload's database. The workload is BASELINE config 2: the
Move, Zero and Matmul phases of `precompute --target avx2 --through matmul 8` over {u32, f32} with
serial-only bounds (the reference's Matmul phase also enumerates Broadcast / Max / Softmax bounds,
which the Matmul closure does not need and which are not built): 10.6 M goal logical Specs, 14.7 M
with their dependency closure, 400 M candidate records. `--size 4` and `--size 2` run the smaller
precomputes (size 2 contains the closure of `morello matmul 2`, BASELINE config 1); `--through move`
stops after the Move phase (a small case with large launches, for profilers). All inputs are
synthetic by construction: the Spec space is generated from the size alone.

Unit of work ("Spec resolved"): one (logical Spec, memory limits) entry of the database made
answerable. Both arms cover the same kind of entry - a goal logical Spec of the workload over the
whole 17 x 17 x 12 x 27 limits lattice of the target - so the figure is goal Specs x 93 636 divided
by each arm's time. It is not a solve rate: the CUDA arm also reports the cells it solved and the
candidates it evaluated, the reference arm its `put`s. Beyond size 2 the CPU arm cannot finish in
bench time: every phase (Move, Zero, Matmul) runs its own stage order under a third of the time
budget, on what the phases before it left in the database, and the goal Specs whose limits
staircase was completed are counted.

Outside the timed region the CUDA arm checks what it timed (`parity`): the table against the
reference algorithm's puts of the CPU leg (N = 1), the fill's recurrence at sampled points, and at
N > 1 that every rank holds the same table and that it equals a single-GPU fill.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LATTICE_POINTS = 17 * 17 * 12 * 27  # RF 0..16, VRF 0..16, L1 and GL as bit lengths (avx2.rs:59-65)
SIZE = 8
THROUGH = 2
THROUGH_NAMES = ["move", "zero", "matmul"]
DTYPES = (4, 6)   # u32, f32: DTYPES of precompute/src/main.rs:55
DTYPE_NAMES = {4: "u32", 6: "f32"}


def workload_name():
    return ("precompute --target avx2 --through %s %d: Move%s phases only, %s, serial-only bounds"
            % (THROUGH_NAMES[THROUGH], SIZE, ["", "+Zero", "+Zero+Matmul"][THROUGH],
               "+".join(DTYPE_NAMES[d] for d in DTYPES)))


def dtype_mask():
    return sum({4: 1, 6: 2}[d] for d in DTYPES)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index=0):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                                         text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_oracle(threads, budget_s):
    """The reference's algorithm (top-down memoised search with a range-filling memo table and the
    precompute driver) restated in C++ under oracle/, on the host cores. Returns (report, oracle);
    the caller closes the oracle."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_lib
    o = oracle_lib.load().new()
    n_phases = THROUGH + 1
    if SIZE <= 2:
        r = o.precompute(SIZE, through=THROUGH, dtype_mask=dtype_mask(), threads=threads)
        r["phases"] = None
    else:
        r = o.precompute_phases(SIZE, [budget_s / n_phases] * n_phases, through=THROUGH, dtype_mask=dtype_mask(), threads=threads)
        r["finished"] = all(p["finished"] for p in r["phases"])
    r["utilisation"] = r["busy_seconds"] / (r["seconds"] * threads) if r["seconds"] > 0 else None
    return r, o


def cpu_sample_text(rep, budget_s):
    if rep["finished"]:
        return "the whole workload (C++ restatement of the reference algorithm; the Rust reference cannot be built here)"
    return ("%.0f s of the workload: each phase (%s) runs its own stage order for a third of that, on what the phases "
            "before it left in the database; goal Specs whose limits staircase was completed are counted (C++ "
            "restatement of the reference algorithm; the Rust reference cannot be built here)"
            % (budget_s, ", ".join(THROUGH_NAMES[:THROUGH + 1])))


def cpu_baseline_object(rep, cores, budget_s):
    value = rep["logical_specs"] * LATTICE_POINTS / rep["seconds"]
    return {"value": value, "unit": "specs/s", "cores": cores, "kind": "port", "sample": cpu_sample_text(rep, budget_s),
            "wall_s": rep["seconds"], "goal_specs_completed": rep["logical_specs"], "reference_puts": rep["puts"],
            "puts_per_s": rep["puts"] / rep["seconds"], "core_utilisation": rep["utilisation"], "phases": rep["phases"]}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    times, last = [], None
    # each step is one bounded sample; the samples are sized so that the whole run stays within five minutes
    budget = min(args.cpu_budget, max(3.0, 300.0 / max(1, args.steps)))
    for i in range((0 if SIZE > 2 else args.warmup) + args.steps):
        rep, o = run_oracle(cores, budget)
        o.close()
        if SIZE > 2 or i >= args.warmup:
            times.append(rep["seconds"])
            last = rep
    per_step = sum(times) / len(times)
    base = cpu_baseline_object(last, cores, budget)
    line = {
        "impl": "reference", "metric": "specs_resolved_per_s", "value": base["value"], "unit": "specs/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
        "config": {"workload": workload_name(), "lattice_points_per_spec": LATTICE_POINTS,
                   "goal_specs_completed_in_sample": last["logical_specs"], "reference_puts": last["puts"]},
        "wall_s_full_db": per_step if last["finished"] else None,
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "specs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def compare_with_oracle_puts(db, oracle_obj):
    """Every oracle put says: the whole rectangle [lo..hi] of the limits lattice has this decision.
    Looks the GPU table up at both corners of every rectangle; returns (lookups, mismatches)."""
    import oracle_lib
    keys, key_off, rect, dec = oracle_obj.dump()
    kb = keys.tobytes()
    blobs = [kb[int(key_off[i]):int(key_off[i + 1])] for i in range(len(key_off) - 1)]
    checked = bad = 0
    for codes in (rect[:, 4:], rect[:, :4]):
        limits = oracle_lib.codes_to_limits(codes)
        for lo in range(0, len(blobs), 200000):
            hi = min(len(blobs), lo + 200000)
            got = db.get_many(blobs[lo:hi], limits[lo:hi].tolist())
            for i, g in enumerate(got):
                want = dec[lo + i]
                checked += 1
                if g.found != int(want["found"]) or (g.found == 1 and (
                        g.action != int(want["action"]) or g.main_cost != int(want["main"]) or g.depth != int(want["depth"]) or
                        tuple(g.peaks) != tuple(int(x) for x in want["peaks"]))):
                    bad += 1
    return checked, bad


def cuda_arm(args):
    import torch
    import torch.distributed as dist
    import morello_b200 as m

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # stdout carries exactly one JSON line: whatever libraries print while the job runs (the NCCL
    # version banner, for one) goes to stderr
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device: the fill has no CPU path")

    # N > 1: ONE database fill sharded over the ranks (the Specs of a stage are split between the
    # GPUs; masks and rows are exchanged per stage), so total work is fixed: strong scaling.
    from morello_b200 import sharded
    db = m.SynthesisDatabase(device=local_rank)

    def one_fill():
        if world > 1:
            sharded.fill_sharded(db, dist, torch)
        else:
            db.fill()

    if world > 1:
        sharded.precompute_sharded(db, SIZE, dist, torch, through=THROUGH, dtypes=DTYPES)
    else:
        db.precompute(SIZE, through=THROUGH, dtypes=DTYPES)  # plans, uploads, fills: leaves plan and tables on the device
    for _ in range(max(args.warmup, 3) - 1):
        one_fill()

    # End to end through the public call: host planning, host->device copy of the plan, the fill,
    # and a device->host read of a sample of the goal Specs' decisions at the top limits.
    n_specs = db.num_specs()
    goal_blobs = [db.spec_blob(i) for i in range(0, n_specs, max(1, n_specs // 512))]
    e2e_s = []
    e2e_runs = 1 if SIZE >= 8 else 3
    for i in range((0 if SIZE >= 8 else 1) + e2e_runs):   # small sizes: one untimed run first
        fresh = m.SynthesisDatabase(device=local_rank)  # a new database: nothing carried over
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        if world > 1:
            sharded.precompute_sharded(fresh, SIZE, dist, torch, through=THROUGH, dtypes=DTYPES)
        else:
            fresh.precompute(SIZE, through=THROUGH, dtypes=DTYPES)
        got = fresh.get_many(goal_blobs, [m.MAX_MEM] * len(goal_blobs))
        dt = time.perf_counter() - t0
        e2e_s.append(dt)
        st2 = fresh.stats()
        fresh.close()
    e2e_s = e2e_s[-e2e_runs:]
    assert all(g.found in (0, 1) for g in got)
    e2e_step = sorted(e2e_s)[len(e2e_s) // 2]  # median
    if world > 1:
        t = torch.tensor([e2e_step], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_step = float(t.item())

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2
    fill_ms, launches = [], 0
    for _ in range(args.steps):
        flush.fill_(1)
        torch.cuda.synchronize()
        one_fill()  # device time measured inside with CUDA events on the launching stream
        s1 = db.stats()
        fill_ms.append(s1["fill_ms"])
        launches += int(s1["n_launches"])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    st = db.stats()
    total_ms = sum(fill_ms)
    cells_by_rank = [int(st["n_cells_solved"])]
    alg_bytes = float(st["algorithmic_bytes"])   # of the final rows this rank computed
    if world > 1:
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
        t = torch.tensor([float(launches), alg_bytes], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        launches, alg_bytes = int(t[0].item()), float(t[1].item())
        t = torch.zeros(world, device="cuda", dtype=torch.float64)
        t[rank] = float(st["n_cells_solved"])
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        cells_by_rank = [int(x) for x in t.tolist()]
    ms_per_step = total_ms / args.steps

    # ---- what was timed, checked (outside the timed region) ----
    parity = {}
    checked, bad = db.verify(args.verify_samples, seed=11)
    parity["recurrence_points_checked"], parity["recurrence_mismatches"] = checked, bad
    my_sum = db.checksum()
    parity["table_checksum"] = "%016x" % my_sum
    if world > 1:
        lo = torch.tensor([my_sum & 0x7FFFFFFF, my_sum >> 31 & 0x7FFFFFFF, my_sum >> 62], device="cuda", dtype=torch.int64)
        mn, mx = lo.clone(), lo.clone()
        dist.all_reduce(mn, op=dist.ReduceOp.MIN)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        parity["checksum_equal_on_all_ranks"] = bool(torch.equal(mn, mx))
        solo_sum = None
        if rank == 0 and SIZE >= 16:
            parity["equals_single_gpu"] = None   # records, table and working rows of this size do not fit one GPU
        elif rank == 0:   # the same workload filled by this GPU alone
            solo = m.SynthesisDatabase(device=local_rank)
            solo.precompute(SIZE, through=THROUGH, dtypes=DTYPES)
            solo_sum = solo.checksum()
            solo.close()
            parity["equals_single_gpu"] = solo_sum == my_sum
        dist.barrier()

    lspecs = st["n_goal_specs"]      # the Specs the workload asks for (the closure adds more rows, not more units)
    units = lspecs * LATTICE_POINTS  # one database, however many GPUs fill it
    hbm_gbs, peak_kind = measured_peaks()
    # the dominant kernel is the stage kernel: every launch of a fill is one, so its time is the fill's
    kernel_ms = ms_per_step
    achieved = alg_bytes / world / (kernel_ms * 1e-3) / 1e9   # per GPU: the bytes of the finished table, split over the ranks
    table_gb = st["n_rows"] * 16 / 1e9
    plan_gb = (st["n_candidates"] * 32 + st["n_specs"] * 48) / 1e9
    line = {
        "metric": "specs_resolved_per_s", "value": units / (ms_per_step * 1e-3), "unit": "specs/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "u32",
        "data": "synthetic",
        "config": {"workload": workload_name(), "logical_specs": lspecs, "lattice_points_per_spec": LATTICE_POINTS,
                   "logical_specs_with_closure": st["n_specs"], "candidate_records": st["n_candidates"],
                   "stages": st["n_stages"], "table_rows": st["n_rows"], "cells_solved_per_step": sum(cells_by_rank),
                   "cells_solved_by_rank": cells_by_rank,
                   "cells_imbalance_max_over_mean": max(cells_by_rank) / (sum(cells_by_rank) / len(cells_by_rank)),
                   "solve_passes_per_step": st["n_passes"],
                   "candidates_evaluated_per_step_rank0": st["n_candidates_evaluated"],
                   "rows_gathered_per_step_rank0": st["n_rows_gathered"], "grid_syncs_per_step_rank0": st["n_grid_syncs"],
                   "solve_phases_ms_rank0": st["combine_ms"], "unordered_phase_ms_rank0": st["early_ms"],
                   "relaxation_sweeps_per_step_rank0": st["n_sweeps"],
                   "cells_of_the_unordered_phase_rank0": st["n_cells_unordered"],
                   "candidates_evaluated_by_sweeps_rank0": st["n_candidates_swept"],
                   "kernel_parts_ms_rank0": dict(zip(["setup", "unordered_phase", "its_real_breakpoints", "pass_setup",
                                                      "cell_init", "first_sweeps", "later_sweeps", "pass_real_breakpoints"],
                                                     [round(x, 2) for x in st["phase_ms"]])),
                   "l2": ("candidate records and headers %.1f GB + table %.2f GB, larger than L2; L2 also flushed "
                          "between fills" % (plan_gb, table_gb)),
                   "multi_gpu": ("Specs of each stage sharded over %d ranks; masks and rows exchanged per stage over "
                                 "NCCL" % world) if world > 1 else "single"},
        "wall_s_full_db": e2e_step,
        "cells_solved_per_s": sum(cells_by_rank) / (ms_per_step * 1e-3),
        "e2e": {"value": units / e2e_step, "unit": "specs/s", "h2d_bytes_per_step": st2["h2d_bytes"],
                "d2h_bytes_per_step": st2["d2h_bytes"], "plan_s": st2["plan_seconds"],
                "plan_parts_s": {"goals": st2["plan_goal_seconds"], "closure_and_records": st2["plan_discover_seconds"],
                                 "ids_and_record_array": st2["plan_layout_seconds"],
                                 "of_which_record_array": st2["plan_layout_step_seconds"][3]},
                "upload_s": st2["upload_seconds"], "fill_ms": st2["fill_ms"], "buffer_growths": st2["n_buffer_growths"],
                "wall_s": e2e_step, "wall_s_runs": e2e_s},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                     "traffic": None, "peak_kind": peak_kind, "kernel": "stage_kernel",
                     "scope": "one GPU" if world == 1 else "per GPU (bytes of the whole job / %d ranks)" % world,
                     "algorithmic_bytes_per_step": alg_bytes,
                     "algorithmic_bytes_how": ("final table rows only: per row 12 B out, 16 B per candidate record of its "
                                               "Spec, 16 B per child of each candidate that fits the row's limits"),
                     "kernel_ms_per_step": kernel_ms, "kernel_launches_per_step": launches // args.steps,
                     "limiter": ("instruction issue (55-60 % of cycles in the stages that carry the time) and the latency of "
                                 "dependent loads at 32 resident warps per SM; DRAM at 0.13 of peak (profiles/)")},
        "parity": parity,
        "clocks": clocks,
    }
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            rep, o = run_oracle(cores, args.cpu_budget)
            line["cpu_baseline"] = cpu_baseline_object(rep, cores, args.cpu_budget)
            n_lookups, n_bad = compare_with_oracle_puts(db, o)
            o.close()
            parity["oracle_put_corners_checked"], parity["oracle_mismatches"] = n_lookups, n_bad
        traffic_path = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(traffic_path):
            with open(traffic_path) as f:
                t = json.load(f).get(str(SIZE) if THROUGH == 2 else "")
            if t and "dram_bytes_per_cell" in t:  # measured DRAM bytes per solved working cell on a small case, scaled to this step (see the file's "how")
                traffic = t["dram_bytes_per_cell"] * sum(cells_by_rank)
                line["roofline"]["traffic"] = traffic
                line["roofline"]["traffic_how"] = ("DRAM bytes of one single-GPU fill of this workload (one ncu pass per launch), "
                                                   "scaled by the working cells solved: profiles/traffic.json")
                line["roofline"]["dram_GBps"] = traffic / world / (kernel_ms * 1e-3) / 1e9   # per GPU
                line["roofline"]["dram_frac_of_peak"] = traffic / world / (kernel_ms * 1e-3) / 1e9 / hbm_gbs
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(line), flush=True)
        os.dup2(2, 1)
    db.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--size", type=int, default=8, choices=[1, 2, 4, 8, 16], help="largest Spec dimension of the workload")
    ap.add_argument("--dtypes", default="u32,f32", help="u32,f32 (the reference's DTYPES) or one of them")
    ap.add_argument("--through", default="matmul", choices=THROUGH_NAMES, help="last phase of the workload")
    ap.add_argument("--cpu-budget", type=float, default=21.0, help="seconds of CPU work per reference sample")
    ap.add_argument("--verify-samples", type=int, default=100_000_000,
                    help="(Spec, limits) points at which the timed table is checked against its recurrence")
    args = ap.parse_args()
    global SIZE, THROUGH, DTYPES
    SIZE = args.size
    THROUGH = THROUGH_NAMES.index(args.through)
    DTYPES = tuple({"u32": 4, "f32": 6}[d] for d in args.dtypes.split(","))
    if args.impl == "reference":
        reference_arm(args)
    else:
        cuda_arm(args)


if __name__ == "__main__":
    main()

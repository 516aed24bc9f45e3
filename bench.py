#!/usr/bin/env python
"""Benchmark of the synthesis-database fill.

  python bench.py --gpus N --steps K --warmup W            # the CUDA path
  python bench.py --impl reference --gpus N --steps K ...  # the reference algorithm on host cores

One step = one complete fill of the workload's database. The workload is BASELINE config 2:
the precompute of every canonical Move / Zero / Matmul Spec with dimensions in {1, 2, 4, 8} over
{u32, f32} on the Avx2 target with default memory limits (`precompute --target avx2 --through
matmul 8`): 10.6 M goal logical Specs, 14.7 M with their dependency closure, 400 M candidate
records. `--size 4` and `--size 2` run the smaller precomputes (size 2 is the closure of `morello
matmul 2`, BASELINE config 1). All inputs are synthetic by construction: the Spec space is
generated from the size alone.

Unit of work ("Spec resolved"): one (logical Spec, memory limits) entry of the database made
answerable. Both arms cover the same entries - every goal logical Spec of the workload over the
whole 17 x 17 x 12 x 27 limits lattice of the target - so the figure is the same numerator
divided by each arm's time. The CUDA arm also reports how many cells it solved directly and
the reference arm how many solves (`put`s) it needed. Beyond size 2 the CPU arm cannot finish in
bench time: it runs the reference's stage order under a time budget and counts the goal Specs
it completed (the cheap early stages - Moves, small shapes - come first, so this sample
flatters the CPU).
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
GOAL_SPECS = {1: 180, 2: 10454, 4: 410954, 8: 10613126}  # canonical goal Specs of the precompute of each size


def workload_name():
    return "precompute --target avx2 --through matmul %d (Move+Zero+Matmul, u32+f32, serial)" % SIZE


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


def run_oracle(threads, steps, warmup, budget_s=0.0):
    """The reference's algorithm (top-down memoised search with a range-filling memo table and
    the precompute driver) restated in C++ under oracle/, on the host cores."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_lib
    fac = oracle_lib.load()
    times, puts, lspecs = [], 0, 0
    for i in range(warmup + steps):
        o = fac.new()
        r = o.precompute(SIZE, through=2, dtype_mask=3, threads=threads, budget_s=budget_s)
        o.close()
        if i >= warmup:
            times.append(r["seconds"])
        puts, lspecs, finished = r["puts"], r["logical_specs"], r["finished"]
    return times, puts, lspecs, finished


def cpu_sample_text(finished, budget_s):
    if finished:
        return "the whole workload (C++ restatement of the reference algorithm, all host cores)"
    return ("the first %.0f s of the workload in the reference's stage order (Move phase first); goal Specs "
            "completed in that time; C++ restatement of the reference algorithm, all host cores" % budget_s)


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    budget = 0.0 if SIZE <= 2 else args.cpu_budget
    times, puts, lspecs, finished = run_oracle(cores, args.steps, 0 if budget else args.warmup, budget)
    per_step = sum(times) / len(times)
    value = lspecs * LATTICE_POINTS / per_step
    line = {
        "impl": "reference", "metric": "specs_resolved_per_s", "value": value, "unit": "specs/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
        "config": {"workload": workload_name(), "logical_specs": GOAL_SPECS[SIZE],
                   "lattice_points_per_spec": LATTICE_POINTS, "goal_specs_completed_in_sample": lspecs,
                   "reference_puts": puts},
        "wall_s_full_db": per_step if finished else None,
        "cpu_baseline": {"value": value, "unit": "specs/s", "cores": cores, "kind": "port",
                         "sample": cpu_sample_text(finished, budget) + " (the Rust reference cannot be built here)",
                         "puts_per_s": puts / per_step},
        "e2e": {"value": value, "unit": "specs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


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

    # N > 1: ONE database fill sharded over the ranks (the families of a stage are split between
    # the GPUs, masks and rows are summed over the ranks per stage), so total work is fixed:
    # strong scaling.
    from morello_b200 import sharded
    db = m.SynthesisDatabase(device=local_rank)

    def one_fill():
        if world > 1:
            sharded.fill_sharded(db, dist, torch)
        else:
            db.fill()

    if world > 1:
        sharded.precompute_sharded(db, SIZE, dist, torch)
    else:
        db.precompute(SIZE)  # plans, uploads, fills: leaves plan and tables on the device
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
            sharded.precompute_sharded(fresh, SIZE, dist, torch)
        else:
            fresh.precompute(SIZE)
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
    fill_ms, combine_ms, launches = [], [], 0
    for _ in range(args.steps):
        flush.fill_(1)
        torch.cuda.synchronize()
        one_fill()  # device time measured inside with CUDA events on the launching stream
        s1 = db.stats()
        fill_ms.append(s1["fill_ms"])
        combine_ms.append(s1["combine_ms"])
        launches += int(s1["n_launches"])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    st = db.stats()
    total_ms = sum(fill_ms)
    alg_bytes = float(st["algorithmic_bytes"])   # of this rank's solves
    if world > 1:
        t = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
        t = torch.tensor([float(launches)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        launches = int(t.item())
    ms_per_step = total_ms / args.steps
    combine_ms_per_step = sum(combine_ms) / args.steps

    lspecs = st["n_goal_specs"]      # the Specs the workload asks for (the closure adds more rows, not more units)
    units = lspecs * LATTICE_POINTS  # one database, however many GPUs fill it
    hbm_gbs, peak_kind = measured_peaks()
    # the dominant kernel: algorithmic bytes of its launches / CUDA-event time inside its launches
    achieved = alg_bytes / (combine_ms_per_step * 1e-3) / 1e9
    table_gb = st["n_rows"] * 16 / 1e9
    plan_gb = (st["n_candidates"] * 32 + st["n_specs"] * 48) / 1e9
    line = {
        "metric": "specs_resolved_per_s", "value": units / (ms_per_step * 1e-3), "unit": "specs/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None, "dtype": "u32",
        "data": "synthetic",
        "config": {"workload": workload_name(), "logical_specs": lspecs, "lattice_points_per_spec": LATTICE_POINTS,
                   "logical_specs_with_closure": st["n_specs"], "candidate_records": st["n_candidates"],
                   "stages": st["n_stages"], "table_rows": st["n_rows"], "cells_solved_per_step": st["n_cells_solved"],
                   "solve_passes_per_step": st["n_passes"],
                   "candidates_evaluated_per_step": st["n_candidates_evaluated"],
                   "rows_gathered_per_step": st["n_rows_gathered"], "grid_syncs_per_step": st["n_grid_syncs"],
                   "combine_phase_ms_per_step": st["combine_ms"],
                   "l2": ("candidate records and headers %.1f GB + table %.2f GB, larger than L2; L2 also flushed "
                          "between fills" % (plan_gb, table_gb)),
                   "multi_gpu": ("families of each stage sharded over %d ranks; masks and rows summed over the ranks "
                                 "per stage (NCCL all-reduce)" % world) if world > 1 else "single"},
        "wall_s_full_db": e2e_step,
        "cells_solved_per_s": st["n_cells_solved"] / (ms_per_step * 1e-3),
        "e2e": {"value": units / e2e_step, "unit": "specs/s", "h2d_bytes_per_step": st2["h2d_bytes"],
                "d2h_bytes_per_step": st2["d2h_bytes"], "plan_s": st2["plan_seconds"],
                "upload_s": st2["upload_seconds"], "fill_ms": st2["fill_ms"], "wall_s": e2e_step, "wall_s_runs": e2e_s},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_gbs, "unit": "GB/s", "frac": achieved / hbm_gbs,
                     "traffic": None, "peak_kind": peak_kind, "kernel": "combine_argmin_kernel",
                     "algorithmic_bytes_per_step": st["algorithmic_bytes"], "kernel_ms_per_step": combine_ms_per_step,
                     "kernel_launches_per_step": st["n_launches"],
                     "whole_fill_GBps": alg_bytes / (ms_per_step * 1e-3) / 1e9},
        "clocks": clocks,
    }
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            budget = 0.0 if SIZE <= 2 else args.cpu_budget
            times, puts, done, finished = run_oracle(cores, 1, 0, budget)
            line["cpu_baseline"] = {
                "value": done * LATTICE_POINTS / times[0], "unit": "specs/s", "cores": cores, "kind": "port",
                "sample": cpu_sample_text(finished, budget), "wall_s": times[0], "goal_specs_completed": done,
                "reference_puts": puts, "puts_per_s": puts / times[0]}
        traffic_path = os.path.join(ROOT, "profiles", "traffic.json")
        if os.path.exists(traffic_path):
            with open(traffic_path) as f:
                t = json.load(f).get(str(SIZE))
            if t:  # measured DRAM bytes per algorithmic byte on a small case, scaled to this step (see the file's "how")
                line["roofline"]["traffic"] = t["dram_over_algorithmic"] * st["algorithmic_bytes"]
                line["roofline"]["traffic_how"] = "scaled from a small-case ncu capture: profiles/traffic.json"
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
    ap.add_argument("--size", type=int, default=8, choices=[1, 2, 4, 8], help="largest Spec dimension of the workload")
    ap.add_argument("--cpu-budget", type=float, default=20.0, help="seconds of CPU work per reference sample")
    args = ap.parse_args()
    global SIZE
    SIZE = args.size
    if args.impl == "reference":
        reference_arm(args)
    else:
        cuda_arm(args)


if __name__ == "__main__":
    main()

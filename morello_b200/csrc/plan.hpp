// Host-side planner of the database fill.
//
// Turns a set of goal logical Specs into the flat arrays the combine kernel walks:
//   * the dependency closure of the goals (every sub-Spec any candidate action can ask for),
//   * per Spec its candidate records (action number, combine kind, immediates, child ids),
//   * per Spec the breakpoints of its memory-limits lattice (one bit mask per memory), which
//     give the Spec a dense 4-D grid of cells; one table row per cell,
//   * the schedule: groups of Specs ordered by (phase, log-shape sum) crossed with limits
//     diagonals, a total order in which every child row precedes its parent row.
//
// This replaces, for the path built here, the reference's on-demand recursion
// (morello/src/search/algo.rs:61-95) and its paged R-tree tables
// (morello/src/db/mod.rs:538-573,650-766): every (logical Spec, limits) point gets its own
// direct solve, so a point lookup is an index computation instead of a rectangle search.
#pragma once
#include "model/actions.hpp"
#include "model/space.hpp"
#include "device_types.h"
#include <string>
#include <vector>

namespace mrl {

struct PlanStats {
  u64 n_specs = 0;
  u64 n_goal_specs = 0;
  u64 n_cands = 0;
  u64 n_children = 0;
  u64 n_rows = 0;
  u64 n_columns = 0;
  u64 n_groups = 0;
  u64 n_steps = 0;
  u64 max_diag = 0;
  u64 algorithmic_bytes = 0;  // per full fill
  u64 mask_sweeps = 0;
  double seconds_discover = 0, seconds_masks = 0, seconds_layout = 0;
};

struct Group {          // Specs with the same phase and log-shape sum: no dependencies inside
  u32 spec_lo = 0, spec_hi = 0;  // id range
  u32 chunk_lo = 0, chunk_hi = 0;
  u32 max_diag = 0;     // largest limits diagonal any member has a cell on
  u8 free_dim = 3;      // memory whose slot the diagonal fixes; a thread owns a column of the other three
  u8 phase = 0;
  u8 shape_sum = 0;
};

// Specs of one group with the same dtype and shape. Moves never change either, so families of
// a group do not depend on each other: the unit of work handed to one GPU.
struct Family {
  u32 spec_lo = 0, spec_hi = 0;
  u32 group = 0;
  u32 owner = 0;        // rank that computes it
  u64 row_lo = 0, row_hi = 0;
};

struct Step {           // one kernel launch
  u32 group;
  u32 diag;             // sum of the four limit slots of the cells this launch evaluates
};

struct Plan {
  std::vector<LogicalSpec> specs;        // by id
  std::vector<SpecHdr> hdrs;             // by id
  std::vector<CandRec> cands;
  // warp_prefix[i] = number of warp-sized column chunks of the Specs with id < i that this rank
  // computes (n_specs + 1 entries). The chunk list itself is expanded on the device.
  std::vector<u32> warp_prefix;
  int n_threads = 1;
  // Lanes of a warp that share one cell (each takes every lanes_per_cell-th candidate); a warp
  // covers 32 / lanes_per_cell neighbouring columns. 1 or 2.
  int lanes_per_cell = 1;
  std::vector<Group> groups;
  std::vector<Family> families;
  std::vector<Step> steps;
  // Sharding: this process computes the families whose owner == rank; every rank keeps the
  // whole table. world == 1: everything is local.
  u32 rank = 0, world = 1;
  std::vector<u32> goal_ids;
  u32 top_code[NMEM] = {0, 0, 0, 0};   // lattice codes of the top limits the plan covers
  // Lattice compression. In a compressed memory k the table keeps the codes 0..cap_code[k] and
  // the top code only ("slots" 0..cap and cap+1); limits strictly between map to the cap slot.
  // That is exact as long as no optimal peak exceeds the cap (checked after every fill): a
  // result whose peak fits under the cap is already available at the cap, so nothing changes
  // between cap and top. cap_code[k] == top_code[k] means memory k is not compressed.
  u32 cap_code[NMEM] = {0, 0, 0, 0};
  bool compressed(int k) const { return cap_code[k] + 1 < top_code[k]; }
  u32 slot_of_code(int k, u32 code) const {
    if (!compressed(k)) return code;
    if (code == top_code[k]) return cap_code[k] + 1;
    return code < cap_code[k] ? code : cap_code[k];
  }
  // Smallest slot whose limit is >= the limit `code` (for feasibility thresholds).
  u32 slot_ceil(int k, u32 code) const {
    if (!compressed(k) || code <= cap_code[k]) return code;
    return cap_code[k] + 1;
  }
  u32 cap_pack() const {   // one byte per memory, 255 = not compressed
    u32 r = 0;
    for (int k = 0; k < NMEM; k++) r |= (compressed(k) ? cap_code[k] : 255u) << (8 * k);
    return r;
  }
  u32 top_pack() const {
    u32 r = 0;
    for (int k = 0; k < NMEM; k++) r |= top_code[k] << (8 * k);
    return r;
  }
  PlanStats stats;

  // id of a logical Spec (canonical form), or -1.
  long find(const LogicalSpec& ls) const;
  // Row index of (spec id, limits) or -1 when limits exceed the planned top.
  long row_of(u32 id, const u64 limits[NMEM]) const;

 private:
  friend Plan build_plan(const std::vector<LogicalSpec>&, int, const u64*, const int*, u32, u32);
  std::vector<std::pair<std::string, u32>> sorted_keys_;  // (key, id), sorted by key
};

// Top limits are Avx2Target::max_mem() unless overridden. caps: per memory the largest lattice
// code kept below the top (negative or >= top: no compression), see Plan::cap_code.
Plan build_plan(const std::vector<LogicalSpec>& goals, int n_threads, const u64* top_limits = nullptr,
                const int* caps = nullptr, u32 rank = 0, u32 world = 1);

// Recomputes everything that depends on the lattice caps (breakpoint masks, row offsets, chunk
// lists, schedule, byte accounting) and leaves Specs and candidate records alone.
void relayout_plan(Plan& plan, const int* caps);

// Goal sets.
std::vector<LogicalSpec> precompute_goals(u32 size, Through through, const std::vector<Dtype>& dtypes,
                                          int n_threads = 1);

// Lattice code <-> value helpers shared by planner and lookups.
inline u32 limit_code(int mem, u64 value) { return mem_counts_registers((Mem)mem) ? (u32)value : bit_length(value); }
inline u64 limit_value(int mem, u32 code) { return mem_counts_registers((Mem)mem) ? code : bit_length_inverse(code); }

}  // namespace mrl

// TEST INFRASTRUCTURE — NOT PART OF THE PRODUCT PATH.
//
// CPU oracle for the synthesis-database fill: a restatement, in plain C++17, of the
// reference's top-down memoised search, its Cost arithmetic, its range-filling memo
// table and its precompute driver. Only tests/, the smoke check and the CPU-baseline
// leg of the benchmark may build, link or call this; the CUDA path never does.
//
// What is shared with the product: the Spec/Layout/action-enumeration model under
// morello_b200/csrc/model/ (host code that defines WHICH candidates a Spec has). What is
// restated independently here: how candidate costs are combined (Cost, MemVec rules),
// feasibility under memory limits, the argmin, the search order, the memo semantics and
// the driver.
//
// Parity status: the reference is Rust and cannot be built where this was written, and
// it ships no fixture of filled-database contents. The pieces below are pinned by the
// reference's in-tree known-answer tests (see oracle/kat.cpp); whole-database contents
// are "parity unpinned" against the Rust binary itself.
//
// Reference anchors (paths inside the Morello repository):
//   morello/src/cost.rs:52-104                     Cost, ordering
//   morello/src/memorylimits.rs:159-224,303-470    peaks, MemVec snapping, limit subtraction
//   morello/src/imp/loops.rs:207-242               loop main cost
//   morello/src/scheduling/mod.rs:286-368          per-action cost combine
//   morello/src/scheduling/select.rs:34-47         kernel memory check
//   morello/src/search/{algo,spectask,reducer}.rs  search, task coroutine, argmin
//   morello/src/db/mod.rs:538-573,650-766,1782-1819; morello/src/db/pagecontents.rs:103-210
//                                                  get / put range fill / dominance
//   precompute/src/main.rs:275-441,738-759         stage driver, next_limits
#pragma once
#include "../morello_b200/csrc/model/actions.hpp"
#include "../morello_b200/csrc/model/space.hpp"
#include <array>
#include <atomic>
#include <mutex>
#include <optional>
#include <unordered_map>

namespace orc {
using namespace mrl;

using Limits = std::array<u64, NMEM>;  // decoded values: registers, or cache lines

struct Cost {
  u32 main = 0;
  Limits peaks = {0, 0, 0, 0};
  u8 depth = 0;
};

struct Decision {  // ActionCostVec with k = 1: empty (unsat) or one (action, cost)
  bool found = false;
  u16 action = 0;
  Cost cost;
};

// ---- MemVec rules on decoded values ----
// set_snap_up (memorylimits.rs:352-363)
inline u64 snap_up_value(u64 v) { return v < 128 ? v : (is_pow2(v) ? v : next_pow2(v)); }
// snap_up_for_target (memorylimits.rs:458-470)
inline Limits snap_up_for_target(Limits p) {
  for (int i = 0; i < NMEM; i++)
    if (!mem_counts_registers((Mem)i) && p[i] != 0) p[i] = next_pow2(p[i]);
  return p;
}
// MemVec::lex_cmp (memorylimits.rs:315-321)
inline int lex_cmp(const Limits& a, const Limits& b) {
  for (int i = 0; i < NMEM; i++) if (a[i] != b[i]) return a[i] < b[i] ? -1 : 1;
  return 0;
}
// Cost::cmp (cost.rs:87-104)
inline int cost_cmp(const Cost& a, const Cost& b) {
  if (a.main != b.main) return a.main < b.main ? -1 : 1;
  int p = lex_cmp(a.peaks, b.peaks);
  if (p) return p;
  if (a.depth != b.depth) return a.depth < b.depth ? -1 : 1;
  return 0;
}
// checked_sub_snap_down (memorylimits.rs:409-436). Returns false when out of memory.
inline bool checked_sub_snap_down(const Limits& cur, const Limits& rhs, Limits& out) {
  for (int i = 0; i < NMEM; i++) {
    if (cur[i] < rhs[i]) return false;
    u64 rem = cur[i] - rhs[i];
    out[i] = mem_counts_registers((Mem)i) ? rem : prev_power_of_two(rem);
  }
  return true;
}
// MemoryAllocation::Simple peak propagation (memorylimits.rs:159-187)
inline Limits peaks_simple(const Limits& own, const std::vector<Limits>& child_peaks) {
  Limits peak = {0, 0, 0, 0};
  if (child_peaks.empty()) {
    for (int i = 0; i < NMEM; i++) {
      u64 v = own[i];
      if (!mem_counts_registers((Mem)i)) v = next_binary_power(v);
      peak[i] = snap_up_value(v);
    }
    return peak;
  }
  for (const Limits& cp : child_peaks) {
    for (int i = 0; i < NMEM; i++) {
      u64 v = std::max(peak[i], own[i] + cp[i]);
      if (!mem_counts_registers((Mem)i)) v = next_binary_power(v);
      peak[i] = snap_up_value(v);
    }
  }
  return peak;
}
// MemoryAllocation::Pipeline peak propagation (memorylimits.rs:198-221)
inline Limits peaks_pipeline(const std::vector<Limits>& inter, const std::vector<Limits>& child_peaks) {
  Limits peak = {0, 0, 0, 0};
  const Limits z = {0, 0, 0, 0};
  for (size_t c = 0; c < child_peaks.size(); c++) {
    const Limits& before = c == 0 ? z : inter[c - 1];
    const Limits& after = c < inter.size() ? inter[c] : z;
    for (int i = 0; i < NMEM; i++) {
      u64 v = std::max(peak[i], before[i] + child_peaks[c][i] + after[i]);
      if (!mem_counts_registers((Mem)i)) v = next_binary_power(v);
      peak[i] = snap_up_value(v);
    }
  }
  return peak;
}

// compute_loop_main_cost (imp/loops.rs:207-242), Avx2 constants (:14-15).
inline u32 compute_loop_main_cost(const std::vector<std::pair<u32, u32>>& dims, bool parallel,
                                  const std::vector<u32>& body_costs) {
  u64 iterations = 1;
  for (auto& d : dims) {
    iterations *= d.second;
    if (iterations > 0xFFFFFFFFull) throw ModelError("number of full iterations overflows");
  }
  u32 it = (u32)iterations;
  if (parallel) it = (it + AVX2_PROCESSORS - 1) / AVX2_PROCESSORS;
  u32 total = sat_mul_u32(body_costs[0], it);
  for (size_t i = 1; i < body_costs.size(); i++) total = sat_add_u32(total, body_costs[i]);
  if (parallel) total = sat_add_u32(total, 230000u + 60u * it);
  return total;
}

// ActionSolver::compute_cost (scheduling/mod.rs:286-368) for one tabulated candidate.
inline Cost combine(const Candidate& c, const LogicalSpec& parent, const std::vector<Cost>& kids) {
  Cost out;
  switch (c.kind) {
    case CK_LEAF: {  // Cost::from_node_and_child_costs on a KernelApp (cost.rs:52-78)
      Limits own = {0, 0, 0, 0};
      own[c.level] = c.units;
      out.main = c.imm;
      out.peaks = snap_up_for_target(peaks_simple(own, {}));
      out.depth = 1;
      return out;
    }
    case CK_LOOP: {  // PrimitiveTileOut (mod.rs:291-343)
      const LogicalSpec& body = c.child[0];
      std::vector<std::pair<u32, u32>> dims;
      for (int d = 0; d < parent.spec_shape.n; d++) {
        u32 o = parent.spec_shape[d], t = body.spec_shape[d];
        dims.push_back({(o + t - 1) / t, o / t});
      }
      std::vector<u32> mains;
      u8 max_depth = 0;
      for (size_t i = 0; i < kids.size(); i++) {
        mains.push_back(kids[i].main);
        if (i > 0) max_depth = std::max(max_depth, kids[i].depth);  // first child's depth is skipped
      }
      out = kids[0];
      out.main = compute_loop_main_cost(dims, false, mains);
      out.depth = (u8)(max_depth + 1);
      return out;
    }
    case CK_MOVE: {  // Move (mod.rs:347-363)
      u32 main = c.imm;
      u8 depth = 0;
      std::vector<Limits> cps;
      for (const Cost& k : kids) {
        main = sat_add_u32(main, k.main);
        depth = std::max(depth, k.depth);
        cps.push_back(k.peaks);
      }
      Limits own = {0, 0, 0, 0};
      own[c.level] = c.units;
      out.main = main;
      out.depth = (u8)(depth + 1);
      out.peaks = snap_up_for_target(peaks_simple(own, cps));
      return out;
    }
    default: {  // Block via the fallback path (mod.rs:364-366,599-615; imp/blocks.rs:28-38)
      u32 main = kids[0].main;
      u8 depth = kids[0].depth;
      std::vector<Limits> cps = {kids[0].peaks};
      for (size_t i = 1; i < kids.size(); i++) {
        main = sat_add_u32(main, kids[i].main);
        depth = std::max(depth, kids[i].depth);
        cps.push_back(kids[i].peaks);
      }
      out.main = main;
      out.depth = depth == 255 ? 255 : (u8)(depth + 1);  // saturating_add(1)
      out.peaks = snap_up_for_target(peaks_simple({0, 0, 0, 0}, cps));
      return out;
    }
  }
}

// ImplReducer with k = 1 (search/reducer.rs:22-99): minimum of (Cost, ActionNum).
struct Reducer {
  bool has = false;
  Cost cost;
  u16 action = 0;
  void insert(u16 a, const Cost& c) {
    if (!has) { has = true; cost = c; action = a; return; }
    int cmp = cost_cmp(cost, c);
    if (cmp > 0 || (cmp == 0 && action > a)) { cost = c; action = a; }
  }
  Decision finalize() const {
    Decision d;
    d.found = has;
    if (has) { d.action = action; d.cost = cost; }
    return d;
  }
};

// ---- limits <-> database coordinates (MemoryLimitsBimap, memorylimits.rs:696-734) ----
using Codes = std::array<u8, NMEM>;
inline Codes limits_to_codes(const Limits& l) {
  Codes c;
  for (int i = 0; i < NMEM; i++) {
    if (mem_counts_registers((Mem)i)) c[i] = (u8)l[i];
    else {
      if (l[i] != 0 && !is_pow2(l[i])) throw ModelError("cache limit is not a power of two");
      c[i] = (u8)bit_length(l[i]);
    }
  }
  return c;
}
inline Limits codes_to_limits(const Codes& c) {
  Limits l;
  for (int i = 0; i < NMEM; i++) l[i] = mem_counts_registers((Mem)i) ? c[i] : bit_length_inverse(c[i]);
  return l;
}

// One `put`: the rectangle [peaks .. limits] of the limits lattice and its value.
struct PutRect {
  Codes lo, hi;
  Decision value;
};

// next_limits (precompute/src/main.rs:738-759)
inline std::vector<Limits> next_limits(const Limits& limits, const Limits& peaks) {
  std::vector<Limits> r;
  for (int i = 0; i < NMEM; i++) {
    u64 p = peaks[i];
    if (p == 0) continue;
    u64 lower;
    if (p == 1) lower = 0;
    else if (mem_counts_registers((Mem)i)) lower = p - 1;
    else lower = u64(1) << (bit_length(p) - 2);
    Limits n = limits;
    n[i] = lower;
    r.push_back(n);
  }
  return r;
}

// The memo table. Per logical Spec it keeps every put rectangle; a get returns the
// dominance-minimum over the rectangles covering the point, which is the pointwise state
// the reference's fill_region maintains (db/pagecontents.rs:125-210).
class Database {
 public:
  static constexpr int NSHARDS = 256;
  // Rectangles of one logical Spec, corners packed one byte per memory so that a
  // containment test is two word operations (codes are < 128, bit 7 is a borrow guard).
  struct Entry {
    std::vector<u32> lo, hi;
    std::vector<Decision> val;
  };
  struct Shard {
    std::mutex mu;
    std::unordered_map<std::string, Entry> map;
  };
  static u32 pack(const Codes& c) { return u32(c[0]) | (u32(c[1]) << 8) | (u32(c[2]) << 16) | (u32(c[3]) << 24); }
  Shard shards[NSHARDS];
  std::atomic<u64> puts{0}, gets{0}, hits{0}, dominance_conflicts{0};

  Shard& shard_for(const std::string& key) { return shards[std::hash<std::string>()(key) % NSHARDS]; }

  // -1 miss, else fills `out`.
  bool get(const std::string& key, const Codes& pt, Decision& out);
  void put(const std::string& key, const Limits& limits, const Decision& d);
};

struct SolveStats {
  u64 solves = 0;          // SpecTask::start calls (misses that were computed)
  u64 candidates_seen = 0; // applicable actions examined
};

class Search {
 public:
  // cache_candidates: keep each logical Spec's tabulated action list for later solves at
  // other limits. The reference re-enumerates actions on every solve
  // (search/spectask.rs:66); the cache only makes this baseline faster, never different.
  explicit Search(Database& db, bool cache_candidates = false) : db_(db), cache_(cache_candidates) {}
  Decision solve(const LogicalSpec& ls, const Limits& limits);  // algo::solve_node
  SolveStats stats;
  // A timed run gives up in the middle of a recursion: solve() throws OutOfTime once this
  // returns true. Nothing half-done reaches the database (puts happen when a solve completes).
  std::function<bool()> out_of_time;
  struct OutOfTime {};
 private:
  const std::vector<Candidate>& candidates_for(const LogicalSpec& ls, const std::string& key,
                                               std::vector<Candidate>& scratch);
  Database& db_;
  bool cache_;
  std::unordered_map<std::string, std::vector<Candidate>> cand_cache_;
};

// The precompute driver (precompute/src/main.rs:172-386).
struct PrecomputeReport {
  double seconds = 0;        // wall
  double busy_seconds = 0;   // summed over the workers: time spent inside tasks
  u64 puts = 0;
  u64 logical_specs = 0;     // goal Specs whose whole limits staircase was completed
  u64 solves = 0;
};
struct PhaseReport {
  double seconds = 0;
  u64 logical_specs = 0, puts = 0;
  bool finished = false;
};
// time_budget_s > 0: stop when the whole run has taken that long. phase_budget_s (one entry per
// phase): stop a phase when it has, and go on with the next one.
PrecomputeReport precompute(Database& db, u32 size, Through through, const std::vector<Dtype>& dtypes, int threads,
                            double time_budget_s /* <=0: none */, bool* finished, bool cache_candidates = false,
                            const double* phase_budget_s = nullptr, PhaseReport* phase_reports = nullptr);

}  // namespace orc

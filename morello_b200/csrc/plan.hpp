// Host-side planner of the database fill.
//
// Turns a set of goal logical Specs into the flat arrays the device side walks:
//   * the dependency closure of the goals (every sub-Spec any candidate action can ask for),
//   * per Spec its candidate records (action number, combine kind, immediates, child ids),
//   * the order: Specs sorted into stages by (phase, log-shape sum, memory-level sum). Every
//     child of a Spec lies in an earlier stage, except the children of same-memory relayout
//     Moves, which stay in the stage but sit at strictly lower memory limits.
// The limits grids (which lattice codes each Spec's table distinguishes) are not planned here:
// the device derives them stage by stage from the finished tables of the children.
//
// This replaces, for the path built here, the reference's on-demand recursion
// (morello/src/search/algo.rs:61-95) and its paged R-tree tables
// (morello/src/db/mod.rs:538-573,650-766): every cell of a Spec's limits grid gets its own
// direct solve, so a point lookup is an index computation instead of a rectangle search.
#pragma once
#include "model/actions.hpp"
#include "model/space.hpp"
#include "device_types.h"
#include <cstdlib>
#include <new>
#include <string>
#include <memory>
#include <vector>

namespace mrl {

// Uninitialised storage for plain records. Nothing is written at allocation, so the pages of a
// large array are first touched by the threads that fill it, in parallel.
template <class T>
class RawVec {
 public:
  RawVec() {}
  ~RawVec() { free(p_); }
  RawVec(const RawVec&) = delete;
  RawVec& operator=(const RawVec&) = delete;
  RawVec(RawVec&& o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr; o.n_ = 0; }
  RawVec& operator=(RawVec&& o) noexcept {
    if (this != &o) { free(p_); p_ = o.p_; n_ = o.n_; o.p_ = nullptr; o.n_ = 0; }
    return *this;
  }
  void reset(size_t n) {
    free(p_);
    p_ = nullptr;
    n_ = 0;
    if (n) {
      const size_t bytes = n * sizeof(T);
      if (bytes >= (size_t(64) << 20)) {
        // large arrays are 2 MiB-aligned (huge-page advice was measured: no gain on a GPU host,
        // eight times slower page faults where the kernel has to compact memory to grant them)
        void* q = nullptr;
        if (posix_memalign(&q, size_t(2) << 20, bytes) != 0) throw std::bad_alloc();
        p_ = static_cast<T*>(q);
      } else {
        p_ = static_cast<T*>(malloc(bytes));
      }
      if (!p_) throw std::bad_alloc();
      n_ = n;
    }
  }
  size_t size() const { return n_; }
  bool empty() const { return n_ == 0; }
  T* data() { return p_; }
  const T* data() const { return p_; }
  T& operator[](size_t i) { return p_[i]; }
  const T& operator[](size_t i) const { return p_[i]; }

 private:
  T* p_ = nullptr;
  size_t n_ = 0;
};

struct PlanStats {
  u64 n_specs = 0;
  u64 n_goal_specs = 0;
  u64 n_cands = 0;
  u64 n_children = 0;
  u64 n_stages = 0;
  u64 n_families = 0;
  double seconds_discover = 0, seconds_layout = 0;
  double seconds_layout_step[8] = {};   // key sort, final ids, twin leaves and offsets, record array, id table, stages and families, checks, release of temporaries
};

// Specs with the same phase (kind), log-shape sum and memory-level rank (sum over operands of
// the memory index RF 0, VRF 1, L1 2, GL 3; for Move Specs the largest index instead). Tile-outs
// and splits shrink the shape, ToAccum and the Move prologues/epilogues of Matmul and Fill Specs
// go to an earlier phase, Moves to a faster memory lower the level sum: only relayout Moves
// (same memory, other layout) - and, in the Move phase, Moves that keep the slowest memory -
// keep a child inside the stage.
struct Stage {
  u32 spec_lo = 0, spec_hi = 0;  // id range
  u32 fam_lo = 0, fam_hi = 0;    // family range
  u8 phase = 0;
  u8 shape_sum = 0;
  u8 level_rank = 0;
};

// Specs of one stage with the same dtype and shape. Moves never change either, so families of
// a stage do not depend on each other. Outside the Move phase a family splits further into
// independent units by the operands' memories (Plan::owner is per Spec).
struct Family {
  u32 spec_lo = 0, spec_hi = 0;
  u32 stage = 0;
  u32 owner = 0;        // rank that computes its first Spec (informational)
  u64 weight = 0;       // candidate records (the load-balancing estimate)
};

struct Plan {
  RawVec<LogicalSpec> specs;             // by id
  RawVec<SpecHdr> hdrs;                  // by id; masks and row_base are filled in on the device
  RawVec<CandRec> cands;
  int n_threads = 1;
  std::vector<Stage> stages;
  std::vector<Family> families;
  // Sharding: this process computes the families whose owner == rank; every rank keeps the
  // whole table. world == 1: everything is local.
  u32 rank = 0, world = 1;
  std::vector<u8> owner;                 // by id: rank that computes the Spec (empty when world == 1)
  std::vector<u8> mine;                  // by id: 1 = computed by this rank (empty when world == 1)
  std::vector<u32> goal_ids;
  u32 top_code[NMEM] = {0, 0, 0, 0};   // lattice codes of the top limits the plan covers
  u32 top_pack() const {
    u32 r = 0;
    for (int k = 0; k < NMEM; k++) r |= top_code[k] << (8 * k);
    return r;
  }
  PlanStats stats;

  // A plan as eight flat byte ranges (0 meta, 1 specs, 2 hdrs, 3 cands, 4 stages, 5 families,
  // 6 goal ids, 7 id lookup table), so that one process can plan and hand the result to others
  // (ranks of a multi-GPU fill on one node share the host cores; only one of them should plan).
  static constexpr int N_BLOBS = 8;
  void share_blobs(void* ptrs[N_BLOBS], u64 sizes[N_BLOBS]);
  // Receiving side: allocate by size, let the caller fill the ranges (share_blobs gives the
  // pointers), then adopt_done() for this rank of `world`.
  void adopt_alloc(const u64 sizes[N_BLOBS]);
  // have_cands: the candidate records were received too (they are checked as well).
  void adopt_done(u32 rank, u32 world, int n_threads, bool have_cands);
  // 64-bit fingerprint of the job: every Spec key in id order, the candidate count, the top
  // limits. Two plans with one fingerprint address one table layout.
  u64 fingerprint(int n_threads) const;

  // id of a logical Spec (canonical form), or -1.
  long find(const LogicalSpec& ls) const;
  // Limits as packed lattice codes (RF in byte 0 .. GL in byte 3); false when the limits are
  // not lattice points or exceed the planned top.
  bool pack_limits(const u64 limits[NMEM], u32* out) const;

 private:
  friend Plan build_plan(const std::vector<LogicalSpec>&, int, const u64*, u32, u32, int, u32);
  friend Plan table_only_plan(RawVec<LogicalSpec>&&, RawVec<SpecHdr>&&, const u32*, int);
  std::shared_ptr<void> cleanup_;  // background release of planning temporaries; joined when dropped
  std::vector<u32> find_tab_;  // open-addressing table of ids by Spec key hash (0xFFFFFFFF = empty)
  struct Meta {                // blob 0
    u32 top_code[NMEM];
    u32 world, pad;
    PlanStats stats;
  } meta_;
  void assign_owners_();
};

// Cross-check modes of the planner: slower, same plan (tests compare).
enum : u32 {
  PLAN_NO_TWINS = 1,   // tabulate both dtypes of a mirrored goal set instead of deriving one from the other
  PLAN_NO_MEMO = 2,    // tabulate every Spec from scratch instead of re-using per-operand results
};

// Top limits are Avx2Target::max_mem() unless overridden. mirror_dtype >= 0: the goals come in
// one dtype and the plan also covers their images in that second dtype of the same byte size
// (what build_plan otherwise detects by itself when handed both goal sets).
Plan build_plan(const std::vector<LogicalSpec>& goals, int n_threads, const u64* top_limits = nullptr,
                u32 rank = 0, u32 world = 1, int mirror_dtype = -1, u32 flags = 0);

// A plan that can only answer lookups: Specs and their table headers as a saved database holds
// them; no candidate records, no stages.
Plan table_only_plan(RawVec<LogicalSpec>&& specs, RawVec<SpecHdr>&& hdrs, const u32* top_code, int n_threads);

// Goal sets.
std::vector<LogicalSpec> precompute_goals(u32 size, Through through, const std::vector<Dtype>& dtypes,
                                          int n_threads = 1);

// Lattice code <-> value helpers shared by planner and lookups.
inline u32 limit_code(int mem, u64 value) { return mem_counts_registers((Mem)mem) ? (u32)value : bit_length(value); }
inline u64 limit_value(int mem, u32 code) { return mem_counts_registers((Mem)mem) ? code : bit_length_inverse(code); }

}  // namespace mrl

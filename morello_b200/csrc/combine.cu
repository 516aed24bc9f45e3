// The CUDA side of the synthesis-database fill (sm_100a).
//
// Specs are processed stage by stage (plan.hpp). One cooperative launch solves a whole stage
// on the device, with grid-wide barriers between its phases and nothing for the host to decide.
// A limits grid of a Spec = per memory the lattice codes at which its result can change; a cell
// = one combination of slots; evaluating a candidate record at a cell = feasibility under the
// cell's limits, gather of the child rows at the children's limits, combine into a Cost,
// lexicographic minimum.
//   0. corners: below its corner a Spec has no implementation at all; every grid of the stage is
//      clipped there (phase_minsat, phase_corner);
//   1. once per stage, the records whose children all lie in earlier stages are solved on a grid
//      of their own - their thresholds plus the (shifted) breakpoints of those children's
//      finished tables - in no particular order: a warp takes a piece of one Spec's grid, stages
//      the Spec's records and the headers of their children in shared memory, and its lanes take
//      32 cells at a time and walk the staged records together (phase_derive_early,
//      phase_place, phase_early); the real breakpoints of the result are found at once
//      (phase_real_masks);
//   2. the rest - relayout Moves, whose body is a Spec of the same stage at strictly lower limits
//      - is solved on working grids: the real breakpoints of step 1's result, the thresholds of
//      those records and the shifted breakpoints of their children (phase_derive_late). Every
//      working cell starts from step 1's result at its limits (phase_late_init) and is recomputed
//      in place, sweep after sweep, from that and its records at the children's current values,
//      until a sweep changes nothing (phase_late): the dependencies between cells form no cycle,
//      so that fixpoint is the direct solve;
//   3. breakpoints at which some pair of neighbouring cells differs are real
//      (phase_real_masks); 2-3 repeat for the Specs whose working grid still lacks a breakpoint
//      that a same-stage child turned out to have, and for the Specs above them (phase_spread);
//   4. the working grids are compacted to the real breakpoints and appended to the table
//      (phase_final_count, phase_scan_sums, phase_compact).
// Step 3's fixpoint is exact: when every Spec's grid contains all thresholds and all shifted
// breakpoints of the computed tables of its children, induction over the limits lattice shows
// every computed cell equals the direct solve at every limit inside it.
//
// What the combine replaces in the reference (paths inside the Morello repository):
//   morello/src/scheduling/mod.rs:286-368     ActionSolver::compute_cost
//   morello/src/imp/loops.rs:207-242          loop main cost (serial, no boundary regions)
//   morello/src/memorylimits.rs:159-224,409-470  peak propagation, limit subtraction
//   morello/src/scheduling/select.rs:34-47    kernel-allocation feasibility
//   morello/src/search/reducer.rs:40-99       argmin on (Cost, ActionNum)
//   morello/src/db/pagecontents.rs:103-123    child lookup (here: an index computation)
//   precompute/src/main.rs:304-385            the stage loop (here: on the device)
// Integer-only work; no tensor cores.
#include "device_types.h"
#include "fill.hpp"
#include "../../include/morello_b200.h"
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include <chrono>
#include <mutex>
#include <thread>

namespace cg = cooperative_groups;

static_assert(MRL_STATIC_SCRATCH_BYTES == MRL_NOALLOC_MAX_BYTES,
              "the fixed device array and the limit the header promises are one number");

namespace {

constexpr int kBlock = 128;      // threads per block of every kernel here
constexpr int kMinBlocks = 8;   // resident blocks per SM the stage kernel is compiled for
constexpr int kMaxPasses = 128;
constexpr int kMaxSweeps = 256;   // per pass; a dependency chain is shorter than the 70 diagonals of the limits lattice

__device__ __forceinline__ uint32_t sat_add(uint32_t a, uint32_t b) {
  uint32_t s = a + b;
  return s < a ? 0xFFFFFFFFu : s;
}
__device__ __forceinline__ uint32_t sat_mul(uint32_t a, uint32_t b) {
  unsigned long long p = (unsigned long long)a * b;
  return p > 0xFFFFFFFFull ? 0xFFFFFFFFu : (uint32_t)p;
}
// cpack: limit codes packed one per byte, RF in byte 0 .. GL in byte 3.
__device__ __forceinline__ uint32_t code_of(uint32_t cpack, uint32_t level) { return (cpack >> (8 * level)) & 0xFFu; }
// peaks word: RF in byte 3 .. GL in byte 0 (so that a plain u32 compare is lexicographic).
__device__ __forceinline__ uint32_t peak_shift(uint32_t level) { return 8 * (3 - level); }

// Code of the power-of-two-rounded line count x (0 -> 0, 1 -> 1, 2 -> 2, 3..4 -> 3, ...).
__device__ __forceinline__ uint32_t cache_code_ceil(uint32_t x) {
  if (x == 0) return 0;
  if (x == 1) return 1;
  return (32 - __clz(x - 1)) + 1;
}
__device__ __forceinline__ uint32_t cache_value(uint32_t code) { return code ? (1u << (code - 1)) : 0u; }

// The limit code a Move's children see in the memory it allocates in, given the parent's code
// there (at or above the Move's threshold): registers subtract, caches subtract and snap down
// to a power of two (morello/src/memorylimits.rs:409-436).
__device__ __forceinline__ uint32_t child_code(uint32_t level, uint32_t lv, uint32_t units) {
  return level < 2 ? lv - units : 32 - __clz(cache_value(lv) - units);
}

// Position of the n-th (0-based) set bit of m; m has more than n bits set.
__device__ __forceinline__ uint32_t nth_set_bit(uint32_t m, uint32_t n) {
  uint32_t pos = 0;
#pragma unroll
  for (int w = 16; w > 0; w >>= 1) {
    const uint32_t low = __popc(m & ((1u << w) - 1u));
    const bool up = n >= low;
    n -= up ? low : 0u;
    m = up ? (m >> w) : m;
    pos += up ? (uint32_t)w : 0u;
  }
  return pos;
}

__device__ __forceinline__ uint32_t sel4(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t k) {
  return k == 0 ? a0 : (k == 1 ? a1 : (k == 2 ? a2 : a3));
}
__device__ __forceinline__ uint32_t below(uint32_t code) { return (2u << code) - 1u; }   // codes <= code

// The running optimum of a cell: the row's three key words and the index of the winning
// candidate record within its Spec.
struct Best {
  uint32_t main, peaks, tail, ci;
};
__device__ __forceinline__ bool key_less(uint32_t m, uint32_t p, uint32_t t, const Best& b) {
  if (m != b.main) return m < b.main;
  if (p != b.peaks) return p < b.peaks;
  return t < b.tail;
}

struct Tally {   // what a thread's solves touched
  uint32_t cands, lookups;
};

// Row `base` of the table: bit 63 set = a working row of the stage being solved.
#define MRL_TEMP_FLAG (1ull << 63)
__device__ __forceinline__ const MrlRow* row_at(const MrlRow* rows, const MrlRow* temp, unsigned long long base) {
  return ((base & MRL_TEMP_FLAG) ? temp : rows) + (base & ~MRL_TEMP_FLAG);
}

// Row of a child Spec at given limits: the cell whose breakpoints are the largest ones not
// above the limits. b_k = mask of the codes <= the limit's code in memory k. One 32-byte
// header and one 16-byte row. Plain loads: headers and working rows of the stage being solved
// are written by earlier phases of the same launch.
__device__ __forceinline__ const MrlRow* row_of(const MrlRow* rows, const MrlRow* temp, const uint4 m,
                                                unsigned long long base, uint32_t b0, uint32_t b1, uint32_t b2,
                                                uint32_t b3) {
  const uint32_t i0 = __popc(m.x & b0) - 1;
  const uint32_t i1 = __popc(m.y & b1) - 1;
  const uint32_t i2 = __popc(m.z & b2) - 1;
  const uint32_t i3 = __popc(m.w & b3) - 1;
  const uint32_t off = ((i3 * __popc(m.z) + i2) * __popc(m.y) + i1) * __popc(m.x) + i0;  // cells per Spec < 2^32
  return row_at(rows, temp, base) + off;
}
__device__ __forceinline__ uint4 lookup(const SpecHdr* hdrs, const MrlRow* rows, const MrlRow* temp, uint32_t child,
                                        uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
  const uint4 m = *reinterpret_cast<const uint4*>(&hdrs[child]);
  const unsigned long long base = hdrs[child].row_base;
  return *reinterpret_cast<const uint4*>(row_of(rows, temp, m, base, b0, b1, b2, b3));
}

// One candidate record of a Spec at one limits point: feasibility under the limits, the child
// rows at the children's limits, the combined Cost, and the running minimum. The fill is bound by
// the latency of dependent loads (record -> child header -> child row), so the headers of all
// children are requested together, then all rows: two round trips per candidate whatever the
// number of children.
// kFinished: every child lies in a finished stage, so headers and rows are read-only for the whole
// launch and may take the non-coherent load path.
template <bool kFinished>
__device__ __forceinline__ void eval_candidate(const SpecHdr* hdrs, const CandRec* __restrict__ cands, const MrlRow* rows,
                                               const MrlRow* temp, uint32_t rec, const uint4 a, uint32_t ci, uint32_t cpack,
                                               uint32_t bm0, uint32_t bm1, uint32_t bm2, uint32_t bm3, Best& best,
                                               Tally& tally) {
  const uint32_t action = a.x & 0xFFFFu, kind = (a.x >> 16) & 0xFFu, nchild = a.x >> 24;
  const uint32_t imm = a.y;
  const uint32_t level = a.z & 0xFFu, thr = (a.z >> 8) & 0xFFu, pcode = (a.z >> 16) & 0xFFu;
  const uint32_t units = a.w;
  const uint32_t lv = code_of(cpack, level);  // the cell's limit in `level`
  tally.cands++;
  uint32_t k_main, k_peaks, k_tail;
  if (kind == MRL_CK_LEAF) {
    if (lv < thr) return;
    k_main = imm;
    k_peaks = pcode << peak_shift(level);
    k_tail = (1u << 16) | action;
  } else {
    uint32_t c0 = bm0, c1 = bm1, c2 = bm2, c3 = bm3;
    const uint32_t sh = peak_shift(level);
    if (kind == MRL_CK_MOVE) {
      if (lv < thr) return;
      // Branch and bound: a Move costs at least its own base cost.
      if (imm > best.main) return;
      const uint32_t cb = below(child_code(level, lv, units));
      c0 = (level == 0) ? cb : c0;
      c1 = (level == 1) ? cb : c1;
      c2 = (level == 2) ? cb : c2;
      c3 = (level == 3) ? cb : c3;
    }
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(&cands[rec]) + 1);
    const uint32_t ch1 = nchild > 1 ? b.y : b.x, ch2 = nchild > 2 ? b.z : b.x;   // absent children repeat the first
    uint4 m0, m1, m2, r0, r1, r2;
    unsigned long long base0, base1, base2;
    if (kFinished) {
      m0 = __ldg(reinterpret_cast<const uint4*>(&hdrs[b.x]));
      m1 = __ldg(reinterpret_cast<const uint4*>(&hdrs[ch1]));
      m2 = __ldg(reinterpret_cast<const uint4*>(&hdrs[ch2]));
      base0 = __ldg(&hdrs[b.x].row_base); base1 = __ldg(&hdrs[ch1].row_base); base2 = __ldg(&hdrs[ch2].row_base);
      r0 = __ldg(reinterpret_cast<const uint4*>(row_of(rows, temp, m0, base0, c0, c1, c2, c3)));
      r1 = __ldg(reinterpret_cast<const uint4*>(row_of(rows, temp, m1, base1, c0, c1, c2, c3)));
      r2 = __ldg(reinterpret_cast<const uint4*>(row_of(rows, temp, m2, base2, c0, c1, c2, c3)));
    } else {
      m0 = *reinterpret_cast<const uint4*>(&hdrs[b.x]);
      m1 = *reinterpret_cast<const uint4*>(&hdrs[ch1]);
      m2 = *reinterpret_cast<const uint4*>(&hdrs[ch2]);
      base0 = hdrs[b.x].row_base; base1 = hdrs[ch1].row_base; base2 = hdrs[ch2].row_base;
      r0 = *reinterpret_cast<const uint4*>(row_of(rows, temp, m0, base0, c0, c1, c2, c3));
      r1 = *reinterpret_cast<const uint4*>(row_of(rows, temp, m1, base1, c0, c1, c2, c3));
      r2 = *reinterpret_cast<const uint4*>(row_of(rows, temp, m2, base2, c0, c1, c2, c3));
    }
    tally.lookups += nchild;
    if (r0.z == MRL_UNSAT || r1.z == MRL_UNSAT || r2.z == MRL_UNSAT) return;
    uint32_t depth;
    if (kind == MRL_CK_LOOP) {
      k_main = sat_mul(r0.x, imm);
      k_peaks = r0.y;
      depth = 1u;  // a single-body tile loop has depth 1 whatever its body's depth
    } else {
      k_main = (kind == MRL_CK_MOVE) ? sat_add(imm, r0.x) : r0.x;
      if (nchild > 1) k_main = sat_add(k_main, r1.x);
      if (nchild > 2) k_main = sat_add(k_main, r2.x);
      if (k_main > best.main) return;
      k_peaks = __vmaxu4(__vmaxu4(r0.y, r1.y), r2.y);
      if (kind == MRL_CK_MOVE) {
        // own allocation sits on top of the deepest child's peak in `level`; rounding to the
        // lattice is monotone, so max-then-round equals the reference's round-per-child
        const uint32_t cc = (k_peaks >> sh) & 0xFFu;
        const uint32_t ncode = level < 2 ? units + cc : cache_code_ceil(units + cache_value(cc));
        k_peaks = (k_peaks & ~(0xFFu << sh)) | (ncode << sh);
      }
      depth = min(max(max(r0.z >> 16, r1.z >> 16), r2.z >> 16) + 1u, 255u);
    }
    k_tail = (depth << 16) | action;
  }
  if (key_less(k_main, k_peaks, k_tail, best)) {
    best.main = k_main;
    best.peaks = k_peaks;
    best.tail = k_tail;
    best.ci = ci;
  }
}

// The direct solve of one (Spec, limits) point from the tables of the Spec's children: every
// candidate record of the Spec. cpack = the limits as lattice codes.
__device__ __forceinline__ Best solve_point(const SpecHdr* hdrs, const CandRec* __restrict__ cands, const MrlRow* rows,
                                            const MrlRow* temp, uint32_t spec, uint32_t cpack, Tally& tally) {
  const uint32_t bm0 = below(code_of(cpack, 0)), bm1 = below(code_of(cpack, 1)), bm2 = below(code_of(cpack, 2)),
                 bm3 = below(code_of(cpack, 3));
  const uint2 cl = *reinterpret_cast<const uint2*>(&hdrs[spec].cand_off);
  Best best = {MRL_UNSAT, MRL_UNSAT, MRL_UNSAT, MRL_UNSAT};
  for (uint32_t ci = 0; ci < cl.y; ci++) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(&cands[cl.x + ci]));
    eval_candidate<false>(hdrs, cands, rows, temp, cl.x + ci, a, ci, cpack, bm0, bm1, bm2, bm3, best, tally);
  }
  return best;
}

// ---- working grids ---------------------------------------------------------------------

struct Grid {   // what a Spec's masks imply
  uint32_t nn[4];
  unsigned long long cells;
  uint32_t F, cols, warps;
};
__device__ __forceinline__ Grid grid_of(const uint4 m) {
  Grid g;
  g.nn[0] = __popc(m.x); g.nn[1] = __popc(m.y); g.nn[2] = __popc(m.z); g.nn[3] = __popc(m.w);
  g.cells = (unsigned long long)g.nn[0] * g.nn[1] * g.nn[2] * g.nn[3];
  // The free memory is the one with the most slots (lowest index on ties): the longest columns,
  // so the fewest chunks.
  g.F = 0;
  uint32_t best = g.nn[0];
#pragma unroll
  for (int k = 1; k < 4; k++)
    if (g.nn[k] > best) { best = g.nn[k]; g.F = k; }
  g.cols = (uint32_t)(g.cells / best);
  g.warps = (g.cols + 31u) / 32u;
  return g;
}

// Geometry of one thread's column. A column fixes the slot index in the three memories other
// than the Spec's free memory F.
struct Column {
  uint32_t spec, F;
  uint32_t mm[4], nn[4], idx[4];
  bool valid;
};
__device__ __forceinline__ Column decode_column(const SpecHdr* hdrs, const Chunk ch, uint32_t lane) {
  Column c;
  c.spec = ch.spec;
  c.F = ch.col_start >> 30;
  const uint4 m = *reinterpret_cast<const uint4*>(&hdrs[ch.spec]);
  c.mm[0] = m.x; c.mm[1] = m.y; c.mm[2] = m.z; c.mm[3] = m.w;
  uint32_t rest = (ch.col_start & 0x3FFFFFFFu) + lane;
#pragma unroll
  for (int k = 0; k < 4; k++) {
    c.nn[k] = (uint32_t)__popc(c.mm[k]);
    const uint32_t nk = ((uint32_t)k == c.F) ? 1u : c.nn[k];
    c.idx[k] = rest % nk;   // for F: slot 0
    rest /= nk;
  }
  c.valid = rest == 0;  // false: column index beyond this Spec's grid
  return c;
}

__device__ __forceinline__ void or_level(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t level,
                                         uint32_t bits) {
  r0 |= (level == 0) ? bits : 0u;
  r1 |= (level == 1) ? bits : 0u;
  r2 |= (level == 2) ? bits : 0u;
  r3 |= (level == 3) ? bits : 0u;
}

// Where a child's breakpoints in the destination memory of a Move show up in the parent: the
// child sees limit - units (registers) or that snapped down to a power of two (caches), so a
// child breakpoint at code b becomes the smallest parent code whose child code reaches b.
__device__ __forceinline__ uint32_t shift_mask(uint32_t cm, uint32_t level, uint32_t units, uint32_t top) {
  const uint32_t keep = (2u << top) - 1u;   // top <= 30
  if (level < 2) return units >= 32 ? 0u : (uint32_t)(((unsigned long long)cm << units) & keep);
  uint32_t out = 0;
  while (cm) {
    const uint32_t b = __ffs(cm) - 1;
    cm &= cm - 1;
    const unsigned long long v = (unsigned long long)cache_value(b) + units;
    if (v > 0x40000000ull) continue;
    const uint32_t code = cache_code_ceil((uint32_t)v);
    if (code <= top) out |= 1u << code;
  }
  return out;
}

// Exclusive prefix of v over the block (kBlock threads); *total = the block's sum.
__device__ __forceinline__ unsigned long long block_excl_scan(unsigned long long v, unsigned long long* total) {
  __shared__ unsigned long long warp_sum[kBlock / 32];
  __shared__ unsigned long long block_total;
  const uint32_t lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  unsigned long long inc = v;
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xFFFFFFFFu, inc, o);
    if (lane >= (uint32_t)o) inc += t;
  }
  __syncthreads();   // protects the shared arrays across consecutive calls
  if (lane == 31) warp_sum[w] = inc;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long run = 0;
    for (int k = 0; k < kBlock / 32; k++) { const unsigned long long t = warp_sum[k]; warp_sum[k] = run; run += t; }
    block_total = run;
  }
  __syncthreads();
  *total = block_total;
  return warp_sum[w] + inc - v;
}

// Everything a stage kernel needs; passed by value.
struct StageArgs {
  SpecHdr* hdrs;
  const CandRec* cands;
  uint4* rmask;
  const uint8_t* mine;    // null: every Spec is computed here
  uint8_t* dirty;         // by Spec id: 0 keep, 1 solve in the coming pass, 2 being solved in this pass
  Chunk* chunks;
  WorkItem* items;
  MrlRow* rows;
  MrlRow* temp;
  MrlRow* base;                   // as many rows again: the grids of the unordered phase
  SpecHdr* ehdr;                  // by position in the stage: masks and first row (in base) of the Spec's grid of the unordered phase
  uint32_t* fcount;
  unsigned long long* block_sums;
  uint32_t* minsat;               // by Spec id: lower corner of the satisfiable region (see phase_minsat)
  uint32_t* corner;               // by position in the stage: the corner its working grids are clipped at
  uint32_t* stamp;                // by position in the stage: last relaxation sweep that improved a cell of the Spec
  FillCtl* ctl;
  uint32_t lo, hi;                // the stage's Spec ids
  uint32_t prev_lo, prev_hi;      // the stage before it
  uint32_t top_pack;
  uint32_t stage;
  unsigned long long temp_cap, chunk_cap, item_cap, row_cap;
  int solve, place;               // which halves to run
};

__device__ __forceinline__ bool computed_here(const StageArgs& a, uint32_t i) { return !a.mine || a.mine[i]; }

// Lower corner of a Spec's satisfiable region: per memory the smallest limit code at which any
// implementation exists at all, 5 bits each (RF in the low bits); 31 = none anywhere. More memory
// never loses an implementation, so every limits point with a coordinate below the corner is
// unsatisfiable. For a finished Spec the corner is exact (read off its table); for a Spec of the
// stage being solved it is a lower bound worked out from its candidates before anything is solved.
#define MRL_NEVER 31u
__device__ __forceinline__ uint32_t corner_of(uint32_t pack, uint32_t k) { return (pack >> (5 * k)) & 31u; }

// Exact corners of the Specs of the stage before this one (their rows are complete, also where
// another rank computed them). Along memory k the cell with the top slot in every other memory is
// satisfiable as soon as any cell with that slot in k is.
__device__ __noinline__ void phase_minsat(const StageArgs& a, uint32_t gtid, uint32_t gthreads) {
  for (uint32_t i = a.prev_lo + gtid; i < a.prev_hi; i += gthreads) {
    const uint4 m = *reinterpret_cast<const uint4*>(&a.hdrs[i]);
    const MrlRow* grid = a.rows + a.hdrs[i].row_base;
    const uint32_t mm[4] = {m.x, m.y, m.z, m.w};
    uint32_t nn[4], st[4];
#pragma unroll
    for (int k = 0; k < 4; k++) nn[k] = __popc(mm[k]);
    st[0] = 1; st[1] = nn[0]; st[2] = nn[0] * nn[1]; st[3] = nn[0] * nn[1] * nn[2];
    uint32_t top = 0;
#pragma unroll
    for (int k = 0; k < 4; k++) top += (nn[k] - 1) * st[k];
    uint32_t pack = 0;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      uint32_t code = MRL_NEVER;
      for (uint32_t sl = 0; sl < nn[k]; sl++) {
        if (grid[top - (nn[k] - 1 - sl) * st[k]].tail != MRL_UNSAT) { code = nth_set_bit(mm[k], sl); break; }
      }
      pack |= code << (5 * k);
    }
    a.minsat[i] = pack;
  }
}

// Step 0: the corner of every Spec of the stage, per memory the minimum over its candidates of
// what each needs at least (its threshold; its children's corners, shifted by what a Move
// takes). Two rounds: the first knows nothing about same-stage children (bound zero) and leaves
// its result in minsat, the second reads those for same-stage children and writes the array the
// grids are clipped with, so that no thread reads what another writes.
__device__ __noinline__ void phase_corner(const StageArgs& a, uint32_t gtid, uint32_t gthreads, int round) {
  for (uint32_t i = a.lo + gtid; i < a.hi; i += gthreads) {
    if (!computed_here(a, i)) continue;
    const uint2 cl = *reinterpret_cast<const uint2*>(&a.hdrs[i].cand_off);
    uint32_t l0 = MRL_NEVER, l1 = MRL_NEVER, l2 = MRL_NEVER, l3 = MRL_NEVER;
    for (uint32_t ci = 0; ci < cl.y; ci++) {
      const uint4 c = __ldg(reinterpret_cast<const uint4*>(&a.cands[cl.x + ci]));
      const uint32_t kind = (c.x >> 16) & 0xFFu, nchild = c.x >> 24;
      const uint32_t level = c.z & 0xFFu, thr = (c.z >> 8) & 0xFFu, units = c.w;
      uint32_t q0 = 0, q1 = 0, q2 = 0, q3 = 0;   // this candidate's corner
      if (kind == MRL_CK_LEAF || kind == MRL_CK_MOVE) {
        q0 = level == 0 ? thr : 0u; q1 = level == 1 ? thr : 0u; q2 = level == 2 ? thr : 0u; q3 = level == 3 ? thr : 0u;
      }
      bool never = false;
      if (kind != MRL_CK_LEAF) {
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(&a.cands[cl.x + ci]) + 1);
        for (uint32_t j = 0; j < nchild; j++) {
          const uint32_t child = j == 0 ? b.x : (j == 1 ? b.y : b.z);
          // a finished child's exact corner; a same-stage child's bound from the first round
          const uint32_t cp = (child < a.lo || round) ? a.minsat[child] : 0u;
          uint32_t e0 = corner_of(cp, 0), e1 = corner_of(cp, 1), e2 = corner_of(cp, 2), e3 = corner_of(cp, 3);
          if (e0 == MRL_NEVER) { never = true; break; }
          if (kind == MRL_CK_MOVE) {
            const uint32_t e = sel4(e0, e1, e2, e3, level);
            uint32_t sh = 0;
            if (e) {
              const uint32_t bit = shift_mask(1u << e, level, units, code_of(a.top_pack, level));
              if (!bit) { never = true; break; }
              sh = __ffs(bit) - 1;
            }
            e0 = level == 0 ? sh : e0; e1 = level == 1 ? sh : e1; e2 = level == 2 ? sh : e2; e3 = level == 3 ? sh : e3;
          }
          q0 = max(q0, e0); q1 = max(q1, e1); q2 = max(q2, e2); q3 = max(q3, e3);
        }
      }
      if (!never) { l0 = min(l0, q0); l1 = min(l1, q1); l2 = min(l2, q2); l3 = min(l3, q3); }
    }
    const uint32_t t0 = code_of(a.top_pack, 0), t1 = code_of(a.top_pack, 1), t2 = code_of(a.top_pack, 2), t3 = code_of(a.top_pack, 3);
    if (l0 > t0 || l1 > t1 || l2 > t2 || l3 > t3) l0 = l1 = l2 = l3 = MRL_NEVER;   // no limits inside the lattice reach it
    const uint32_t corner = l0 | (l1 << 5) | (l2 << 10) | (l3 << 15);
    if (round == 0) a.minsat[i] = corner;
    a.corner[i - a.lo] = corner;
  }
}

// Clips a grid at the corner: below it everything is unsatisfiable, so one cell [0, corner) per
// memory is enough.
__device__ __forceinline__ uint4 clip_at_corner(uint4 nm, uint32_t corner) {
  const uint32_t k0 = corner_of(corner, 0), k1 = corner_of(corner, 1), k2 = corner_of(corner, 2), k3 = corner_of(corner, 3);
  if (k0 == MRL_NEVER) return make_uint4(1u, 1u, 1u, 1u);   // unsatisfiable at every limit: a single cell
  if (k0) nm.x = (nm.x & ~((1u << k0) - 1u)) | 1u | (1u << k0);
  if (k1) nm.y = (nm.y & ~((1u << k1) - 1u)) | 1u | (1u << k1);
  if (k2) nm.z = (nm.z & ~((1u << k2) - 1u)) | 1u | (1u << k2);
  if (k3) nm.w = (nm.w & ~((1u << k3) - 1u)) | 1u | (1u << k3);
  return nm;
}

// ORs into r the breakpoints one record puts into its Spec's grid: its own threshold, and its
// children's breakpoints (for a Move, shifted in the memory it allocates in). Children of
// finished stages contribute their final masks, same-stage children what rmask holds for them.
__device__ __forceinline__ void record_breakpoints(const StageArgs& a, uint32_t rec, const uint4 c, uint32_t& r0, uint32_t& r1,
                                                   uint32_t& r2, uint32_t& r3) {
  const uint32_t kind = (c.x >> 16) & 0xFFu, nchild = c.x >> 24;
  const uint32_t level = c.z & 0xFFu, thr = (c.z >> 8) & 0xFFu, units = c.w;
  if (kind == MRL_CK_LEAF || kind == MRL_CK_MOVE) or_level(r0, r1, r2, r3, level, 1u << thr);
  if (kind == MRL_CK_LEAF) return;
  const uint4 b = __ldg(reinterpret_cast<const uint4*>(&a.cands[rec]) + 1);
  for (uint32_t j = 0; j < nchild; j++) {
    const uint32_t child = j == 0 ? b.x : (j == 1 ? b.y : b.z);
    const uint4 cm = child < a.lo ? *reinterpret_cast<const uint4*>(&a.hdrs[child]) : a.rmask[child];
    if (kind == MRL_CK_MOVE) {
      const uint32_t s = shift_mask(sel4(cm.x, cm.y, cm.z, cm.w, level), level, units, code_of(a.top_pack, level));
      r0 |= (level == 0) ? s : cm.x;
      r1 |= (level == 1) ? s : cm.y;
      r2 |= (level == 2) ? s : cm.z;
      r3 |= (level == 3) ? s : cm.w;
    } else {
      r0 |= cm.x; r1 |= cm.y; r2 |= cm.z; r3 |= cm.w;
    }
  }
}

// Step 1: per Spec of the stage the grid of the unordered phase: the breakpoints of the records
// whose children all lie in finished stages (they come first). Nothing of it depends on the
// stage itself, so it is derived, and solved, once.
__device__ __noinline__ void phase_derive_early(const StageArgs& a, uint32_t gtid, uint32_t gthreads) {
  for (uint32_t i = a.lo + gtid; i < a.hi; i += gthreads) {
    if (!computed_here(a, i)) continue;
    const uint2 cl = *reinterpret_cast<const uint2*>(&a.hdrs[i].cand_off);
    uint32_t r0 = 1, r1 = 1, r2 = 1, r3 = 1;
    for (uint32_t ci = 0; ci < cl.y; ci++) {
      const uint4 c = __ldg(reinterpret_cast<const uint4*>(&a.cands[cl.x + ci]));
      if ((c.z >> 24) & 1u) break;   // records with a same-stage child come last
      record_breakpoints(a, cl.x + ci, c, r0, r1, r2, r3);
    }
    *reinterpret_cast<uint4*>(&a.ehdr[i - a.lo]) = clip_at_corner(make_uint4(r0, r1, r2, r3), a.corner[i - a.lo]);
  }
}

// Pass step 1: per Spec of the stage the grid the records with a same-stage child are solved on:
// the real breakpoints of what the unordered phase found (first pass: they are in rmask), the
// breakpoints of those records, and for their same-stage children the breakpoints in rmask -
// first pass: of what the unordered phase found for the child; later passes: found real by the
// pass before. Grids only grow; a Spec whose masks grew is marked for solving.
__device__ __noinline__ void phase_derive_late(const StageArgs& a, uint32_t gtid, uint32_t gthreads, int first) {
  for (uint32_t i = a.lo + gtid; i < a.hi; i += gthreads) {
    if (!computed_here(a, i)) continue;
    const uint4 old = first ? a.rmask[i] : *reinterpret_cast<const uint4*>(&a.hdrs[i]);
    const uint2 cl = *reinterpret_cast<const uint2*>(&a.hdrs[i].cand_off);
    uint32_t r0 = old.x, r1 = old.y, r2 = old.z, r3 = old.w;
    for (uint32_t back = 0; back < cl.y; back++) {
      const uint32_t ci = cl.y - 1 - back;
      const uint4 c = __ldg(reinterpret_cast<const uint4*>(&a.cands[cl.x + ci]));
      if (!((c.z >> 24) & 1u)) break;
      record_breakpoints(a, cl.x + ci, c, r0, r1, r2, r3);
    }
    const uint4 nm = clip_at_corner(make_uint4(r0, r1, r2, r3), a.corner[i - a.lo]);
    if (first || nm.x != old.x || nm.y != old.y || nm.z != old.z || nm.w != old.w) {
      *reinterpret_cast<uint4*>(&a.hdrs[i]) = nm;
      a.dirty[i] = 1;
    }
  }
}

// A Spec with a marked same-stage child has to be solved again too (its lookups may change).
// Monotone, so racing with other threads' marks is harmless; repeated until a round marks nothing.
__device__ __noinline__ void phase_spread(const StageArgs& a, uint32_t gtid, uint32_t gthreads, uint32_t epoch) {
  for (uint32_t i = a.lo + gtid; i < a.hi; i += gthreads) {
    if (!computed_here(a, i) || a.dirty[i]) continue;
    const uint2 cl = *reinterpret_cast<const uint2*>(&a.hdrs[i].cand_off);
    bool hit = false;
    for (uint32_t ci = 0; ci < cl.y && !hit; ci++) {
      const uint4 c = __ldg(reinterpret_cast<const uint4*>(&a.cands[cl.x + ci]));
      const uint32_t kind = (c.x >> 16) & 0xFFu, nchild = c.x >> 24;
      if (kind != MRL_CK_MOVE) continue;   // only Moves have same-stage children
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(&a.cands[cl.x + ci]) + 1);
      for (uint32_t j = 0; j < nchild; j++) {
        const uint32_t child = j == 0 ? b.x : (j == 1 ? b.y : b.z);
        if (child >= a.lo && a.dirty[child]) hit = true;
      }
    }
    if (hit) {
      a.dirty[i] = 1;
      a.ctl->spread_epoch = epoch;   // every writer of a round stores the same value
    }
  }
}

// Totals of what the coming solve takes: the grids of the unordered phase of all the stage's
// Specs (early), or the grids of the marked Specs (else).
__device__ __noinline__ void phase_totals(const StageArgs& a, uint32_t gtid, uint32_t gthreads, bool early) {
  unsigned long long cells = 0, warps = 0;
  for (uint32_t i = a.lo + gtid; i < a.hi; i += gthreads) {
    if (!computed_here(a, i) || !(early || a.dirty[i])) continue;
    const Grid g = grid_of(*reinterpret_cast<const uint4*>(early ? &a.ehdr[i - a.lo] : &a.hdrs[i]));
    cells += g.cells;
    warps += g.warps;
  }
  for (int o = 16; o > 0; o >>= 1) {
    cells += __shfl_xor_sync(0xFFFFFFFFu, cells, o);
    warps += __shfl_xor_sync(0xFFFFFFFFu, warps, o);
  }
  if ((threadIdx.x & 31) == 0 && cells) {
    atomicAdd(&a.ctl->cells, cells);
    atomicAdd(&a.ctl->warps, warps);
  }
}

// Gives every Spec of the stage the rows of its grid of the unordered phase (early: in the base
// rows, from row 0), or every marked Spec fresh working rows (from temp_top up; Specs that are not
// solved again keep theirs), with its work items and chunks, and resets its real-breakpoint
// masks. Capacities were checked against the totals before.
__device__ __noinline__ void phase_place(const StageArgs& a, unsigned long long temp_top, uint32_t item_cells, bool early) {
  __shared__ unsigned long long row0, chunk0, item0;
  for (uint32_t base = a.lo + blockIdx.x * kBlock; base < a.hi; base += gridDim.x * kBlock) {
    const uint32_t i = base + threadIdx.x;
    const bool active = i < a.hi && computed_here(a, i) && (early || a.dirty[i] == 1);
    Grid g;
    g.cells = 0; g.warps = 0; g.F = 0;
    if (active) g = grid_of(*reinterpret_cast<const uint4*>(early ? &a.ehdr[i - a.lo] : &a.hdrs[i]));
    const uint32_t n_items = (uint32_t)((g.cells + item_cells - 1) / item_cells);
    unsigned long long tot_cells, tot_warps, tot_items;
    const unsigned long long my_row = block_excl_scan(g.cells, &tot_cells);
    const unsigned long long my_chunk = block_excl_scan(active ? g.warps : 0ull, &tot_warps);
    const unsigned long long my_item = block_excl_scan(n_items, &tot_items);
    if (threadIdx.x == 0) {
      row0 = atomicAdd(&a.ctl->row_cursor, tot_cells);
      chunk0 = atomicAdd(&a.ctl->chunk_cursor, (uint32_t)tot_warps);
      item0 = atomicAdd(&a.ctl->item_cursor, (uint32_t)tot_items);
    }
    __syncthreads();
    if (active) {
      const unsigned long long cb = chunk0 + my_chunk;
      for (uint32_t w = 0; w < n_items; w++) {
        WorkItem it;
        it.spec = i;
        it.first_cell = w * item_cells;
        a.items[item0 + my_item + w] = it;
      }
      if (early) {
        a.ehdr[i - a.lo].row_base = row0 + my_row;
      } else {
        a.hdrs[i].row_base = (temp_top + row0 + my_row) | MRL_TEMP_FLAG;
        a.dirty[i] = 2;   // solved by this pass
      }
      a.rmask[i] = make_uint4(1u, 1u, 1u, 1u);
      for (uint32_t w = 0; w < g.warps; w++) {
        Chunk c;
        c.spec = i;
        c.col_start = (w * 32u) | (g.F << 30);
        a.chunks[cb + w] = c;
      }
    }
    __syncthreads();   // row0 / chunk0 / item0 are rewritten by the next round
  }
}

// A candidate record whose body is a Spec of the same stage (a relayout Move): the planner flags
// it and stores these records after all others, dearest first.
__device__ __forceinline__ bool is_late(const uint4 a) { return (a.z >> 24) & 1u; }

// Step 2: the candidates whose children all lie in earlier stages, for every cell of every
// Spec's grid of the unordered phase. No order is needed. A warp takes a work item (up to MRL_ITEM_CELLS cells of one
// Spec) at a time as it finishes others. Per item it first stages the Spec's records and the
// headers of their children in shared memory, one record per lane, so that the chain record ->
// child header -> child row costs two round trips per batch of records instead of two per record;
// then its lanes take 32 cells at a time and walk the staged records together, and the only
// global loads left in that loop are the child rows.
struct HotArgs {   // what the two solve phases read, by value: registers instead of the argument block in local memory
  const SpecHdr* hdrs;
  const CandRec* cands;
  const MrlRow* rows;
  MrlRow* temp;
  MrlRow* base;             // the grids of the unordered phase
  const SpecHdr* ehdr;      // their masks and first rows; already offset: indexed by Spec id
  const uint32_t* corner;   // already offset: indexed by Spec id
};
__device__ __forceinline__ HotArgs hot_args(const StageArgs& s) {
  HotArgs h;
  h.hdrs = s.hdrs; h.cands = s.cands; h.rows = s.rows; h.temp = s.temp; h.base = s.base; h.ehdr = s.ehdr - s.lo; h.corner = s.corner - s.lo;
  return h;
}
// A cell with a limit below its Spec's corner has no implementation; no record needs to be read.
__device__ __forceinline__ bool below_corner(uint32_t corner, uint32_t cpack) {
  return code_of(cpack, 0) < corner_of(corner, 0) || code_of(cpack, 1) < corner_of(corner, 1) ||
         code_of(cpack, 2) < corner_of(corner, 2) || code_of(cpack, 3) < corner_of(corner, 3);
}

constexpr int kBatch = 16;   // records staged at a time
struct StagedRec {           // a record with what the row lookups of its children need
  uint4 rec;                 // action | kind << 16 | nchild << 24, imm, level | thr << 8 | peak << 16, units
  uint4 mask[3];
  const MrlRow* grid[3];     // per child: the first row of its grid, in the table or in the working rows
  uint32_t stride[3][3];     // per child: rows per step in memories 1, 2, 3 of its grid
  uint8_t in_temp[4];        // per child: its grid lies in the working rows (it may change during a sweep)
};
static_assert(sizeof(StagedRec) == 128, "staged record");

// What the lookups of one child need, into its slot of a staged record.
__device__ __forceinline__ void stage_child(StagedRec& s, uint32_t j, const uint4 m, unsigned long long base, const MrlRow* rows,
                                            const MrlRow* temp) {
  s.mask[j] = m;
  s.grid[j] = row_at(rows, temp, base);
  s.in_temp[j] = (base & MRL_TEMP_FLAG) ? 1 : 0;
  const uint32_t n0 = __popc(m.x), n1 = __popc(m.y), n2 = __popc(m.z);
  s.stride[j][0] = n0;
  s.stride[j][1] = n0 * n1;
  s.stride[j][2] = n0 * n1 * n2;
}
// row_of with the child's header and strides at hand.
__device__ __forceinline__ const MrlRow* staged_row(const StagedRec& s, uint32_t j, uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
  const uint4 m = s.mask[j];
  const uint32_t i0 = __popc(m.x & b0) - 1, i1 = __popc(m.y & b1) - 1, i2 = __popc(m.z & b2) - 1, i3 = __popc(m.w & b3) - 1;
  const uint32_t off = i3 * s.stride[j][2] + i2 * s.stride[j][1] + i1 * s.stride[j][0] + i0;   // cells per Spec < 2^32
  return s.grid[j] + off;
}

// The lattice code of every slot of a grid, memory after memory, for the lanes of a warp to look
// up instead of counting bits (a grid has at most 17 + 17 + 12 + 27 slots).
constexpr int kMaxSlots = 80;
__device__ __forceinline__ void stage_slot_codes(uint8_t* codes, const uint4 m, uint32_t n0, uint32_t n1, uint32_t n2, uint32_t n3,
                                                 uint32_t lane) {
  __syncwarp();   // the previous item's codes have been read by every lane
  for (uint32_t t = lane; t < n0 + n1 + n2 + n3; t += 32) {
    uint32_t mk = m.x, slot = t;
    if (slot >= n0) { slot -= n0; mk = m.y; if (slot >= n1) { slot -= n1; mk = m.z; if (slot >= n2) { slot -= n2; mk = m.w; } } }
    codes[t] = (uint8_t)nth_set_bit(mk, slot);
  }
  __syncwarp();
}

// A staged record at one limits point; eval_candidate with the record and the child headers
// already at hand. All children are finished, so the rows come from the table on the read-only path.
__device__ __forceinline__ void eval_staged(const StagedRec& s, const MrlRow* __restrict__ rows, uint32_t ci,
                                            uint32_t cpack, uint32_t bm0, uint32_t bm1, uint32_t bm2, uint32_t bm3,
                                            Best& best, Tally& tally) {
  const uint4 a = s.rec;
  const uint32_t action = a.x & 0xFFFFu, kind = (a.x >> 16) & 0xFFu, nchild = a.x >> 24;   // the same in all lanes
  const uint32_t imm = a.y;
  const uint32_t level = a.z & 0xFFu, thr = (a.z >> 8) & 0xFFu, pcode = (a.z >> 16) & 0xFFu;
  const uint32_t units = a.w;
  const uint32_t lv = code_of(cpack, level);
  tally.cands++;
  uint32_t k_main, k_peaks, k_tail;
  if (kind == MRL_CK_LEAF) {
    if (lv < thr) return;
    k_main = imm;
    k_peaks = pcode << peak_shift(level);
    k_tail = (1u << 16) | action;
  } else {
    uint32_t c0 = bm0, c1 = bm1, c2 = bm2, c3 = bm3;
    const uint32_t sh = peak_shift(level);
    if (kind == MRL_CK_MOVE) {
      if (lv < thr) return;
      if (imm > best.main) return;   // a Move costs at least its own base cost
      const uint32_t cb = below(child_code(level, lv, units));
      c0 = (level == 0) ? cb : c0;
      c1 = (level == 1) ? cb : c1;
      c2 = (level == 2) ? cb : c2;
      c3 = (level == 3) ? cb : c3;
    }
    const uint4 r0 = __ldg(reinterpret_cast<const uint4*>(staged_row(s, 0, c0, c1, c2, c3)));
    uint4 r1 = r0, r2 = r0;
    if (nchild > 1) r1 = __ldg(reinterpret_cast<const uint4*>(staged_row(s, 1, c0, c1, c2, c3)));
    if (nchild > 2) r2 = __ldg(reinterpret_cast<const uint4*>(staged_row(s, 2, c0, c1, c2, c3)));
    tally.lookups += nchild;
    if (r0.z == MRL_UNSAT || r1.z == MRL_UNSAT || r2.z == MRL_UNSAT) return;
    uint32_t depth;
    if (kind == MRL_CK_LOOP) {
      k_main = sat_mul(r0.x, imm);
      k_peaks = r0.y;
      depth = 1u;
    } else {
      k_main = (kind == MRL_CK_MOVE) ? sat_add(imm, r0.x) : r0.x;
      if (nchild > 1) k_main = sat_add(k_main, r1.x);
      if (nchild > 2) k_main = sat_add(k_main, r2.x);
      if (k_main > best.main) return;
      k_peaks = __vmaxu4(__vmaxu4(r0.y, r1.y), r2.y);
      if (kind == MRL_CK_MOVE) {
        const uint32_t cc = (k_peaks >> sh) & 0xFFu;
        const uint32_t ncode = level < 2 ? units + cc : cache_code_ceil(units + cache_value(cc));
        k_peaks = (k_peaks & ~(0xFFu << sh)) | (ncode << sh);
      }
      depth = min(max(max(r0.z >> 16, r1.z >> 16), r2.z >> 16) + 1u, 255u);
    }
    k_tail = (depth << 16) | action;
  }
  if (key_less(k_main, k_peaks, k_tail, best)) {
    best.main = k_main;
    best.peaks = k_peaks;
    best.tail = k_tail;
    best.ci = ci;
  }
}

__device__ __noinline__ void phase_early(const HotArgs a, const WorkItem* items, uint32_t n_items, uint32_t item_cells,
                                         uint32_t* next_item, unsigned long long* block_stats) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t gwarps = gridDim.x * (kBlock / 32);
  __shared__ StagedRec staged_all[kBlock / 32][kBatch];
  __shared__ uint8_t codes_all[kBlock / 32][kMaxSlots];
  StagedRec* const staged = staged_all[threadIdx.x >> 5];   // this warp's
  uint8_t* const codes = codes_all[threadIdx.x >> 5];
  Tally tally = {0, 0};
  // every warp starts with the item of its own number; further items are handed out by a counter
  // (no atomics at all when there are fewer items than warps)
  for (uint32_t w = blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); w < n_items;) {
    const WorkItem it = items[w];
    const uint32_t i = it.spec;
    const uint4 m = *reinterpret_cast<const uint4*>(&a.ehdr[i]);
    const uint2 cl = *reinterpret_cast<const uint2*>(&a.hdrs[i].cand_off);
    MrlRow* const grid = a.base + a.ehdr[i].row_base;
    const uint32_t n0 = __popc(m.x), n1 = __popc(m.y), n2 = __popc(m.z), n3 = __popc(m.w);
    const uint32_t cells = n0 * n1 * n2 * n3;
    const uint32_t c_end = min(cells, it.first_cell + item_cells);
    const uint32_t corner = a.corner[i];
    stage_slot_codes(codes, m, n0, n1, n2, n3, lane);
    uint32_t b0 = 0;
    do {
      // stage the next records (those with a same-stage child come last and end the walk) ...
      const uint32_t nb = min((uint32_t)kBatch, cl.y - b0);
      __syncwarp();   // the previous batch has been read by every lane
      bool late = false;
      if (lane < nb) {
        const uint4 c = __ldg(reinterpret_cast<const uint4*>(&a.cands[cl.x + b0 + lane]));
        staged[lane].rec = c;
        late = is_late(c);
      }
      const uint32_t late_lanes = __ballot_sync(0xFFFFFFFFu, late);
      const uint32_t n_here = late_lanes ? (uint32_t)__ffs(late_lanes) - 1u : nb;
      __syncwarp();
      // ... and the headers of their children, one (record, child) per lane
      for (uint32_t t = lane; t < n_here * 3u; t += 32) {
        const uint32_t r = t / 3u, j = t - r * 3u;
        if (j < (staged[r].rec.x >> 24)) {
          const uint32_t child = __ldg(&a.cands[cl.x + b0 + r].child[j]);
          stage_child(staged[r], j, __ldg(reinterpret_cast<const uint4*>(&a.hdrs[child])), __ldg(&a.hdrs[child].row_base), a.rows, a.rows);
        }
      }
      __syncwarp();
      for (uint32_t c0 = it.first_cell; c0 < c_end; c0 += 32) {
        const uint32_t cell = c0 + lane;
        const bool valid = cell < c_end;
        uint32_t rest = valid ? cell : 0u;
        const uint32_t k0 = codes[rest % n0]; rest /= n0;
        const uint32_t k1 = codes[n0 + rest % n1]; rest /= n1;
        const uint32_t k2 = codes[n0 + n1 + rest % n2]; rest /= n2;
        const uint32_t k3 = codes[n0 + n1 + n2 + rest];
        const uint32_t cpack = k0 | (k1 << 8) | (k2 << 16) | (k3 << 24);
        const bool live = valid && !below_corner(corner, cpack);
        Best best = {MRL_UNSAT, MRL_UNSAT, MRL_UNSAT, MRL_UNSAT};
        if (!__any_sync(0xFFFFFFFFu, live)) {
          if (valid && b0 == 0) *reinterpret_cast<uint4*>(grid + cell) = make_uint4(best.main, best.peaks, best.tail, best.ci);
          continue;
        }
        if (b0 && live) {   // what the earlier batches found
          const uint4 r = *reinterpret_cast<const uint4*>(grid + cell);
          best.main = r.x; best.peaks = r.y; best.tail = r.z; best.ci = r.w;
        }
        const uint32_t bm0 = below(k0), bm1 = below(k1), bm2 = below(k2), bm3 = below(k3);
        if (live) {
          for (uint32_t r = 0; r < n_here; r++) eval_staged(staged[r], a.rows, b0 + r, cpack, bm0, bm1, bm2, bm3, best, tally);
        }
        if (valid && (b0 == 0 || live))
          *reinterpret_cast<uint4*>(grid + cell) = make_uint4(best.main, best.peaks, best.tail, best.ci);
      }
      if (late_lanes) break;
      b0 += nb;
    } while (b0 < cl.y);
    if (n_items <= gwarps) break;
    if (lane == 0) w = gwarps + atomicAdd(next_item, 1u);
    w = __shfl_sync(0xFFFFFFFFu, w, 0);
  }
  uint32_t tc = tally.cands, tl = tally.lookups;
  for (int o = 16; o > 0; o >>= 1) {
    tc += __shfl_xor_sync(0xFFFFFFFFu, tc, o);
    tl += __shfl_xor_sync(0xFFFFFFFFu, tl, o);
  }
  if (lane == 0 && (tc | tl)) {
    atomicAdd(&block_stats[0], (unsigned long long)tc);
    atomicAdd(&block_stats[1], (unsigned long long)tl);
  }
}

// Whole-row accesses to working rows that other warps may be writing at the same time: one
// 128-bit access each, so a reader sees a row either before or after an update, never a mix.
__device__ __forceinline__ uint4 ld_row_shared(const MrlRow* p) {
  unsigned long long lo, hi;
  asm volatile("{\n\t.reg .b128 q;\n\tld.relaxed.gpu.global.b128 q, [%2];\n\tmov.b128 {%0, %1}, q;\n\t}"
               : "=l"(lo), "=l"(hi) : "l"(p) : "memory");
  return make_uint4((uint32_t)lo, (uint32_t)(lo >> 32), (uint32_t)hi, (uint32_t)(hi >> 32));
}
__device__ __forceinline__ void st_row_shared(MrlRow* p, const uint4 v) {
  const unsigned long long lo = v.x | ((unsigned long long)v.y << 32), hi = v.z | ((unsigned long long)v.w << 32);
  asm volatile("{\n\t.reg .b128 q;\n\tmov.b128 q, {%1, %2};\n\tst.relaxed.gpu.global.b128 [%0], q;\n\t}"
               :: "l"(p), "l"(lo), "l"(hi) : "memory");
}

// A staged record with a same-stage child at one limits point. Children of the stage being solved
// live in the working rows and may improve while this runs; finished children are read-only.
__device__ __forceinline__ void eval_staged_late(const StagedRec& s, const MrlRow* __restrict__ rows, const MrlRow* temp,
                                                 uint32_t ci, uint32_t cpack, uint32_t bm0, uint32_t bm1, uint32_t bm2,
                                                 uint32_t bm3, Best& best, Tally& tally) {
  const uint4 a = s.rec;
  const uint32_t action = a.x & 0xFFFFu, kind = (a.x >> 16) & 0xFFu, nchild = a.x >> 24;   // the same in all lanes
  const uint32_t imm = a.y;
  const uint32_t level = a.z & 0xFFu, thr = (a.z >> 8) & 0xFFu;
  const uint32_t units = a.w;
  const uint32_t lv = code_of(cpack, level);
  tally.cands++;
  uint32_t c0 = bm0, c1 = bm1, c2 = bm2, c3 = bm3;
  const uint32_t sh = peak_shift(level);
  if (kind == MRL_CK_MOVE) {
    if (lv < thr) return;
    if (imm > best.main) return;   // a Move costs at least its own base cost
    const uint32_t cb = below(child_code(level, lv, units));
    c0 = (level == 0) ? cb : c0;
    c1 = (level == 1) ? cb : c1;
    c2 = (level == 2) ? cb : c2;
    c3 = (level == 3) ? cb : c3;
  }
  uint4 r[3];
#pragma unroll
  for (int j = 0; j < 3; j++) {
    if ((uint32_t)j < nchild) {
      const MrlRow* const p = staged_row(s, j, c0, c1, c2, c3);
      r[j] = s.in_temp[j] ? ld_row_shared(p) : __ldg(reinterpret_cast<const uint4*>(p));
    } else {
      r[j] = r[0];
    }
  }
  tally.lookups += nchild;
  if (r[0].z == MRL_UNSAT || r[1].z == MRL_UNSAT || r[2].z == MRL_UNSAT) return;
  uint32_t k_main, k_peaks, depth;
  if (kind == MRL_CK_LOOP) {
    k_main = sat_mul(r[0].x, imm);
    k_peaks = r[0].y;
    depth = 1u;
  } else {
    k_main = (kind == MRL_CK_MOVE) ? sat_add(imm, r[0].x) : r[0].x;
    if (nchild > 1) k_main = sat_add(k_main, r[1].x);
    if (nchild > 2) k_main = sat_add(k_main, r[2].x);
    if (k_main > best.main) return;
    k_peaks = __vmaxu4(__vmaxu4(r[0].y, r[1].y), r[2].y);
    if (kind == MRL_CK_MOVE) {
      const uint32_t cc = (k_peaks >> sh) & 0xFFu;
      const uint32_t ncode = level < 2 ? units + cc : cache_code_ceil(units + cache_value(cc));
      k_peaks = (k_peaks & ~(0xFFu << sh)) | (ncode << sh);
    }
    depth = min(max(max(r[0].z >> 16, r[1].z >> 16), r[2].z >> 16) + 1u, 255u);
  }
  const uint32_t k_tail = (depth << 16) | action;
  if (key_less(k_main, k_peaks, k_tail, best)) {
    best.main = k_main;
    best.peaks = k_peaks;
    best.tail = k_tail;
    best.ci = ci;
  }
}

// Pass step 4b, one relaxation sweep: the candidates with a child in the Spec's own stage (relayout
// Moves). Such a child is read at limits reduced by what the Move allocates, so the dependencies
// between cells form no cycle and the system "cell = best of its candidates at its children's
// values" has exactly one solution. A sweep recomputes every cell from what phase_early found at
// its limits (in the base rows) and all its same-stage records at the children's current values, in
// place, while other warps read and write their own cells; a cell whose children all hold their
// final values gets its final value, so every sweep settles at least one more level of the
// dependency order, and the pass is finished after a sweep that changed nothing anywhere. (Keeping
// the better of the old and the new value instead of recomputing would be wrong: a child that
// improves can make the parent's peaks or depth worse.) From the second sweep on a Spec is looked
// at again only if one of its same-stage children changed since the sweep before last began
// (stamp = number of the last sweep that changed any cell of a Spec).
// The records come dearest first and are staged from the end, so the cheapest Move is tried first.
__device__ __forceinline__ void stage_late_batch(const HotArgs& a, StagedRec* staged, uint32_t last_rec, uint32_t n_here,
                                                 uint32_t lane) {
  __syncwarp();   // the previous batch has been read by every lane
  if (lane < n_here) staged[lane].rec = __ldg(reinterpret_cast<const uint4*>(&a.cands[last_rec - lane]));
  __syncwarp();
  for (uint32_t t = lane; t < n_here * 3u; t += 32) {
    const uint32_t r = t / 3u, j = t - r * 3u;
    if (j < (staged[r].rec.x >> 24)) {
      const uint32_t child = __ldg(&a.cands[last_rec - r].child[j]);
      stage_child(staged[r], j, *reinterpret_cast<const uint4*>(&a.hdrs[child]), a.hdrs[child].row_base, a.rows, a.temp);   // same-stage headers: written earlier in this launch
    }
  }
  __syncwarp();
}

// Pass step 3: every cell of the grids placed by this pass starts from what the unordered phase
// found at the cell's limits. For a Spec without same-stage records that is its final value.
__device__ __noinline__ void phase_late_init(const HotArgs a, const WorkItem* items, uint32_t n_items, uint32_t item_cells,
                                             uint32_t* next_item) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t gwarps = gridDim.x * (kBlock / 32);
  for (uint32_t w = blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); w < n_items;) {
    const WorkItem it = items[w];
    const uint32_t i = it.spec;
    const uint4 m = *reinterpret_cast<const uint4*>(&a.hdrs[i]);
    MrlRow* const grid = a.temp + (a.hdrs[i].row_base & ~MRL_TEMP_FLAG);
    const uint4 em = *reinterpret_cast<const uint4*>(&a.ehdr[i]);
    const unsigned long long ebase = a.ehdr[i].row_base;
    const uint32_t n0 = __popc(m.x), n1 = __popc(m.y), n2 = __popc(m.z), n3 = __popc(m.w);
    const uint32_t c_end = min(n0 * n1 * n2 * n3, it.first_cell + item_cells);
    for (uint32_t cell = it.first_cell + lane; cell < c_end; cell += 32) {
      uint32_t rest = cell;
      const uint32_t k0 = nth_set_bit(m.x, rest % n0); rest /= n0;
      const uint32_t k1 = nth_set_bit(m.y, rest % n1); rest /= n1;
      const uint32_t k2 = nth_set_bit(m.z, rest % n2); rest /= n2;
      const uint32_t k3 = nth_set_bit(m.w, rest);
      *reinterpret_cast<uint4*>(grid + cell) =
          *reinterpret_cast<const uint4*>(row_of(a.base, a.base, em, ebase, below(k0), below(k1), below(k2), below(k3)));
    }
    if (n_items <= gwarps) break;
    if (lane == 0) w = gwarps + atomicAdd(next_item, 1u);
    w = __shfl_sync(0xFFFFFFFFu, w, 0);
  }
}

__device__ __noinline__ void phase_late(const HotArgs a, const WorkItem* items, uint32_t n_items, uint32_t item_cells,
                                        uint32_t* next_item, uint32_t lo, uint32_t* stamp /* by position in the stage */,
                                        uint32_t sweep, bool first_sweep, uint32_t* changed,
                                        unsigned long long* block_stats) {
  __shared__ StagedRec staged_all[kBlock / 32][kBatch];
  __shared__ uint8_t codes_all[kBlock / 32][kMaxSlots];
  StagedRec* const staged = staged_all[threadIdx.x >> 5];   // this warp's
  uint8_t* const codes = codes_all[threadIdx.x >> 5];
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t gwarps = gridDim.x * (kBlock / 32);
  Tally tally = {0, 0};
  for (uint32_t w = blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); w < n_items;) {
    const WorkItem it = items[w];
    const uint32_t i = it.spec;
    const uint2 cl = *reinterpret_cast<const uint2*>(&a.hdrs[i].cand_off);
    // the records with a same-stage child are the last ones
    uint32_t n_late = 0;
    for (uint32_t k = 0; k < cl.y; k += 32) {
      const bool late = k + lane < cl.y && ((__ldg(&reinterpret_cast<const uint32_t*>(&a.cands[cl.x + cl.y - 1 - k - lane])[2]) >> 24) & 1u);
      const uint32_t not_late = ~__ballot_sync(0xFFFFFFFFu, late);
      const uint32_t run = not_late ? (uint32_t)__ffs(not_late) - 1u : 32u;
      n_late += run;
      if (run < 32) break;
    }
    bool fresh = first_sweep && n_late;   // some same-stage child changed lately
    if (n_late && !first_sweep) {
      for (uint32_t t = lane; t < n_late * 3u; t += 32) {
        const uint32_t r = t / 3u, j = t - r * 3u;
        const CandRec* const rec = &a.cands[cl.x + cl.y - 1 - r];
        if (j < (__ldg(reinterpret_cast<const uint32_t*>(rec)) >> 24)) {
          const uint32_t child = __ldg(&rec->child[j]);
          if (child >= lo && stamp[child - lo] + 1u >= sweep) fresh = true;
        }
      }
      fresh = __any_sync(0xFFFFFFFFu, fresh);
    }
    if (fresh) {
      if (lane == 0) atomicAdd(&block_stats[4], 1ull);
      const uint4 m = *reinterpret_cast<const uint4*>(&a.hdrs[i]);
      MrlRow* const grid = a.temp + (a.hdrs[i].row_base & ~MRL_TEMP_FLAG);
      const uint4 em = *reinterpret_cast<const uint4*>(&a.ehdr[i]);   // where the unordered phase left its result
      const unsigned long long ebase = a.ehdr[i].row_base;
      const uint32_t n0 = __popc(m.x), n1 = __popc(m.y), n2 = __popc(m.z), n3 = __popc(m.w);
      const uint32_t cells = n0 * n1 * n2 * n3;
      const uint32_t corner = a.corner[i];
      // Grids are clipped at the corner, so the cells below it are exactly those in slot 0 of a
      // clipped memory; they stay unsatisfiable and are left out: the lanes walk the live cells
      // only. The item's share of them: its range of all cells, scaled (the items of a Spec tile
      // its cells, so the scaled ranges tile the live ones).
      const uint32_t z0 = corner_of(corner, 0) ? 1u : 0u, z1 = corner_of(corner, 1) ? 1u : 0u, z2 = corner_of(corner, 2) ? 1u : 0u,
                     z3 = corner_of(corner, 3) ? 1u : 0u;
      const uint32_t v0 = n0 - z0, v1 = n1 - z1, v2 = n2 - z2, v3 = n3 - z3;
      const unsigned long long live_cells = (corner_of(corner, 0) == MRL_NEVER) ? 0ull : (unsigned long long)v0 * v1 * v2 * v3;
      const uint32_t c_hi = min(cells, it.first_cell + item_cells);
      const uint32_t l_begin = (uint32_t)(live_cells * it.first_cell / cells), l_end = (uint32_t)(live_cells * c_hi / cells);
      const bool single = n_late <= (uint32_t)kBatch;   // all records staged once for the whole item
      stage_slot_codes(codes, m, n0, n1, n2, n3, lane);
      if (single) stage_late_batch(a, staged, cl.x + cl.y - 1, n_late, lane);
      bool changed_any = false;
      for (uint32_t c0 = l_begin; c0 < l_end; c0 += 32) {
        const bool live = c0 + lane < l_end;
        uint32_t rest = live ? c0 + lane : l_begin;
        const uint32_t s0 = rest % v0 + z0; rest /= v0;
        const uint32_t s1 = rest % v1 + z1; rest /= v1;
        const uint32_t s2 = rest % v2 + z2;
        const uint32_t s3 = rest / v2 + z3;
        const uint32_t cell = ((s3 * n2 + s2) * n1 + s1) * n0 + s0;
        const uint32_t k0 = codes[s0], k1 = codes[n0 + s1], k2 = codes[n0 + n1 + s2], k3 = codes[n0 + n1 + n2 + s3];
        const uint32_t cpack = k0 | (k1 << 8) | (k2 << 16) | (k3 << 24);
        Best best = {MRL_UNSAT, MRL_UNSAT, MRL_UNSAT, MRL_UNSAT};
        const uint32_t bm0 = below(k0), bm1 = below(k1), bm2 = below(k2), bm3 = below(k3);
        if (live) {
          const uint4 f = *reinterpret_cast<const uint4*>(row_of(a.base, a.base, em, ebase, bm0, bm1, bm2, bm3));
          best.main = f.x; best.peaks = f.y; best.tail = f.z; best.ci = f.w;
        }
        for (uint32_t b = 0; b < n_late; b += kBatch) {
          const uint32_t n_here = min((uint32_t)kBatch, n_late - b);
          if (!single) stage_late_batch(a, staged, cl.x + cl.y - 1 - b, n_here, lane);
          if (live)
            for (uint32_t r = 0; r < n_here; r++)
              eval_staged_late(staged[r], a.rows, a.temp, cl.y - 1 - b - r, cpack, bm0, bm1, bm2, bm3, best, tally);
        }
        if (live) {
          const uint4 was = *reinterpret_cast<const uint4*>(grid + cell);   // only this warp writes the cell in this sweep
          if (best.main != was.x || best.peaks != was.y || best.tail != was.z) {
            st_row_shared(grid + cell, make_uint4(best.main, best.peaks, best.tail, best.ci));
            changed_any = true;
          }
        }
      }
      if (__any_sync(0xFFFFFFFFu, changed_any) && lane == 0) {
        stamp[i - lo] = sweep;
        *changed = sweep;
      }
    }
    if (n_items <= gwarps) break;
    if (lane == 0) w = gwarps + atomicAdd(next_item, 1u);
    w = __shfl_sync(0xFFFFFFFFu, w, 0);
  }
  uint32_t tc = tally.cands, tl = tally.lookups;
  for (int o = 16; o > 0; o >>= 1) {
    tc += __shfl_xor_sync(0xFFFFFFFFu, tc, o);
    tl += __shfl_xor_sync(0xFFFFFFFFu, tl, o);
  }
  if (lane == 0 && (tc | tl)) {
    atomicAdd(&block_stats[2], (unsigned long long)tc);
    atomicAdd(&block_stats[3], (unsigned long long)tl);
  }
}

// Pass step 5: which breakpoints of the working grids are real. A breakpoint (memory k, code c)
// is real when some cell starting at c differs from its neighbour one slot lower in k.
// early: of the grids of the unordered phase (in the base rows), else of the working grids.
__device__ __noinline__ void phase_real_masks(const StageArgs& a, uint32_t n_chunks, bool early) {
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t gwarps = gridDim.x * (kBlock / 32);
  const SpecHdr* const H = early ? a.ehdr - a.lo : a.hdrs;
  const MrlRow* const R = early ? a.base : a.temp;
  for (uint32_t w = blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); w < n_chunks; w += gwarps) {
    const Chunk ch = a.chunks[w];
    const Column c = decode_column(H, ch, lane);
    uint32_t bits[4] = {0, 0, 0, 0};
    if (c.valid) {
      const unsigned long long base = H[ch.spec].row_base & ~MRL_TEMP_FLAG;
      const uint32_t st[4] = {1u, c.nn[0], c.nn[0] * c.nn[1], c.nn[0] * c.nn[1] * c.nn[2]};
      const uint32_t mF = sel4(c.mm[0], c.mm[1], c.mm[2], c.mm[3], c.F);
      const uint32_t nF = sel4(c.nn[0], c.nn[1], c.nn[2], c.nn[3], c.F);
      const uint32_t stF = sel4(st[0], st[1], st[2], st[3], c.F);
      uint32_t off0 = 0;
#pragma unroll
      for (int k = 0; k < 4; k++) off0 += c.idx[k] * st[k];   // idx[F] is 0
      uint4 prev = make_uint4(0, 0, 0, 0);
      uint32_t fbits = 0, mrest = mF, differs = 0;   // differs: memories in which some cell of the column differs from its lower neighbour
      for (uint32_t s = 0; s < nF; s++) {
        const uint32_t codeF = __ffs(mrest) - 1;
        mrest &= mrest - 1;
        const unsigned long long r_at = base + off0 + (unsigned long long)s * stF;
        const uint4 r = *reinterpret_cast<const uint4*>(R + r_at);
#pragma unroll
        for (int k = 0; k < 4; k++) {
          if ((uint32_t)k == c.F || c.idx[k] == 0) continue;
          const uint4 nb = *reinterpret_cast<const uint4*>(R + r_at - st[k]);
          if (nb.x != r.x || nb.y != r.y || nb.z != r.z) differs |= 1u << k;
        }
        if (s > 0 && (prev.x != r.x || prev.y != r.y || prev.z != r.z)) fbits |= 1u << codeF;
        prev = r;
      }
#pragma unroll
      for (int k = 0; k < 4; k++) {
        if ((uint32_t)k == c.F) bits[k] = fbits;
        else if ((differs >> k) & 1u) bits[k] = 1u << nth_set_bit(c.mm[k], c.idx[k]);   // the column's slot in that memory starts at a real breakpoint
      }
    }
#pragma unroll
    for (int k = 0; k < 4; k++) bits[k] = __reduce_or_sync(0xFFFFFFFFu, bits[k]);
    if (lane == 0) {
      uint32_t* out = reinterpret_cast<uint32_t*>(&a.rmask[ch.spec]);
#pragma unroll
      for (int k = 0; k < 4; k++)
        if (bits[k]) atomicOr(out + k, bits[k]);
    }
  }
}

// ---- compaction: working grids -> final table ---------------------------------------------

// Final cell count per Spec of the stage, the sum per run of kBlock Specs, and the algorithmic
// bytes of the stage's final rows.
__device__ __noinline__ void phase_final_count(const StageArgs& a) {
  unsigned long long bytes = 0;
  for (uint32_t base = a.lo + blockIdx.x * kBlock; base < a.hi; base += gridDim.x * kBlock) {
    const uint32_t i = base + threadIdx.x;
    unsigned long long n = 0;
    if (i < a.hi) {
      const uint4 m = a.rmask[i];
      n = (unsigned long long)__popc(m.x) * __popc(m.y) * __popc(m.z) * __popc(m.w);
      a.fcount[i - a.lo] = (uint32_t)n;
      if (computed_here(a, i)) {
        const uint2 cl = *reinterpret_cast<const uint2*>(&a.hdrs[i].cand_off);
        bytes += n * (12ull + 16ull * cl.y);
        for (uint32_t ci = 0; ci < cl.y; ci++) {
          const uint4 c = __ldg(reinterpret_cast<const uint4*>(&a.cands[cl.x + ci]));
          const uint32_t kind = (c.x >> 16) & 0xFFu, nchild = c.x >> 24;
          if (!nchild) continue;
          unsigned long long feasible = n;
          if (kind == MRL_CK_MOVE) {
            const uint32_t ml = sel4(m.x, m.y, m.z, m.w, c.z & 0xFFu), thr = (c.z >> 8) & 0xFFu;
            feasible = n / (uint32_t)__popc(ml) * (uint32_t)__popc(ml >> thr);   // final cells at or above the threshold
          }
          bytes += feasible * nchild * 16ull;
        }
      }
    }
    unsigned long long total;
    block_excl_scan(n, &total);
    if (threadIdx.x == 0) a.block_sums[(base - a.lo) / kBlock] = total;
  }
  for (int o = 16; o > 0; o >>= 1) bytes += __shfl_xor_sync(0xFFFFFFFFu, bytes, o);
  if ((threadIdx.x & 31) == 0 && bytes) atomicAdd(&a.ctl->st_final_bytes, bytes);
}

// Exclusive scan of the run sums (one block), and the stage's place in the table.
__device__ __noinline__ void phase_scan_sums(const StageArgs& a) {
  const uint32_t n_runs = (a.hi - a.lo + kBlock - 1) / kBlock;
  unsigned long long carry = 0;
  for (uint32_t b0 = 0; b0 < n_runs; b0 += kBlock) {
    const uint32_t b = b0 + threadIdx.x;
    const unsigned long long v = b < n_runs ? a.block_sums[b] : 0ull;
    unsigned long long total;
    const unsigned long long ex = block_excl_scan(v, &total);
    if (b < n_runs) a.block_sums[b] = carry + ex;
    carry += total;
  }
  if (threadIdx.x == 0) {
    FillCtl* ctl = a.ctl;
    ctl->stage_first_row = ctl->final_top;
    ctl->stage_rows = carry;
    if (ctl->final_top + carry > a.row_cap) {
      if (!ctl->error) ctl->failed_stage = a.stage;
      ctl->error |= MRL_ERR_TABLE;
      ctl->need_rows = ctl->final_top + carry;
    } else {
      ctl->final_top += carry;
    }
  }
}

// Copies each Spec's real cells from its working grid to its final rows and repoints the header.
// Specs computed by another rank get zero rows (the exchange adds the owner's rows onto them).
__device__ __noinline__ void phase_compact(const StageArgs& a) {
  const unsigned long long first_row = a.ctl->stage_first_row;
  for (uint32_t base = a.lo + blockIdx.x * kBlock; base < a.hi; base += gridDim.x * kBlock) {
    const uint32_t i = base + threadIdx.x;
    const unsigned long long n = i < a.hi ? a.fcount[i - a.lo] : 0u;
    unsigned long long total;
    const unsigned long long ex = block_excl_scan(n, &total);
    if (i >= a.hi) continue;
    const unsigned long long fbase = first_row + a.block_sums[(base - a.lo) / kBlock] + ex;
    const uint4 fm = a.rmask[i];
    if (computed_here(a, i)) {
      const uint4 tm = *reinterpret_cast<const uint4*>(&a.hdrs[i]);
      const unsigned long long tbase = a.hdrs[i].row_base & ~MRL_TEMP_FLAG;
      const uint32_t f0 = __popc(fm.x), f1 = __popc(fm.y), f2 = __popc(fm.z);
      const uint32_t t0 = __popc(tm.x), t1 = __popc(tm.y), t2 = __popc(tm.z);
      for (uint32_t j = 0; j < (uint32_t)n; j++) {
        uint32_t rest = j;
        const uint32_t j0 = rest % f0; rest /= f0;
        const uint32_t j1 = rest % f1; rest /= f1;
        const uint32_t j2 = rest % f2; rest /= f2;
        const uint32_t j3 = rest;
        const uint32_t i0 = __popc(tm.x & below(nth_set_bit(fm.x, j0))) - 1;
        const uint32_t i1 = __popc(tm.y & below(nth_set_bit(fm.y, j1))) - 1;
        const uint32_t i2 = __popc(tm.z & below(nth_set_bit(fm.z, j2))) - 1;
        const uint32_t i3 = __popc(tm.w & below(nth_set_bit(fm.w, j3))) - 1;
        const uint32_t toff = ((i3 * t2 + i2) * t1 + i1) * t0 + i0;
        uint4 r = *reinterpret_cast<const uint4*>(a.temp + tbase + toff);
        r.w = 0;
        *reinterpret_cast<uint4*>(a.rows + fbase + j) = r;
      }
    } else {
      for (uint32_t j = 0; j < (uint32_t)n; j++) *reinterpret_cast<uint4*>(a.rows + fbase + j) = make_uint4(0, 0, 0, 0);
    }
    *reinterpret_cast<uint4*>(&a.hdrs[i]) = fm;
    a.hdrs[i].row_base = fbase;
  }
}

// One stage, start to finish, in one cooperative launch. Every thread of the grid reaches every
// barrier: what decides the control flow (totals, the closure epoch, the sweep that last changed
// a cell, the error word) is read from device memory after a barrier and written again only
// after a later one, so all threads take the same branches.
__global__ void __launch_bounds__(kBlock, kMinBlocks) stage_kernel(const StageArgs a) {
  cg::grid_group grid = cg::this_grid();
  const uint32_t gtid = blockIdx.x * kBlock + threadIdx.x;
  const uint32_t gthreads = gridDim.x * kBlock;
  FillCtl* const ctl = a.ctl;
  uint32_t syncs = 0;
#define GRID_SYNC() do { grid.sync(); syncs++; } while (0)
  if (ctl->error) return;   // an earlier stage failed: the host repairs and resumes (uniform: nothing writes it before the first barrier)
  __shared__ unsigned long long block_stats[5];   // candidates evaluated and rows gathered by the unordered phase; by the sweeps; items the sweeps evaluated
  if (threadIdx.x < 5) block_stats[threadIdx.x] = 0;
  __syncthreads();
  if (a.solve) {
    if (gtid == 0) {
      ctl->cells = ctl->warps = ctl->row_cursor = 0;
      ctl->chunk_cursor = ctl->item_cursor = ctl->item_next = 0;
      ctl->spread_epoch = 0;
      ctl->temp_top = 0;
      ctl->sweep_next[0] = ctl->sweep_next[1] = 0;
      ctl->late_changed = 0;
    }
    for (uint32_t i = gtid; i < a.hi - a.lo; i += gthreads) a.stamp[i] = 0;
    if (a.mine)
      for (uint32_t i = a.lo + gtid; i < a.hi; i += gthreads) a.rmask[i] = make_uint4(0, 0, 0, 0);   // other ranks' Specs: zero until the exchange
    for (uint32_t i = a.lo + gtid; i < a.hi; i += gthreads) a.dirty[i] = 0;
    phase_minsat(a, gtid, gthreads);
    GRID_SYNC();
    uint32_t epoch = 0, sweep = 0, sweep_before = 0;
    unsigned long long n_sweeps = 0, t_last = 0;
    if (gtid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_last));
    // device time since the last mark goes to part ph (thread 0 only; after a barrier)
#define MARK(ph) do { if (gtid == 0) { unsigned long long t_now; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_now)); \
                                       ctl->st_phase_ns[ph] += t_now - t_last; t_last = t_now; } } while (0)
    bool failed = false;
    const uint32_t gwarps = gridDim.x * (kBlock / 32);
    // ---- once per stage: the corners, then the candidates whose children are all finished, on grids of their own
    phase_corner(a, gtid, gthreads, 0);
    GRID_SYNC();
    phase_corner(a, gtid, gthreads, 1);
    GRID_SYNC();
    phase_derive_early(a, gtid, gthreads);
    GRID_SYNC();
    phase_totals(a, gtid, gthreads, true);
    GRID_SYNC();
    {
      const unsigned long long cells = ctl->cells, warps = ctl->warps;
      // Work items: an even share of the cells per warp, in whole warp-wide steps, at most
      // MRL_ITEM_CELLS; every Spec adds at most one partial item.
      const uint32_t item_cells = (uint32_t)min((unsigned long long)MRL_ITEM_CELLS, max(32ull, ((cells + gwarps - 1) / gwarps + 31ull) & ~31ull));
      const unsigned long long max_items = cells / item_cells + (a.hi - a.lo);
      if (cells > a.temp_cap || warps > a.chunk_cap || max_items > a.item_cap || cells >= 0xFFFFFFF0ull || warps >= 0xFFFFFFF0ull) {
        failed = true;
        if (gtid == 0) {
          ctl->failed_stage = a.stage;
          ctl->error |= MRL_ERR_WORKING;
          ctl->need_temp = cells;
          ctl->need_chunks = warps;
          ctl->need_items = max_items;
        }
      } else if (cells) {
        phase_place(a, 0, item_cells, true);
        GRID_SYNC();
        MARK(MRL_PH_SETUP);
        const uint32_t n_items = ctl->item_cursor;
        phase_early(hot_args(a), a.items, n_items, item_cells, &ctl->item_next, block_stats);
        GRID_SYNC();
        MARK(MRL_PH_EARLY);
        phase_real_masks(a, (uint32_t)warps, true);   // into rmask: what the first pass seeds the working grids with
        if (gtid == 0) {
          ctl->st_cells += cells;
          ctl->st_early_cells += cells;
          ctl->cells = ctl->warps = ctl->row_cursor = 0;
          ctl->chunk_cursor = ctl->item_cursor = ctl->item_next = 0;
        }
        GRID_SYNC();
        MARK(MRL_PH_EARLY_MASKS);
      }
    }
    // ---- passes: the candidates with a same-stage child, until every working grid is consistent
    for (int pass = 0; !failed; pass++) {
      if (pass >= kMaxPasses) { failed = true; if (gtid == 0) { ctl->failed_stage = a.stage; ctl->error |= MRL_ERR_PASSES; } break; }
      phase_derive_late(a, gtid, gthreads, pass == 0);
      GRID_SYNC();
      if (pass > 0) {
        // close the marks under "has a marked same-stage child"
        for (;;) {
          epoch++;
          phase_spread(a, gtid, gthreads, epoch);
          GRID_SYNC();
          if (ctl->spread_epoch != epoch) break;
        }
      }
      phase_totals(a, gtid, gthreads, false);
      GRID_SYNC();
      const unsigned long long cells = ctl->cells, warps = ctl->warps, temp_top = ctl->temp_top;
      const uint32_t item_cells = (uint32_t)min((unsigned long long)MRL_ITEM_CELLS, max(32ull, ((cells + gwarps - 1) / gwarps + 31ull) & ~31ull));
      const unsigned long long max_items = cells / item_cells + (a.hi - a.lo);
      if (cells == 0) break;   // nothing left to solve: every working grid is consistent
      if (temp_top + cells > a.temp_cap || warps > a.chunk_cap || max_items > a.item_cap ||
          cells >= 0xFFFFFFF0ull || warps >= 0xFFFFFFF0ull) {
        failed = true;
        if (gtid == 0) {
          ctl->failed_stage = a.stage;
          ctl->error |= MRL_ERR_WORKING;
          ctl->need_temp = temp_top + cells;
          ctl->need_chunks = warps;
          ctl->need_items = max_items;
        }
        break;
      }
      phase_place(a, temp_top, item_cells, false);
      GRID_SYNC();
      MARK(MRL_PH_PASS_SETUP);
      const uint32_t n_chunks = (uint32_t)warps;
      const uint32_t n_items = ctl->item_cursor;
      phase_late_init(hot_args(a), a.items, n_items, item_cells, &ctl->item_next);
      GRID_SYNC();
      MARK(MRL_PH_INIT);
      for (bool first_sweep = true;; first_sweep = false) {
        sweep++;
        if (gtid == 0) ctl->sweep_next[(sweep + 1) & 1] = 0;   // the other counter is idle during this sweep
        phase_late(hot_args(a), a.items, n_items, item_cells, &ctl->sweep_next[sweep & 1], a.lo, a.stamp, sweep, first_sweep,
                   &ctl->late_changed, block_stats);
        GRID_SYNC();
        MARK(first_sweep ? MRL_PH_SWEEP_FIRST : MRL_PH_SWEEP_MORE);
        if (ctl->late_changed != sweep) break;   // nothing changed anywhere: the stage's cells are consistent
        if (sweep - sweep_before >= (uint32_t)kMaxSweeps) {   // more sweeps than the limits lattice has diagonals: give up rather than spin
          failed = true;
          if (gtid == 0) { ctl->failed_stage = a.stage; ctl->error |= MRL_ERR_PASSES; }
          break;
        }
      }
      if (failed) break;
      n_sweeps += sweep - sweep_before;
      sweep_before = sweep;
      phase_real_masks(a, n_chunks, false);
      for (uint32_t i = a.lo + gtid; i < a.hi; i += gthreads)
        if (a.dirty[i] == 2) a.dirty[i] = 0;
      if (gtid == 0) {
        ctl->temp_top = temp_top + cells;
        ctl->st_cells += cells;
        ctl->st_passes += 1;
        ctl->cells = ctl->warps = ctl->row_cursor = 0;
        ctl->chunk_cursor = ctl->item_cursor = ctl->item_next = 0;
      }
      GRID_SYNC();
      MARK(MRL_PH_PASS_MASKS);
    }
    MARK(MRL_PH_PASS_SETUP);   // of a pass that found nothing left to solve
#undef MARK
    __syncthreads();
    if (threadIdx.x == 0 && (block_stats[0] | block_stats[1] | block_stats[2] | block_stats[4])) {
      atomicAdd(&ctl->st_cands, block_stats[0] + block_stats[2]);
      atomicAdd(&ctl->st_lookups, block_stats[1] + block_stats[3]);
      atomicAdd(&ctl->st_late_cands, block_stats[2]);
      atomicAdd(&ctl->st_late_items, block_stats[4]);
    }
    if (gtid == 0) ctl->st_sweeps += n_sweeps;
    if (failed) {
      if (gtid == 0) ctl->st_syncs += syncs;
      return;   // uniform
    }
  }
  if (a.place) {
    phase_final_count(a);
    GRID_SYNC();
    if (blockIdx.x == 0) phase_scan_sums(a);
    GRID_SYNC();
    if (!(ctl->error & MRL_ERR_TABLE)) phase_compact(a);   // uniform: set by phase_scan_sums only
  }
  if (gtid == 0) ctl->st_syncs += syncs;
#undef GRID_SYNC
}

// Consistency check of a finished table: at sampled (or all) points of the limits lattice, for
// sampled (or all) Specs, the direct solve from the children's tables - every candidate record,
// no re-use of neighbouring cells - must equal what the Spec's own table returns there. Every
// point where that holds is a point where the table satisfies the defining recurrence of the
// fill, whatever grid the table is stored on.
__global__ void __launch_bounds__(kBlock)
verify_points_kernel(const SpecHdr* hdrs, const CandRec* __restrict__ cands, const MrlRow* rows, uint32_t n_specs,
                     uint32_t top_pack, unsigned long long first, unsigned long long count,
                     unsigned long long total_points, unsigned long long seed, int exhaustive,
                     unsigned long long* out /* [0] mismatches, [1] first bad sample */) {
  const unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const uint32_t e0 = code_of(top_pack, 0) + 1, e1 = code_of(top_pack, 1) + 1, e2 = code_of(top_pack, 2) + 1,
                 e3 = code_of(top_pack, 3) + 1;
  const unsigned long long per_spec = (unsigned long long)e0 * e1 * e2 * e3;
  unsigned long long s = first + i;
  if (!exhaustive) {
    // splitmix64 of (seed, sample index): a point of the (Spec x lattice) product
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (s + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    s = z % total_points;
  }
  const uint32_t spec = (uint32_t)(s / per_spec);
  uint32_t p = (uint32_t)(s % per_spec);
  const uint32_t c0 = p % e0; p /= e0;
  const uint32_t c1 = p % e1; p /= e1;
  const uint32_t c2 = p % e2;
  const uint32_t c3 = p / e2;
  const uint32_t cpack = c0 | (c1 << 8) | (c2 << 16) | (c3 << 24);
  Tally tally = {0, 0};
  const Best k = solve_point(hdrs, cands, rows, rows, spec, cpack, tally);
  const uint4 r = lookup(hdrs, rows, rows, spec, below(c0), below(c1), below(c2), below(c3));
  if (k.main != r.x || k.peaks != r.y || k.tail != r.z) {
    atomicAdd(&out[0], 1ull);
    atomicMin(&out[1], first + i);
  }
}

// Point lookups for get: the row of (Spec id, packed limit codes), into a dense buffer.
__global__ void lookup_rows_kernel(const SpecHdr* hdrs, const MrlRow* rows, const uint2* __restrict__ queries,
                                   unsigned long long n, MrlRow* __restrict__ out) {
  const unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint2 q = queries[i];
  const uint4 r = lookup(hdrs, rows, rows, q.x, below(code_of(q.y, 0)), below(code_of(q.y, 1)), below(code_of(q.y, 2)),
                         below(code_of(q.y, 3)));
  *reinterpret_cast<uint4*>(out + i) = r;
}

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// Sum over all Specs of a hash of (id, masks, rows in cell order). The sum commutes, and where a
// Spec's rows lie in the table does not enter, so two fills of one plan agree however their
// tables are laid out.
__global__ void __launch_bounds__(kBlock)
checksum_kernel(const SpecHdr* hdrs, const MrlRow* rows, uint32_t n_specs, unsigned long long* out) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  unsigned long long h = 0;
  if (i < n_specs) {
    const uint4 m = *reinterpret_cast<const uint4*>(&hdrs[i]);
    const unsigned long long base = hdrs[i].row_base;
    const unsigned long long n = (unsigned long long)__popc(m.x) * __popc(m.y) * __popc(m.z) * __popc(m.w);
    h = mix64(0x9E3779B97F4A7C15ull * (i + 1ull));
    h = mix64(h ^ (((unsigned long long)m.x << 32) | m.y));
    h = mix64(h ^ (((unsigned long long)m.z << 32) | m.w));
    for (unsigned long long j = 0; j < n; j++) {
      const uint4 r = *reinterpret_cast<const uint4*>(rows + base + j);
      h = mix64(h ^ (((unsigned long long)r.x << 32) | r.y));
      h = mix64(h ^ r.z);
    }
  }
  for (int o = 16; o > 0; o >>= 1) h += __shfl_xor_sync(0xFFFFFFFFu, h, o);
  if ((threadIdx.x & 31) == 0 && h) atomicAdd(out, h);
}

// Candidate records that arrived on the device without passing through this host's planner:
// every field a kernel indexes with must be in range.
__global__ void __launch_bounds__(kBlock)
check_records_kernel(const SpecHdr* hdrs, const CandRec* __restrict__ cands, uint32_t n_specs, unsigned long long n_cands,
                     uint32_t* error) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_specs) return;
  const uint2 cl = *reinterpret_cast<const uint2*>(&hdrs[i].cand_off);
  bool bad = (unsigned long long)cl.x + cl.y > n_cands;
  for (uint32_t ci = 0; ci < cl.y && !bad; ci++) {
    const CandRec c = cands[cl.x + ci];
    bad = c.kind > MRL_CK_BLOCK || c.nchild > 3 || c.level > 3 || c.thr_code > 30 || c.peak_code > 31 || c.late > 1 ||
          (c.kind == MRL_CK_LEAF) != (c.nchild == 0);
    for (uint32_t j = 0; j < c.nchild && !bad; j++) bad = c.child[j] >= n_specs;
  }
  if (bad) atomicOr(error, (uint32_t)MRL_ERR_CHILD);
}

}  // namespace

namespace mrl {

#define CK(x)                                                                              \
  do {                                                                                     \
    cudaError_t e_ = (x);                                                                  \
    if (e_ != cudaSuccess) {                                                               \
      snprintf(err_, sizeof(err_), "%s failed: %s", #x, cudaGetErrorString(e_));           \
      return -1;                                                                           \
    }                                                                                      \
  } while (0)

static size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

DeviceFill::~DeviceFill() { release(); }

int DeviceFill::too_large_() {
  snprintf(err_, sizeof(err_),
           "this fill needs more than the %zu bytes of device memory the no-allocation entry point has; "
           "use mrl_top_down_many for it", buf_bytes_);
  return -5;
}

int DeviceFill::alloc_(void** p, size_t bytes) {
  bytes = std::max<size_t>(bytes, 256);
  if (fixed_) {
    const size_t off = align256(buf_off_);
    if (off + bytes > buf_bytes_) return too_large_();
    *p = buf_ + off;
    buf_off_ = off + bytes;
    return 0;
  }
  cudaError_t e = cudaMalloc(p, bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    snprintf(err_, sizeof(err_), "out of device memory: cudaMalloc of %zu bytes failed (%s)", bytes, cudaGetErrorString(e));
    return -6;
  }
  return 0;
}

void DeviceFill::free_(void* p) {
  if (p && !fixed_) cudaFree(p);
}

void DeviceFill::release() {
  wait_upload();
  free_(d_hdrs_); free_(d_cands_); free_(d_rmask_); free_(d_mine_); free_(d_chunks_); free_(d_items_); free_(d_minsat_); free_(d_corner_); free_(d_stamp_); free_(d_ehdr_); free_(d_rows_);
  free_(d_temp_); free_(d_fcount_); free_(d_block_sums_); free_(d_ctl_); free_(d_stage_);
  free_(d_dirty_);
  d_hdrs_ = nullptr; d_cands_ = nullptr; d_rmask_ = nullptr; d_mine_ = nullptr; d_chunks_ = nullptr; d_items_ = nullptr; d_minsat_ = nullptr; d_corner_ = nullptr; d_stamp_ = nullptr; d_ehdr_ = nullptr;
  d_rows_ = nullptr; d_temp_ = nullptr; d_fcount_ = nullptr; d_block_sums_ = nullptr; d_ctl_ = nullptr;
  d_stage_ = nullptr; d_dirty_ = nullptr;
  stage_bytes_ = 0;
  row_cap_ = temp_cap_ = chunk_cap_ = item_cap_ = 0;
  buf_off_ = 0;
  cands_present_ = false;
  if (h_ctl_ && h_ctl_ != &ctl_pageable_) cudaFreeHost(h_ctl_);
  h_ctl_ = nullptr;
  if (ev0_) cudaEventDestroy(ev0_);
  if (ev1_) cudaEventDestroy(ev1_);
  ev0_ = ev1_ = nullptr;
  if (own_stream_ && stream_) cudaStreamDestroy(stream_);
  stream_ = nullptr;
  own_stream_ = false;
}

int DeviceFill::init(int device) {
  device_ = device;
  CK(cudaSetDevice(device));
  if (!stream_) {
    CK(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    own_stream_ = true;
  }
  return init_events();
}

int DeviceFill::init_events() {
  if (!ev0_) CK(cudaEventCreate(&ev0_));
  if (!ev1_) CK(cudaEventCreate(&ev1_));
  int coop = 0, per_sm = 0;
  CK(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device_));
  CK(cudaDeviceGetAttribute(&n_sm_, cudaDevAttrMultiProcessorCount, device_));
  if (!coop) { snprintf(err_, sizeof(err_), "the device does not support cooperative launches"); return -1; }
  CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, stage_kernel, kBlock, 0));
  if (per_sm < 1) { snprintf(err_, sizeof(err_), "the stage kernel does not fit an SM"); return -1; }
  coop_blocks_ = per_sm * n_sm_;
  return 0;
}

void DeviceFill::attach_buffer(void* base, size_t bytes, cudaStream_t stream, int device) {
  fixed_ = true;
  buf_ = static_cast<unsigned char*>(base);
  buf_bytes_ = bytes;
  buf_off_ = 0;
  stream_ = stream;
  own_stream_ = false;
  device_ = device;
}

int DeviceFill::set_stream(cudaStream_t s) {
  if (own_stream_ && stream_) cudaStreamDestroy(stream_);
  stream_ = s;
  own_stream_ = false;
  return 0;
}

int DeviceFill::wait_cands_(uint64_t upto_bytes) {
  if (up_threads_.empty()) return 0;
  const size_t need = std::min<uint64_t>(up_pieces_, (upto_bytes + up_piece_bytes_ - 1) / up_piece_bytes_);
  while (up_ready_ < need) {
    if (up_done_[up_ready_].load(std::memory_order_acquire)) up_ready_++;
    else if (up_err_.load(std::memory_order_relaxed) != 0) break;
    else std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  const int e = up_err_.load();
  if (up_ready_ == up_pieces_ || e != 0) {
    for (auto& th : up_threads_) th.join();
    up_threads_.clear();
  }
  if (e != 0) {
    snprintf(err_, sizeof(err_), "candidate upload failed: %s", cudaGetErrorString((cudaError_t)e));
    return -1;
  }
  return 0;
}

int DeviceFill::wait_upload() { return wait_cands_(~uint64_t(0) >> 1); }

int DeviceFill::upload(const Plan& plan, bool skip_cands) {
  CK(cudaSetDevice(device_));
  wait_upload();   // of an earlier plan
  free_(d_hdrs_); free_(d_cands_); free_(d_rmask_); free_(d_mine_); free_(d_chunks_); free_(d_items_); free_(d_minsat_); free_(d_corner_); free_(d_stamp_); free_(d_ehdr_); free_(d_rows_);
  free_(d_temp_); free_(d_fcount_); free_(d_block_sums_); free_(d_ctl_); free_(d_stage_);
  free_(d_dirty_);
  d_hdrs_ = nullptr; d_cands_ = nullptr; d_rmask_ = nullptr; d_mine_ = nullptr; d_chunks_ = nullptr; d_items_ = nullptr; d_minsat_ = nullptr; d_corner_ = nullptr; d_stamp_ = nullptr; d_ehdr_ = nullptr;
  d_rows_ = nullptr; d_temp_ = nullptr; d_fcount_ = nullptr; d_block_sums_ = nullptr; d_ctl_ = nullptr;
  d_stage_ = nullptr; d_dirty_ = nullptr;
  stage_bytes_ = 0;
  buf_off_ = 0;
  cands_present_ = false;
  n_specs_ = (uint32_t)plan.hdrs.size();
  max_stage_ = 1;
  for (const Stage& st : plan.stages) max_stage_ = std::max(max_stage_, st.spec_hi - st.spec_lo);
  int rc;
  if ((rc = alloc_((void**)&d_ctl_, 512))) return rc;
  if ((rc = alloc_((void**)&d_hdrs_, plan.hdrs.size() * sizeof(SpecHdr)))) return rc;
  if ((rc = alloc_((void**)&d_cands_, plan.cands.size() * sizeof(CandRec)))) return rc;
  if ((rc = alloc_((void**)&d_rmask_, plan.hdrs.size() * sizeof(uint4)))) return rc;
  if ((rc = alloc_((void**)&d_dirty_, plan.hdrs.size()))) return rc;
  if ((rc = alloc_((void**)&d_minsat_, plan.hdrs.size() * sizeof(uint32_t)))) return rc;
  if ((rc = alloc_((void**)&d_corner_, (size_t)max_stage_ * sizeof(uint32_t)))) return rc;
  if ((rc = alloc_((void**)&d_stamp_, (size_t)max_stage_ * sizeof(uint32_t)))) return rc;
  if ((rc = alloc_((void**)&d_ehdr_, (size_t)max_stage_ * sizeof(SpecHdr)))) return rc;
  if (!plan.mine.empty() && (rc = alloc_((void**)&d_mine_, plan.mine.size()))) return rc;
  if ((rc = alloc_((void**)&d_fcount_, (size_t)max_stage_ * sizeof(uint32_t)))) return rc;
  if ((rc = alloc_((void**)&d_block_sums_, ((size_t)max_stage_ / kBlock + 1) * sizeof(unsigned long long)))) return rc;
  if (fixed_) {
    // Everything left is split once: lookup staging, chunks, work items, working rows and final rows.
    stage_bytes_ = 64 << 10;
    if ((rc = alloc_(&d_stage_, stage_bytes_))) return rc;
    const size_t left = buf_bytes_ > align256(buf_off_) + 2048 ? buf_bytes_ - align256(buf_off_) - 2048 : 0;
    // per working cell: two rows of 16 bytes (the cell and what the unordered phase found for it),
    // under 1 byte of chunks and work items; the rest is the table
    chunk_cap_ = left / 64 / sizeof(Chunk);
    item_cap_ = left / 64 / sizeof(WorkItem);
    temp_cap_ = left * 10 / 32 / (2 * sizeof(MrlRow));
    row_cap_ = (left - 2 * (left / 64) - left * 10 / 32) / sizeof(MrlRow);
    if (item_cap_ < temp_cap_ / 32 + max_stage_ + 1) return too_large_();
    if (chunk_cap_ == 0 || row_cap_ == 0) return too_large_();
    h_ctl_ = &ctl_pageable_;
  } else {
    // Starting sizes from what fills of this kind ended with (about 45 table rows per Spec; 1000
    // working cells per Spec of the largest stage, of which a rank of a sharded fill sees its
    // share), each within a part of the free memory. The table gets the largest
    // part: enlarging it later needs the old and the new copy at once. A stage that needs more than
    // these reports what it needs and is run again with larger buffers.
    size_t free_b = 0, total_b = 0;
    CK(cudaMemGetInfo(&free_b, &total_b));
    const uint64_t shard = std::max<uint32_t>(1, plan.world);
    const uint64_t stage_part = ((uint64_t)max_stage_ * 3 / 2 + shard - 1) / shard;   // Specs of the largest stage a rank solves, with slack
    chunk_cap_ = std::max<uint64_t>(1u << 16, stage_part * 32);
    temp_cap_ = std::max<uint64_t>(1u << 20, std::min<uint64_t>(stage_part * 1000, free_b / 4 / (2 * sizeof(MrlRow))));
    row_cap_ = std::max<uint64_t>(1u << 20, std::min<uint64_t>((uint64_t)n_specs_ * 48, free_b / 2 / sizeof(MrlRow)));
    item_cap_ = temp_cap_ / 32 + max_stage_ + 1;   // a work item holds at least 32 cells, and every Spec at most one partial item
    if (!h_ctl_) CK(cudaHostAlloc((void**)&h_ctl_, sizeof(FillCtl), cudaHostAllocDefault));
  }
  if ((rc = alloc_((void**)&d_chunks_, chunk_cap_ * sizeof(Chunk)))) return rc;
  if ((rc = alloc_((void**)&d_items_, item_cap_ * sizeof(WorkItem)))) return rc;
  if ((rc = alloc_((void**)&d_temp_, temp_cap_ * 2 * sizeof(MrlRow)))) return rc;   // the cells, then what the unordered phase found for them
  if ((rc = alloc_((void**)&d_rows_, row_cap_ * sizeof(MrlRow)))) return rc;
  h2d_bytes_ = plan.hdrs.size() * sizeof(SpecHdr) + (skip_cands ? 0 : plan.cands.size() * sizeof(CandRec)) + plan.mine.size();
  CK(cudaMemsetAsync(d_ctl_, 0, 512, stream_));
  if (!plan.hdrs.empty())
    CK(cudaMemcpyAsync(d_hdrs_, plan.hdrs.data(), plan.hdrs.size() * sizeof(SpecHdr), cudaMemcpyHostToDevice, stream_));
  n_cand_bytes_ = plan.cands.size() * sizeof(CandRec);
  if (skip_cands) {
    if (n_cand_bytes_) CK(cudaMemsetAsync(d_cands_, 0, n_cand_bytes_, stream_));   // defined until the caller's records arrive
  } else {
    cands_present_ = true;
    if (!plan.cands.empty()) {
      // The candidate records are gigabytes of pageable memory and one host thread stages about
      // 11 GB/s, so four threads copy them on their own streams, piece by piece in id order, and
      // go on after this call has returned (wait_cands_).
      const size_t total = n_cand_bytes_;
      if (fixed_ || total < (size_t(1) << 30)) {
        CK(cudaMemcpyAsync(d_cands_, plan.cands.data(), total, cudaMemcpyHostToDevice, stream_));
      } else {
        up_piece_bytes_ = size_t(128) << 20;
        up_pieces_ = (total + up_piece_bytes_ - 1) / up_piece_bytes_;
        up_done_.reset(new std::atomic<uint8_t>[up_pieces_]);
        for (size_t k = 0; k < up_pieces_; k++) up_done_[k].store(0, std::memory_order_relaxed);
        up_next_ = 0;
        up_err_ = 0;
        up_ready_ = 0;
        const unsigned char* src = reinterpret_cast<const unsigned char*>(plan.cands.data());
        unsigned char* dst = reinterpret_cast<unsigned char*>(d_cands_);
        for (int t = 0; t < 4; t++)
          up_threads_.emplace_back([this, src, dst, total]() {
            // Each thread stages through two small pinned buffers of its own: the copy into them
            // is a plain memcpy outside the driver, and the transfer out of them is asynchronous,
            // so the thread that launches the fill's kernels is not held up behind driver-side
            // staging of pageable memory.
            const size_t sub = size_t(8) << 20;
            unsigned char* pin[2] = {nullptr, nullptr};
            cudaEvent_t ev[2] = {nullptr, nullptr};
            bool used[2] = {false, false};
            cudaError_t e = cudaSetDevice(device_);
            cudaStream_t st = nullptr;
            if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
            for (int b = 0; b < 2 && e == cudaSuccess; b++) {
              e = cudaHostAlloc((void**)&pin[b], sub, cudaHostAllocDefault);
              if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ev[b], cudaEventDisableTiming);
            }
            unsigned turn = 0;
            while (e == cudaSuccess && up_err_.load(std::memory_order_relaxed) == 0) {
              const size_t k = up_next_.fetch_add(1);
              if (k >= up_pieces_) break;
              const size_t lo = k * up_piece_bytes_, hi = std::min(total, lo + up_piece_bytes_);
              for (size_t off = lo; off < hi && e == cudaSuccess; off += sub, turn++) {
                const int b = turn & 1;
                const size_t len = std::min(sub, hi - off);
                if (used[b]) e = cudaEventSynchronize(ev[b]);   // the buffer's last transfer is done
                if (e != cudaSuccess) break;
                memcpy(pin[b], src + off, len);
                e = cudaMemcpyAsync(dst + off, pin[b], len, cudaMemcpyHostToDevice, st);
                if (e == cudaSuccess) e = cudaEventRecord(ev[b], st);
                used[b] = true;
              }
              if (e == cudaSuccess) e = cudaStreamSynchronize(st);
              if (e == cudaSuccess) up_done_[k].store(1, std::memory_order_release);
            }
            if (st) { cudaStreamSynchronize(st); cudaStreamDestroy(st); }
            for (int b = 0; b < 2; b++) {
              if (ev[b]) cudaEventDestroy(ev[b]);
              if (pin[b]) cudaFreeHost(pin[b]);
            }
            if (e != cudaSuccess) {
              int expect = 0;
              up_err_.compare_exchange_strong(expect, (int)e);
            }
          });
      }
    }
  }
  if (d_mine_) CK(cudaMemcpyAsync(d_mine_, plan.mine.data(), plan.mine.size(), cudaMemcpyHostToDevice, stream_));
  CK(cudaStreamSynchronize(stream_));
  stats_ = FillStats();
  return 0;
}

int DeviceFill::cands_arrived() {
  CK(cudaSetDevice(device_));
  if (cands_present_) return 0;
  if (n_specs_) {
    check_records_kernel<<<(n_specs_ + kBlock - 1) / kBlock, kBlock, 0, stream_>>>(d_hdrs_, d_cands_, n_specs_,
                                                                                   n_cand_bytes_ / sizeof(CandRec), &d_ctl_->error);
    CK(cudaGetLastError());
  }
  if (read_ctl_() != 0) return -1;
  if (h_ctl_->error) {
    CK(cudaMemsetAsync(&d_ctl_->error, 0, sizeof(uint32_t), stream_));
    snprintf(err_, sizeof(err_), "the candidate records on the device do not describe this plan (a field is out of range)");
    return -2;
  }
  cands_present_ = true;
  return 0;
}

int DeviceFill::read_ctl_() {
  CK(cudaMemcpyAsync(h_ctl_, d_ctl_, sizeof(FillCtl), cudaMemcpyDeviceToHost, stream_));
  CK(cudaStreamSynchronize(stream_));
  return 0;
}

// After a stage asked for more room than a buffer had: enlarges what it named. Working buffers
// hold nothing worth keeping between stages; the rows placed so far move along.
int DeviceFill::grow_after_error_(uint32_t bits) {
  if (fixed_) return too_large_();
  stats_.growths++;
  CK(cudaStreamSynchronize(stream_));
  auto regrow = [&](void** p, uint64_t* cap, uint64_t need, size_t elem) -> int {
    if (need <= *cap) return 0;
    cudaFree(*p);
    *p = nullptr;
    *cap = 0;
    const uint64_t want = need + need / 4;
    int rc = alloc_(p, want * elem);
    if (rc) return rc;
    *cap = want;
    return 0;
  };
  int rc;
  if (bits & MRL_ERR_WORKING) {
    if ((rc = regrow((void**)&d_temp_, &temp_cap_, h_ctl_->need_temp, 2 * sizeof(MrlRow)))) return rc;
    if ((rc = regrow((void**)&d_chunks_, &chunk_cap_, h_ctl_->need_chunks, sizeof(Chunk)))) return rc;
    if ((rc = regrow((void**)&d_items_, &item_cap_, h_ctl_->need_items, sizeof(WorkItem)))) return rc;
  }
  if (bits & MRL_ERR_TABLE) {
    const uint64_t need = h_ctl_->need_rows;
    size_t free_b = 0, total_b = 0;
    CK(cudaMemGetInfo(&free_b, &total_b));
    uint64_t cap = std::max<uint64_t>(need + need / 8, row_cap_ * 2);
    if (cap * sizeof(MrlRow) + (1ull << 30) > free_b) cap = need + need / 16;
    MrlRow* nr = nullptr;
    if ((rc = alloc_((void**)&nr, cap * sizeof(MrlRow)))) {
      snprintf(err_, sizeof(err_), "out of device memory: the table needs %llu rows", (unsigned long long)need);
      return -6;
    }
    if (h_ctl_->final_top) CK(cudaMemcpyAsync(nr, d_rows_, h_ctl_->final_top * sizeof(MrlRow), cudaMemcpyDeviceToDevice, stream_));
    CK(cudaStreamSynchronize(stream_));
    cudaFree(d_rows_);
    d_rows_ = nr;
    row_cap_ = cap;
  }
  return 0;
}

int DeviceFill::begin_fill() {
  CK(cudaSetDevice(device_));
  if (!cands_present_) {
    snprintf(err_, sizeof(err_), "the candidate records are not on the device yet (mrl_device_cands hands out the buffer; "
             "mrl_cands_arrived checks what was written)");
    return -3;
  }
  stats_ = FillStats();
  CK(cudaMemsetAsync(d_ctl_, 0, 512, stream_));
  CK(cudaEventRecord(ev0_, stream_));
  filling_ = true;
  return 0;
}

int DeviceFill::launch_solve_(const Plan& plan, uint32_t si, bool place_too) {
  const Stage& st = plan.stages[si];
  const uint32_t n = st.spec_hi - st.spec_lo;
  if (n == 0) return 0;
  {
    // the stage reads its own Specs' candidate records (ids, and with them the records, are in
    // stage order): wait for that much of a background upload
    const SpecHdr& last = plan.hdrs[st.spec_hi - 1];
    int rc = wait_cands_(((uint64_t)last.cand_off + last.ncand) * sizeof(CandRec));
    if (rc) return rc;
  }
  StageArgs a;
  a.hdrs = d_hdrs_; a.cands = d_cands_; a.rmask = d_rmask_; a.mine = d_mine_; a.dirty = d_dirty_;
  a.chunks = d_chunks_; a.items = d_items_; a.rows = d_rows_; a.temp = d_temp_; a.base = d_temp_ + temp_cap_; a.ehdr = d_ehdr_;
  a.fcount = d_fcount_; a.block_sums = d_block_sums_; a.minsat = d_minsat_; a.corner = d_corner_; a.stamp = d_stamp_; a.ctl = d_ctl_;
  a.lo = st.spec_lo; a.hi = st.spec_hi; a.top_pack = plan.top_pack(); a.stage = si;
  a.prev_lo = si ? plan.stages[si - 1].spec_lo : 0; a.prev_hi = si ? plan.stages[si - 1].spec_hi : 0;
  a.temp_cap = temp_cap_; a.chunk_cap = chunk_cap_; a.item_cap = item_cap_; a.row_cap = row_cap_;
  a.solve = 1;
  a.place = place_too ? 1 : 0;
  // Small stages run on fewer blocks: a grid-wide barrier costs less, and there is no work for more.
  const uint64_t want = ((uint64_t)n * 24 + kBlock - 1) / kBlock;
  const int blocks = (int)std::min<uint64_t>((uint64_t)coop_blocks_, std::max<uint64_t>((uint64_t)n_sm_, want));
  void* args[] = {&a};
  CK(cudaLaunchCooperativeKernel((const void*)stage_kernel, dim3(blocks), dim3(kBlock), args, 0, stream_));
  stats_.launches++;
  return 0;
}

int DeviceFill::launch_place_(const Plan& plan, uint32_t si) {
  const Stage& st = plan.stages[si];
  const uint32_t n = st.spec_hi - st.spec_lo;
  if (n == 0) return 0;
  StageArgs a;
  a.hdrs = d_hdrs_; a.cands = d_cands_; a.rmask = d_rmask_; a.mine = d_mine_; a.dirty = d_dirty_;
  a.chunks = d_chunks_; a.items = d_items_; a.rows = d_rows_; a.temp = d_temp_; a.base = d_temp_ + temp_cap_; a.ehdr = d_ehdr_;
  a.fcount = d_fcount_; a.block_sums = d_block_sums_; a.minsat = d_minsat_; a.corner = d_corner_; a.stamp = d_stamp_; a.ctl = d_ctl_;
  a.lo = st.spec_lo; a.hi = st.spec_hi; a.top_pack = plan.top_pack(); a.stage = si;
  a.prev_lo = si ? plan.stages[si - 1].spec_lo : 0; a.prev_hi = si ? plan.stages[si - 1].spec_hi : 0;
  a.temp_cap = temp_cap_; a.chunk_cap = chunk_cap_; a.item_cap = item_cap_; a.row_cap = row_cap_;
  a.solve = 0;
  a.place = 1;
  const uint64_t want = ((uint64_t)n + kBlock - 1) / kBlock;
  const int blocks = (int)std::min<uint64_t>((uint64_t)coop_blocks_, std::max<uint64_t>(1, want));
  void* args[] = {&a};
  CK(cudaLaunchCooperativeKernel((const void*)stage_kernel, dim3(blocks), dim3(kBlock), args, 0, stream_));
  stats_.launches++;
  return 0;
}

int DeviceFill::solve_stage(const Plan& plan, uint32_t si) {
  if (si >= plan.stages.size()) { snprintf(err_, sizeof(err_), "stage index out of range"); return -3; }
  if (!filling_) { snprintf(err_, sizeof(err_), "no fill in progress"); return -3; }
  return launch_solve_(plan, si, false);
}

static const char* kErrorBits = "(1: candidate record out of range, 2: working buffers too small, 4: row table too small, "
                                "8: no consistent limits grid)";

// Where the stage's real-breakpoint masks lie (what the ranks exchange before any of them places
// the stage). The masks must be final before they travel, so this is where a rank learns that its
// solve ran out of working room: it enlarges its own buffers and solves the stage again; the other
// ranks wait in the exchange.
int DeviceFill::stage_masks(const Plan& plan, uint32_t si, void** ptr, uint64_t* bytes) {
  if (si >= plan.stages.size()) { snprintf(err_, sizeof(err_), "stage index out of range"); return -3; }
  const Stage& st = plan.stages[si];
  if (filling_ && st.spec_hi != st.spec_lo) {
    int rc;
    if (read_ctl_() != 0) return -1;
    if (h_ctl_->error & MRL_ERR_WORKING) {
      const uint32_t bits = h_ctl_->error;
      if (bits & ~(uint32_t)(MRL_ERR_WORKING | MRL_ERR_TABLE)) {
        snprintf(err_, sizeof(err_), "a fill kernel reported error bits 0x%x in stage %u %s", bits, h_ctl_->failed_stage, kErrorBits);
        return -2;
      }
      if ((rc = grow_after_error_(MRL_ERR_WORKING))) return rc;
      CK(cudaMemsetAsync(&d_ctl_->error, 0, sizeof(uint32_t), stream_));
      if ((rc = launch_solve_(plan, si, false))) return rc;
      if (read_ctl_() != 0) return -1;
      if (h_ctl_->error) {
        snprintf(err_, sizeof(err_), "stage %u failed again after its working buffers were enlarged (0x%x)", si, h_ctl_->error);
        return -2;
      }
    }
  }
  if (ptr) *ptr = d_rmask_ + st.spec_lo;
  if (bytes) *bytes = (uint64_t)(st.spec_hi - st.spec_lo) * sizeof(uint4);
  return 0;
}

// Appends the stage's compacted grids to the table and reports where they went (the slice other
// ranks need), which costs the one synchronisation of the stage. A stage that ran out of room is
// run again here, whole, after its buffers have grown: its masks cannot have been exchanged yet.
int DeviceFill::place_stage(const Plan& plan, uint32_t si, void** rows_ptr, uint64_t* bytes) {
  if (si >= plan.stages.size()) { snprintf(err_, sizeof(err_), "stage index out of range"); return -3; }
  if (!filling_) { snprintf(err_, sizeof(err_), "no fill in progress"); return -3; }
  if (rows_ptr) *rows_ptr = d_rows_;
  if (bytes) *bytes = 0;
  const Stage& st = plan.stages[si];
  if (st.spec_hi == st.spec_lo) return 0;
  int rc;
  if ((rc = launch_place_(plan, si))) return rc;
  if (read_ctl_() != 0) return -1;
  if (h_ctl_->error) {
    const uint32_t bits = h_ctl_->error;
    if (bits & MRL_ERR_WORKING) {
      snprintf(err_, sizeof(err_), "stage %u needs larger working buffers than a sharded fill starts with "
               "(%llu working rows); fill once unsharded, or with fewer Specs per stage", si,
               (unsigned long long)h_ctl_->need_temp);
      return -6;
    }
    if (bits & ~(uint32_t)MRL_ERR_TABLE) {
      snprintf(err_, sizeof(err_), "a fill kernel reported error bits 0x%x in stage %u %s", bits, h_ctl_->failed_stage, kErrorBits);
      return -2;
    }
    if ((rc = grow_after_error_(bits))) return rc;
    CK(cudaMemsetAsync(&d_ctl_->error, 0, sizeof(uint32_t), stream_));
    if ((rc = launch_place_(plan, si))) return rc;
    if (read_ctl_() != 0) return -1;
    if (h_ctl_->error) { snprintf(err_, sizeof(err_), "stage %u failed again after its buffers were enlarged (0x%x)", si, h_ctl_->error); return -2; }
  }
  if (rows_ptr) *rows_ptr = d_rows_ + h_ctl_->stage_first_row;
  if (bytes) *bytes = h_ctl_->stage_rows * sizeof(MrlRow);
  return 0;
}

void DeviceFill::take_stats_() {
  const FillCtl& c = *h_ctl_;
  stats_.n_rows = c.final_top;
  stats_.cells_solved = c.st_cells;
  stats_.cands_evaluated = c.st_cands;
  stats_.lookups = c.st_lookups;
  stats_.alg_bytes = c.st_final_bytes;
  stats_.passes = c.st_passes;
  stats_.grid_syncs = c.st_syncs;
  stats_.sweeps = c.st_sweeps;
  stats_.early_cells = c.st_early_cells;
  stats_.late_cands = c.st_late_cands;
  stats_.late_items = c.st_late_items;
  for (int k = 0; k < 8; k++) stats_.phase_ms[k] = (float)(c.st_phase_ns[k] * 1e-6);
  stats_.early_ms = stats_.phase_ms[MRL_PH_EARLY];
  stats_.combine_ms = stats_.early_ms + stats_.phase_ms[MRL_PH_INIT] + stats_.phase_ms[MRL_PH_SWEEP_FIRST] + stats_.phase_ms[MRL_PH_SWEEP_MORE];
}

int DeviceFill::end_fill() {
  CK(cudaEventRecord(ev1_, stream_));
  if (read_ctl_() != 0) return -1;
  filling_ = false;
  CK(cudaEventElapsedTime(&stats_.fill_ms, ev0_, ev1_));
  take_stats_();
  if (h_ctl_->error) {
    snprintf(err_, sizeof(err_), "a fill kernel reported error bits 0x%x in stage %u %s", h_ctl_->error, h_ctl_->failed_stage, kErrorBits);
    return -2;
  }
  return 0;
}

// Every stage is enqueued without waiting for the one before: sizes, pass counts and launch
// geometry are all decided on the device. A stage that runs out of room raises an error word
// that turns the stages behind it into no-ops; the host then enlarges the buffers it named and
// resumes from that stage.
int DeviceFill::run(const Plan& plan) {
  int rc;
  if ((rc = begin_fill())) return rc;
  uint32_t from = 0;
  for (int attempt = 0;; attempt++) {
    for (uint32_t s = from; s < plan.stages.size(); s++)
      if ((rc = launch_solve_(plan, s, true))) return rc;
    CK(cudaEventRecord(ev1_, stream_));
    if (read_ctl_() != 0) return -1;
    const uint32_t bits = h_ctl_->error;
    if (!bits) break;
    if ((bits & ~(uint32_t)(MRL_ERR_WORKING | MRL_ERR_TABLE)) || attempt >= 64) {
      filling_ = false;
      take_stats_();
      snprintf(err_, sizeof(err_), "a fill kernel reported error bits 0x%x in stage %u %s", bits, h_ctl_->failed_stage, kErrorBits);
      return -2;
    }
    from = h_ctl_->failed_stage;
    if ((rc = grow_after_error_(bits))) { filling_ = false; return rc; }
    CK(cudaMemsetAsync(&d_ctl_->error, 0, sizeof(uint32_t), stream_));
  }
  filling_ = false;
  CK(cudaEventElapsedTime(&stats_.fill_ms, ev0_, ev1_));
  take_stats_();
  return 0;
}

int DeviceFill::lookup(const uint32_t* spec_ids, const uint32_t* cpacks, size_t n, MrlRow* out) {
  std::lock_guard<std::mutex> guard(lookup_mu_);   // callers on several threads share the staging buffer and the stream
  CK(cudaSetDevice(device_));
  if (n == 0) return 0;
  for (size_t i = 0; i < n; i++)
    if (spec_ids[i] >= n_specs_) { snprintf(err_, sizeof(err_), "Spec id out of range"); return -3; }
  const size_t per = sizeof(uint2) + sizeof(MrlRow);
  size_t batch = std::min<size_t>(n, size_t(1) << 22);
  if (fixed_) batch = std::min(n, stage_bytes_ / 2 / per);
  else if (stage_bytes_ < 2 * align256(batch * sizeof(MrlRow))) {
    CK(cudaStreamSynchronize(stream_));
    if (d_stage_) cudaFree(d_stage_);
    d_stage_ = nullptr;
    stage_bytes_ = 0;
    int rc = alloc_(&d_stage_, 2 * align256(batch * sizeof(MrlRow)));
    if (rc) return rc;
    stage_bytes_ = 2 * align256(batch * sizeof(MrlRow));
  }
  if (batch == 0) { snprintf(err_, sizeof(err_), "lookup staging too small"); return -5; }
  std::vector<uint2> q(batch);
  for (size_t done = 0; done < n; done += batch) {
    const size_t m = std::min(batch, n - done);
    for (size_t i = 0; i < m; i++) q[i] = make_uint2(spec_ids[done + i], cpacks[done + i]);
    uint2* d_q = static_cast<uint2*>(d_stage_);
    MrlRow* d_out = reinterpret_cast<MrlRow*>(static_cast<unsigned char*>(d_stage_) + stage_bytes_ / 2);
    CK(cudaMemcpyAsync(d_q, q.data(), m * sizeof(uint2), cudaMemcpyHostToDevice, stream_));
    lookup_rows_kernel<<<(unsigned)((m + 255) / 256), 256, 0, stream_>>>(d_hdrs_, d_rows_, d_q, m, d_out);
    CK(cudaGetLastError());
    CK(cudaMemcpyAsync(out + done, d_out, m * sizeof(MrlRow), cudaMemcpyDeviceToHost, stream_));
    CK(cudaStreamSynchronize(stream_));
  }
  return 0;
}

// Checks the finished table against its defining recurrence at n_samples pseudo-random points of
// (Spec x limits lattice), or at every point when n_samples == 0.
int DeviceFill::verify(const Plan& plan, uint64_t n_samples, uint64_t seed, uint64_t* checked, uint64_t* mismatches,
                       uint64_t* first_bad) {
  CK(cudaSetDevice(device_));
  if (wait_upload()) return -1;
  const uint32_t top = plan.top_pack();
  unsigned long long per_spec = 1;
  for (int k = 0; k < 4; k++) per_spec *= ((top >> (8 * k)) & 0xFFu) + 1u;
  const unsigned long long total = per_spec * n_specs_;
  const bool exhaustive = n_samples == 0;
  const unsigned long long count = exhaustive ? total : n_samples;
  unsigned long long* d_out = d_ctl_->scratch;
  const unsigned long long init[2] = {0ull, ~0ull};
  CK(cudaMemcpyAsync(d_out, init, sizeof(init), cudaMemcpyHostToDevice, stream_));
  CK(cudaStreamSynchronize(stream_));
  const unsigned long long batch = 1ull << 28;
  for (unsigned long long first = 0; first < count && total; first += batch) {
    const unsigned long long n = std::min(batch, count - first);
    verify_points_kernel<<<(unsigned)((n + kBlock - 1) / kBlock), kBlock, 0, stream_>>>(d_hdrs_, d_cands_, d_rows_, n_specs_, top, first, n,
                                                                                       total, seed, exhaustive ? 1 : 0, d_out);
    CK(cudaGetLastError());
  }
  unsigned long long res[2] = {0, 0};
  CK(cudaMemcpyAsync(res, d_out, sizeof(res), cudaMemcpyDeviceToHost, stream_));
  CK(cudaStreamSynchronize(stream_));
  if (checked) *checked = total ? count : 0;
  if (mismatches) *mismatches = res[0];
  if (first_bad) *first_bad = res[1];
  return 0;
}

int DeviceFill::checksum(uint64_t* out) {
  CK(cudaSetDevice(device_));
  unsigned long long* d_out = d_ctl_->scratch + 2;
  CK(cudaMemsetAsync(d_out, 0, sizeof(unsigned long long), stream_));
  if (n_specs_) {
    checksum_kernel<<<(n_specs_ + kBlock - 1) / kBlock, kBlock, 0, stream_>>>(d_hdrs_, d_rows_, n_specs_, d_out);
    CK(cudaGetLastError());
  }
  unsigned long long v = 0;
  CK(cudaMemcpyAsync(&v, d_out, sizeof(v), cudaMemcpyDeviceToHost, stream_));
  CK(cudaStreamSynchronize(stream_));
  *out = v;
  return 0;
}

int DeviceFill::read_table(SpecHdr* hdrs_out, MrlRow* rows_out) {
  CK(cudaSetDevice(device_));
  if (n_specs_) CK(cudaMemcpyAsync(hdrs_out, d_hdrs_, (size_t)n_specs_ * sizeof(SpecHdr), cudaMemcpyDeviceToHost, stream_));
  if (stats_.n_rows) CK(cudaMemcpyAsync(rows_out, d_rows_, stats_.n_rows * sizeof(MrlRow), cudaMemcpyDeviceToHost, stream_));
  CK(cudaStreamSynchronize(stream_));
  return 0;
}

int DeviceFill::load_table(const Plan& plan, const SpecHdr* hdrs, const MrlRow* rows, uint64_t n_rows) {
  CK(cudaSetDevice(device_));
  if (plan.hdrs.size() != n_specs_) { snprintf(err_, sizeof(err_), "the saved table belongs to another plan"); return -3; }
  if (n_rows > row_cap_) {
    if (fixed_) return too_large_();
    CK(cudaStreamSynchronize(stream_));
    cudaFree(d_rows_);
    d_rows_ = nullptr;
    row_cap_ = 0;
    int rc = alloc_((void**)&d_rows_, n_rows * sizeof(MrlRow));
    if (rc) return rc;
    row_cap_ = n_rows;
  }
  if (n_specs_) CK(cudaMemcpyAsync(d_hdrs_, hdrs, (size_t)n_specs_ * sizeof(SpecHdr), cudaMemcpyHostToDevice, stream_));
  if (n_rows) CK(cudaMemcpyAsync(d_rows_, rows, n_rows * sizeof(MrlRow), cudaMemcpyHostToDevice, stream_));
  CK(cudaStreamSynchronize(stream_));
  stats_ = FillStats();
  stats_.n_rows = n_rows;
  return 0;
}

int DeviceFill::read_hdr(uint32_t spec, SpecHdr* out) {
  CK(cudaSetDevice(device_));
  if (spec >= n_specs_) { snprintf(err_, sizeof(err_), "Spec id out of range"); return -3; }
  CK(cudaMemcpyAsync(out, d_hdrs_ + spec, sizeof(SpecHdr), cudaMemcpyDeviceToHost, stream_));
  CK(cudaStreamSynchronize(stream_));
  return 0;
}

int DeviceFill::read_rows(uint64_t first, uint64_t n, MrlRow* out) {
  CK(cudaSetDevice(device_));
  if (first + n > stats_.n_rows) { snprintf(err_, sizeof(err_), "row range out of the table"); return -3; }
  if (n == 0) return 0;
  CK(cudaMemcpyAsync(out, d_rows_ + first, n * sizeof(MrlRow), cudaMemcpyDeviceToHost, stream_));
  CK(cudaStreamSynchronize(stream_));
  return 0;
}

// ---------------------------------------------------------------------------------------
// Fill without device allocation.
//
// Some callers of this library must not allocate device memory while they run: a host that
// reserved all of HBM for its replicated tables at start-up has nothing left to hand out, and
// a worker pool that calls top_down_many from many threads would be serialised by the
// device-wide synchronisation every cudaMalloc / cudaFree implies. For them the whole device
// working set of one small fill - plan arrays, working buffers, row table, lookup staging - is
// carved out of the fixed array below instead of being allocated per call. Every GPU that
// loads this library holds the array until the process exits.
//
// In host code `g_static_scratch` is only a stand-in for the device array, not a device
// address; the address a kernel may use comes from cudaGetSymbolAddress, asked once per
// device with that device current (static_scratch_address).
namespace {
__device__ __align__(256) unsigned char g_static_scratch[MRL_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mu;

// Device address of the static array on `device`, resolved on first use. The caller's current
// device is left as it was.
cudaError_t static_scratch_address(int device, void** out) {
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> g(g_scratch_mu);
  if (!g_scratch_addr[device]) {
    int before = -1;
    cudaError_t e = cudaGetDevice(&before);
    if (e != cudaSuccess) return e;
    e = cudaSetDevice(device);
    if (e != cudaSuccess) return e;
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (before != device) cudaSetDevice(before);
    if (e != cudaSuccess) return e;
    g_scratch_addr[device] = p;
  }
  *out = g_scratch_addr[device];
  return cudaSuccess;
}
}  // namespace

// Runs `plan` entirely inside the static array and copies the rows of the given (Spec id,
// packed limit codes) queries to `out` (host). No cudaMalloc / cudaFree. Returns -5 with a
// message when the fill does not fit.
int fill_static(int device, cudaStream_t stream, const Plan& plan, const uint32_t* spec_ids, const uint32_t* cpacks,
                size_t n, MrlRow* out, char* err, size_t err_len) {
  void* base = nullptr;
  cudaError_t e = static_scratch_address(device, &base);
  if (e == cudaSuccess) e = cudaSetDevice(device);
  if (e != cudaSuccess) {
    snprintf(err, err_len, "static scratch unavailable: %s", cudaGetErrorString(e));
    return -1;
  }
  DeviceFill f;
  f.attach_buffer(base, (size_t)MRL_STATIC_SCRATCH_BYTES, stream, device);
  int rc = f.init_events();
  if (rc == 0) rc = f.upload(plan);
  if (rc == 0) rc = f.run(plan);
  if (rc == 0) rc = f.lookup(spec_ids, cpacks, n, out);
  if (rc != 0) snprintf(err, err_len, "%s", f.error());
  return rc;
}

}  // namespace mrl

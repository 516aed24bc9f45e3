// The CUDA side of the synthesis-database fill (sm_100a).
//
// Specs are processed stage by stage (plan.hpp). For one stage the device
//   1. derives each Spec's working limits grid: per memory the lattice codes at which its
//      result can change - thresholds of its own candidates plus the (shifted) breakpoints of
//      the finished tables of its children (derive_masks_kernel; totals_kernel, place_kernel);
//   2. lists the working cells by limits diagonal (diag_histogram_kernel, scatter_cells_kernel)
//      and solves them directly, one launch per occupied diagonal (combine_argmin_kernel): a
//      thread (or 4, 8, 32 lanes in small launches) takes one cell, walks the Spec's candidate
//      records, gathers the child rows each candidate needs at the child's limits, combines
//      them into a Cost and keeps the lexicographic minimum;
//   3. finds which breakpoints are real - some pair of neighbouring cells differs
//      (real_masks_kernel) - and repeats 1-3 for the Specs whose grid still lacks a breakpoint
//      that a same-stage child turned out to have, and for the Specs above them
//      (spread_dirty_kernel); relayout Moves are the only same-stage dependency;
//   4. compacts the working grids to the real breakpoints and appends them to the table
//      (final_count_kernel, scan_block_sums_kernel, compact_kernel).
// Step 3's fixpoint is exact: when every Spec's grid contains all thresholds and all shifted
// breakpoints of the computed tables of its children, induction over the limits lattice shows
// every computed cell equals the direct solve at every limit inside the cell.
//
// What the combine replaces in the reference (paths inside the Morello repository):
//   morello/src/scheduling/mod.rs:286-368     ActionSolver::compute_cost
//   morello/src/imp/loops.rs:207-242          loop main cost (serial, no boundary regions)
//   morello/src/memorylimits.rs:159-224,409-470  peak propagation, limit subtraction
//   morello/src/scheduling/select.rs:34-47    kernel-allocation feasibility
//   morello/src/search/reducer.rs:40-99       argmin on (Cost, ActionNum)
//   morello/src/db/pagecontents.rs:103-123    child lookup (here: an index computation)
// Integer-only work bounded by HBM/L2 bandwidth; no tensor cores.
#include "device_types.h"
#include "fill.hpp"
#include <cuda_runtime.h>
#include <cuda_profiler_api.h>
#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include <chrono>
#include <mutex>
#include <thread>

#ifndef MRL_MIN_BLOCKS
#define MRL_MIN_BLOCKS 12
#endif

namespace {

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

struct Key {
  uint32_t main, peaks, tail;
};
__device__ __forceinline__ bool key_less(const Key& a, const Key& b) {
  if (a.main != b.main) return a.main < b.main;
  if (a.peaks != b.peaks) return a.peaks < b.peaks;
  return a.tail < b.tail;
}

// Row of a child Spec at given limits: the cell whose breakpoints are the largest ones not
// above the limits. b_k = mask of the codes <= the limit's code in memory k. One 32-byte
// header (two loads) and one 16-byte row.
// Row `base` of the table: bit 63 set = a working row of the stage being solved (temp buffer).
#define MRL_TEMP_FLAG (1ull << 63)
__device__ __forceinline__ const MrlRow* row_at(const MrlRow* rows, const MrlRow* temp, unsigned long long base) {
  return ((base & MRL_TEMP_FLAG) ? temp : rows) + (base & ~MRL_TEMP_FLAG);
}

__device__ __forceinline__ uint4 lookup(const SpecHdr* __restrict__ hdrs, const MrlRow* __restrict__ rows,
                                        const MrlRow* __restrict__ temp, uint32_t child, uint32_t b0, uint32_t b1,
                                        uint32_t b2, uint32_t b3) {
  const uint4 m = __ldg(reinterpret_cast<const uint4*>(&hdrs[child]));
  const unsigned long long base = __ldg(reinterpret_cast<const unsigned long long*>(&hdrs[child].row_base));
  const uint32_t i0 = __popc(m.x & b0) - 1;
  const uint32_t i1 = __popc(m.y & b1) - 1;
  const uint32_t i2 = __popc(m.z & b2) - 1;
  const uint32_t i3 = __popc(m.w & b3) - 1;
  const uint32_t off = ((i3 * __popc(m.z) + i2) * __popc(m.y) + i1) * __popc(m.x) + i0;  // cells per Spec < 2^32
  // Rows read here were written by earlier launches (lower diagonal or earlier stage), never by
  // this one, so the read-only path is safe.
  return __ldg(reinterpret_cast<const uint4*>(row_at(rows, temp, base) + off));
}

// Geometry of one thread's column. A column fixes the slot index in the three memories other
// than the Spec's free memory F.
struct Column {
  uint32_t spec, F;
  uint32_t mm[4], nn[4], idx[4], code[4];
  uint32_t others;  // sum of the codes of the fixed memories
  bool valid;
};
__device__ __forceinline__ Column decode_column(const SpecHdr* __restrict__ hdrs, const Chunk ch, uint32_t lane) {
  Column c;
  c.spec = ch.spec;
  c.F = ch.col_start >> 30;
  const uint4 m = __ldg(reinterpret_cast<const uint4*>(&hdrs[ch.spec]));
  c.mm[0] = m.x; c.mm[1] = m.y; c.mm[2] = m.z; c.mm[3] = m.w;
  uint32_t rest = (ch.col_start & 0x3FFFFFFFu) + lane;
  c.others = 0;
#pragma unroll
  for (int k = 0; k < 4; k++) {
    c.nn[k] = (uint32_t)__popc(c.mm[k]);
    const uint32_t nk = ((uint32_t)k == c.F) ? 1u : c.nn[k];
    c.idx[k] = rest % nk;
    rest /= nk;
    c.code[k] = nth_set_bit(c.mm[k], c.idx[k]);  // for F: slot 0, code 0
    c.others += c.code[k];
  }
  c.valid = rest == 0;  // false: column index beyond this Spec's grid
  return c;
}

// The direct solve of one (Spec, limits) point from the tables of the Spec's children: walks the
// candidate records, applies the limits-dependent feasibility tests, gathers the child rows at
// the children's limits, combines them and keeps the lexicographic minimum. cpack = the limits
// as lattice codes (RF in byte 0 .. GL in byte 3).
__device__ __forceinline__ Key solve_point(const SpecHdr* __restrict__ hdrs, const CandRec* __restrict__ cands,
                                           const MrlRow* __restrict__ rows, const MrlRow* __restrict__ temp,
                                           uint32_t spec, uint32_t cpack, uint32_t n_specs,
                                           uint32_t* __restrict__ error_flag, uint32_t first_cand = 0,
                                           uint32_t cand_stride = 1) {
  // "codes at or below this point's limit", per memory: what a child lookup at the same limits needs
  const uint32_t bm0 = (2u << code_of(cpack, 0)) - 1u, bm1 = (2u << code_of(cpack, 1)) - 1u,
                 bm2 = (2u << code_of(cpack, 2)) - 1u, bm3 = (2u << code_of(cpack, 3)) - 1u;
  const uint2 cl = __ldg(reinterpret_cast<const uint2*>(&hdrs[spec].cand_off));
  const uint32_t cand_off = cl.x, ncand = cl.y;

  Key best = {MRL_UNSAT, MRL_UNSAT, MRL_UNSAT};
  for (uint32_t ci = first_cand; ci < ncand; ci += cand_stride) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(&cands[cand_off + ci]));
    const uint32_t action = a.x & 0xFFFFu, kind = (a.x >> 16) & 0xFFu, nchild = a.x >> 24;
    const uint32_t imm = a.y;
    const uint32_t level = a.z & 0xFFu, thr = (a.z >> 8) & 0xFFu, pcode = (a.z >> 16) & 0xFFu;
    const uint32_t units = a.w;
    const uint32_t lv = code_of(cpack, level);  // the cell's limit in `level`
    Key k;
    if (kind == MRL_CK_LEAF) {
      if (lv < thr) continue;
      k.main = imm;
      k.peaks = pcode << peak_shift(level);
      k.tail = (1u << 16) | action;
    } else {
      const uint4 b = __ldg(reinterpret_cast<const uint4*>(&cands[cand_off + ci]) + 1);
      uint32_t c0 = bm0, c1 = bm1, c2 = bm2, c3 = bm3;
      const uint32_t sh = peak_shift(level);
      if (kind == MRL_CK_MOVE) {
        if (lv < thr) continue;
        // Branch and bound: a Move costs at least its own base cost. Candidates are stored
        // cheapest-first (kernels, loops, then Moves by base cost), so most Moves end here.
        if (imm > best.main) continue;
        uint32_t ccode;
        if (level < 2) ccode = lv - units;                      // registers: exact
        else ccode = 32 - __clz(cache_value(lv) - units);       // caches: snap down to 2^k
        const uint32_t cb = (2u << ccode) - 1u;
        c0 = (level == 0) ? cb : c0;
        c1 = (level == 1) ? cb : c1;
        c2 = (level == 2) ? cb : c2;
        c3 = (level == 3) ? cb : c3;
      }
#ifdef MRL_CHECK_CHILD_IDS
      if (b.x >= n_specs || (nchild > 1 && b.y >= n_specs) || (nchild > 2 && b.z >= n_specs)) {
        if (error_flag) atomicExch(error_flag, 1u);
        continue;
      }
#endif
      // Children one at a time: a child without an implementation, or a partial sum that already
      // exceeds the best main cost, ends the candidate before the remaining rows are fetched.
      const uint4 r0 = lookup(hdrs, rows, temp, b.x, c0, c1, c2, c3);
      if (r0.z == MRL_UNSAT) continue;
      uint4 r1 = r0, r2 = r0;
      if (nchild > 1) {
        if (kind == MRL_CK_MOVE && sat_add(imm, r0.x) > best.main) continue;
        r1 = lookup(hdrs, rows, temp, b.y, c0, c1, c2, c3);
        if (r1.z == MRL_UNSAT) continue;
        if (nchild > 2) {
          r2 = lookup(hdrs, rows, temp, b.z, c0, c1, c2, c3);
          if (r2.z == MRL_UNSAT) continue;
        }
      }
      uint32_t main, peaks, depth;
      if (kind == MRL_CK_LOOP) {
        main = sat_mul(r0.x, imm);
        peaks = r0.y;
        depth = 1u;  // a single-body tile loop has depth 1 whatever its body's depth
      } else {
        main = (kind == MRL_CK_MOVE) ? sat_add(imm, r0.x) : r0.x;
        if (nchild > 1) main = sat_add(main, r1.x);
        if (nchild > 2) main = sat_add(main, r2.x);
        peaks = __vmaxu4(__vmaxu4(r0.y, r1.y), r2.y);
        if (kind == MRL_CK_MOVE) {
          // own allocation sits on top of the deepest child's peak in `level`; rounding to the
          // lattice is monotone, so max-then-round equals the reference's round-per-child
          const uint32_t child_code = (peaks >> sh) & 0xFFu;
          uint32_t ncode;
          if (level < 2) ncode = units + child_code;
          else ncode = cache_code_ceil(units + cache_value(child_code));
          peaks = (peaks & ~(0xFFu << sh)) | (ncode << sh);
        }
        depth = min(max(max(r0.z >> 16, r1.z >> 16), r2.z >> 16) + 1u, 255u);
      }
      k.main = main;
      k.peaks = peaks;
      k.tail = (depth << 16) | action;
    }
    if (key_less(k, best)) best = k;
  }
  return best;
}

// One launch = the cells of one stage that lie on one limits diagonal (sum of the four codes),
// listed by scatter_cells_kernel: every thread has a cell, and neighbouring threads mostly have
// neighbouring cells of one Spec. G = lanes per cell. A launch with few cells cannot fill the
// GPU and lasts as long as one cell's chain of dependent loads (tens of microseconds with ~30
// candidates); there the G lanes of a cell take every G-th candidate each and min-reduce their
// keys with shuffles, which shortens the chain G-fold. Large launches use G = 1, which keeps the
// lower-bound cut across all candidates of a cell.
template <int G>
__global__ void __launch_bounds__(128, MRL_MIN_BLOCKS)
combine_argmin_kernel(const SpecHdr* __restrict__ hdrs, const CandRec* __restrict__ cands,
                      const CellRef* __restrict__ cells, uint32_t n_cells,
                      const MrlRow* __restrict__ rows, MrlRow* __restrict__ temp, uint32_t n_specs,
                      uint32_t* __restrict__ error_flag) {
  const uint32_t t = (blockIdx.x * blockDim.x + threadIdx.x) / G;
  const uint32_t sub = threadIdx.x % G;
  const bool valid = t < n_cells;   // the G lanes of a cell agree; no lane leaves before the shuffles
  Key best = {MRL_UNSAT, MRL_UNSAT, MRL_UNSAT};
  CellRef ref;
  ref.spec = 0;
  ref.cpack = 0;
  uint32_t cell = 0;
  unsigned long long base = 0;
  if (valid) {
    ref = cells[t];
    // the cell's place in its Spec's working grid: slot = breakpoints at or below the code, minus one
    const uint4 m = __ldg(reinterpret_cast<const uint4*>(&hdrs[ref.spec]));
    const uint32_t i0 = __popc(m.x & ((2u << code_of(ref.cpack, 0)) - 1u)) - 1;
    const uint32_t i1 = __popc(m.y & ((2u << code_of(ref.cpack, 1)) - 1u)) - 1;
    const uint32_t i2 = __popc(m.z & ((2u << code_of(ref.cpack, 2)) - 1u)) - 1;
    const uint32_t i3 = __popc(m.w & ((2u << code_of(ref.cpack, 3)) - 1u)) - 1;
    cell = ((i3 * __popc(m.z) + i2) * __popc(m.y) + i1) * __popc(m.x) + i0;
    base = __ldg(reinterpret_cast<const unsigned long long*>(&hdrs[ref.spec].row_base));
    best = solve_point(hdrs, cands, rows, temp, ref.spec, ref.cpack, n_specs, error_flag, sub, G);
  }
  if (G > 1) {
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) {
      Key other;
      other.main = __shfl_xor_sync(0xFFFFFFFFu, best.main, o);
      other.peaks = __shfl_xor_sync(0xFFFFFFFFu, best.peaks, o);
      other.tail = __shfl_xor_sync(0xFFFFFFFFu, best.tail, o);
      if (key_less(other, best)) best = other;
    }
  }
  // Specs of the stage being solved always live in the working buffer.
  if (valid && sub == 0)
    *reinterpret_cast<uint4*>(temp + (base & ~MRL_TEMP_FLAG) + cell) = make_uint4(best.main, best.peaks, best.tail, 0u);
}

// Consistency check of a finished table: at sampled (or all) points of the limits lattice, for
// sampled (or all) Specs, the direct solve from the children's tables must equal what the Spec's
// own table returns there. Every point where that holds is a point where the table satisfies
// the defining recurrence of the fill, whatever grid the table is stored on.
__global__ void __launch_bounds__(128, MRL_MIN_BLOCKS)
verify_points_kernel(const SpecHdr* __restrict__ hdrs, const CandRec* __restrict__ cands,
                     const MrlRow* __restrict__ rows, uint32_t n_specs, uint32_t top_pack, unsigned long long first,
                     unsigned long long count, unsigned long long total_points, unsigned long long seed, int exhaustive,
                     unsigned long long* __restrict__ out /* [0] mismatches, [1] first bad sample + 1 */) {
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
  const Key k = solve_point(hdrs, cands, rows, rows, spec, cpack, n_specs, nullptr);
  const uint4 r = lookup(hdrs, rows, rows, spec, (2u << c0) - 1u, (2u << c1) - 1u, (2u << c2) - 1u, (2u << c3) - 1u);
  if (k.main != r.x || k.peaks != r.y || k.tail != r.z) {
    atomicAdd(&out[0], 1ull);
    atomicMin(&out[1], first + i);
  }
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
  // The free memory is the one with the most slots (lowest index on ties): a column then has
  // a cell on as many diagonals as possible.
  g.F = 0;
  uint32_t best = g.nn[0];
#pragma unroll
  for (int k = 1; k < 4; k++)
    if (g.nn[k] > best) { best = g.nn[k]; g.F = k; }
  g.cols = (uint32_t)(g.cells / best);
  g.warps = (g.cols + 31u) / 32u;
  return g;
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

// Pass step 1: per Spec of the stage, the masks its working grid needs. child_source says what
// is known about same-stage children: 0 = nothing (first pass: they are ignored), 1 = the
// breakpoints in rmask (found real by the previous pass; or, when seeding, the children's own
// first working masks). A Spec whose masks grew is marked dirty. seed_copy: also copy the new
// masks to rmask (so that a following launch can read them as the children's breakpoints).
__global__ void __launch_bounds__(128)
derive_masks_kernel(SpecHdr* __restrict__ hdrs, const CandRec* __restrict__ cands, uint4* __restrict__ rmask,
                    const uint8_t* __restrict__ mine, uint8_t* __restrict__ dirty, uint32_t lo, uint32_t hi,
                    int first, int child_source, int seed_copy, uint32_t top_pack) {
  const uint32_t i = lo + blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= hi || (mine && !mine[i])) return;
  const uint4 old = *reinterpret_cast<const uint4*>(&hdrs[i]);
  const uint2 cl = *reinterpret_cast<const uint2*>(&hdrs[i].cand_off);
  uint32_t r0 = 1, r1 = 1, r2 = 1, r3 = 1;
  for (uint32_t ci = 0; ci < cl.y; ci++) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(&cands[cl.x + ci]));
    const uint32_t kind = (a.x >> 16) & 0xFFu, nchild = a.x >> 24;
    const uint32_t level = a.z & 0xFFu, thr = (a.z >> 8) & 0xFFu, units = a.w;
    if (kind == MRL_CK_LEAF || kind == MRL_CK_MOVE) or_level(r0, r1, r2, r3, level, 1u << thr);
    if (kind == MRL_CK_LEAF) continue;
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(&cands[cl.x + ci]) + 1);
    for (uint32_t j = 0; j < nchild; j++) {
      const uint32_t child = j == 0 ? b.x : (j == 1 ? b.y : b.z);
      uint4 cm;
      if (child < lo) cm = *reinterpret_cast<const uint4*>(&hdrs[child]);   // finished stage: final masks
      else if (child_source == 0) continue;
      else cm = rmask[child];
      if (kind == MRL_CK_MOVE) {
        const uint32_t s = shift_mask(sel4(cm.x, cm.y, cm.z, cm.w, level), level, units, code_of(top_pack, level));
        r0 |= (level == 0) ? s : cm.x;
        r1 |= (level == 1) ? s : cm.y;
        r2 |= (level == 2) ? s : cm.z;
        r3 |= (level == 3) ? s : cm.w;
      } else {
        r0 |= cm.x; r1 |= cm.y; r2 |= cm.z; r3 |= cm.w;
      }
    }
  }
  const uint4 nm = first ? make_uint4(r0, r1, r2, r3) : make_uint4(old.x | r0, old.y | r1, old.z | r2, old.w | r3);
  const bool changed = first || nm.x != old.x || nm.y != old.y || nm.z != old.z || nm.w != old.w;
  if (changed) {
    *reinterpret_cast<uint4*>(&hdrs[i]) = nm;
    dirty[i] = 1;
  }
  if (seed_copy) rmask[i] = nm;
}

// A Spec with a dirty same-stage child has to be solved again too (its lookups may change).
// Monotone, so racing with other threads' marks is harmless; run until totals_kernel reports
// no unmarked Spec with a dirty child.
__global__ void __launch_bounds__(128)
spread_dirty_kernel(const SpecHdr* __restrict__ hdrs, const CandRec* __restrict__ cands,
                    const uint8_t* __restrict__ mine, uint8_t* __restrict__ dirty, uint32_t lo, uint32_t hi) {
  const uint32_t i = lo + blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= hi || (mine && !mine[i]) || dirty[i]) return;
  const uint2 cl = *reinterpret_cast<const uint2*>(&hdrs[i].cand_off);
  for (uint32_t ci = 0; ci < cl.y; ci++) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(&cands[cl.x + ci]));
    const uint32_t kind = (a.x >> 16) & 0xFFu, nchild = a.x >> 24;
    if (kind != MRL_CK_MOVE) continue;   // only Moves have same-stage children
    const uint4 b = __ldg(reinterpret_cast<const uint4*>(&cands[cl.x + ci]) + 1);
    for (uint32_t j = 0; j < nchild; j++) {
      const uint32_t child = j == 0 ? b.x : (j == 1 ? b.y : b.z);
      if (child >= lo && dirty[child]) { dirty[i] = 1; return; }
    }
  }
}

// Totals of what the coming solve takes (dirty Specs only), the working cells of the whole stage,
// and whether the dirty marks are closed under "has a dirty same-stage child".
__global__ void __launch_bounds__(128)
totals_kernel(const SpecHdr* __restrict__ hdrs, const CandRec* __restrict__ cands, const uint8_t* __restrict__ mine,
              uint8_t* __restrict__ dirty, uint32_t lo, uint32_t hi, PassCounters* __restrict__ ctr) {
  const uint32_t i = lo + blockIdx.x * blockDim.x + threadIdx.x;
  const bool active = i < hi && (!mine || mine[i]);
  unsigned long long cells = 0, warps = 0, bytes = 0, all_cells = 0;
  uint32_t open_marks = 0;
  if (active) {
    const uint4 nm = *reinterpret_cast<const uint4*>(&hdrs[i]);
    const uint2 cl = *reinterpret_cast<const uint2*>(&hdrs[i].cand_off);
    const Grid g = grid_of(nm);
    all_cells = g.cells;
    bool is_dirty = dirty[i] != 0;
    if (!is_dirty) {
      for (uint32_t ci = 0; ci < cl.y && !is_dirty; ci++) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(&cands[cl.x + ci]));
        const uint32_t kind = (a.x >> 16) & 0xFFu, nchild = a.x >> 24;
        if (kind != MRL_CK_MOVE) continue;
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(&cands[cl.x + ci]) + 1);
        for (uint32_t j = 0; j < nchild; j++) {
          const uint32_t child = j == 0 ? b.x : (j == 1 ? b.y : b.z);
          if (child >= lo && dirty[child]) is_dirty = true;
        }
      }
      if (is_dirty) { dirty[i] = 1; open_marks = 1; }
    }
    if (is_dirty) {
      cells = g.cells;
      warps = g.warps;
      // algorithmic bytes of one solve: a 12-byte row out; per candidate a 16-byte header; per
      // child of a candidate that fits the cell's limits a 4-byte index and a 12-byte row in
      bytes = cells * 12ull;
      for (uint32_t ci = 0; ci < cl.y; ci++) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(&cands[cl.x + ci]));
        const uint32_t kind = (a.x >> 16) & 0xFFu, nchild = a.x >> 24;
        const uint32_t level = a.z & 0xFFu, thr = (a.z >> 8) & 0xFFu;
        bytes += cells * 16ull;
        if (nchild) {
          unsigned long long feasible = cells;
          if (kind == MRL_CK_MOVE) {
            const uint32_t ml = sel4(nm.x, nm.y, nm.z, nm.w, level);
            feasible = cells / (uint32_t)__popc(ml) * (uint32_t)__popc(ml >> thr);
          }
          bytes += feasible * nchild * 16ull;
        }
      }
    }
  }
  // warp totals, then one atomic per warp and counter
  for (int o = 16; o > 0; o >>= 1) {
    cells += __shfl_xor_sync(0xFFFFFFFFu, cells, o);
    warps += __shfl_xor_sync(0xFFFFFFFFu, warps, o);
    bytes += __shfl_xor_sync(0xFFFFFFFFu, bytes, o);
    all_cells += __shfl_xor_sync(0xFFFFFFFFu, all_cells, o);
  }
  open_marks = __reduce_or_sync(0xFFFFFFFFu, open_marks);
  if ((threadIdx.x & 31) == 0) {
    if (cells) {
      atomicAdd(&ctr->cells, cells);
      atomicAdd(&ctr->warps, warps);
      atomicAdd(&ctr->alg_bytes, bytes);
    }
    if (all_cells) atomicAdd(&ctr->all_cells, all_cells);
    if (open_marks) atomicOr(&ctr->changed, 1u);
  }
}

// Exclusive prefix of v over the block (blockDim.x == 256); *total = the block's sum.
__device__ __forceinline__ unsigned long long block_excl_scan(unsigned long long v, unsigned long long* total) {
  __shared__ unsigned long long warp_sum[8];
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
    for (int k = 0; k < 8; k++) { const unsigned long long t = warp_sum[k]; warp_sum[k] = run; run += t; }
    block_total = run;
  }
  __syncthreads();
  *total = block_total;
  return warp_sum[w] + inc - v;
}

// Pass step 2: gives every dirty Spec of the stage fresh working rows (in the temp buffer, from
// temp_top up; Specs that are not solved again keep theirs) and its chunks, and resets its
// real-breakpoint masks.
__global__ void __launch_bounds__(256)
place_kernel(SpecHdr* __restrict__ hdrs, uint4* __restrict__ rmask, const uint8_t* __restrict__ mine,
             uint8_t* __restrict__ dirty, uint32_t lo, uint32_t hi, unsigned long long temp_top,
             unsigned long long temp_cap, Chunk* __restrict__ chunks, unsigned long long chunk_cap,
             PassCounters* __restrict__ ctr) {
  const uint32_t i = lo + blockIdx.x * blockDim.x + threadIdx.x;
  const bool active = i < hi && (!mine || mine[i]) && dirty[i];
  Grid g;
  g.cells = 0; g.warps = 0; g.F = 0;
  if (active) g = grid_of(*reinterpret_cast<const uint4*>(&hdrs[i]));
  unsigned long long tot_cells, tot_warps;
  const unsigned long long my_row = block_excl_scan(g.cells, &tot_cells);
  const unsigned long long my_chunk = block_excl_scan(active ? g.warps : 0ull, &tot_warps);
  __shared__ unsigned long long row0, chunk0;
  if (threadIdx.x == 0) {
    row0 = atomicAdd(&ctr->temp_rows, tot_cells);
    chunk0 = atomicAdd(&ctr->n_chunks, (uint32_t)tot_warps);
  }
  __syncthreads();
  if (!active) return;
  const unsigned long long rb = temp_top + row0 + my_row;
  const unsigned long long cb = chunk0 + my_chunk;
  if (rb + g.cells > temp_cap || cb + g.warps > chunk_cap) { atomicOr(&ctr->error, 2u); return; }
  hdrs[i].row_base = rb | MRL_TEMP_FLAG;
  rmask[i] = make_uint4(1u, 1u, 1u, 1u);
  dirty[i] = 0;   // solved by this pass
  for (uint32_t w = 0; w < g.warps; w++) {
    Chunk c;
    c.spec = i;
    c.col_start = (w * 32u) | (g.F << 30);
    chunks[cb + w] = c;
  }
}

// Pass step 3a: how many working cells lie on each limits diagonal. Thread per column.
__global__ void __launch_bounds__(128)
diag_histogram_kernel(const SpecHdr* __restrict__ hdrs, const Chunk* __restrict__ chunks, uint32_t n_chunks,
                      DiagTable* __restrict__ diag) {
  __shared__ uint32_t hist[MRL_MAX_DIAG];
  for (uint32_t k = threadIdx.x; k < MRL_MAX_DIAG; k += blockDim.x) hist[k] = 0;
  __syncthreads();
  const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (warp < n_chunks) {
    const Column c = decode_column(hdrs, chunks[warp], lane);
    if (c.valid) {
      uint32_t mrest = sel4(c.mm[0], c.mm[1], c.mm[2], c.mm[3], c.F);
      while (mrest) {
        const uint32_t codeF = __ffs(mrest) - 1;
        mrest &= mrest - 1;
        atomicAdd(&hist[(c.others + codeF) & (MRL_MAX_DIAG - 1)], 1u);
      }
    }
  }
  __syncthreads();
  for (uint32_t k = threadIdx.x; k < MRL_MAX_DIAG; k += blockDim.x)
    if (hist[k]) atomicAdd(&diag->count[k], hist[k]);
}

// Pass step 3b: lists the working cells diagonal by diagonal (diag->base set by the host from the
// histogram). Every warp counts its own cells per diagonal; the block reserves list slots per
// diagonal with one atomic each and hands every warp a contiguous piece, so that the cells one
// warp (one Spec) has on a diagonal stay neighbours in the list - and neighbours in a combine warp.
__global__ void __launch_bounds__(128)
scatter_cells_kernel(const SpecHdr* __restrict__ hdrs, const Chunk* __restrict__ chunks, uint32_t n_chunks,
                     DiagTable* __restrict__ diag, CellRef* __restrict__ cells) {
  __shared__ uint32_t hist[4][MRL_MAX_DIAG];
  __shared__ unsigned long long start[4][MRL_MAX_DIAG];
  for (uint32_t k = threadIdx.x; k < 4 * MRL_MAX_DIAG; k += blockDim.x) hist[k / MRL_MAX_DIAG][k % MRL_MAX_DIAG] = 0;
  __syncthreads();
  const uint32_t wib = threadIdx.x >> 5;   // warp in block
  const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  Column c;
  c.valid = false;
  if (warp < n_chunks) c = decode_column(hdrs, chunks[warp], lane);
  const uint32_t mF = c.valid ? sel4(c.mm[0], c.mm[1], c.mm[2], c.mm[3], c.F) : 0u;
  for (uint32_t mrest = mF; mrest; mrest &= mrest - 1)
    atomicAdd(&hist[wib][(c.others + __ffs(mrest) - 1) & (MRL_MAX_DIAG - 1)], 1u);
  __syncthreads();
  for (uint32_t k = threadIdx.x; k < MRL_MAX_DIAG; k += blockDim.x) {
    const uint32_t n0 = hist[0][k], n1 = hist[1][k], n2 = hist[2][k], n3 = hist[3][k];
    const uint32_t n = n0 + n1 + n2 + n3;
    if (n) {
      const unsigned long long base = diag->base[k] + atomicAdd(&diag->cursor[k], n);
      start[0][k] = base;
      start[1][k] = base + n0;
      start[2][k] = base + n0 + n1;
      start[3][k] = base + n0 + n1 + n2;
    }
    hist[0][k] = hist[1][k] = hist[2][k] = hist[3][k] = 0;   // become the warps' cursors
  }
  __syncthreads();
  if (!c.valid) return;
  // the fixed memories' codes, one per byte (RF in byte 0 .. GL in byte 3); the byte of F is 0
  const uint32_t fixed = c.code[0] | (c.code[1] << 8) | (c.code[2] << 16) | (c.code[3] << 24);
  for (uint32_t mrest = mF; mrest; mrest &= mrest - 1) {
    const uint32_t codeF = __ffs(mrest) - 1;
    const uint32_t d = (c.others + codeF) & (MRL_MAX_DIAG - 1);
    const uint32_t pos = atomicAdd(&hist[wib][d], 1u);
    CellRef r;
    r.spec = c.spec;
    r.cpack = fixed | (codeF << (8 * c.F));
    cells[start[wib][d] + pos] = r;
  }
}

// Pass step 4: which breakpoints of the working grids are real. A breakpoint (memory k, code c)
// is real when some cell starting at c differs from its neighbour one slot lower in k.
__global__ void __launch_bounds__(128)
real_masks_kernel(const SpecHdr* __restrict__ hdrs, const Chunk* __restrict__ chunks, uint32_t n_chunks,
                  const MrlRow* __restrict__ temp, uint4* __restrict__ rmask) {
  const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (warp >= n_chunks) return;   // whole warps leave together
  const Chunk ch = chunks[warp];
  const Column c = decode_column(hdrs, ch, lane);
  uint32_t bits[4] = {0, 0, 0, 0};
  if (c.valid) {
    const unsigned long long base = hdrs[ch.spec].row_base & ~MRL_TEMP_FLAG;
    const uint32_t st[4] = {1u, c.nn[0], c.nn[0] * c.nn[1], c.nn[0] * c.nn[1] * c.nn[2]};
    const uint32_t mF = sel4(c.mm[0], c.mm[1], c.mm[2], c.mm[3], c.F);
    const uint32_t nF = sel4(c.nn[0], c.nn[1], c.nn[2], c.nn[3], c.F);
    const uint32_t stF = sel4(st[0], st[1], st[2], st[3], c.F);
    uint32_t off0 = 0;
#pragma unroll
    for (int k = 0; k < 4; k++) off0 += c.idx[k] * st[k];   // idx[F] is 0
    uint4 prev = make_uint4(0, 0, 0, 0);
    uint32_t fbits = 0, mrest = mF;
    for (uint32_t s = 0; s < nF; s++) {
      const uint32_t codeF = __ffs(mrest) - 1;
      mrest &= mrest - 1;
      const unsigned long long r_at = base + off0 + (unsigned long long)s * stF;
      const uint4 r = *reinterpret_cast<const uint4*>(temp + r_at);
#pragma unroll
      for (int k = 0; k < 4; k++) {
        if ((uint32_t)k == c.F || c.idx[k] == 0) continue;
        const uint4 nb = *reinterpret_cast<const uint4*>(temp + r_at - st[k]);
        if (nb.x != r.x || nb.y != r.y || nb.z != r.z) bits[k] |= 1u << c.code[k];
      }
      if (s > 0 && (prev.x != r.x || prev.y != r.y || prev.z != r.z)) fbits |= 1u << codeF;
      prev = r;
    }
#pragma unroll
    for (int k = 0; k < 4; k++)
      if ((uint32_t)k == c.F) bits[k] = fbits;
  }
#pragma unroll
  for (int k = 0; k < 4; k++) bits[k] = __reduce_or_sync(0xFFFFFFFFu, bits[k]);
  if (lane == 0) {
    uint32_t* out = reinterpret_cast<uint32_t*>(&rmask[ch.spec]);
#pragma unroll
    for (int k = 0; k < 4; k++)
      if (bits[k]) atomicOr(out + k, bits[k]);
  }
}

// ---- compaction: working grids -> final table ---------------------------------------------

// Final cell count per Spec of the stage and the sum per block of 256 Specs.
__global__ void __launch_bounds__(256)
final_count_kernel(const uint4* __restrict__ rmask, uint32_t lo, uint32_t hi, uint32_t* __restrict__ fcount,
                   unsigned long long* __restrict__ block_sums) {
  const uint32_t i = lo + blockIdx.x * blockDim.x + threadIdx.x;
  unsigned long long n = 0;
  if (i < hi) {
    const uint4 m = rmask[i];
    n = (unsigned long long)__popc(m.x) * __popc(m.y) * __popc(m.z) * __popc(m.w);
    fcount[i - lo] = (uint32_t)n;
  }
  unsigned long long total;
  block_excl_scan(n, &total);
  if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
}

// Exclusive scan of the block sums (one block), and the stage's place in the table:
// stage_info[0] = first final row of the stage, stage_info[1] = its row count.
__global__ void __launch_bounds__(256)
scan_block_sums_kernel(unsigned long long* __restrict__ block_sums, uint32_t n_blocks,
                       unsigned long long* __restrict__ final_top, unsigned long long* __restrict__ stage_info) {
  unsigned long long carry = 0;
  for (uint32_t b0 = 0; b0 < n_blocks; b0 += 256) {
    const uint32_t b = b0 + threadIdx.x;
    const unsigned long long v = b < n_blocks ? block_sums[b] : 0ull;
    unsigned long long total;
    const unsigned long long ex = block_excl_scan(v, &total);
    if (b < n_blocks) block_sums[b] = carry + ex;
    carry += total;
  }
  if (threadIdx.x == 0) {
    stage_info[0] = *final_top;
    stage_info[1] = carry;
    *final_top += carry;
  }
}

// Copies each Spec's real cells from its working grid to its final rows and repoints the header.
// Specs computed by another rank get zero rows (the exchange adds the owner's rows onto them).
__global__ void __launch_bounds__(256)
compact_kernel(SpecHdr* __restrict__ hdrs, const uint4* __restrict__ rmask, const uint8_t* __restrict__ mine,
               uint32_t lo, uint32_t hi, const uint32_t* __restrict__ fcount,
               const unsigned long long* __restrict__ block_sums, const unsigned long long* __restrict__ stage_info,
               MrlRow* __restrict__ rows, unsigned long long row_cap, const MrlRow* __restrict__ temp,
               PassCounters* __restrict__ ctr) {
  const uint32_t i = lo + blockIdx.x * blockDim.x + threadIdx.x;
  const unsigned long long n = i < hi ? fcount[i - lo] : 0u;
  unsigned long long total;
  const unsigned long long ex = block_excl_scan(n, &total);
  if (i >= hi) return;
  const unsigned long long fbase = stage_info[0] + block_sums[blockIdx.x] + ex;
  if (fbase + n > row_cap) { atomicOr(&ctr->error, 4u); return; }
  const uint4 fm = rmask[i];
  if (!mine || mine[i]) {
    const uint4 tm = *reinterpret_cast<const uint4*>(&hdrs[i]);
    const unsigned long long tbase = hdrs[i].row_base & ~MRL_TEMP_FLAG;
    const uint32_t f0 = __popc(fm.x), f1 = __popc(fm.y), f2 = __popc(fm.z);
    const uint32_t t0 = __popc(tm.x), t1 = __popc(tm.y), t2 = __popc(tm.z);
    for (uint32_t j = 0; j < (uint32_t)n; j++) {
      uint32_t rest = j;
      const uint32_t j0 = rest % f0; rest /= f0;
      const uint32_t j1 = rest % f1; rest /= f1;
      const uint32_t j2 = rest % f2; rest /= f2;
      const uint32_t j3 = rest;
      const uint32_t i0 = __popc(tm.x & ((2u << nth_set_bit(fm.x, j0)) - 1u)) - 1;
      const uint32_t i1 = __popc(tm.y & ((2u << nth_set_bit(fm.y, j1)) - 1u)) - 1;
      const uint32_t i2 = __popc(tm.z & ((2u << nth_set_bit(fm.z, j2)) - 1u)) - 1;
      const uint32_t i3 = __popc(tm.w & ((2u << nth_set_bit(fm.w, j3)) - 1u)) - 1;
      const uint32_t toff = ((i3 * t2 + i2) * t1 + i1) * t0 + i0;
      *reinterpret_cast<uint4*>(rows + fbase + j) = *reinterpret_cast<const uint4*>(temp + tbase + toff);
    }
  } else {
    for (uint32_t j = 0; j < (uint32_t)n; j++) *reinterpret_cast<uint4*>(rows + fbase + j) = make_uint4(0, 0, 0, 0);
  }
  *reinterpret_cast<uint4*>(&hdrs[i]) = fm;
  hdrs[i].row_base = fbase;
}

// Point lookups for get: the row of (Spec id, packed limit codes), into a dense buffer.
__global__ void lookup_rows_kernel(const SpecHdr* __restrict__ hdrs, const MrlRow* __restrict__ rows,
                                   const uint2* __restrict__ queries, unsigned long long n, MrlRow* __restrict__ out) {
  const unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint2 q = queries[i];
  const uint4 r = lookup(hdrs, rows, rows, q.x, (2u << code_of(q.y, 0)) - 1u, (2u << code_of(q.y, 1)) - 1u,
                         (2u << code_of(q.y, 2)) - 1u, (2u << code_of(q.y, 3)) - 1u);
  *reinterpret_cast<uint4*>(out + i) = r;
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

int DeviceFill::alloc_(void** p, size_t bytes) {
  bytes = std::max<size_t>(bytes, 256);
  if (fixed_) {
    const size_t off = align256(buf_off_);
    if (off + bytes > buf_bytes_) {
      snprintf(err_, sizeof(err_),
               "this fill needs more than the %zu bytes of device memory the no-allocation entry point has; "
               "use mrl_top_down_many for it", buf_bytes_);
      return -4;
    }
    *p = buf_ + off;
    buf_off_ = off + bytes;
    return 0;
  }
  CK(cudaMalloc(p, bytes));
  return 0;
}

void DeviceFill::free_(void* p) {
  if (p && !fixed_) cudaFree(p);
}

void DeviceFill::release() {
  wait_upload();
  free_(d_hdrs_); free_(d_cands_); free_(d_rmask_); free_(d_mine_); free_(d_chunks_); free_(d_rows_);
  free_(d_temp_); free_(d_fcount_); free_(d_block_sums_); free_(d_ctr_); free_(d_stage_); free_(d_cells_); free_(d_diag_); free_(d_dirty_);
  d_hdrs_ = nullptr; d_cands_ = nullptr; d_rmask_ = nullptr; d_mine_ = nullptr; d_chunks_ = nullptr;
  d_rows_ = nullptr; d_temp_ = nullptr; d_fcount_ = nullptr; d_block_sums_ = nullptr; d_ctr_ = nullptr;
  d_stage_ = nullptr; d_cells_ = nullptr; d_diag_ = nullptr; d_dirty_ = nullptr;
  stage_bytes_ = 0;
  row_cap_ = temp_cap_ = chunk_cap_ = cell_cap_ = 0;
  buf_off_ = 0;
  if (h_ctr_) { cudaFreeHost(h_ctr_); h_ctr_ = nullptr; }
  if (h_diag_) { cudaFreeHost(h_diag_); h_diag_ = nullptr; }
  for (cudaEvent_t e : ev_pool_) cudaEventDestroy(e);
  ev_pool_.clear();
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
  stage_log_ = getenv("MRL_STAGE_LOG") != nullptr;
  if (const char* e = getenv("MRL_SEED_HOPS")) seed_hops_ = std::max(0, std::min(8, atoi(e)));
  // For profilers started with capture off (ncu --profile-from-start off): only combine launches
  // with at least this many cells are bracketed by cudaProfilerStart / Stop.
  if (const char* e = getenv("MRL_PROFILE_MIN_CELLS")) profile_min_cells_ = (uint32_t)strtoul(e, nullptr, 10);
  if (!ev0_) CK(cudaEventCreate(&ev0_));
  if (!ev1_) CK(cudaEventCreate(&ev1_));
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
  free_(d_hdrs_); free_(d_cands_); free_(d_rmask_); free_(d_mine_); free_(d_chunks_); free_(d_rows_);
  free_(d_temp_); free_(d_fcount_); free_(d_block_sums_); free_(d_ctr_); free_(d_stage_); free_(d_cells_); free_(d_diag_); free_(d_dirty_);
  d_hdrs_ = nullptr; d_cands_ = nullptr; d_rmask_ = nullptr; d_mine_ = nullptr; d_chunks_ = nullptr;
  d_rows_ = nullptr; d_temp_ = nullptr; d_fcount_ = nullptr; d_block_sums_ = nullptr; d_ctr_ = nullptr;
  d_stage_ = nullptr; d_cells_ = nullptr; d_diag_ = nullptr; d_dirty_ = nullptr;
  stage_bytes_ = 0;
  buf_off_ = 0;
  n_specs_ = (uint32_t)plan.hdrs.size();
  uint32_t max_stage = 1;
  for (const Stage& st : plan.stages) max_stage = std::max(max_stage, st.spec_hi - st.spec_lo);
  int rc;
  if ((rc = alloc_((void**)&d_ctr_, 256))) return rc;
  if ((rc = alloc_((void**)&d_diag_, sizeof(DiagTable)))) return rc;
  d_final_top_ = reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(d_ctr_) + 64);
  d_stage_info_ = d_final_top_ + 1;
  if ((rc = alloc_((void**)&d_hdrs_, plan.hdrs.size() * sizeof(SpecHdr)))) return rc;
  if ((rc = alloc_((void**)&d_cands_, plan.cands.size() * sizeof(CandRec)))) return rc;
  if ((rc = alloc_((void**)&d_rmask_, plan.hdrs.size() * sizeof(uint4)))) return rc;
  if ((rc = alloc_((void**)&d_dirty_, plan.hdrs.size()))) return rc;
  if (!plan.mine.empty() && (rc = alloc_((void**)&d_mine_, plan.mine.size()))) return rc;
  if ((rc = alloc_((void**)&d_fcount_, (size_t)max_stage * sizeof(uint32_t)))) return rc;
  if ((rc = alloc_((void**)&d_block_sums_, ((size_t)max_stage / 256 + 1) * sizeof(unsigned long long)))) return rc;
  if (fixed_) {
    // Everything left is split once: lookup staging, chunks, working rows and final rows.
    stage_bytes_ = 64 << 10;
    if ((rc = alloc_(&d_stage_, stage_bytes_))) return rc;
    const size_t left = buf_bytes_ > align256(buf_off_) + 1024 ? buf_bytes_ - align256(buf_off_) - 1024 : 0;
    // per working cell: 16 bytes of row, 8 of cell list, under 1 of chunks; the rest is the table
    chunk_cap_ = left / 32 / sizeof(Chunk);
    temp_cap_ = left * 14 / 32 / sizeof(MrlRow);
    cell_cap_ = left * 7 / 32 / sizeof(CellRef);
    row_cap_ = (left - left / 32 - left * 14 / 32 - left * 7 / 32) / sizeof(MrlRow);
    if (chunk_cap_ == 0 || row_cap_ == 0) {
      snprintf(err_, sizeof(err_), "this fill needs more than the %zu bytes of device memory the no-allocation "
               "entry point has; use mrl_top_down_many for it", buf_bytes_);
      return -4;
    }
    if ((rc = alloc_((void**)&d_chunks_, chunk_cap_ * sizeof(Chunk)))) return rc;
    if ((rc = alloc_((void**)&d_temp_, temp_cap_ * sizeof(MrlRow)))) return rc;
    if ((rc = alloc_((void**)&d_cells_, cell_cap_ * sizeof(CellRef)))) return rc;
    if ((rc = alloc_((void**)&d_rows_, row_cap_ * sizeof(MrlRow)))) return rc;
  } else {
    // Starting sizes from what fills of this kind ended with (about 40 table rows per Spec and
    // 700 working cells per Spec of the largest stage at size 8), within a quarter of the free
    // memory each; every buffer still grows on demand.
    size_t free_b = 0, total_b = 0;
    CK(cudaMemGetInfo(&free_b, &total_b));
    const uint64_t quarter = free_b / 4;
    chunk_cap_ = std::max<uint64_t>(1u << 16, (uint64_t)max_stage * 32);
    temp_cap_ = std::max<uint64_t>(1u << 20, std::min<uint64_t>((uint64_t)max_stage * 700, quarter / sizeof(MrlRow)));
    cell_cap_ = std::max<uint64_t>(1u << 20, std::min<uint64_t>((uint64_t)max_stage * 400, quarter / sizeof(CellRef)));
    row_cap_ = std::max<uint64_t>(1u << 20, std::min<uint64_t>((uint64_t)n_specs_ * 40, quarter / sizeof(MrlRow)));
    if ((rc = alloc_((void**)&d_chunks_, chunk_cap_ * sizeof(Chunk)))) return rc;
    if ((rc = alloc_((void**)&d_temp_, temp_cap_ * sizeof(MrlRow)))) return rc;
    if ((rc = alloc_((void**)&d_cells_, cell_cap_ * sizeof(CellRef)))) return rc;
    if ((rc = alloc_((void**)&d_rows_, row_cap_ * sizeof(MrlRow)))) return rc;
    if (!h_ctr_) CK(cudaHostAlloc((void**)&h_ctr_, 256, cudaHostAllocDefault));
    if (!h_diag_) CK(cudaHostAlloc((void**)&h_diag_, sizeof(DiagTable), cudaHostAllocDefault));
  }
  h2d_bytes_ = plan.hdrs.size() * sizeof(SpecHdr) + (skip_cands ? 0 : plan.cands.size() * sizeof(CandRec)) + plan.mine.size();
  CK(cudaMemsetAsync(d_ctr_, 0, 256, stream_));
  if (!plan.hdrs.empty())
    CK(cudaMemcpyAsync(d_hdrs_, plan.hdrs.data(), plan.hdrs.size() * sizeof(SpecHdr), cudaMemcpyHostToDevice, stream_));
  n_cand_bytes_ = plan.cands.size() * sizeof(CandRec);
  if (!plan.cands.empty() && !skip_cands) {
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
  if (d_mine_) CK(cudaMemcpyAsync(d_mine_, plan.mine.data(), plan.mine.size(), cudaMemcpyHostToDevice, stream_));
  CK(cudaStreamSynchronize(stream_));
  stats_ = FillStats();
  final_bound_ = 0;
  return 0;
}

int DeviceFill::read_counters_(PassCounters* out) {
  if (h_ctr_) {
    CK(cudaMemcpyAsync(h_ctr_, d_ctr_, sizeof(PassCounters) + 24, cudaMemcpyDeviceToHost, stream_));
    CK(cudaStreamSynchronize(stream_));
    *out = *h_ctr_;
    final_top_seen_ = reinterpret_cast<const unsigned long long*>(h_ctr_ + 1)[0];
    stage_info_seen_[0] = reinterpret_cast<const unsigned long long*>(h_ctr_ + 1)[1];
    stage_info_seen_[1] = reinterpret_cast<const unsigned long long*>(h_ctr_ + 1)[2];
  } else {
    unsigned char tmp[sizeof(PassCounters) + 24];
    CK(cudaMemcpyAsync(tmp, d_ctr_, sizeof(tmp), cudaMemcpyDeviceToHost, stream_));
    CK(cudaStreamSynchronize(stream_));
    memcpy(out, tmp, sizeof(PassCounters));
    unsigned long long v[3];
    memcpy(v, tmp + sizeof(PassCounters), 24);
    final_top_seen_ = v[0];
    stage_info_seen_[0] = v[1];
    stage_info_seen_[1] = v[2];
  }
  return 0;
}

// Makes room for `need` final rows; the rows placed so far move along.
int DeviceFill::ensure_rows_(uint64_t need, bool refresh) {
  if (need <= row_cap_) return 0;
  if (refresh) {
    // The bound on the rows placed so far may be loose: use the exact count before growing.
    PassCounters c;
    if (read_counters_(&c) != 0) return -1;
    need = need - final_bound_ + final_top_seen_;
    final_bound_ = final_top_seen_;
    if (need <= row_cap_) return 0;
  }
  if (fixed_) {
    snprintf(err_, sizeof(err_), "this fill needs more than the %zu bytes of device memory the no-allocation "
             "entry point has; use mrl_top_down_many for it", buf_bytes_);
    return -4;
  }
  size_t free_b = 0, total_b = 0;
  CK(cudaMemGetInfo(&free_b, &total_b));
  uint64_t cap = std::max<uint64_t>(need, row_cap_ * 2);
  if (cap * sizeof(MrlRow) + (1ull << 30) > free_b) cap = need;
  if (cap * sizeof(MrlRow) + (256ull << 20) > free_b) {
    snprintf(err_, sizeof(err_), "out of device memory: the table needs %llu rows", (unsigned long long)need);
    return -6;
  }
  MrlRow* nr = nullptr;
  CK(cudaMalloc((void**)&nr, cap * sizeof(MrlRow)));
  if (final_bound_) CK(cudaMemcpyAsync(nr, d_rows_, final_bound_ * sizeof(MrlRow), cudaMemcpyDeviceToDevice, stream_));
  CK(cudaStreamSynchronize(stream_));
  cudaFree(d_rows_);
  d_rows_ = nr;
  row_cap_ = cap;
  return 0;
}

// Room for `need` working rows; the first `keep` rows (grids of Specs that are not solved again
// in this pass) move along.
int DeviceFill::ensure_temp_(uint64_t need, uint64_t keep) {
  if (need <= temp_cap_) return 0;
  if (fixed_) {
    snprintf(err_, sizeof(err_), "this fill needs more than the %zu bytes of device memory the no-allocation "
             "entry point has; use mrl_top_down_many for it", buf_bytes_);
    return -4;
  }
  const uint64_t cap = need + need / 4;
  MrlRow* nt = nullptr;
  CK(cudaMalloc((void**)&nt, cap * sizeof(MrlRow)));
  if (keep) CK(cudaMemcpyAsync(nt, d_temp_, keep * sizeof(MrlRow), cudaMemcpyDeviceToDevice, stream_));
  CK(cudaStreamSynchronize(stream_));
  cudaFree(d_temp_);
  d_temp_ = nt;
  temp_cap_ = cap;
  return 0;
}

int DeviceFill::ensure_cells_(uint64_t need) {
  if (need <= cell_cap_) return 0;
  if (fixed_) {
    snprintf(err_, sizeof(err_), "this fill needs more than the %zu bytes of device memory the no-allocation "
             "entry point has; use mrl_top_down_many for it", buf_bytes_);
    return -4;
  }
  CK(cudaStreamSynchronize(stream_));
  cudaFree(d_cells_);
  d_cells_ = nullptr;
  cell_cap_ = 0;
  const uint64_t cap = need + need / 4;
  CK(cudaMalloc((void**)&d_cells_, cap * sizeof(CellRef)));
  cell_cap_ = cap;
  return 0;
}

int DeviceFill::ensure_chunks_(uint64_t need) {
  if (need <= chunk_cap_) return 0;
  if (need > 0xFFFFFFF0ull) { snprintf(err_, sizeof(err_), "stage too large: %llu chunks", (unsigned long long)need); return -6; }
  if (fixed_) {
    snprintf(err_, sizeof(err_), "this fill needs more than the %zu bytes of device memory the no-allocation "
             "entry point has; use mrl_top_down_many for it", buf_bytes_);
    return -4;
  }
  CK(cudaStreamSynchronize(stream_));
  cudaFree(d_chunks_);
  d_chunks_ = nullptr;
  chunk_cap_ = 0;
  const uint64_t cap = need + need / 4;
  CK(cudaMalloc((void**)&d_chunks_, cap * sizeof(Chunk)));
  chunk_cap_ = cap;
  return 0;
}

int DeviceFill::begin_fill() {
  CK(cudaSetDevice(device_));
  stats_ = FillStats();
  final_bound_ = 0;
  ev_used_ = 0;
  CK(cudaMemsetAsync(d_ctr_, 0, 256, stream_));
  CK(cudaEventRecord(ev0_, stream_));
  filling_ = true;
  return 0;
}

// Solves one stage: passes of (derive masks, place, one combine launch per occupied diagonal,
// find real breakpoints) until no working grid lacks a breakpoint of a same-stage child.
int DeviceFill::solve_stage(const Plan& plan, uint32_t si) {
  if (si >= plan.stages.size()) { snprintf(err_, sizeof(err_), "stage index out of range"); return -3; }
  const Stage& st = plan.stages[si];
  const uint32_t lo = st.spec_lo, hi = st.spec_hi, n = hi - lo;
  last_cells_ = 0;
  if (n == 0) return 0;
  {
    // the stage reads its own Specs' candidate records (ids, and with them the records, are in
    // stage order): wait for that much of a background upload
    const SpecHdr& last = plan.hdrs[hi - 1];
    int rc = wait_cands_(((uint64_t)last.cand_off + last.ncand) * sizeof(CandRec));
    if (rc) return rc;
  }
  if (d_mine_) CK(cudaMemsetAsync(d_rmask_ + lo, 0, (size_t)n * sizeof(uint4), stream_));
  CK(cudaMemsetAsync(d_dirty_ + lo, 0, n, stream_));
  const uint32_t top_pack = plan.top_pack();
  const uint32_t nb128 = (n + 127) / 128;
  uint64_t temp_top = 0;   // working rows handed out so far in this stage
  for (int pass = 0;; pass++) {
    if (pass >= 128) { snprintf(err_, sizeof(err_), "stage %u did not reach a consistent limits grid", si); return -2; }
    // masks: the first pass knows nothing about same-stage children; later passes add the real
    // breakpoints the previous passes found in them. Specs whose masks grew become dirty.
    derive_masks_kernel<<<nb128, 128, 0, stream_>>>(d_hdrs_, d_cands_, d_rmask_, d_mine_, d_dirty_, lo, hi, pass == 0,
                                                    pass == 0 ? 0 : 1, pass == 0 && seed_hops_ > 0, top_pack);
    stats_.launches++;
    if (pass == 0)
      for (int h = 0; h < seed_hops_; h++) {
        // optional seeding: assume the same-stage children's breakpoints are their own first masks
        derive_masks_kernel<<<nb128, 128, 0, stream_>>>(d_hdrs_, d_cands_, d_rmask_, d_mine_, d_dirty_, lo, hi, 0, 1,
                                                        h + 1 < seed_hops_, top_pack);
        stats_.launches++;
      }
    // close the dirty marks under "has a dirty same-stage child", then total the pass
    PassCounters c;
    for (int round = 0;; round++) {
      if (round >= 4096) { snprintf(err_, sizeof(err_), "stage %u: dirty marks did not settle", si); return -2; }
      if (pass > 0)
        for (int k = 0; k < 3; k++) {
          spread_dirty_kernel<<<nb128, 128, 0, stream_>>>(d_hdrs_, d_cands_, d_mine_, d_dirty_, lo, hi);
          stats_.launches++;
        }
      CK(cudaMemsetAsync(d_ctr_, 0, offsetof(PassCounters, error), stream_));   // the error word is sticky
      totals_kernel<<<nb128, 128, 0, stream_>>>(d_hdrs_, d_cands_, d_mine_, d_dirty_, lo, hi, d_ctr_);
      stats_.launches++;
      if (read_counters_(&c) != 0) return -1;
      if (c.error) {
        snprintf(err_, sizeof(err_), "a fill kernel reported error bits 0x%x in stage %u (1: bad child index, 2: working "
                 "buffers too small, 4: row arena too small)", c.error, si);
        return -2;
      }
      if (pass == 0 || !c.changed) break;
    }
    last_cells_ = c.all_cells;
    if (c.cells == 0) break;   // nothing left to solve: every working grid is consistent
    int rc;
    if ((rc = ensure_chunks_(c.warps))) return rc;
    if ((rc = ensure_temp_(temp_top + c.cells, temp_top))) return rc;
    if (c.cells >= 0xFFFFFFF0ull) { snprintf(err_, sizeof(err_), "stage %u too large: %llu working cells", si, (unsigned long long)c.cells); return -6; }
    if ((rc = ensure_cells_(c.cells))) return rc;
    place_kernel<<<(n + 255) / 256, 256, 0, stream_>>>(d_hdrs_, d_rmask_, d_mine_, d_dirty_, lo, hi, temp_top, temp_cap_,
                                                       d_chunks_, chunk_cap_, d_ctr_);
    temp_top += c.cells;
    const uint32_t n_chunks = (uint32_t)c.warps;
    const uint32_t blocks = (n_chunks + 3) / 4;
    // cells per limits diagonal, then the cell lists
    CK(cudaMemsetAsync(d_diag_, 0, sizeof(DiagTable), stream_));
    diag_histogram_kernel<<<blocks, 128, 0, stream_>>>(d_hdrs_, d_chunks_, n_chunks, d_diag_);
    DiagTable* hd = h_diag_ ? h_diag_ : &diag_pageable_;
    CK(cudaMemcpyAsync(hd->count, d_diag_->count, sizeof(hd->count), cudaMemcpyDeviceToHost, stream_));
    CK(cudaStreamSynchronize(stream_));
    unsigned long long run = 0;
    for (int d = 0; d < MRL_MAX_DIAG; d++) { hd->base[d] = run; run += hd->count[d]; }
    if (run != c.cells) { snprintf(err_, sizeof(err_), "stage %u: diagonal histogram counts %llu cells, expected %llu", si, run, (unsigned long long)c.cells); return -2; }
    CK(cudaMemcpyAsync(d_diag_->base, hd->base, sizeof(hd->base), cudaMemcpyHostToDevice, stream_));
    scatter_cells_kernel<<<blocks, 128, 0, stream_>>>(d_hdrs_, d_chunks_, n_chunks, d_diag_, d_cells_);
    if (ev_used_ + 2 > ev_pool_.size()) {
      for (int k = 0; k < 64; k++) {
        cudaEvent_t e;
        CK(cudaEventCreate(&e));
        ev_pool_.push_back(e);
      }
    }
    CK(cudaEventRecord(ev_pool_[ev_used_++], stream_));
    for (uint32_t d = 0; d < MRL_MAX_DIAG; d++) {
      const uint32_t nd = hd->count[d];
      if (!nd) continue;
      // lanes per cell by launch size: what fills the GPU (227 k threads) runs one lane per cell
      const CellRef* list = d_cells_ + hd->base[d];
      const bool mark = profile_min_cells_ && nd >= profile_min_cells_;   // MRL_PROFILE_MIN_CELLS: see init_events
      if (mark) cudaProfilerStart();
      if (nd > 65536)
        combine_argmin_kernel<1><<<(nd + 127) / 128, 128, 0, stream_>>>(d_hdrs_, d_cands_, list, nd, d_rows_, d_temp_, n_specs_, &d_ctr_->error);
      else if (nd > 16384)
        combine_argmin_kernel<4><<<(nd + 31) / 32, 128, 0, stream_>>>(d_hdrs_, d_cands_, list, nd, d_rows_, d_temp_, n_specs_, &d_ctr_->error);
      else if (nd > 4096)
        combine_argmin_kernel<8><<<(nd + 15) / 16, 128, 0, stream_>>>(d_hdrs_, d_cands_, list, nd, d_rows_, d_temp_, n_specs_, &d_ctr_->error);
      else
        combine_argmin_kernel<32><<<(nd + 3) / 4, 128, 0, stream_>>>(d_hdrs_, d_cands_, list, nd, d_rows_, d_temp_, n_specs_, &d_ctr_->error);
      if (mark) cudaProfilerStop();
      stats_.combine_launches++;
    }
    CK(cudaEventRecord(ev_pool_[ev_used_++], stream_));
    real_masks_kernel<<<blocks, 128, 0, stream_>>>(d_hdrs_, d_chunks_, n_chunks, d_temp_, d_rmask_);
    CK(cudaGetLastError());
    if (stage_log_) fprintf(stderr, "[fill] stage %u (phase %u, shape %u, level %u, %u Specs) pass %d: %llu cells, %u chunks\n", si,
                            st.phase, st.shape_sum, st.level_rank, n, pass, (unsigned long long)c.cells, n_chunks);
    stats_.launches += 4;
    stats_.passes++;
    stats_.cells_solved += c.cells;
    stats_.alg_bytes += c.alg_bytes;
  }
  return 0;
}

int DeviceFill::stage_masks(const Plan& plan, uint32_t si, void** ptr, uint64_t* bytes) {
  if (si >= plan.stages.size()) { snprintf(err_, sizeof(err_), "stage index out of range"); return -3; }
  const Stage& st = plan.stages[si];
  if (ptr) *ptr = d_rmask_ + st.spec_lo;
  if (bytes) *bytes = (uint64_t)(st.spec_hi - st.spec_lo) * sizeof(uint4);
  return 0;
}

// Appends the stage's compacted grids to the table. With rows_ptr: also reports where they
// went (the slice other ranks need), which costs one synchronisation.
int DeviceFill::place_stage(const Plan& plan, uint32_t si, void** rows_ptr, uint64_t* bytes) {
  if (si >= plan.stages.size()) { snprintf(err_, sizeof(err_), "stage index out of range"); return -3; }
  const Stage& st = plan.stages[si];
  const uint32_t lo = st.spec_lo, hi = st.spec_hi, n = hi - lo;
  if (rows_ptr) *rows_ptr = d_rows_;
  if (bytes) *bytes = 0;
  if (n == 0) return 0;
  const uint32_t nb = (n + 255) / 256;
  int rc;
  const bool exact = d_mine_ || rows_ptr;
  if (!exact) {
    // final cells <= working cells of the last pass: room for that many is enough
    if ((rc = ensure_rows_(final_bound_ + last_cells_, true))) return rc;
    final_bound_ += last_cells_;
  }
  final_count_kernel<<<nb, 256, 0, stream_>>>(d_rmask_, lo, hi, d_fcount_, d_block_sums_);
  scan_block_sums_kernel<<<1, 256, 0, stream_>>>(d_block_sums_, nb, d_final_top_, d_stage_info_);
  stats_.launches += 2;
  if (exact) {
    // other ranks' Specs count too: ask the device how many rows the stage takes
    PassCounters c;
    if (read_counters_(&c) != 0) return -1;
    final_bound_ = stage_info_seen_[0];   // rows to keep if the arena has to grow
    if ((rc = ensure_rows_(final_bound_ + stage_info_seen_[1], false))) return rc;
    final_bound_ += stage_info_seen_[1];
  }
  compact_kernel<<<nb, 256, 0, stream_>>>(d_hdrs_, d_rmask_, d_mine_, lo, hi, d_fcount_, d_block_sums_, d_stage_info_,
                                          d_rows_, row_cap_, d_temp_, d_ctr_);
  CK(cudaGetLastError());
  stats_.launches++;
  if (rows_ptr) {
    *rows_ptr = d_rows_ + stage_info_seen_[0];
    if (bytes) *bytes = stage_info_seen_[1] * sizeof(MrlRow);
  }
  return 0;
}

int DeviceFill::end_fill() {
  CK(cudaEventRecord(ev1_, stream_));
  PassCounters c;
  if (read_counters_(&c) != 0) return -1;
  filling_ = false;
  CK(cudaEventElapsedTime(&stats_.fill_ms, ev0_, ev1_));
  float cms = 0;
  for (size_t k = 0; k + 1 < ev_used_; k += 2) {
    float t = 0;
    CK(cudaEventElapsedTime(&t, ev_pool_[k], ev_pool_[k + 1]));
    cms += t;
  }
  stats_.combine_ms = cms;
  stats_.launches += stats_.combine_launches;
  stats_.n_rows = final_top_seen_;
  final_bound_ = final_top_seen_;
  if (c.error) {
    snprintf(err_, sizeof(err_), "a fill kernel reported error bits 0x%x (1: bad child index, 2: working buffers too small, "
             "4: row arena too small)", c.error);
    return -2;
  }
  return 0;
}

int DeviceFill::run(const Plan& plan) {
  int rc;
  if ((rc = begin_fill())) return rc;
  for (uint32_t s = 0; s < plan.stages.size(); s++) {
    if ((rc = solve_stage(plan, s))) return rc;
    if ((rc = place_stage(plan, s, nullptr, nullptr))) return rc;
  }
  return end_fill();
}

int DeviceFill::lookup(const uint32_t* spec_ids, const uint32_t* cpacks, size_t n, MrlRow* out) {
  std::lock_guard<std::mutex> guard(lookup_mu_);   // callers on several threads share the staging buffer and the stream
  CK(cudaSetDevice(device_));
  if (n == 0) return 0;
  for (size_t i = 0; i < n; i++)
    if (spec_ids[i] >= n_specs_) { snprintf(err_, sizeof(err_), "Spec id out of range"); return -3; }
  const size_t per = sizeof(uint2) + sizeof(MrlRow);
  size_t batch = n;
  if (fixed_) batch = std::min(n, stage_bytes_ / 2 / per);
  else if (stage_bytes_ < 2 * align256(n * sizeof(MrlRow))) {
    CK(cudaStreamSynchronize(stream_));
    if (d_stage_) cudaFree(d_stage_);
    d_stage_ = nullptr;
    stage_bytes_ = 0;
    CK(cudaMalloc(&d_stage_, 2 * align256(n * sizeof(MrlRow))));
    stage_bytes_ = 2 * align256(n * sizeof(MrlRow));
  }
  if (batch == 0) { snprintf(err_, sizeof(err_), "lookup staging too small"); return -4; }
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
  unsigned long long* d_out = reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(d_ctr_) + 96);
  const unsigned long long init[2] = {0ull, ~0ull};
  CK(cudaMemcpyAsync(d_out, init, sizeof(init), cudaMemcpyHostToDevice, stream_));
  CK(cudaStreamSynchronize(stream_));
  const unsigned long long batch = 1ull << 28;
  for (unsigned long long first = 0; first < count && total; first += batch) {
    const unsigned long long n = std::min(batch, count - first);
    verify_points_kernel<<<(unsigned)((n + 127) / 128), 128, 0, stream_>>>(d_hdrs_, d_cands_, d_rows_, n_specs_, top, first, n,
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

// Device address of the static array on `device`, resolved on first use.
cudaError_t static_scratch_address(int device, void** out) {
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> g(g_scratch_mu);
  if (!g_scratch_addr[device]) {
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return e;
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_addr[device] = p;
  }
  *out = g_scratch_addr[device];
  return cudaSuccess;
}
}  // namespace

// Runs `plan` entirely inside the static array and copies the rows of the given (Spec id,
// packed limit codes) queries to `out` (host). No cudaMalloc / cudaFree. Returns -4 with a
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

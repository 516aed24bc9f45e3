// combine_argmin: the CUDA side of the synthesis-database fill (sm_100a).
//
// One launch evaluates, for one group of logical Specs (same phase and log-shape sum, so no
// dependencies among them), every table cell that lies on one diagonal of the memory-limits
// lattice. A thread owns one "column" of a Spec's cell grid (RF, VRF and L1 indices fixed;
// the GL index is whatever puts the cell on the launch's diagonal), loops over the Spec's
// candidate records, gathers the child rows each candidate needs at the child's limits,
// combines them into a Cost and keeps the lexicographic minimum. Lanes of a warp hold
// neighbouring RF indices of the same Spec, so the rows they gather from one child are
// neighbours in memory.
//
// What it replaces in the reference (paths inside the Morello repository):
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
#include <stdio.h>
#include <mutex>

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
__device__ __forceinline__ uint32_t with_code(uint32_t cpack, uint32_t level, uint32_t code) {
  return (cpack & ~(0xFFu << (8 * level))) | (code << (8 * level));
}
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

struct Key {
  uint32_t main, peaks, tail;
};
__device__ __forceinline__ bool key_less(const Key& a, const Key& b) {
  if (a.main != b.main) return a.main < b.main;
  if (a.peaks != b.peaks) return a.peaks < b.peaks;
  return a.tail < b.tail;
}

// Row of a child Spec at given limits: the cell whose breakpoints are the largest ones not
// above the limits. bm[k] = mask of the slots <= the limit's slot in memory k. One 32-byte
// header (two loads, warp-uniform) and one 16-byte row.
__device__ __forceinline__ uint4 lookup(const SpecHdr* __restrict__ hdrs, const MrlRow* __restrict__ rows,
                                        uint32_t child, uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
  const uint4 m = __ldg(reinterpret_cast<const uint4*>(&hdrs[child]));
  const unsigned long long base = __ldg(reinterpret_cast<const unsigned long long*>(&hdrs[child].row_base));
  const uint32_t i0 = __popc(m.x & b0) - 1;
  const uint32_t i1 = __popc(m.y & b1) - 1;
  const uint32_t i2 = __popc(m.z & b2) - 1;
  const uint32_t i3 = __popc(m.w & b3) - 1;
  const uint32_t off = ((i3 * __popc(m.z) + i2) * __popc(m.y) + i1) * __popc(m.x) + i0;  // cells per Spec < 2^32
  // Rows read here were written by earlier launches (lower diagonal or earlier group), never by
  // this one, so the read-only path is safe.
  return __ldg(reinterpret_cast<const uint4*>(rows + base + off));
}

// G = lanes per cell: the G lanes of a cell take every G-th candidate each and min-reduce
// their keys with warp shuffles; a warp covers 32 / G neighbouring columns.
// F = the memory whose slot is fixed by the diagonal (chosen per group: the memory with the
// most slots, so that most columns have a cell on the launch's diagonal).
template <int G, int F>
__global__ void __launch_bounds__(128, MRL_MIN_BLOCKS)
combine_argmin_kernel(const SpecHdr* __restrict__ hdrs, const CandRec* __restrict__ cands,
                      const Chunk* __restrict__ chunks, uint32_t n_chunks, uint32_t diag,
                      MrlRow* __restrict__ rows, uint32_t n_specs, uint32_t cap_pack, uint32_t top_pack,
                      int* __restrict__ error_flag) {
  const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const uint32_t lane = threadIdx.x & 31;
  if (warp >= n_chunks) return;
  const Chunk ch = chunks[warp];
  const uint4 m = __ldg(reinterpret_cast<const uint4*>(&hdrs[ch.spec]));
  const uint32_t sub = lane % G;
  const uint32_t col = ch.col_start + lane / G;
  // A column fixes the slot index in the three memories other than F; the launch's diagonal
  // then fixes the code in F, and the cell exists if that code is one of the Spec's slots.
  const uint32_t mm[4] = {m.x, m.y, m.z, m.w};
  const uint32_t nn[4] = {(uint32_t)__popc(m.x), (uint32_t)__popc(m.y), (uint32_t)__popc(m.z), (uint32_t)__popc(m.w)};
  uint32_t idx[4], code[4];
  uint32_t rest = col, others = 0;
#pragma unroll
  for (int k = 0; k < 4; k++) {
    if (k == F) continue;
    idx[k] = rest % nn[k];
    rest /= nn[k];
    code[k] = nth_set_bit(mm[k], idx[k]);
    others += code[k];
  }
  if (rest != 0) return;  // column index beyond this Spec's grid
  const int cfs = (int)diag - (int)others;
  if (cfs < 0 || cfs > 31 || !((mm[F] >> cfs) & 1u)) return;
  code[F] = (uint32_t)cfs;
  idx[F] = __popc(mm[F] & ((1u << cfs) - 1u));
  const uint32_t cpack = code[0] | (code[1] << 8) | (code[2] << 16) | (code[3] << 24);
  // "slots at or below this cell's limit", per memory: what a child lookup at the same limits needs
  const uint32_t bm0 = (2u << code[0]) - 1u, bm1 = (2u << code[1]) - 1u, bm2 = (2u << code[2]) - 1u,
                 bm3 = (2u << code[3]) - 1u;

  // The cell's limits as lattice codes: in a compressed memory slot cap+1 stands for the top code.
  uint32_t lvpack = 0;
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const uint32_t capk = code_of(cap_pack, k);
    lvpack |= ((code[k] == capk + 1u) ? code_of(top_pack, k) : code[k]) << (8 * k);
  }

  const unsigned long long base = __ldg(reinterpret_cast<const unsigned long long*>(&hdrs[ch.spec].row_base));
  const uint2 cl = __ldg(reinterpret_cast<const uint2*>(&hdrs[ch.spec].cand_off));
  const uint32_t cand_off = cl.x, ncand = cl.y;

  Key best = {MRL_UNSAT, MRL_UNSAT, MRL_UNSAT};
  for (uint32_t ci = sub; ci < ncand; ci += G) {
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(&cands[cand_off + ci]));
    const uint32_t action = a.x & 0xFFFFu, kind = (a.x >> 16) & 0xFFu, nchild = a.x >> 24;
    const uint32_t imm = a.y;
    const uint32_t level = a.z & 0xFFu, thr = (a.z >> 8) & 0xFFu, pcode = (a.z >> 16) & 0xFFu;
    const uint32_t units = a.w;
    // The cell's limit in `level` as a lattice code. In a compressed memory the grid keeps the
    // codes 0..cap and, as slot cap+1, the top code.
    const uint32_t lv = code_of(lvpack, level);
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
        // The child's limit is below the top; codes above the cap read the cap slot (nothing
        // changes between cap and top while no optimal peak exceeds the cap).
        const uint32_t cb = (2u << min(ccode, code_of(cap_pack, level))) - 1u;
        c0 = (level == 0) ? cb : c0;
        c1 = (level == 1) ? cb : c1;
        c2 = (level == 2) ? cb : c2;
        c3 = (level == 3) ? cb : c3;
      }
#ifdef MRL_CHECK_CHILD_IDS
      if (b.x >= n_specs || (nchild > 1 && b.y >= n_specs) || (nchild > 2 && b.z >= n_specs)) {
        atomicExch(error_flag, 1);
        continue;
      }
#endif
      // Children one at a time: a child without an implementation, or a partial sum that already
      // exceeds the best main cost, ends the candidate before the remaining rows are fetched.
      const uint4 r0 = lookup(hdrs, rows, b.x, c0, c1, c2, c3);
      if (r0.z == MRL_UNSAT) continue;
      uint4 r1 = r0, r2 = r0;
      if (nchild > 1) {
        if (kind == MRL_CK_MOVE && sat_add(imm, r0.x) > best.main) continue;
        r1 = lookup(hdrs, rows, b.y, c0, c1, c2, c3);
        if (r1.z == MRL_UNSAT) continue;
        if (nchild > 2) {
          r2 = lookup(hdrs, rows, b.z, c0, c1, c2, c3);
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
  if (G > 1) {
    // The G lanes of this cell are all here (a cell is active or not as a whole).
    const unsigned gmask = (G == 32) ? 0xFFFFFFFFu : (((1u << G) - 1u) << (lane & ~(G - 1)));
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) {
      Key other;
      other.main = __shfl_xor_sync(gmask, best.main, o);
      other.peaks = __shfl_xor_sync(gmask, best.peaks, o);
      other.tail = __shfl_xor_sync(gmask, best.tail, o);
      if (key_less(other, best)) best = other;
    }
    if (sub != 0) return;
  }
  const uint32_t off = ((idx[3] * nn[2] + idx[2]) * nn[1] + idx[1]) * nn[0] + idx[0];
  *reinterpret_cast<uint4*>(rows + base + off) = make_uint4(best.main, best.peaks, best.tail, 0u);
}

// Largest peak code per memory over all satisfiable rows (checks the lattice compression).
__global__ void max_peaks_kernel(const MrlRow* __restrict__ rows, unsigned long long n, uint32_t* __restrict__ out4) {
  uint32_t mx = 0;
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (unsigned long long)gridDim.x * blockDim.x) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(rows + i));
    if (r.z != MRL_UNSAT) mx = __vmaxu4(mx, r.y);
  }
  for (int o = 16; o > 0; o >>= 1) mx = __vmaxu4(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
  if ((threadIdx.x & 31) == 0) {
    atomicMax(&out4[0], (mx >> 24) & 0xFFu);
    atomicMax(&out4[1], (mx >> 16) & 0xFFu);
    atomicMax(&out4[2], (mx >> 8) & 0xFFu);
    atomicMax(&out4[3], mx & 0xFFu);
  }
}

// Expands the per-Spec warp counts into the chunk list the combine kernel walks.
__global__ void expand_chunks_kernel(const uint32_t* __restrict__ warp_prefix, uint32_t n_specs,
                                     uint32_t cols_per_warp, Chunk* __restrict__ chunks) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_specs) return;
  const uint32_t lo = warp_prefix[i], hi = warp_prefix[i + 1];
  for (uint32_t w = lo; w < hi; w++) {
    chunks[w].spec = i;
    chunks[w].col_start = (w - lo) * cols_per_warp;
  }
}

// Point lookups for get: copies the rows at the given indices into a dense buffer.
__global__ void gather_rows_kernel(const MrlRow* __restrict__ rows, const unsigned long long* __restrict__ idx,
                                   unsigned long long n, MrlRow* __restrict__ out) {
  unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  *reinterpret_cast<uint4*>(out + i) = *reinterpret_cast<const uint4*>(rows + idx[i]);
}

}  // namespace

namespace mrl {

// One (group, diagonal) launch.
static void launch_combine(int lanes, int free_dim, uint32_t blocks, cudaStream_t stream, const SpecHdr* hdrs,
                           const CandRec* cands, const Chunk* chunks, uint32_t n_chunks, uint32_t diag, MrlRow* rows,
                           uint32_t n_specs, uint32_t cap_pack, uint32_t top_pack, int* err) {
#define MRL_LAUNCH(G, F)                                                                                         \
  combine_argmin_kernel<G, F><<<blocks, 128, 0, stream>>>(hdrs, cands, chunks, n_chunks, diag, rows, n_specs,    \
                                                          cap_pack, top_pack, err)
  if (lanes == 2) {
    switch (free_dim) {
      case 0: MRL_LAUNCH(2, 0); break;
      case 1: MRL_LAUNCH(2, 1); break;
      case 2: MRL_LAUNCH(2, 2); break;
      default: MRL_LAUNCH(2, 3); break;
    }
  } else {
    switch (free_dim) {
      case 0: MRL_LAUNCH(1, 0); break;
      case 1: MRL_LAUNCH(1, 1); break;
      case 2: MRL_LAUNCH(1, 2); break;
      default: MRL_LAUNCH(1, 3); break;
    }
  }
#undef MRL_LAUNCH
}

#define CK(x)                                                                              \
  do {                                                                                     \
    cudaError_t e_ = (x);                                                                  \
    if (e_ != cudaSuccess) {                                                               \
      snprintf(err_, sizeof(err_), "%s failed: %s", #x, cudaGetErrorString(e_));           \
      return -1;                                                                           \
    }                                                                                      \
  } while (0)

DeviceFill::~DeviceFill() { release(); }

void DeviceFill::release() {
  if (d_hdrs_) cudaFree(d_hdrs_);
  if (d_cands_) cudaFree(d_cands_);
  if (d_chunks_) cudaFree(d_chunks_);
  if (d_rows_) cudaFree(d_rows_);
  if (d_err_) cudaFree(d_err_);
  if (d_peaks_) cudaFree(d_peaks_);
  d_peaks_ = nullptr;
  d_hdrs_ = nullptr; d_cands_ = nullptr; d_chunks_ = nullptr; d_rows_ = nullptr; d_err_ = nullptr;
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
  if (!ev0_) CK(cudaEventCreate(&ev0_));
  if (!ev1_) CK(cudaEventCreate(&ev1_));
  return 0;
}

int DeviceFill::upload(const Plan& plan) {
  CK(cudaSetDevice(device_));
  if (d_hdrs_) { cudaFree(d_hdrs_); d_hdrs_ = nullptr; }
  if (d_cands_) { cudaFree(d_cands_); d_cands_ = nullptr; }
  if (d_chunks_) { cudaFree(d_chunks_); d_chunks_ = nullptr; }
  if (d_rows_) { cudaFree(d_rows_); d_rows_ = nullptr; }
  if (!d_err_) CK(cudaMalloc(&d_err_, sizeof(int)));
  n_specs_ = (uint32_t)plan.hdrs.size();
  n_rows_ = plan.stats.n_rows;
  const size_t n_warps = plan.warp_prefix.empty() ? 0 : plan.warp_prefix.back();
  h2d_bytes_ = plan.hdrs.size() * sizeof(SpecHdr) + plan.cands.size() * sizeof(CandRec) +
               plan.warp_prefix.size() * sizeof(uint32_t);
  uint32_t* d_prefix = nullptr;
  CK(cudaMalloc(&d_hdrs_, std::max<size_t>(plan.hdrs.size(), 1) * sizeof(SpecHdr)));
  CK(cudaMalloc(&d_cands_, std::max<size_t>(plan.cands.size(), 1) * sizeof(CandRec)));
  CK(cudaMalloc(&d_chunks_, std::max<size_t>(n_warps, 1) * sizeof(Chunk)));
  CK(cudaMalloc(&d_rows_, std::max<uint64_t>(n_rows_, 1) * sizeof(MrlRow)));
  CK(cudaMalloc(&d_prefix, std::max<size_t>(plan.warp_prefix.size(), 1) * sizeof(uint32_t)));
  CK(cudaMemcpyAsync(d_hdrs_, plan.hdrs.data(), plan.hdrs.size() * sizeof(SpecHdr), cudaMemcpyHostToDevice, stream_));
  CK(cudaMemcpyAsync(d_cands_, plan.cands.data(), plan.cands.size() * sizeof(CandRec), cudaMemcpyHostToDevice, stream_));
  CK(cudaMemcpyAsync(d_prefix, plan.warp_prefix.data(), plan.warp_prefix.size() * sizeof(uint32_t), cudaMemcpyHostToDevice, stream_));
  if (n_specs_) expand_chunks_kernel<<<(n_specs_ + 127) / 128, 128, 0, stream_>>>(d_prefix, n_specs_, 32u / plan.lanes_per_cell, d_chunks_);
  CK(cudaGetLastError());
  CK(cudaMemsetAsync(d_err_, 0, sizeof(int), stream_));
  CK(cudaStreamSynchronize(stream_));
  cudaFree(d_prefix);
  CK(cudaStreamSynchronize(stream_));
  return 0;
}

int DeviceFill::run(const Plan& plan, float* ms_out, uint64_t* launches_out) {
  CK(cudaSetDevice(device_));
  // No clearing pass: every cell lies on exactly one (group, diagonal) step and is written
  // there, and no cell is read before its step.
  CK(cudaEventRecord(ev0_, stream_));
  uint64_t launches = 0;
  for (const Step& st : plan.steps) {
    const Group& g = plan.groups[st.group];
    const uint32_t n_chunks = g.chunk_hi - g.chunk_lo;
    const uint32_t blocks = (n_chunks + 3) / 4;
    launch_combine(plan.lanes_per_cell, g.free_dim, blocks, stream_, d_hdrs_, d_cands_, d_chunks_ + g.chunk_lo, n_chunks, st.diag,
                   d_rows_, n_specs_, plan.cap_pack(), plan.top_pack(), d_err_);
    launches++;
  }
  CK(cudaGetLastError());
  CK(cudaEventRecord(ev1_, stream_));
  CK(cudaStreamSynchronize(stream_));
  float ms = 0;
  CK(cudaEventElapsedTime(&ms, ev0_, ev1_));
  int flag = 0;
  CK(cudaMemcpy(&flag, d_err_, sizeof(int), cudaMemcpyDeviceToHost));
  if (flag) {
    snprintf(err_, sizeof(err_), "combine kernel reported a bad child index");
    return -2;
  }
  if (ms_out) *ms_out = ms;
  if (launches_out) *launches_out = launches;
  return 0;
}

int DeviceFill::set_stream(cudaStream_t s) {
  if (own_stream_ && stream_) cudaStreamDestroy(stream_);
  stream_ = s;
  own_stream_ = false;
  return 0;
}

int DeviceFill::begin_fill() {
  CK(cudaSetDevice(device_));
  CK(cudaEventRecord(ev0_, stream_));
  launches_ = 0;
  return 0;
}

// Enqueues every diagonal of one group (this rank's chunks only); does not synchronise.
int DeviceFill::run_group(const Plan& plan, uint32_t gi) {
  if (gi >= plan.groups.size()) { snprintf(err_, sizeof(err_), "group index out of range"); return -3; }
  const Group& g = plan.groups[gi];
  const uint32_t n_chunks = g.chunk_hi - g.chunk_lo;
  if (n_chunks == 0) return 0;
  const uint32_t blocks = (n_chunks + 3) / 4;
  for (uint32_t d = 0; d <= g.max_diag; d++) {
    launch_combine(plan.lanes_per_cell, g.free_dim, blocks, stream_, d_hdrs_, d_cands_, d_chunks_ + g.chunk_lo, n_chunks, d, d_rows_,
                   n_specs_, plan.cap_pack(), plan.top_pack(), d_err_);
    launches_++;
  }
  CK(cudaGetLastError());
  return 0;
}

int DeviceFill::end_fill(float* ms_out, uint64_t* launches_out) {
  CK(cudaEventRecord(ev1_, stream_));
  CK(cudaStreamSynchronize(stream_));
  float ms = 0;
  CK(cudaEventElapsedTime(&ms, ev0_, ev1_));
  int flag = 0;
  CK(cudaMemcpy(&flag, d_err_, sizeof(int), cudaMemcpyDeviceToHost));
  if (flag) {
    snprintf(err_, sizeof(err_), "combine kernel reported a bad child index");
    return -2;
  }
  if (ms_out) *ms_out = ms;
  if (launches_out) *launches_out = launches_;
  return 0;
}

int DeviceFill::max_peaks(uint32_t out[4]) {
  CK(cudaSetDevice(device_));
  if (!d_peaks_) CK(cudaMalloc(&d_peaks_, 4 * sizeof(uint32_t)));
  CK(cudaMemsetAsync(d_peaks_, 0, 4 * sizeof(uint32_t), stream_));
  if (n_rows_) max_peaks_kernel<<<148 * 8, 256, 0, stream_>>>(d_rows_, n_rows_, d_peaks_);
  CK(cudaGetLastError());
  CK(cudaMemcpyAsync(out, d_peaks_, 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost, stream_));
  CK(cudaStreamSynchronize(stream_));
  return 0;
}

int DeviceFill::read_rows(const uint64_t* row_idx, size_t n, MrlRow* out) {
  CK(cudaSetDevice(device_));
  if (n == 0) return 0;
  for (size_t i = 0; i < n; i++)
    if (row_idx[i] >= n_rows_) { snprintf(err_, sizeof(err_), "row index out of range"); return -3; }
  unsigned long long* d_idx = nullptr;
  MrlRow* d_out = nullptr;
  CK(cudaMalloc(&d_idx, n * sizeof(unsigned long long)));
  if (cudaMalloc(&d_out, n * sizeof(MrlRow)) != cudaSuccess) {
    cudaFree(d_idx);
    snprintf(err_, sizeof(err_), "cudaMalloc failed in read_rows");
    return -1;
  }
  cudaError_t e = cudaMemcpyAsync(d_idx, row_idx, n * sizeof(unsigned long long), cudaMemcpyHostToDevice, stream_);
  if (e == cudaSuccess) {
    gather_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream_>>>(d_rows_, d_idx, n, d_out);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaMemcpyAsync(out, d_out, n * sizeof(MrlRow), cudaMemcpyDeviceToHost, stream_);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream_);
  cudaFree(d_idx);
  cudaFree(d_out);
  if (e != cudaSuccess) { snprintf(err_, sizeof(err_), "read_rows failed: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}

int DeviceFill::download(std::vector<MrlRow>& out) {
  CK(cudaSetDevice(device_));
  out.resize(n_rows_);
  CK(cudaMemcpyAsync(out.data(), d_rows_, n_rows_ * sizeof(MrlRow), cudaMemcpyDeviceToHost, stream_));
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
// working set of one small fill - plan arrays, row table, lookup staging - is carved out of
// the fixed array below instead of being allocated per call. Every GPU that loads this
// library holds the array until the process exits.
//
// In host code `g_static_scratch` is only a stand-in for the device array, not a device
// address; the address a kernel may use comes from cudaGetSymbolAddress, asked once per
// device with that device current (static_scratch_address).
namespace {
__device__ __align__(256) unsigned char g_static_scratch[MRL_STATIC_SCRATCH_BYTES];
}

namespace {
constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mu;

size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

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

// Runs `plan` entirely inside the static array and copies the rows at `row_idx` to `out`
// (host). No cudaMalloc / cudaFree. Returns -4 with a message when the plan does not fit.
int fill_static(int device, cudaStream_t stream, const Plan& plan, const uint64_t* row_idx, size_t n,
                MrlRow* out, char* err, size_t err_len) {
#define CKS(x)                                                                        \
  do {                                                                                \
    cudaError_t e_ = (x);                                                             \
    if (e_ != cudaSuccess) {                                                          \
      snprintf(err, err_len, "%s failed: %s", #x, cudaGetErrorString(e_));            \
      return -1;                                                                      \
    }                                                                                 \
  } while (0)
  const size_t hdr_b = plan.hdrs.size() * sizeof(SpecHdr);
  const size_t cand_b = plan.cands.size() * sizeof(CandRec);
  const size_t n_warps = plan.warp_prefix.empty() ? 0 : plan.warp_prefix.back();
  const size_t chunk_b = n_warps * sizeof(Chunk);
  const size_t prefix_b = plan.warp_prefix.size() * sizeof(uint32_t);
  const size_t row_b = (size_t)plan.stats.n_rows * sizeof(MrlRow);
  const size_t idx_b = n * sizeof(unsigned long long);
  const size_t out_b = n * sizeof(MrlRow);
  size_t off = 256;  // first 256 bytes: the error flag
  const size_t o_hdr = off; off = align256(off + hdr_b);
  const size_t o_cand = off; off = align256(off + cand_b);
  const size_t o_chunk = off; off = align256(off + chunk_b);
  const size_t o_prefix = off; off = align256(off + prefix_b);
  const size_t o_rows = off; off = align256(off + row_b);
  const size_t o_idx = off; off = align256(off + idx_b);
  const size_t o_out = off; off = align256(off + out_b);
  if (off > (size_t)MRL_STATIC_SCRATCH_BYTES) {
    snprintf(err, err_len,
             "this fill needs %zu bytes of device memory but the no-allocation entry point has a fixed %zu; "
             "use mrl_top_down_many for it", off, (size_t)MRL_STATIC_SCRATCH_BYTES);
    return -4;
  }
  for (size_t i = 0; i < n; i++)
    if (row_idx[i] >= plan.stats.n_rows) { snprintf(err, err_len, "row index out of range"); return -3; }

  void* base_v = nullptr;
  CKS(static_scratch_address(device, &base_v));
  CKS(cudaSetDevice(device));
  unsigned char* base = static_cast<unsigned char*>(base_v);
  int* d_err = reinterpret_cast<int*>(base);
  SpecHdr* d_hdrs = reinterpret_cast<SpecHdr*>(base + o_hdr);
  CandRec* d_cands = reinterpret_cast<CandRec*>(base + o_cand);
  Chunk* d_chunks = reinterpret_cast<Chunk*>(base + o_chunk);
  uint32_t* d_prefix = reinterpret_cast<uint32_t*>(base + o_prefix);
  MrlRow* d_rows = reinterpret_cast<MrlRow*>(base + o_rows);
  unsigned long long* d_idx = reinterpret_cast<unsigned long long*>(base + o_idx);
  MrlRow* d_out = reinterpret_cast<MrlRow*>(base + o_out);

  // The array keeps whatever the previous call left. Only the error flag has to start at
  // zero; every table cell is written by its own step before anything reads it.
  CKS(cudaMemsetAsync(d_err, 0, 256, stream));
  if (hdr_b) CKS(cudaMemcpyAsync(d_hdrs, plan.hdrs.data(), hdr_b, cudaMemcpyHostToDevice, stream));
  if (cand_b) CKS(cudaMemcpyAsync(d_cands, plan.cands.data(), cand_b, cudaMemcpyHostToDevice, stream));
  if (prefix_b) CKS(cudaMemcpyAsync(d_prefix, plan.warp_prefix.data(), prefix_b, cudaMemcpyHostToDevice, stream));
  if (idx_b) CKS(cudaMemcpyAsync(d_idx, row_idx, idx_b, cudaMemcpyHostToDevice, stream));
  const uint32_t n_specs = (uint32_t)plan.hdrs.size();
  if (n_specs) expand_chunks_kernel<<<(n_specs + 127) / 128, 128, 0, stream>>>(d_prefix, n_specs, 32u / plan.lanes_per_cell, d_chunks);
  for (const Step& st : plan.steps) {
    const Group& g = plan.groups[st.group];
    const uint32_t n_chunks = g.chunk_hi - g.chunk_lo;
    launch_combine(plan.lanes_per_cell, g.free_dim, (n_chunks + 3) / 4, stream, d_hdrs, d_cands, d_chunks + g.chunk_lo, n_chunks,
                   st.diag, d_rows, n_specs, plan.cap_pack(), plan.top_pack(), d_err);
  }
  if (n) gather_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(d_rows, d_idx, n, d_out);
  CKS(cudaGetLastError());
  int flag = 0;
  if (out_b) CKS(cudaMemcpyAsync(out, d_out, out_b, cudaMemcpyDeviceToHost, stream));
  CKS(cudaMemcpyAsync(&flag, d_err, sizeof(int), cudaMemcpyDeviceToHost, stream));
  CKS(cudaStreamSynchronize(stream));
  if (flag) { snprintf(err, err_len, "combine kernel reported a bad child index"); return -2; }
  return 0;
#undef CKS
}

}  // namespace mrl

// The Spec space of a precompute job: goal phases, task points and the logical Specs
// at each task point.
//
// Restates precompute/src/main.rs:454-507,651-736 (goal phases and their bound Specs),
// :275-325 (bound point -> anti-diagonals -> task points -> canonical logical Specs),
// morello/src/spec.rs:2256-2454 + morello/src/tensorspec.rs:439-485 (the task map and
// its inverse) and morello/src/utils.rs:356-406 (diagonals / sum_seqs).
// Only the Move, Zero and Matmul phases over {u32, f32} are built; the reduction,
// softmax and Conv bounds of the reference's phases are not needed by the Matmul closure.
#pragma once
#include "spec.hpp"
#include <functional>

namespace mrl {

// sum_seqs (utils.rs:366-406): all vectors v with v[i] <= maxes[i] and sum(v) == total,
// in the reference's order (first coordinate ascending, then recursively).
inline void sum_seqs(const std::vector<u32>& maxes, size_t from, u32 total, std::vector<u32>& prefix,
                     const std::function<void(const std::vector<u32>&)>& visit) {
  size_t len = maxes.size() - from;
  if (len == 0) return;
  if (len == 1) {
    if (maxes[from] >= total) { prefix.push_back(total); visit(prefix); prefix.pop_back(); }
    return;
  }
  u32 obligation = total;
  for (size_t i = from + 1; i < maxes.size(); i++) obligation = obligation > maxes[i] ? obligation - maxes[i] : 0;
  u32 hi = maxes[from] < total ? maxes[from] : total;
  for (u32 v = obligation; v <= hi; v++) {
    prefix.push_back(v);
    sum_seqs(maxes, from + 1, total - v, prefix, visit);
    prefix.pop_back();
  }
}

// diagonals (utils.rs:356-362, 74-85): stage s holds every point with coordinate sum s.
inline std::vector<std::vector<std::vector<u32>>> diagonals(const std::vector<u32>& maxes) {
  std::vector<std::vector<std::vector<u32>>> stages;
  for (u32 stage = 0;; stage++) {
    std::vector<std::vector<u32>> pts;
    std::vector<u32> prefix;
    sum_seqs(maxes, 0, stage, prefix, [&](const std::vector<u32>& p) { pts.push_back(p); });
    if (pts.empty()) break;
    stages.push_back(std::move(pts));
  }
  return stages;
}

// TensorSpecAuxSurMap::apply_inverse (tensorspec.rs:453-484): every (layout, vector size,
// contiguousness) variant of an operand at a memory level.
inline std::vector<Aux> aux_variants(const Shape& shape, Dtype dt, Mem mem) {
  std::vector<u32> vopts;
  for (u32 vb : mem_vector_bytes(mem)) vopts.push_back(vb / dtype_size(dt));
  if (vopts.empty()) vopts.push_back(0);
  std::vector<Layout> layouts;
  if (mem_has_layout(mem)) layouts = all_layouts_for_shape(shape, dt);
  else layouts.push_back(Layout());
  std::vector<Aux> r;
  for (const Layout& l : layouts)
    for (u32 vs : vopts)
      for (int contig = 0; contig <= l.n; contig++) {
        Aux a;
        a.mem = mem;
        a.vector_size = (u8)vs;
        a.layout = l;
        a.layout.contig = (u8)contig;
        r.push_back(a);
      }
  return r;
}

// A bound Spec of a goal phase (precompute/src/main.rs:651-736): everything in GL,
// row-major, serial only.
struct Bound {
  SpecKind kind;   // K_MATMUL stands for the Matmul table (both accum values)
  Dtype dtype;
  Shape spec_shape;
};

// Task point layout (spec.rs:2256-2290, 2727-2760, 2839-2860): [!accum]? ++ log2(dims)
// ++ one level per operand ++ [!serial_only].
inline std::vector<u32> bound_point(const Bound& b) {
  std::vector<u32> pt;
  if (b.kind == K_MATMUL || b.kind == K_MATMUL_ACCUM) pt.push_back(b.kind == K_MATMUL ? 1 : 0);
  for (int i = 0; i < b.spec_shape.n; i++) {
    if (!is_pow2(b.spec_shape[i])) throw ModelError("task grid needs power-of-two dims");
    pt.push_back(bit_length(b.spec_shape[i]) - 1);
  }
  for (int i = 0; i < kind_operand_count(b.kind); i++) pt.push_back(GL);
  pt.push_back(0);  // serial_only = true
  return pt;
}

// LogicalSpecSurMap::apply_inverse followed by the is_canonical filter
// (precompute/src/main.rs:312-324).
inline std::vector<LogicalSpec> task_point_specs(const Bound& b, const std::vector<u32>& pt) {
  LogicalSpec proto;
  size_t p = 0;
  bool is_mm = (b.kind == K_MATMUL || b.kind == K_MATMUL_ACCUM);
  if (is_mm) proto.kind = pt[p++] == 0 ? K_MATMUL_ACCUM : K_MATMUL;
  else proto.kind = b.kind;
  proto.dtype = b.dtype;
  proto.spec_shape.n = b.spec_shape.n;
  for (int i = 0; i < b.spec_shape.n; i++) proto.spec_shape.d[i] = 1u << pt[p++];
  int nops = proto.nops();
  std::vector<std::vector<Aux>> variants(nops);
  for (int i = 0; i < nops; i++) {
    // is_canonical is per operand (plus one cross-operand rule for Moves, checked below), so
    // the operand's variants are filtered before the product is taken.
    const Shape shp = proto.operand_shape(i);
    for (const Aux& a : aux_variants(shp, b.dtype, (Mem)pt[p++]))
      if (check_tensor_vector_size(shp, b.dtype, a.mem, a.vector_size) == CANON_OK && aux_is_canonical(a, shp))
        variants[i].push_back(a);
    if (variants[i].empty()) return {};
  }
  proto.serial_only = pt[p++] == 0;
  std::vector<LogicalSpec> out;
  std::vector<size_t> idx(nops, 0);
  while (true) {
    LogicalSpec l = proto;
    for (int i = 0; i < nops; i++) l.aux[i] = variants[i][idx[i]];
    if (logicalspec_is_canonical(l)) out.push_back(l);
    int k = nops - 1;
    while (k >= 0) {
      if (++idx[k] < variants[k].size()) break;
      idx[k] = 0;
      k--;
    }
    if (k < 0) break;
  }
  return out;
}

enum Through : u8 { THROUGH_MOVE = 0, THROUGH_ZERO = 1, THROUGH_MATMUL = 2 };

// goal_phases (precompute/src/main.rs:454-507) restricted to the Move, Zero and Matmul
// bounds. DTYPES = [u32, f32] (:55); Move/Zero ranks 1..=3.
inline std::vector<std::vector<Bound>> goal_phases(u32 size, Through through, const std::vector<Dtype>& dtypes) {
  std::vector<std::vector<Bound>> phases;
  std::vector<Bound> moves;
  for (int rank = 1; rank <= 3; rank++)
    for (Dtype dt : dtypes) {
      Bound b{K_MOVE, dt, Shape()};
      b.spec_shape.n = (u8)rank;
      for (int i = 0; i < rank; i++) b.spec_shape.d[i] = size;
      moves.push_back(b);
    }
  phases.push_back(moves);
  if (through == THROUGH_MOVE) return phases;
  std::vector<Bound> zeros;
  for (int rank = 1; rank <= 3; rank++)
    for (Dtype dt : dtypes) {
      Bound b{K_FILL_ZERO, dt, Shape()};
      b.spec_shape.n = (u8)rank;
      for (int i = 0; i < rank; i++) b.spec_shape.d[i] = size;
      zeros.push_back(b);
    }
  phases.push_back(zeros);
  if (through == THROUGH_ZERO) return phases;
  std::vector<Bound> mms;
  for (Dtype dt : dtypes) mms.push_back(Bound{K_MATMUL, dt, Shape{1, size, size, size}});
  phases.push_back(mms);
  return phases;
}

}  // namespace mrl

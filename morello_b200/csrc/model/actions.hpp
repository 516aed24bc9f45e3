// Candidate tabulation: the ordered action list of a logical Spec, reduced to the
// limits-independent facts the combine kernel needs.
//
// The action list of a Spec depends only on its logical part; memory limits decide
// applicability at evaluation time (morello/src/spec.rs:4551-4553). For every action
// that can apply at SOME limits this emits one Candidate: its ActionNum (index in the
// reference's enumeration order, counting inapplicable actions too,
// morello/src/search/spectask.rs:66), a combine kind, integer immediates, the memory
// it consumes and its sub-Specs in request order.
//
// Restates: morello/src/target/cpu.rs:455-823 (Target::actions), :896-1879 (kernel
// applicability), :1881-1998 (kernel memory), :2000-2380 (kernel cost), :2719-2808
// (broadcastvecmult_side); morello/src/target/common_actions.rs:37-121 (tile-outs),
// :123-249 (splits), :301-376 (moves); morello/src/scheduling/tiling.rs:132-228,478-541
// (TileOut/Split solvers); morello/src/scheduling/moves.rs:118-138,275-381,383-528
// (Move solver); morello/src/scheduling/to_accum.rs:12-62; morello/src/scheduling/select.rs:13-56.
#pragma once
#include "spec.hpp"
#include <cstring>
#include <memory>
#include <unordered_map>

namespace mrl {

// How a candidate's Cost is combined from its children (morello/src/scheduling/mod.rs:286-368).
enum CombineKind : u8 {
  CK_LEAF = 0,   // Select(kernel): no children; cost and allocation are constants
  CK_LOOP = 1,   // TileOut / Split without boundary: main = child.main * iters (saturating),
                 //   peaks = child's, depth = 1
  CK_MOVE = 2,   // Move: main = base + sum(children) (saturating), peaks fold own + child,
                 //   depth = max + 1; children see limits lowered by `units` in `level`
  CK_BLOCK = 3,  // ToAccum: main = sum(children) (saturating), peaks = fold with no own
                 //   allocation, depth = max + 1; same limits
};

struct Candidate {
  u16 action = 0;
  u8 kind = CK_LEAF;
  u8 nchild = 0;
  u32 imm = 0;    // LEAF: kernel main cost; LOOP: iteration count; MOVE: base main cost
  u8 level = 0;   // memory index that `units` refers to
  u32 units = 0;  // MOVE: units consumed in `level`; LEAF: kernel allocation in `level`
  LogicalSpec child[3];
  // Optional memo slots for the ids a caller gives to child[j] (see MoveMemo): Move prologues
  // and epilogues depend on the moved operand only and recur across thousands of parent Specs.
  u32* child_id_slot[3] = {nullptr, nullptr, nullptr};
  // What the action is, for printing a reconstructed implementation (no effect on the fill).
  u8 what = 0;    // ActionWhat
  u8 arg0 = 0;    // Move: operand index; TileOut: dimension; Kernel: LeafKernel
  u8 arg1 = 0;    // Move: destination memory
  u32 arg2 = 0;   // Move: vector size; TileOut: tile size; Split: k
  Layout lay;     // Move: destination layout as enumerated
};

enum ActionWhat : u8 { ACT_MOVE = 0, ACT_TILE_OUT = 1, ACT_SPLIT = 2, ACT_KERNEL = 3, ACT_TO_ACCUM = 4 };

// ---- leaf kernels ----
inline bool is_rf_or_l1(Mem m) { return m == RF || m == L1; }

// broadcastvecmult_side(..).is_some() (cpu.rs:2719-2808)
inline bool broadcastvecmult_applies(const TensorSpec* op) {
  const TensorSpec& out = op[2];
  if (out.aux.mem != VRF || !out.is_contiguous()) return false;
  if (!op[0].is_contiguous() || !op[1].is_contiguous()) return false;
  if (op[0].shape[0] != out.shape[0] || op[1].shape[0] != out.shape[0]) return false;
  u32 ovs = out.aux.vector_size;
  if (ovs == 0) return false;
  if (out.volume() % ovs != 0) return false;
  const int pairs[2][2] = {{0, 1}, {1, 0}};
  for (auto& pr : pairs) {
    const TensorSpec& scalar = op[pr[0]];
    const TensorSpec& bcast = op[pr[1]];
    if (!is_rf_or_l1(scalar.aux.mem) || !scalar.is_contiguous() || bcast.aux.mem != VRF || !bcast.is_contiguous()) continue;
    if (!scalar.shape.all_ones()) continue;
    if (bcast.aux.vector_size != ovs || bcast.volume() % ovs != 0) continue;
    u32 b1 = bcast.shape[1], b2 = bcast.shape[2], s1 = scalar.shape[1], s2 = scalar.shape[2];
    u32 o1 = out.shape[1], o2 = out.shape[2];
    if (s1 == o1 && s2 == 1 && b1 == 1 && b2 == o2) return true;
    if (s1 == 1 && s2 == o2 && b1 == o1 && b2 == 1) return true;
  }
  return false;
}

struct LeafInfo { bool applies = false; u32 main = 0; u8 level = 0; u32 units = 0; };

enum LeafKernel : u8 { LK_MULTADD, LK_BCAST_VEC_MULTADD, LK_DOT_PRODUCT_LOOP, LK_ASSIGN, LK_MEMSET_ZERO, LK_VALUE_ZERO, LK_VECTOR_ZERO };

inline LeafInfo leaf_kernel_info(LeafKernel k, const LogicalSpec& spec) {
  LeafInfo r;
  TensorSpec op[MAX_OPS];
  for (int i = 0; i < spec.nops(); i++) op[i] = spec.operand(i);
  // cost of touching every operand once; only the scalar kernels charge it, and it is the
  // expensive part (a layout expansion per operand), so it is computed where it is used
  auto io_cost = [&]() {
    u32 io = 0;
    for (int i = 0; i < spec.nops(); i++) io += move_cost(op[i]);
    return io;
  };
  switch (k) {
    case LK_MULTADD: {  // cpu.rs:914-921, 2315-2340
      if (spec.kind != K_MATMUL_ACCUM) return r;
      for (int i = 0; i < 3; i++) if (!is_rf_or_l1(op[i].aux.mem) || !op[i].shape.all_ones()) return r;
      r.applies = true;
      r.main = (spec.dtype == DT_F32 ? 1 : (spec.dtype == DT_BF16 ? 30 : 2)) + io_cost();
      return r;
    }
    case LK_BCAST_VEC_MULTADD: {  // cpu.rs:922-943, 1884-1897, 2010-2036
      if (spec.kind != K_MATMUL_ACCUM) return r;
      if (spec.dtype == DT_BF16) return r;
      if (!broadcastvecmult_applies(op)) return r;
      r.applies = true;
      u32 vcount = (u32)op[2].volume() / op[2].aux.vector_size;
      r.main = vcount * 2 + 1;
      r.level = VRF; r.units = 1;
      return r;
    }
    case LK_DOT_PRODUCT_LOOP: {  // cpu.rs:988-1031, 1910-1923, 2037-2042
      if (spec.kind != K_MATMUL_ACCUM || spec.dtype != DT_F32) return r;
      const TensorSpec &lhs = op[0], &rhs = op[1], &out = op[2];
      if (lhs.shape[0] != 1 || lhs.shape[1] != 1) return r;
      if (lhs.shape[2] % 8 != 0) return r;  // vector_accum_count(k, 8).is_some()
      if (!out.shape.all_ones()) return r;
      if (!lhs.aux.layout.is_row_major() || !rhs.aux.layout.is_col_major()) return r;
      if (!lhs.is_contiguous() || !rhs.is_contiguous()) return r;
      if (lhs.aux.vector_size != 0 && lhs.aux.vector_size != 8) return r;
      if (rhs.aux.vector_size != 0 && rhs.aux.vector_size != 8) return r;
      if (!(lhs.aux.mem == L1 || (lhs.aux.mem == VRF && lhs.aux.vector_size == 8))) return r;
      if (rhs.aux.mem != L1 || !is_rf_or_l1(out.aux.mem)) return r;
      r.applies = true;
      r.main = 8 * lhs.shape[2] / 32 + move_cost(out);
      r.level = VRF; r.units = 1;
      return r;
    }
    case LK_ASSIGN: {  // cpu.rs:1694-1745, 2351-2370
      if (spec.kind != K_MOVE) return r;
      bool scalar = op[0].shape.all_ones() && op[1].shape.all_ones();
      if (scalar) {
        if (op[0].aux.layout != op[1].aux.layout) return r;
        if (!is_rf_or_l1(op[0].aux.mem) || !is_rf_or_l1(op[1].aux.mem)) return r;
        r.applies = true;
        r.main = io_cost() + 1;
        return r;
      }
      if (!op[0].is_contiguous() || !op[1].is_contiguous()) return r;
      if (op[0].aux.layout != op[1].aux.layout) return r;
      bool has_vrf = false;
      for (int i = 0; i < 2; i++) {
        if (mem_is_vector(op[i].aux.mem)) {
          has_vrf = true;
          if (op[i].volume() % op[i].aux.vector_size != 0) return r;
        }
      }
      if (!has_vrf) return r;
      r.applies = true;
      u32 vs = op[0].aux.vector_size ? op[0].aux.vector_size : op[1].aux.vector_size;
      r.main = (u32)op[0].volume() / vs;
      return r;
    }
    case LK_MEMSET_ZERO: {  // cpu.rs:1812-1821, 2371
      if (spec.kind != K_FILL_ZERO) return r;
      if (op[0].aux.mem == RF || op[0].aux.mem == VRF || !op[0].is_contiguous()) return r;
      r.applies = true; r.main = 1;
      return r;
    }
    case LK_VALUE_ZERO: {  // cpu.rs:1822-1831, 2057-2069
      if (spec.kind != K_FILL_ZERO) return r;
      if (op[0].volume() != 1 || !is_rf_or_l1(op[0].aux.mem)) return r;
      r.applies = true; r.main = io_cost() + 1;
      return r;
    }
    case LK_VECTOR_ZERO: {  // cpu.rs:1832-1856, 2372-2378
      if (spec.kind != K_FILL_ZERO) return r;
      if (!op[0].is_contiguous() || op[0].aux.mem != VRF) return r;
      if (op[0].aux.vector_size == 0 || op[0].aux.vector_size != op[0].volume()) return r;
      r.applies = true; r.main = 1;
      return r;
    }
  }
  return r;
}

// ---- Move planning (scheduling/moves.rs:275-381 plan_alloc_shared, :383-528) ----
struct MovePlan {
  bool applies = false;
  TensorSpec new_spec;
  bool cache_miss = false;
  u64 units = 0;
};

inline MovePlan plan_move(const TensorSpec& src, Mem dest, const Layout& dest_layout, u32 dest_vs) {
  MovePlan p;
  Layout lay;
  bool miss = false;
  if (!mem_has_layout(dest)) {
    lay = Layout();
    miss = false;  // RF is addressed: never a cache miss
  } else if (!mem_is_addressed(dest)) {
    if (!layout_canonicalize(dest_layout, src.shape, lay))
      throw ModelError("destination layout does not apply to the moved tensor");
    miss = (src.aux.layout == lay);
    if (!miss) lay.contig = lay.n;
  } else {
    lay = dest_layout;
    lay.contig = lay.n;
  }
  p.new_spec.shape = src.shape;
  p.new_spec.dtype = src.dtype;
  p.new_spec.aux.mem = dest;
  p.new_spec.aux.layout = lay;
  p.new_spec.aux.vector_size = (u8)dest_vs;
  if (!miss) {
    if (tensorspec_canonicalize(p.new_spec) != CANON_OK) return p;
  }
  if (src == p.new_spec) return p;  // SelfMove
  p.cache_miss = miss;
  p.units = tensorspec_memory_units(p.new_spec);
  p.applies = true;
  return p;
}

inline LogicalSpec make_move_spec(const TensorSpec& left, const TensorSpec& right, bool serial_only) {
  LogicalSpec l;
  l.kind = K_MOVE;
  l.dtype = left.dtype;
  l.serial_only = serial_only;
  l.spec_shape = left.shape;
  l.aux[0] = left.aux;
  l.aux[1] = right.aux;
  canonicalize_matching_contiguous_move_auxes(l);
  return l;
}

// Leaf kernels in per-kind order; inapplicable kernels take no action number (cpu.rs:477-611).
// Appends the applicable ones numbered from first_action and returns the next free number. This
// is the only part of a Spec's candidate list that depends on the dtype itself rather than on
// its byte size.
inline u32 tabulate_leaves(const LogicalSpec& spec, u32 first_action, std::vector<Candidate>& out) {
  u32 action = first_action;
  static const LeafKernel accum_ks[] = {LK_MULTADD, LK_BCAST_VEC_MULTADD, LK_DOT_PRODUCT_LOOP};
  static const LeafKernel move_ks[] = {LK_ASSIGN};
  static const LeafKernel zero_ks[] = {LK_MEMSET_ZERO, LK_VALUE_ZERO, LK_VECTOR_ZERO};
  const LeafKernel* ks = nullptr;
  int nk = 0;
  switch (spec.kind) {
    case K_MATMUL_ACCUM: ks = accum_ks; nk = 3; break;
    case K_MOVE: ks = move_ks; nk = 1; break;
    case K_FILL_ZERO: ks = zero_ks; nk = 3; break;
    default: break;
  }
  for (int i = 0; i < nk; i++) {
    LeafInfo li = leaf_kernel_info(ks[i], spec);
    if (!li.applies) continue;
    Candidate c;
    c.action = (u16)action++;
    c.kind = CK_LEAF;
    c.nchild = 0;
    c.imm = li.main;
    c.level = li.level;
    c.units = li.units;
    c.what = ACT_KERNEL;
    c.arg0 = (u8)ks[i];
    out.push_back(c);
  }
  return action;
}

// ---- Moves of one operand (common_actions.rs:301-376), independent of the rest of the Spec ----
struct MoveOption {
  u16 action_rel = 0;      // position among the operand's enumerated Moves
  u8 mem = 0;              // destination memory
  u32 vs = 0;              // destination vector size
  Layout layout;           // destination layout as enumerated
  Aux new_aux;             // the moved operand afterwards
  bool cache_miss = false;
  u32 units = 0;
  u32 imm = 0;             // move cost of source + destination
  u32 pro_id = 0xFFFFFFFFu, epi_id = 0xFFFFFFFFu;  // memo slots for the caller's ids of the Move Specs below
  LogicalSpec pro, epi;    // prologue Move(source -> new), epilogue Move(new -> source)
};
struct OperandMoves {
  u32 n_actions = 0;       // enumerated Moves of the operand, applicable or not
  std::vector<MoveOption> opts;  // the applicable ones, in enumeration order
};

inline void operand_moves(const TensorSpec& op, bool serial_only, OperandMoves& out) {
  out.n_actions = 0;
  out.opts.clear();
  const u32 src_cost = move_cost(op);
  auto emit = [&](Mem mem, const Layout& layout, u32 vs) {
    const u32 rel = out.n_actions++;
    MovePlan p = plan_move(op, mem, layout, vs);
    if (!p.applies) return;
    MoveOption o;
    o.action_rel = (u16)rel;
    o.mem = (u8)mem;
    o.vs = vs;
    o.layout = layout;
    o.new_aux = p.new_spec.aux;
    o.cache_miss = p.cache_miss;
    o.units = (u32)p.units;
    o.imm = src_cost + move_cost(p.new_spec);
    o.pro = make_move_spec(op, p.new_spec, serial_only);
    o.epi = make_move_spec(p.new_spec, op, serial_only);
    out.opts.push_back(o);
  };
  std::vector<Layout> dest_layouts = move_destination_layouts(op.shape, op.dtype);
  std::vector<Mem> dest_mems = possible_destination_memories(op.aux.mem);
  bool contains_source_layout = false;
  for (const Layout& layout : dest_layouts) {
    if (!contains_source_layout && layout == op.aux.layout) contains_source_layout = true;
    for (Mem mem : dest_mems) {
      const std::vector<u32>& vb = mem_vector_bytes(mem);
      if (vb.empty()) emit(mem, layout, 0);
      else for (u32 b : vb) emit(mem, layout, b / dtype_size(op.dtype));
    }
  }
  if (!contains_source_layout) {
    for (Mem mem : dest_mems) {
      if (mem_is_addressed(mem)) continue;
      emit(mem, op.aux.layout, 0);  // caches have no vector sizes
    }
  }
}

// What tiling does to one operand: its aux after the layout is updated for the tile shape and
// canonicalised (tiling.rs:132-228 per operand; tensorspec.rs:232-236,370-377).
struct TileResult {
  bool applies = false;  // the layout applies to the tile shape (TensorSpec::is_valid_tile_shape)
  bool ok = false;       // ... and the tiled operand canonicalises
  Aux aux;
};
inline TileResult tile_operand(const TensorSpec& op, const Shape& tile) {
  TileResult r;
  r.aux = op.aux;
  if (mem_has_layout(op.aux.mem)) {
    Layout nl;
    if (!layout_update_for_tiling(op.aux.layout, op.shape, tile, nl)) return r;
    r.aux.layout = nl;
  }
  r.applies = true;
  if (check_tensor_vector_size(tile, op.dtype, r.aux.mem, r.aux.vector_size) != CANON_OK) return r;
  if (!aux_canonicalize(r.aux, tile)) return r;
  r.ok = true;
  return r;
}

// Memo of operand_moves and tile_operand by operand (shape, dtype, aux). One per thread;
// entries never move.
class MoveMemo {
 public:
  const TileResult& tile(const TensorSpec& op, const Shape& tile_shape) {
    Key key;
    int p = operand_key(op, false, key.bytes);
    for (int i = 0; i < tile_shape.n; i++) { key.bytes[p++] = (char)(tile_shape[i] & 0xff); key.bytes[p++] = (char)(tile_shape[i] >> 8); }
    key.len = (u8)p;
    auto it = tiles_.find(key);
    if (it != tiles_.end()) return it->second;
    return tiles_.emplace(key, tile_operand(op, tile_shape)).first->second;
  }
  OperandMoves& get(const TensorSpec& op, bool serial_only) {
    Key key;
    key.len = (u8)operand_key(op, serial_only, key.bytes);
    auto it = map_.find(key);
    if (it != map_.end()) return *it->second;
    std::unique_ptr<OperandMoves> om(new OperandMoves());
    operand_moves(op, serial_only, *om);
    OperandMoves& ref = *om;
    map_.emplace(key, std::move(om));
    return ref;
  }
  size_t size() const { return map_.size(); }

 private:
  // An operand (and, for tiles, the tile shape) as bytes, held inline: a lookup allocates nothing.
  struct Key {
    static constexpr int CAP = 8 + 4 * MAX_RANK + 4 + 4 * MAX_PHYS;
    char bytes[CAP];
    u8 len = 0;
    bool operator==(const Key& o) const { return len == o.len && memcmp(bytes, o.bytes, len) == 0; }
  };
  struct KeyHash {
    size_t operator()(const Key& k) const {
      u64 h = 0x9E3779B97F4A7C15ull ^ k.len;
      int i = 0;
      for (; i + 8 <= k.len; i += 8) { u64 w; memcpy(&w, k.bytes + i, 8); h = (h ^ w) * 0xD6E8FEB86659FD93ull; h ^= h >> 32; }
      u64 w = 0;
      if (i < k.len) memcpy(&w, k.bytes + i, (size_t)(k.len - i));
      h = (h ^ w) * 0xD6E8FEB86659FD93ull;
      return (size_t)(h ^ (h >> 29));
    }
  };
  static int operand_key(const TensorSpec& op, bool flag, char* kb) {
    int p = 0;
    kb[p++] = (char)op.dtype; kb[p++] = (char)flag; kb[p++] = (char)op.shape.n; kb[p++] = (char)op.aux.mem;
    kb[p++] = (char)op.aux.vector_size; kb[p++] = (char)op.aux.layout.n; kb[p++] = (char)op.aux.layout.contig; kb[p++] = 0;
    for (int i = 0; i < op.shape.n; i++) { kb[p++] = (char)(op.shape[i] & 0xff); kb[p++] = (char)(op.shape[i] >> 8); }
    for (int j = 0; j < op.aux.layout.n; j++) {
      kb[p++] = (char)op.aux.layout.d[j].ldim; kb[p++] = (char)op.aux.layout.d[j].kind;
      kb[p++] = (char)(op.aux.layout.d[j].size & 0xff); kb[p++] = (char)(op.aux.layout.d[j].size >> 8);
    }
    return p;
  }
  std::unordered_map<Key, std::unique_ptr<OperandMoves>, KeyHash> map_;
  std::unordered_map<Key, TileResult, KeyHash> tiles_;
};

// The body Spec of a tile-out or split: `body` comes in with the new spec_shape; every operand's
// aux is updated for its new shape and canonicalised. False: the action does not apply.
inline bool tile_body(const LogicalSpec& spec, const TensorSpec* ops, int nops, LogicalSpec& body, MoveMemo* memo) {
  if (memo) {
    for (int j = 0; j < nops; j++) {
      const TileResult& t = memo->tile(ops[j], body.operand_shape(j));
      if (!t.ok) return false;
      body.aux[j] = t.aux;
    }
    if (body.kind == K_MOVE) canonicalize_matching_contiguous_move_auxes(body);
    return true;
  }
  for (int j = 0; j < nops; j++) {
    if (!mem_has_layout(ops[j].aux.mem)) continue;
    Layout nl;
    if (!layout_update_for_tiling(ops[j].aux.layout, ops[j].shape, body.operand_shape(j), nl)) return false;
    body.aux[j].layout = nl;
  }
  (void)spec;
  return logicalspec_canonicalize(body) == CANON_OK;
}

// ---- the enumeration ----
// Returns the total number of enumerated actions (applicable or not); [*leaf_first, *leaf_end) =
// the action numbers of the leaf-kernel section.
inline u32 tabulate_candidates(const LogicalSpec& spec, std::vector<Candidate>& out, u32* leaf_first = nullptr,
                               u32* leaf_end = nullptr, MoveMemo* memo = nullptr) {
  if (!spec.serial_only) throw ModelError("only serial-only Specs are tabulated");
  u32 action = 0;
  const int nops = spec.nops();
  TensorSpec ops[MAX_OPS];
  for (int i = 0; i < nops; i++) ops[i] = spec.operand(i);

  // 1. Moves (common_actions.rs:301-376): per operand, from the memo when there is one
  for (int i = 0; i < nops; i++) {
    OperandMoves local;
    OperandMoves* om = &local;
    if (memo) om = &memo->get(ops[i], spec.serial_only);
    else operand_moves(ops[i], spec.serial_only, local);
    const Direction dir = kind_direction(spec.kind, i);
    for (MoveOption& o : om->opts) {
      Candidate c;
      c.action = (u16)(action + o.action_rel);
      c.kind = CK_MOVE;
      c.level = o.mem;
      c.units = o.units;
      c.imm = o.imm;
      const bool prologue = !o.cache_miss && (dir == DIR_IN || dir == DIR_INOUT);
      const bool epilogue = !o.cache_miss && (dir == DIR_OUT || dir == DIR_INOUT);
      int n = 0;
      if (prologue) { c.child[n] = o.pro; c.child_id_slot[n] = memo ? &o.pro_id : nullptr; n++; }
      LogicalSpec body = spec;
      body.aux[i] = o.new_aux;
      if (body.kind == K_MOVE) canonicalize_matching_contiguous_move_auxes(body);
      c.child[n++] = body;
      if (epilogue) { c.child[n] = o.epi; c.child_id_slot[n] = memo ? &o.epi_id : nullptr; n++; }
      c.nchild = (u8)n;
      c.what = ACT_MOVE;
      c.arg0 = (u8)i;
      c.arg1 = o.mem;
      c.arg2 = o.vs;
      c.lay = o.layout;
      out.push_back(c);
    }
    action += om->n_actions;
  }

  // 2. Serial single-loop tile-outs (common_actions.rs:37-121; tiling.rs:132-228)
  {
    const int oi = kind_output_index(spec.kind);
    const Shape out_shape = ops[oi].shape;
    u32 max_dim = 0;
    for (int d = 0; d < out_shape.n; d++) if (out_shape[d] > max_dim) max_dim = out_shape[d];
    for (u32 size : dim_range_pow2(max_dim, true)) {
      for (int dim = 0; dim < out_shape.n; dim++) {
        u32 this_action = action++;
        if (out_shape[dim] == size) continue;  // TileShapeMatchesOriginal
        if (size > out_shape[dim]) continue;   // TileShapeIsLarger
        Shape tile = out_shape;
        tile[dim] = size;
        if (memo ? !memo->tile(ops[oi], tile).applies : !tensorspec_valid_tile_shape(ops[oi], tile)) continue;
        if (out_shape[dim] % size != 0) throw ModelError("boundary tile-outs are outside the tabulated space");
        LogicalSpec body = spec;
        if (spec.kind == K_MATMUL || spec.kind == K_MATMUL_ACCUM) {
          body.spec_shape[0] = tile[0]; body.spec_shape[1] = tile[1]; body.spec_shape[3] = tile[2];
        } else {
          body.spec_shape = tile;
        }
        if (!tile_body(spec, ops, nops, body, memo)) continue;
        Candidate c;
        c.action = (u16)this_action;
        c.kind = CK_LOOP;
        c.nchild = 1;
        u64 iters = 1;
        for (int d = 0; d < spec.spec_shape.n; d++) iters *= spec.spec_shape[d] / body.spec_shape[d];
        if (iters > 0xFFFFFFFFull) throw ModelError("loop iteration count overflows u32");
        c.imm = (u32)iters;
        c.child[0] = body;
        c.what = ACT_TILE_OUT;
        c.arg0 = (u8)dim;
        c.arg2 = size;
        out.push_back(c);
      }
    }
  }

  // 3. Leaf kernels
  if (leaf_first) *leaf_first = action;
  action = tabulate_leaves(spec, action, out);
  if (leaf_end) *leaf_end = action;

  // 4. Kind-specific tail (cpu.rs:685-699)
  if (spec.kind == K_MATMUL) {  // ToAccum (to_accum.rs:12-62; mod.rs:526-546)
    Candidate c;
    c.action = (u16)action++;
    c.kind = CK_BLOCK;
    c.nchild = 2;
    LogicalSpec fill;
    fill.kind = K_FILL_ZERO;
    fill.dtype = spec.dtype;
    fill.serial_only = spec.serial_only;
    fill.spec_shape = ops[2].shape;
    fill.aux[0] = ops[2].aux;
    if (logicalspec_canonicalize(fill) != CANON_OK) throw ModelError("ToAccum: Fill is not canonicalizable");
    LogicalSpec acc = spec;
    acc.kind = K_MATMUL_ACCUM;
    if (logicalspec_canonicalize(acc) != CANON_OK) throw ModelError("ToAccum: accumulating Spec is not canonicalizable");
    c.child[0] = fill;
    c.child[1] = acc;
    c.what = ACT_TO_ACCUM;
    out.push_back(c);
  } else if (spec.kind == K_MATMUL_ACCUM) {  // Split (common_actions.rs:123-197; tiling.rs:478-541)
    const u32 b = spec.spec_shape[0], m = spec.spec_shape[1], K = spec.spec_shape[2], n = spec.spec_shape[3];
    for (u32 k : dim_range_pow2(K, false)) {
      if (memo ? (!memo->tile(ops[0], Shape{b, m, k}).applies || !memo->tile(ops[1], Shape{b, k, n}).applies)
               : (!tensorspec_valid_tile_shape(ops[0], Shape{b, m, k}) || !tensorspec_valid_tile_shape(ops[1], Shape{b, k, n}))) continue;
      u32 this_action = action++;
      if (K % k != 0) throw ModelError("boundary splits are outside the tabulated space");
      LogicalSpec body = spec;
      body.spec_shape[2] = k;
      if (!tile_body(spec, ops, nops, body, memo)) continue;
      Candidate c;
      c.action = (u16)this_action;
      c.kind = CK_LOOP;
      c.nchild = 1;
      c.imm = K / k;
      c.child[0] = body;
      c.what = ACT_SPLIT;
      c.arg2 = k;
      out.push_back(c);
    }
  }
  return action;
}

}  // namespace mrl

// Tensor specs and logical Specs (the scheduling problems the database is keyed by).
//
// Restates, for the Spec kinds the Matmul closure needs (Move, Fill-zero, Matmul,
// MatmulAccum) with serial-only Specs:
//   morello/src/tensorspec.rs:19-32,140-173,232-250,370-388,566-637
//   morello/src/spec.rs:33-53,57-162 (types), :467-583 (parameter shapes),
//     :1204-1282 (operand directions), :1704-1800 (canonicalize), :1801-1850 (is_canonical)
#pragma once
#include "layout.hpp"

namespace mrl {

struct Aux {
  Mem mem = GL;
  u8 vector_size = 0;  // values per vector register; 0 = none (only VRF has one)
  Layout layout;
  bool operator==(const Aux& o) const { return mem == o.mem && vector_size == o.vector_size && layout == o.layout; }
  bool operator!=(const Aux& o) const { return !(*this == o); }
};

struct TensorSpec {
  Shape shape;
  Dtype dtype = DT_U32;
  Aux aux;
  bool operator==(const TensorSpec& o) const { return shape == o.shape && dtype == o.dtype && aux == o.aux; }
  u64 volume() const { return shape.volume(); }
  bool is_contiguous() const { return aux.layout.fully_contiguous(); }
};

enum CanonErr : u8 { CANON_OK = 0, CANON_LAYOUT = 1, CANON_VECTOR_INVALID = 2, CANON_VECTOR_VOLUME = 3 };

// check_tensor_vector_size (tensorspec.rs:608-637)
inline CanonErr check_tensor_vector_size(const Shape& shape, Dtype dt, Mem mem, u32 vector_size) {
  const std::vector<u32>& allowed = mem_vector_bytes(mem);
  if (allowed.empty()) return CANON_OK;
  if (vector_size == 0) throw ModelError("vector memory without a vector size");
  u32 vbytes = vector_size * dtype_size(dt);
  bool found = false;
  for (u32 vb : allowed) if (vb == vbytes) found = true;
  if (!found) return CANON_VECTOR_INVALID;
  u32 volume = (u32)shape.volume();
  u32 bytes = volume * dtype_size(dt);
  bool any = false;
  for (u32 vb : allowed) if (bytes % vb == 0) any = true;
  if (!any) return CANON_VECTOR_INVALID;
  if (volume % vector_size != 0) return CANON_VECTOR_VOLUME;
  return CANON_OK;
}

// TensorSpecAux::canonicalize (tensorspec.rs:370-377)
inline bool aux_canonicalize(Aux& a, const Shape& shape) {
  if (!mem_has_layout(a.mem)) { a.layout = Layout(); return true; }
  Layout out;
  if (!layout_update_for_tiling(a.layout, shape, shape, out)) return false;
  a.layout = out;
  return true;
}
// TensorSpecAux::is_canonical (tensorspec.rs:379-387)
inline bool aux_is_canonical(const Aux& a, const Shape& shape) {
  if (!mem_has_layout(a.mem)) return a.layout.is_empty();
  Layout out;
  if (!layout_update_for_tiling(a.layout, shape, shape, out)) return false;
  return out == a.layout;
}
// TensorSpec::canonicalize (tensorspec.rs:232-236)
inline CanonErr tensorspec_canonicalize(TensorSpec& t) {
  CanonErr e = check_tensor_vector_size(t.shape, t.dtype, t.aux.mem, t.aux.vector_size);
  if (e != CANON_OK) return e;
  return aux_canonicalize(t.aux, t.shape) ? CANON_OK : CANON_LAYOUT;
}
// TensorSpec::is_valid_tile_shape with parallel_loop = false (tensorspec.rs:140-152)
inline bool tensorspec_valid_tile_shape(const TensorSpec& t, const Shape& tile) {
  return !mem_has_layout(t.aux.mem) || layout_applies_to_shape(t.aux.layout, tile);
}
// TensorSpec::memory_units (tensorspec.rs:161-173)
inline u64 tensorspec_memory_units(const TensorSpec& t) {
  if (mem_counts_registers(t.aux.mem)) {
    u32 vol = (u32)t.volume();
    if (t.aux.vector_size) return (vol + t.aux.vector_size - 1) / t.aux.vector_size;
    return vol;
  }
  return layout_estimate_cache_lines(t.aux.layout, t.shape, t.dtype);
}
// move_cost (imp/allocs.rs:156-173)
inline u32 move_cost(const TensorSpec& t) {
  u32 cost = 0;
  if (mem_has_layout(t.aux.mem)) {
    cost = mem_hit_cost(t.aux.mem) * layout_estimate_cache_lines(t.aux.layout, t.shape, t.dtype);
  }
  if (!t.is_contiguous()) cost *= 2;
  return cost;
}

// ---- logical Specs ----
enum SpecKind : u8 { K_MOVE = 0, K_FILL_ZERO = 1, K_MATMUL_ACCUM = 2, K_MATMUL = 3 };
constexpr int MAX_OPS = 3;

inline int kind_operand_count(SpecKind k) { return k == K_MOVE ? 2 : (k == K_FILL_ZERO ? 1 : 3); }
inline int kind_output_index(SpecKind k) { return k == K_MOVE ? 1 : (k == K_FILL_ZERO ? 0 : 2); }
inline const char* kind_name(SpecKind k) {
  static const char* n[] = {"Move", "FillZero", "MatmulAccum", "Matmul"};
  return n[k];
}
enum Direction : u8 { DIR_IN = 0, DIR_OUT = 1, DIR_INOUT = 2 };
inline Direction kind_direction(SpecKind k, int idx) {  // spec.rs:1204-1246
  switch (k) {
    case K_MOVE: return idx == 0 ? DIR_IN : DIR_OUT;
    case K_FILL_ZERO: return DIR_OUT;
    case K_MATMUL_ACCUM: return idx == 2 ? DIR_INOUT : DIR_IN;
    default: return idx == 2 ? DIR_OUT : DIR_IN;
  }
}

struct LogicalSpec {
  SpecKind kind = K_MOVE;
  Dtype dtype = DT_U32;  // every operand has this dtype on the path built here
  bool serial_only = true;
  Shape spec_shape;      // Move/Fill: tensor shape; Matmul: [b, m, k, n]
  Aux aux[MAX_OPS];

  int nops() const { return kind_operand_count(kind); }
  // PrimitiveBasics::parameter_shape (spec.rs:467-583)
  Shape operand_shape(int idx) const {
    if (kind == K_MOVE || kind == K_FILL_ZERO) return spec_shape;
    switch (idx) {
      case 0: return Shape{spec_shape[0], spec_shape[1], spec_shape[2]};
      case 1: return Shape{spec_shape[0], spec_shape[2], spec_shape[3]};
      default: return Shape{spec_shape[0], spec_shape[1], spec_shape[3]};
    }
  }
  TensorSpec operand(int idx) const {
    TensorSpec t;
    t.shape = operand_shape(idx);
    t.dtype = dtype;
    t.aux = aux[idx];
    return t;
  }
  bool operator==(const LogicalSpec& o) const {
    if (kind != o.kind || dtype != o.dtype || serial_only != o.serial_only || spec_shape != o.spec_shape) return false;
    for (int i = 0; i < nops(); i++) if (aux[i] != o.aux[i]) return false;
    return true;
  }
  u64 volume() const { return spec_shape.volume(); }  // spec.rs:2133-2152

  // Compact, injective byte key (hash-map key and the C-ABI's Spec blob).
  static constexpr int MAX_KEY = 4 + 2 * MAX_RANK + MAX_OPS * (4 + 4 * MAX_PHYS);
  int key_into(char* s) const {
    int p = 0;
    s[p++] = (char)kind; s[p++] = (char)dtype; s[p++] = (char)serial_only; s[p++] = (char)spec_shape.n;
    for (int i = 0; i < spec_shape.n; i++) { s[p++] = (char)(spec_shape[i] & 0xff); s[p++] = (char)(spec_shape[i] >> 8); }
    for (int i = 0; i < nops(); i++) {
      const Aux& a = aux[i];
      s[p++] = (char)a.mem; s[p++] = (char)a.vector_size; s[p++] = (char)a.layout.n; s[p++] = (char)a.layout.contig;
      for (int j = 0; j < a.layout.n; j++) {
        s[p++] = (char)a.layout.d[j].ldim; s[p++] = (char)a.layout.d[j].kind;
        s[p++] = (char)(a.layout.d[j].size & 0xff); s[p++] = (char)(a.layout.d[j].size >> 8);
      }
    }
    return p;
  }
  std::string key() const {
    char buf[MAX_KEY];
    return std::string(buf, (size_t)key_into(buf));
  }
  static LogicalSpec from_key(const std::string& s) {
    LogicalSpec l;
    size_t p = 0;
    auto need = [&](size_t k) { if (p + k > s.size()) throw ModelError("truncated Spec key"); };
    need(4);
    l.kind = (SpecKind)(u8)s[p++]; l.dtype = (Dtype)(u8)s[p++]; l.serial_only = s[p++] != 0; l.spec_shape.n = (u8)s[p++];
    if (l.kind > K_MATMUL || l.spec_shape.n > MAX_RANK) throw ModelError("bad Spec key");
    need(2 * l.spec_shape.n);
    for (int i = 0; i < l.spec_shape.n; i++) { l.spec_shape.d[i] = (u8)s[p] | ((u32)(u8)s[p + 1] << 8); p += 2; }
    for (int i = 0; i < l.nops(); i++) {
      need(4);
      Aux& a = l.aux[i];
      a.mem = (Mem)(u8)s[p++]; a.vector_size = (u8)s[p++]; a.layout.n = (u8)s[p++]; a.layout.contig = (u8)s[p++];
      if (a.mem > GL || a.layout.n > MAX_PHYS) throw ModelError("bad Spec key");
      need(4 * a.layout.n);
      for (int j = 0; j < a.layout.n; j++) {
        a.layout.d[j].ldim = (u8)s[p++]; a.layout.d[j].kind = (u8)s[p++];
        a.layout.d[j].size = (u16)((u8)s[p] | ((u32)(u8)s[p + 1] << 8)); p += 2;
      }
    }
    if (p != s.size()) throw ModelError("trailing bytes in Spec key");
    return l;
  }

  std::string str() const {
    std::string s = kind_name(kind);
    s += "(" + spec_shape.str();
    for (int i = 0; i < nops(); i++) {
      s += ", (";
      s += dtype_name(dtype);
      s += ", ";
      s += mem_name(aux[i].mem);
      if (mem_has_layout(aux[i].mem)) s += ", " + aux[i].layout.str();
      if (aux[i].vector_size) s += ", " + std::to_string(aux[i].vector_size);
      s += ")";
    }
    s += serial_only ? ", serial)" : ")";
    return s;
  }
};

// The Move-only symmetry break (spec.rs:1717-1735; scheduling/moves.rs:447-467): equal
// dtypes, equal layouts, all fully contiguous => row-major on every layout-carrying operand.
inline void canonicalize_matching_contiguous_move_auxes(LogicalSpec& l) {
  const Layout& first = l.aux[0].layout;
  for (int i = 0; i < 2; i++) {
    if (l.aux[i].layout != first || !l.aux[i].layout.fully_contiguous()) return;
  }
  for (int i = 0; i < 2; i++) if (mem_has_layout(l.aux[i].mem)) l.aux[i].layout = layout_row_major(l.spec_shape);
}

// LogicalSpec::canonicalize for primitives (spec.rs:1704-1747)
inline CanonErr logicalspec_canonicalize(LogicalSpec& l) {
  for (int i = 0; i < l.nops(); i++) {
    Shape shp = l.operand_shape(i);
    CanonErr e = check_tensor_vector_size(shp, l.dtype, l.aux[i].mem, l.aux[i].vector_size);
    if (e != CANON_OK) return e;
    if (!aux_canonicalize(l.aux[i], shp)) return CANON_LAYOUT;
  }
  if (l.kind == K_MOVE) canonicalize_matching_contiguous_move_auxes(l);
  return CANON_OK;
}

// LogicalSpec::is_canonical for primitives (spec.rs:1801-1850)
inline bool logicalspec_is_canonical(const LogicalSpec& l) {
  for (int i = 0; i < l.nops(); i++) {
    Shape shp = l.operand_shape(i);
    if (check_tensor_vector_size(shp, l.dtype, l.aux[i].mem, l.aux[i].vector_size) != CANON_OK) return false;
    if (!aux_is_canonical(l.aux[i], shp)) return false;
  }
  if (l.kind == K_MOVE) {
    bool all_equal = l.aux[0].layout == l.aux[1].layout;
    bool all_contig = l.aux[0].layout.fully_contiguous() && l.aux[1].layout.fully_contiguous();
    bool any_nonrm = false;
    for (int i = 0; i < 2; i++)
      if (!l.aux[i].layout.is_row_major() || !l.aux[i].layout.fully_contiguous()) any_nonrm = true;
    if (all_equal && all_contig && any_nonrm) return false;
  }
  return true;
}

}  // namespace mrl

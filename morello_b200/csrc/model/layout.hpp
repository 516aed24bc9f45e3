// Tensor layouts: an ordered list of physical dimensions, each bound to a logical
// dimension, plus the length of the physically contiguous suffix.
//
// Restates morello/src/layout.rs (struct :67-81; Layout::new :205-217;
// estimate_cache_lines :318-343; canonicalize :474-484; update_for_tiling :486-499;
// lower_contig_to_first_broken_dimension :503-527; merge_consecutive_dimensions :602-669;
// drop_unneeded_packings :674-766; expand_physical_shape :769-810; builders :1234-1279)
// and the destination-layout generators of morello/src/target/cpu.rs:399-453,2878-3012.
#pragma once
#include "base.hpp"

namespace mrl {

enum PhysKind : u8 { PD_DYNAMIC = 0, PD_PACKED = 1, PD_ODDEVEN = 2 };

struct PhysDim {
  u8 ldim = 0;   // logical dimension this physical dimension walks
  u8 kind = PD_DYNAMIC;
  u16 size = 0;  // strip size for Packed / OddEven, 0 for Dynamic
  bool operator==(const PhysDim& o) const { return ldim == o.ldim && kind == o.kind && size == o.size; }
  bool operator!=(const PhysDim& o) const { return !(*this == o); }
};

constexpr int MAX_PHYS = 10;

struct Layout {
  u8 n = 0;
  u8 contig = 0;
  PhysDim d[MAX_PHYS];

  bool operator==(const Layout& o) const {
    if (n != o.n || contig != o.contig) return false;
    for (int i = 0; i < n; i++) if (d[i] != o.d[i]) return false;
    return true;
  }
  bool operator!=(const Layout& o) const { return !(*this == o); }
  bool is_empty() const { return n == 0 && contig == 0; }
  bool fully_contiguous() const { return contig == n; }
  void push(u8 ldim, u8 kind, u32 size) {
    if (n >= MAX_PHYS) throw ModelError("layout has too many physical dims");
    d[n].ldim = ldim; d[n].kind = kind; d[n].size = (u16)size; n++;
  }
  void erase(int i) { for (int j = i; j + 1 < n; j++) d[j] = d[j + 1]; n--; }

  // All-Dynamic with ascending logical dims (layout.rs:349-352).
  bool is_row_major() const {
    for (int i = 0; i < n; i++) if (d[i].kind != PD_DYNAMIC) return false;
    for (int i = 1; i < n; i++) if (d[i].ldim < d[i - 1].ldim) return false;
    return true;
  }
  // All-Dynamic with strictly descending logical dims (layout.rs:354-357).
  bool is_col_major() const {
    for (int i = 0; i < n; i++) if (d[i].kind != PD_DYNAMIC) return false;
    for (int i = 1; i < n; i++) if (!(d[i].ldim < d[i - 1].ldim)) return false;
    return true;
  }

  std::string str() const {
    std::string s = "[";
    for (int i = 0; i < n; i++) {
      if (i) s += ", ";
      s += std::to_string(d[i].ldim);
      if (d[i].kind == PD_PACKED) s += " p(" + std::to_string(d[i].size) + ")";
      if (d[i].kind == PD_ODDEVEN) s += " oe(" + std::to_string(d[i].size) + ")";
    }
    s += "]";
    if (!fully_contiguous()) s = "(" + s + ", c" + std::to_string(contig) + ")";
    return s;
  }
};

// ---- expand_physical_shape (layout.rs:769-810). Returns false when the layout does
// not apply to the logical shape. ----
inline bool layout_expand(const Layout& l, const Shape& shape, u32* phys /*[l.n]*/) {
  u32 rem[MAX_RANK];
  bool tiled[MAX_RANK];
  for (int i = 0; i < shape.n; i++) { rem[i] = shape[i]; tiled[i] = false; }
  for (int i = l.n - 1; i >= 0; i--) {
    const PhysDim& p = l.d[i];
    u32& r = rem[p.ldim];
    if (p.kind == PD_DYNAMIC) {
      if (r == 0) throw ModelError("layout has two Dynamic dims for one logical dim");
      phys[i] = r;
      r = 0;  // marks "Dynamic seen"
    } else {
      u32 ps = p.size;
      if (r < ps) {
        bool allowed = (p.kind == PD_PACKED) || r == 1;
        if (!allowed || tiled[p.ldim]) return false;
        if (r == 0) throw ModelError("packed dim outside a Dynamic dim");
        phys[i] = r;
        r = 1;
        tiled[p.ldim] = true;
      } else if (r % ps != 0) {
        return false;
      } else {
        phys[i] = ps;
        r /= ps;
      }
    }
  }
  for (int i = 0; i < shape.n; i++) if (rem[i] > 1) return false;
  return true;
}

inline bool layout_applies_to_shape(const Layout& l, const Shape& shape) {
  u32 phys[MAX_PHYS];
  return layout_expand(l, shape, phys);
}

// ---- merge_consecutive_dimensions (layout.rs:602-669) ----
inline void layout_merge_consecutive(Layout& l) {
  if (l.n == 0) return;
  const int first_contig = l.n - l.contig;
  int new_contig = l.contig;
  int w = 1;
  for (int i = 1; i < l.n; i++) {
    PhysDim cur = l.d[i];
    PhysDim& last = l.d[w - 1];
    if (cur.ldim != last.ldim) { l.d[w++] = cur; continue; }
    if (last.kind == PD_PACKED && cur.kind == PD_PACKED) {
      if (i == first_contig) { l.d[w++] = cur; }
      else {
        last.size = (u16)(u32(last.size) * cur.size);
        if (i >= first_contig) new_contig--;
      }
    } else if (last.kind == PD_DYNAMIC && cur.kind == PD_PACKED) {
      if (i <= first_contig) { l.d[w++] = cur; }
      else { new_contig--; }  // swallowed by the Dynamic dim inside the contiguous suffix
    } else if (last.kind == PD_ODDEVEN && cur.kind == PD_ODDEVEN) {
      throw ModelError("adjacent OddEven dims of one logical dim are unsupported");
    } else if (cur.kind == PD_DYNAMIC && last.kind != PD_ODDEVEN) {
      throw ModelError("Dynamic dim inside a Packed/Dynamic dim of the same logical dim");
    } else {
      l.d[w++] = cur;  // any pair involving one OddEven is kept
    }
  }
  l.n = (u8)w;
  l.contig = (u8)new_contig;
}

// Layout::new (layout.rs:205-217): fully contiguous, then merged.
inline Layout layout_new(const Layout& dims_only) {
  Layout l = dims_only;
  l.contig = l.n;
  layout_merge_consecutive(l);
  return l;
}

// ---- prune_size_one_logical_dims_with_contig (layout.rs:455-472) ----
inline u8 layout_prune_size_one(Layout& l, const Shape& shape, u8 contig) {
  const int first_contig = l.n - contig;
  int new_contig = contig;
  int w = 0;
  for (int i = 0; i < l.n; i++) {
    bool keep = shape[l.d[i].ldim] != 1;
    if (!keep && i >= first_contig) new_contig--;
    if (keep) l.d[w++] = l.d[i];
  }
  l.n = (u8)w;
  return (u8)new_contig;
}

// ---- drop_unneeded_packings (layout.rs:674-766) ----
inline void layout_drop_unneeded_packings(Layout& l, const Shape& tile) {
  {
    // Nothing to drop in an all-Dynamic layout (the common case): merged layouts never hold two
    // neighbouring Dynamic dims of one logical dim.
    bool any_strip = false;
    for (int i = 0; i < l.n; i++) any_strip |= l.d[i].kind != PD_DYNAMIC;
    if (!any_strip) {
      bool twin = false;
      for (int i = 1; i < l.n; i++) twin |= l.d[i].ldim == l.d[i - 1].ldim;
      if (!twin) return;
    }
  }
  const int n = l.n;
  const int contig = l.contig;
  const int first_contig = n - contig;

  bool outer_oe_exists[MAX_PHYS];
  {
    bool seen[MAX_RANK] = {false, false, false, false, false, false, false};
    for (int i = 0; i < n; i++) {
      outer_oe_exists[i] = seen[l.d[i].ldim];
      if (l.d[i].kind == PD_ODDEVEN) seen[l.d[i].ldim] = true;
    }
  }

  u32 rem[MAX_RANK];
  int noneified[MAX_RANK];
  for (int i = 0; i < tile.n; i++) { rem[i] = tile[i]; noneified[i] = -1; }
  for (int i = n - 1; i >= 0; i--) {
    PhysDim& p = l.d[i];
    u32& r = rem[p.ldim];
    if (p.kind == PD_PACKED) {
      u32 fs = p.size;
      if (r % fs == 0) {
        if (!outer_oe_exists[i] && r == fs) {
          p.kind = PD_DYNAMIC; p.size = 0;
          if (noneified[p.ldim] < 0) noneified[p.ldim] = i;
        }
        r /= fs;
      } else if (r != 0 && fs >= r) {
        if (!outer_oe_exists[i]) {
          p.kind = PD_DYNAMIC; p.size = 0;
          if (noneified[p.ldim] < 0) noneified[p.ldim] = i;
        }
        r = 1;
      }
    } else if (p.kind == PD_ODDEVEN) {
      u32 oe = p.size;
      if (r % oe == 0) r /= oe;
      else if (r != 0 && oe % r == 0) r = 1;
    }
  }

  int drops_in_contig = 0;
  int w = 0;
  for (int i = 0; i < n; i++) {
    PhysDim p = l.d[i];
    bool skip = false;
    if (noneified[p.ldim] >= 0 && i < noneified[p.ldim]) skip = true;
    else if (w > 0 && l.d[w - 1].ldim == p.ldim && l.d[w - 1].kind == PD_DYNAMIC && p.kind == PD_DYNAMIC) skip = true;
    if (!skip) l.d[w++] = p;
    else if (i >= first_contig) drops_in_contig++;
  }
  l.n = (u8)w;
  int nc = contig - drops_in_contig;
  if (nc < 0) nc = 0;
  if (nc > w) nc = w;
  l.contig = (u8)nc;
}

// ---- update_for_tiling (layout.rs:486-527). False = layout does not apply. ----
inline bool layout_update_for_tiling(const Layout& src, const Shape& parent, const Shape& tile, Layout& out) {
  u32 pp[MAX_PHYS], tp[MAX_PHYS];
  if (!layout_expand(src, parent, pp)) return false;
  if (!layout_expand(src, tile, tp)) return false;
  int matching = -1;  // index from the end of the first differing physical dim
  for (int k = 0; k < src.n; k++) {
    if (pp[src.n - 1 - k] != tp[src.n - 1 - k]) { matching = k; break; }
  }
  int lowered = (matching >= 0) ? matching + 1 : src.n;
  if (lowered > src.contig) lowered = src.contig;
  out = src;
  out.contig = (u8)lowered;
  out.contig = layout_prune_size_one(out, tile, out.contig);
  layout_merge_consecutive(out);
  layout_drop_unneeded_packings(out, tile);
  return true;
}

// ---- Layout::canonicalize (layout.rs:474-484) ----
inline bool layout_canonicalize(const Layout& src, const Shape& shape, Layout& out) {
  u32 phys[MAX_PHYS];
  if (!layout_expand(src, shape, phys)) return false;  // validate_shape_for_canonicalize
  out = src;
  if (out.contig > out.n) out.contig = out.n;
  out.contig = layout_prune_size_one(out, shape, out.contig);
  layout_merge_consecutive(out);
  layout_drop_unneeded_packings(out, shape);
  return true;
}

// ---- estimate_cache_lines (layout.rs:318-343) ----
inline u32 layout_estimate_cache_lines(const Layout& l, const Shape& shape, Dtype dtype) {
  u32 phys[MAX_PHYS];
  if (!layout_expand(l, shape, phys)) throw ModelError("estimate_cache_lines: layout does not apply");
  int first_contig = l.n - l.contig;
  u32 lines = 1;
  for (int i = 0; i < first_contig; i++) lines *= phys[i];
  u32 inner = 1;
  for (int i = first_contig; i < l.n; i++) inner *= phys[i];
  u32 bytes = inner * dtype_size(dtype);
  lines *= (bytes + LINE_SIZE - 1) / LINE_SIZE;
  return lines;
}

// ---- builders (layout.rs:1234-1279) ----
inline Layout layout_row_major(const Shape& shape) {
  Layout l;
  for (int i = 0; i < shape.n; i++) if (shape[i] != 1) l.push((u8)i, PD_DYNAMIC, 0);
  return layout_new(l);
}
inline Layout layout_col_major(const Shape& shape) {
  Layout l = layout_row_major(shape);
  for (int i = 0; i < l.n / 2; i++) std::swap(l.d[i], l.d[l.n - 1 - i]);
  return l;
}
inline Layout layout_nhwc(const Shape& shape) {
  static const u8 order[4] = {0, 2, 3, 1};
  Layout l;
  for (int i = 0; i < 4; i++) if (shape[order[i]] != 1) l.push(order[i], PD_DYNAMIC, 0);
  l.contig = l.n;
  return l;
}

// ---- destination / enumeration layouts (cpu.rs:317-453, 2878-3012) ----
inline std::vector<u32> all_target_vector_bytes() { return {16, 32}; }  // VRF only

inline std::vector<u32> pack_sizes_all(Dtype dt) {
  std::vector<u32> r = {2};
  for (u32 b : all_target_vector_bytes()) if (b % dtype_size(dt) == 0) r.push_back(b / dtype_size(dt));
  return r;
}
inline std::vector<u32> oddeven_sizes_all(Dtype dt) {
  std::vector<u32> r;
  for (u32 b : all_target_vector_bytes()) if ((2 * b) % dtype_size(dt) == 0) r.push_back(2 * b / dtype_size(dt));
  return r;
}

inline std::vector<Layout> base_layouts_for_shape(const Shape& shape) {
  std::vector<Layout> base;
  base.push_back(layout_row_major(shape));
  if (!shape.all_ones()) {
    if (shape.n == 2) {
      Layout c = layout_col_major(shape);
      if (c != base[0]) base.push_back(c);
    } else if (shape.n == 4) {
      Layout c = layout_nhwc(shape);
      if (c != base[0]) base.push_back(c);
    }
  }
  return base;
}

// Target::move_destination_layouts for CpuTarget (cpu.rs:399-453). Note the literal
// quirk of generic_packed_layouts_for_standard_layout (cpu.rs:2980-2991): `end` walks
// PHYSICAL dim indices but tests the LOGICAL shape at that index.
inline std::vector<Layout> move_destination_layouts(const Shape& shape, Dtype dt) {
  std::vector<Layout> base = base_layouts_for_shape(shape);
  std::vector<Layout> result = base;
  for (int pass = 0; pass < 2; pass++) {
    const bool oddeven = pass == 1;
    std::vector<u32> sizes = oddeven ? oddeven_sizes_all(dt) : pack_sizes_all(dt);
    for (const Layout& orig : base) {
      int end = 0;
      if (orig.n != 0) {
        int dd = orig.n - 1;
        while (dd > 0 && shape[dd] == 1) dd--;
        if (oddeven) dd++;
        end = dd;
      }
      for (int i = 0; i < end; i++) {
        u8 dim = orig.d[i].ldim;
        u32 ds = shape[dim];
        if (ds == 1) continue;
        for (u32 s : sizes) {
          bool ok = oddeven ? (s <= ds && ds % s == 0) : (s < ds && ds % s == 0);
          if (!ok) continue;
          Layout l = orig;
          l.push(dim, oddeven ? PD_ODDEVEN : PD_PACKED, s);
          result.push_back(layout_new(l));
        }
      }
    }
  }
  return result;
}

// Target::all_layouts_for_shape for CpuTarget (cpu.rs:317-397): the layouts the task
// grid enumerates per operand.
inline std::vector<Layout> all_layouts_for_shape(const Shape& shape, Dtype dt) {
  std::vector<Layout> base = base_layouts_for_shape(shape);
  std::vector<Layout> result = base;
  for (int pass = 0; pass < 2; pass++) {
    const bool oddeven = pass == 1;
    std::vector<u32> sizes = oddeven ? oddeven_sizes_all(dt) : pack_sizes_all(dt);
    for (const Layout& orig : base) {
      // unique logical dims in first-appearance order
      std::vector<u8> dims;
      for (int i = 0; i < orig.n; i++) {
        bool seen = false;
        for (u8 x : dims) if (x == orig.d[i].ldim) seen = true;
        if (!seen) dims.push_back(orig.d[i].ldim);
      }
      for (u8 dim : dims) {
        for (u32 s : sizes) {
          if (!oddeven && dim == orig.d[orig.n - 1].ldim) continue;
          if (shape[dim] % s != 0) continue;
          Layout l = orig;
          l.push(dim, oddeven ? PD_ODDEVEN : PD_PACKED, s);
          result.push_back(layout_new(l));
        }
      }
    }
  }
  return result;
}

}  // namespace mrl

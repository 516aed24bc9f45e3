// TEST INFRASTRUCTURE — NOT PART OF THE PRODUCT PATH.
//
// Known-answer tests: every deterministic vector the reference's own in-tree unit tests
// hold for the pieces on the database-fill path, replayed against the host model
// (morello_b200/csrc/model) and the oracle's Cost / memo arithmetic. Each block cites the
// reference test it transcribes (file:line inside the Morello repository). The expected
// VALUES come from those tests; the checking code is new.
//
// The last block (hand-derived anchors) is different: those values were derived by reading
// the reference source, not produced by running it, and are labelled as such.
#include "oracle.hpp"
#include <cstdio>

using namespace orc;

static int g_checks = 0, g_fail = 0;
#define CHECK(cond)                                                              \
  do {                                                                           \
    g_checks++;                                                                  \
    if (!(cond)) { g_fail++; fprintf(stderr, "FAIL %s:%d: %s\n", __FILE__, __LINE__, #cond); } \
  } while (0)

struct PD { int ldim; int kind; int size; };
static Layout L(std::initializer_list<PD> dims) {  // layout![..] == Layout::new(..)
  Layout l;
  for (auto& d : dims) l.push((u8)d.ldim, (u8)d.kind, (u32)d.size);
  return layout_new(l);
}
static Layout Lraw(std::initializer_list<PD> dims, int contig) {  // struct literal, no merging
  Layout l;
  for (auto& d : dims) l.push((u8)d.ldim, (u8)d.kind, (u32)d.size);
  l.contig = (u8)contig;
  return l;
}
#define D(x) PD{x, PD_DYNAMIC, 0}
#define P(x, s) PD{x, PD_PACKED, s}
#define OE(x, s) PD{x, PD_ODDEVEN, s}

static bool expand_eq(const Layout& l, const Shape& s, std::initializer_list<u32> want) {
  u32 phys[MAX_PHYS];
  if (!layout_expand(l, s, phys)) return false;
  if ((size_t)l.n != want.size()) return false;
  int i = 0;
  for (u32 w : want) if (phys[i++] != w) return false;
  return true;
}

static void test_layout() {
  // morello/src/layout.rs:1452-1550 test_expand_physical_shape_1..10 and neighbours
  CHECK(expand_eq(L({D(0), D(1), P(0, 4)}), Shape{64, 64}, {16, 64, 4}));
  CHECK(expand_eq(L({D(0), P(1, 2)}), Shape{2, 2}, {2, 2}));
  CHECK(expand_eq(L({P(0, 4), D(1)}), Shape{1, 64}, {1, 64}));
  CHECK(!layout_applies_to_shape(L({P(0, 2)}), Shape{6}));
  CHECK(expand_eq(L({D(0), D(1), P(0, 4)}), Shape{2, 64}, {1, 64, 2}));
  CHECK(expand_eq(L({P(0, 2)}), Shape{1}, {1}));
  CHECK(layout_applies_to_shape(L({P(0, 4)}), Shape{2}));
  CHECK(layout_applies_to_shape(L({OE(0, 4)}), Shape{1}));
  CHECK(!layout_applies_to_shape(L({OE(0, 4)}), Shape{2}));
  CHECK(!layout_applies_to_shape(L({P(0, 4), D(1)}), Shape{8, 64}));
  CHECK(expand_eq(L({D(1), D(0), P(1, 8)}), Shape{10, 4}, {1, 10, 4}));
  CHECK(expand_eq(L({D(1), D(0), P(1, 4), P(0, 2), P(1, 4)}), Shape{10, 8}, {1, 5, 2, 2, 4}));
  CHECK(!layout_applies_to_shape(L({D(1), D(0), P(1, 4), P(0, 2), P(1, 4)}), Shape{10, 6}));

  Layout out;
  // layout.rs:1560-1577 col-major slices
  CHECK(layout_update_for_tiling(layout_col_major(Shape{128, 128}), Shape{128, 128}, Shape{8, 1}, out));
  CHECK(out.n == 1 && out.d[0] == (PhysDim{0, PD_DYNAMIC, 0}) && out.contig == 1 && out.fully_contiguous());
  // layout.rs:1579-1599 tiling a packed dimension to one / to half
  CHECK(layout_update_for_tiling(L({D(1), D(0), P(1, 4)}), Shape{64, 64}, Shape{16, 1}, out));
  CHECK(out.is_row_major() && !out.fully_contiguous());
  CHECK(layout_update_for_tiling(L({D(1), D(0), P(1, 4)}), Shape{64, 64}, Shape{16, 2}, out));
  CHECK(out.is_row_major() && !out.fully_contiguous());
  // layout.rs:1601-1614 odd-even dimension tiled to one
  {
    Layout l = L({OE(0, 4), D(1)});
    l.contig = 0;
    CHECK(layout_update_for_tiling(l, Shape{4, 64}, Shape{1, 1}, out));
    CHECK(out.is_row_major() && out.fully_contiguous());
  }
  // layout.rs:1616-1625 cannot split an odd-even
  CHECK(!layout_update_for_tiling(L({OE(0, 4), D(1)}), Shape{4, 64}, Shape{2, 1}, out));
  CHECK(!layout_update_for_tiling(L({OE(0, 4), D(1)}), Shape{4, 64}, Shape{3, 1}, out));

  // layout.rs:1711-1747 drop_unneeded_packings 1..4
  {
    Layout l = L({D(0), D(1), P(0, 4)});
    layout_drop_unneeded_packings(l, Shape{4, 1024});
    CHECK(l == L({D(1), D(0)}));
    l = L({D(0), D(1), D(2), P(1, 256), P(2, 512), P(1, 4)});
    layout_drop_unneeded_packings(l, Shape{1, 2048, 512});
    layout_merge_consecutive(l);
    CHECK(l == L({D(0), D(1), D(2), P(1, 4)}));
    l = L({D(0), D(1), P(0, 4), D(1), P(0, 4)});
    layout_drop_unneeded_packings(l, Shape{4, 1024});
    CHECK(l == L({D(1), D(0)}));
    l = L({D(0), D(1), P(0, 4), D(1), P(0, 4)});
    layout_drop_unneeded_packings(l, Shape{16, 1024});
    layout_merge_consecutive(l);
    CHECK(l == L({D(1), D(0), D(1), P(0, 4)}));
  }
  // layout.rs:1749-1758 tile inside a packed physical dimension
  CHECK(layout_update_for_tiling(L({D(0), D(2), D(1), P(2, 32)}), Shape{2, 4, 64}, Shape{1, 4, 16}, out));
  {
    Layout want = L({D(1), D(2)});
    want.contig = 1;
    CHECK(out == want);
  }
  // layout.rs:1760-1786 packs that straddle the contiguity boundary are kept
  CHECK(layout_update_for_tiling(L({D(0), D(1), P(0, 2)}), Shape{6, 8}, Shape{6, 1}, out));
  CHECK(out == Lraw({D(0), P(0, 2)}, 1));
  {
    Layout l = L({D(0), D(1), P(0, 2)});
    l.contig = 0;
    CHECK(layout_update_for_tiling(l, Shape{6, 8}, Shape{6, 1}, out));
    CHECK(out == Lraw({D(0), P(0, 2)}, 0));
  }
  // layout.rs:1788-1809
  {
    Layout l = L({D(0), D(1), P(0, 2), D(2)});
    l.contig = 2;
    CHECK(layout_update_for_tiling(l, Shape{6, 8, 5}, Shape{6, 1, 5}, out));
    CHECK(out == Lraw({D(0), P(0, 2), D(2)}, 2));
  }
  // layout.rs:1811-1897 tile sizes vs a pack of 2 after other dims tile to one
  CHECK(!layout_update_for_tiling(L({D(1), D(0), D(2), P(0, 2)}), Shape{6, 8, 8}, Shape{3, 1, 1}, out));
  CHECK(!layout_applies_to_shape(L({D(1), D(0), D(2), P(0, 2)}), Shape{3, 1, 1}));
  for (u32 t : {1u, 2u, 4u, 6u}) {
    CHECK(layout_update_for_tiling(L({D(1), D(0), D(2), P(0, 2)}), Shape{6, 8, 8}, Shape{t, 1, 1}, out));
    CHECK(layout_applies_to_shape(L({D(1), D(0), D(2), P(0, 2)}), Shape{t, 1, 1}));
  }
  // layout.rs:1898-1921 odd-even interplay in drop_unneeded_packings
  {
    Layout l = L({D(1), OE(0, 4), P(0, 2)});
    layout_drop_unneeded_packings(l, Shape{8, 16});
    CHECK(l == L({D(1), OE(0, 4), P(0, 2)}));
    l = L({D(0), D(1), P(0, 2), OE(0, 4)});
    layout_drop_unneeded_packings(l, Shape{8, 16});
    CHECK(l == L({D(1), D(0), OE(0, 4)}));
    l = L({OE(0, 6), D(1), P(0, 4)});
    layout_drop_unneeded_packings(l, Shape{12, 16});
    CHECK(l == L({OE(0, 6), D(1), P(0, 4)}));
  }
  // layout.rs:1923-1975 merge_consecutive_dimensions
  {
    Layout l = Lraw({D(0), P(0, 2)}, 2);
    layout_merge_consecutive(l);
    CHECK(l == L({D(0)}));
    l = Lraw({D(0), P(0, 2)}, 1);
    layout_merge_consecutive(l);
    CHECK(l == Lraw({D(0), P(0, 2)}, 1));
    l = Lraw({P(0, 2), P(0, 3)}, 1);
    layout_merge_consecutive(l);
    CHECK(l == Lraw({P(0, 2), P(0, 3)}, 1));
  }
  // layout.rs:1977-1982
  {
    Layout l = L({D(0), D(1), P(0, 2), D(2), P(0, 2)});
    layout_drop_unneeded_packings(l, Shape{8, 1, 1});
    CHECK(l == L({D(0), D(1), P(0, 2), D(2), P(0, 2)}));
  }
  // layout.rs:2491-2546 estimate_cache_lines
  CHECK(layout_estimate_cache_lines(layout_row_major(Shape{1, 1, 1}), Shape{1, 1, 1}, DT_F32) == 1);
  CHECK(layout_estimate_cache_lines(layout_row_major(Shape{128, 16}), Shape{128, 16}, DT_F32) == 128);
  CHECK(layout_estimate_cache_lines(layout_row_major(Shape{64, 64}), Shape{64, 64}, DT_U8) == 64);
  {
    Layout l = layout_row_major(Shape{6, 128});
    l.contig = 1;
    CHECK(layout_estimate_cache_lines(l, Shape{6, 128}, DT_F32) == 48);
    CHECK(layout_estimate_cache_lines(L({D(2), D(1), P(2, 16)}), Shape{1, 128, 2048}, DT_F32) == 16384);
    CHECK(layout_estimate_cache_lines(layout_row_major(Shape{3, 3}), Shape{3, 3}, DT_F32) == 1);
    l = layout_row_major(Shape{3, 3});
    l.contig = 1;
    CHECK(layout_estimate_cache_lines(l, Shape{3, 3}, DT_F32) == 3);
  }
  // morello/src/target/cpu.rs:3345-3369 destination / enumeration layouts
  {
    bool found = false;
    for (auto& l : all_layouts_for_shape(Shape{1, 1, 2048}, DT_BF16)) if (l == L({D(2), OE(2, 16)})) found = true;
    CHECK(found);
    found = false;
    for (auto& l : move_destination_layouts(Shape{1, 1, 16}, DT_F32)) if (l == L({D(2), OE(2, 16)})) found = true;
    CHECK(found);
  }
}

static void test_utils() {
  // morello/src/utils.rs:545-575 diagonals
  {
    auto d = diagonals({0, 0});
    CHECK(d.size() == 1 && d[0].size() == 1 && d[0][0] == (std::vector<u32>{0, 0}));
    d = diagonals({0, 1});
    CHECK(d.size() == 2 && d[1][0] == (std::vector<u32>{0, 1}));
    d = diagonals({2, 1});
    CHECK(d.size() == 4);
    CHECK(d[1] == (std::vector<std::vector<u32>>{{0, 1}, {1, 0}}));
    CHECK(d[2] == (std::vector<std::vector<u32>>{{1, 1}, {2, 0}}));
    CHECK(d[3] == (std::vector<std::vector<u32>>{{2, 1}}));
  }
  // morello/src/spec.rs:3945-3954 dim_range (PowerOfTwo)
  CHECK(dim_range_pow2(3, false) == (std::vector<u32>{1, 2}));
  CHECK(dim_range_pow2(3, true) == (std::vector<u32>{1, 2, 3}));
  // morello/src/target/common_actions.rs:438-441: tile sizes of a 16-long dim
  CHECK(dim_range_pow2(16, false) == (std::vector<u32>{1, 2, 4, 8}));
  // bit helpers (utils.rs:123-172)
  CHECK(prev_power_of_two(61) == 32 && prev_power_of_two(64) == 64 && prev_power_of_two(0) == 0);
  CHECK(next_binary_power(0) == 0 && next_binary_power(3) == 4 && bit_length(1024) == 11);
}

static void test_cost_and_limits() {
  // morello/src/imp/loops.rs:267-308 compute_loop_main_cost
  CHECK(compute_loop_main_cost({{9, 8}}, false, {5, 4}) == 5 * 8 + 4);
  CHECK(compute_loop_main_cost({{9, 8}}, true, {5, 5}) == (60 + 5) * 1 + 5 + 230000);
  CHECK(compute_loop_main_cost({{8, 8}}, false, {4}) == 32);
  CHECK(compute_loop_main_cost({{3, 2}, {5, 4}}, false, {7, 6, 9, 10}) == 81);
  CHECK(compute_loop_main_cost({{8, 8}, {4, 3}}, false, {2, 3}) == 51);
  // morello/src/scheduling/tiling.rs:1659-1681: 10x10 tiled to 3x3 costs 922
  CHECK(compute_loop_main_cost({{1, 1}, {4, 3}, {4, 3}}, false, {100, 9, 11, 2}) == 922);

  // morello/src/memorylimits.rs:893-908 set_snap_up
  for (u64 i = 0; i <= 128; i++) CHECK(snap_up_value(i) == i);
  CHECK(snap_up_value(256) == 256 && snap_up_value(129) == 256 && snap_up_value(200) == 256 && snap_up_value(257) == 512);
  // memorylimits.rs:910-942 checked_sub_snap_down
  {
    Limits out;
    CHECK(checked_sub_snap_down({16, 16, 64, 64}, {3, 5, 3, 0}, out));
    CHECK(out == (Limits{13, 11, 32, 64}));
    CHECK(!checked_sub_snap_down({1, 0, 0, 0}, {2, 0, 0, 0}, out));
  }
  // memorylimits.rs:812-846 partial order, via the codes used for rectangles
  CHECK(limits_to_codes({16, 16, 1024, 33554432}) == (Codes{16, 16, 11, 26}));
  CHECK(codes_to_limits({16, 16, 11, 26}) == (Limits{16, 16, 1024, 33554432}));

  // morello/src/search/reducer.rs:108-276 with k = 1 (the head of each expected list)
  auto simple = [](u32 m) { Cost c; c.main = m; return c; };
  {
    Reducer r;
    CHECK(!r.finalize().found);
    r.insert(1, simple(1)); r.insert(0, simple(1)); r.insert(2, simple(1));
    CHECK(r.finalize().found && r.finalize().action == 0);
    Reducer s;
    s.insert(0, simple(1)); s.insert(1, simple(3)); s.insert(2, simple(2));
    CHECK(s.finalize().action == 0 && s.finalize().cost.main == 1);
    Reducer t;
    t.insert(1, simple(1)); t.insert(0, simple(2)); t.insert(2, simple(1));
    CHECK(t.finalize().action == 1 && t.finalize().cost.main == 1);
    Reducer u;
    u.insert(0, simple(2)); u.insert(1, simple(2)); u.insert(2, simple(2)); u.insert(3, simple(1));
    CHECK(u.finalize().action == 3);
  }
  // Cost order (cost.rs:87-104): main, then peaks lexicographically, then depth
  {
    Cost a = simple(5), b = simple(5);
    a.peaks = {1, 0, 0, 0}; b.peaks = {0, 9, 9, 9};
    CHECK(cost_cmp(a, b) > 0);
    b.peaks = a.peaks; a.depth = 2; b.depth = 3;
    CHECK(cost_cmp(a, b) < 0);
  }
  // morello/src/db/mod.rs:2462-2519: a put fills [peaks .. limits]; smaller limits inside
  // the rectangle hit, larger limits miss.
  {
    Database db;
    Decision d;
    d.found = true; d.action = 7; d.cost.main = 10; d.cost.peaks = {2, 0, 4, 0}; d.cost.depth = 1;
    db.put("k", {8, 8, 64, 64}, d);
    Decision g;
    CHECK(db.get("k", limits_to_codes({8, 8, 64, 64}), g) && g.action == 7);
    CHECK(db.get("k", limits_to_codes({2, 0, 4, 0}), g));
    CHECK(db.get("k", limits_to_codes({4, 3, 16, 2}), g));
    CHECK(!db.get("k", limits_to_codes({1, 0, 4, 0}), g));
    CHECK(!db.get("k", limits_to_codes({9, 8, 64, 64}), g));
    CHECK(!db.get("other", limits_to_codes({8, 8, 64, 64}), g));
    Decision unsat;
    db.put("u", {3, 3, 8, 8}, unsat);
    CHECK(db.get("u", limits_to_codes({0, 0, 0, 0}), g) && !g.found);
    CHECK(!db.get("u", limits_to_codes({4, 3, 8, 8}), g));
  }
  // next_limits (precompute/src/main.rs:738-759)
  {
    auto n = next_limits({16, 16, 1024, 1024}, {3, 0, 1, 8});
    CHECK(n.size() == 3);
    CHECK(n[0] == (Limits{2, 16, 1024, 1024}));
    CHECK(n[1] == (Limits{16, 16, 0, 1024}));
    CHECK(n[2] == (Limits{16, 16, 1024, 4}));
  }
}

static LogicalSpec mk(SpecKind k, Dtype dt, Shape s, std::initializer_list<Aux> auxes) {
  LogicalSpec l;
  l.kind = k; l.dtype = dt; l.spec_shape = s; l.serial_only = true;
  int i = 0;
  for (auto& a : auxes) l.aux[i++] = a;
  return l;
}
static Aux aux(Mem m, Layout l = Layout(), u32 vs = 0) { Aux a; a.mem = m; a.layout = l; a.vector_size = (u8)vs; return a; }

static void test_kernels_and_actions() {
  // morello/src/target/cpu.rs:3426-3441: Assign of a 2x32 u32 VRF(8) <- L1 costs 8
  {
    Layout rm = layout_row_major(Shape{2, 32});
    LogicalSpec s = mk(K_MOVE, DT_U32, Shape{2, 32}, {aux(VRF, rm, 8), aux(L1, rm)});
    LeafInfo li = leaf_kernel_info(LK_ASSIGN, s);
    CHECK(li.applies && li.main == 8);
  }
  // cpu.rs:3413-3424: BroadcastVecMultAdd with the broadcast operand on the left
  {
    LogicalSpec s = mk(K_MATMUL_ACCUM, DT_F32, Shape{1, 8, 1, 1},
                       {aux(VRF, layout_row_major(Shape{1, 8, 1}), 8), aux(L1, layout_row_major(Shape{1, 1, 1})),
                        aux(VRF, layout_row_major(Shape{1, 8, 1}), 8)});
    CHECK(logicalspec_is_canonical(s));
    CHECK(leaf_kernel_info(LK_BCAST_VEC_MULTADD, s).applies);
  }
  // cpu.rs:3371-3411: the kernel's one VRF register does not fit zero limits
  {
    LogicalSpec s = mk(K_MATMUL_ACCUM, DT_U8, Shape{1, 1, 1, 16},
                       {aux(RF), aux(VRF, layout_row_major(Shape{1, 1, 16}), 16), aux(VRF, layout_row_major(Shape{1, 1, 16}), 16)});
    CHECK(logicalspec_is_canonical(s));
    LeafInfo li = leaf_kernel_info(LK_BCAST_VEC_MULTADD, s);
    CHECK(li.applies && li.level == VRF && li.units == 1);
    Limits zero = {0, 0, 0, 0};
    CHECK(li.units > zero[li.level]);  // => NotApplicable(OutOfMemory) in select.rs:34-47
  }
  // morello/src/target/common_actions.rs:506-541: a 2x2x2 output has serial single-loop
  // tile-outs {dim 0..3} x {size 1, 2}; of those, size 1 applies and size 2 matches the original.
  {
    LogicalSpec s = mk(K_FILL_ZERO, DT_U32, Shape{2, 2, 2}, {aux(RF)});
    std::vector<Candidate> cs;
    u32 total = tabulate_candidates(s, cs);
    // moves: RF -> RF over row-major + 2 packed(2) + 0 odd-even layouts = 3 actions, all self-moves.
    u32 n_loop = 0;
    for (auto& c : cs) if (c.kind == CK_LOOP) { n_loop++; CHECK(c.imm == 2 && c.child[0].spec_shape.volume() == 4); }
    CHECK(n_loop == 3);
    CHECK(total >= 6);
  }
}

// Values derived BY HAND from the reference source (not outputs of the reference):
// Avx2, default features, max_mem limits, serial.
static void test_hand_derived_anchors() {
  Limits top = {16, 16, 1024, 33554432};
  auto solve = [&](const LogicalSpec& s) { Database db; Search se(db); return se.solve(s, top); };
  Layout e;  // empty layout
  {
    Decision d = solve(mk(K_FILL_ZERO, DT_U32, Shape{1}, {aux(RF)}));
    CHECK(d.found && d.action == 2 && d.cost.main == 1 && d.cost.peaks == (Limits{0, 0, 0, 0}) && d.cost.depth == 1);
  }
  {
    Decision d = solve(mk(K_MATMUL_ACCUM, DT_U32, Shape{1, 1, 1, 1}, {aux(RF), aux(RF), aux(RF)}));
    CHECK(d.found && d.action == 6 && d.cost.main == 2 && d.cost.depth == 1);
    d = solve(mk(K_MATMUL_ACCUM, DT_F32, Shape{1, 1, 1, 1}, {aux(RF), aux(RF), aux(RF)}));
    CHECK(d.found && d.action == 6 && d.cost.main == 1);
  }
  {
    Decision d = solve(mk(K_MATMUL, DT_U32, Shape{1, 1, 1, 1}, {aux(RF), aux(RF), aux(RF)}));
    CHECK(d.found && d.action == 6 && d.cost.main == 3 && d.cost.depth == 2);
  }
  {
    Decision d = solve(mk(K_FILL_ZERO, DT_U32, Shape{1}, {aux(L1, e)}));
    CHECK(d.found && d.action == 5 && d.cost.main == 1 && d.cost.depth == 1);
  }
  {
    Decision d = solve(mk(K_MOVE, DT_U32, Shape{1}, {aux(RF), aux(L1, e)}));
    CHECK(d.found && d.action == 6 && d.cost.main == 3 && d.cost.depth == 1);
  }
}

int main() {
  try {
    test_layout();
    test_utils();
    test_cost_and_limits();
    test_kernels_and_actions();
    test_hand_derived_anchors();
  } catch (const std::exception& ex) {
    fprintf(stderr, "exception: %s\n", ex.what());
    return 2;
  }
  printf("known-answer checks: %d, failures: %d\n", g_checks, g_fail);
  return g_fail ? 1 : 0;
}

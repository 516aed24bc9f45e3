// C ABI of the B200 synthesis-database fill (declared in include/morello_b200.h).
#include "../../include/morello_b200.h"
#include "fill.hpp"
#include <algorithm>
#include <chrono>
#include <thread>

using namespace mrl;

struct mrl_ctx {
  int device = 0;
  int n_threads = 1;
  Plan plan;
  bool planned = false, uploaded = false, filled = false;
  DeviceFill dev;
  mrl_stats stats;
  std::string err;
  // Lattice caps per memory (lattice codes; negative = keep every code). Start low: a fill at
  // low caps is cheap, and fill_verified raises them until no optimal peak exceeds its cap.
  int caps[4] = {4, 2, 4, 0};
  bool caps_chosen = false;  // false: pick a starting point from the goals' largest dimension
  bool auto_raise = true;
  uint32_t rank = 0, world = 1;
};

namespace {

double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int fail(mrl_ctx* ctx, int code, const std::string& msg) {
  if (ctx) ctx->err = msg;
  return code;
}

void decode_row(const MrlRow& r, mrl_decision* d) {
  memset(d, 0, sizeof(*d));
  if (r.tail == MRL_UNSAT) { d->found = 0; return; }
  d->found = 1;
  d->action = r.tail & 0xFFFFu;
  d->depth = r.tail >> 16;
  d->main_cost = r.main;
  d->peaks[0] = limit_value(0, (r.peaks >> 24) & 0xFF);
  d->peaks[1] = limit_value(1, (r.peaks >> 16) & 0xFF);
  d->peaks[2] = limit_value(2, (r.peaks >> 8) & 0xFF);
  d->peaks[3] = limit_value(3, r.peaks & 0xFF);
}

std::vector<Dtype> dtypes_of(int mask) {
  std::vector<Dtype> d;
  if (mask & 1) d.push_back(DT_U32);
  if (mask & 2) d.push_back(DT_F32);
  return d;
}

void copy_plan_stats(mrl_ctx* ctx) {
  const PlanStats& ps = ctx->plan.stats;
  ctx->stats.n_specs = ps.n_specs;
  ctx->stats.n_goal_specs = ps.n_goal_specs;
  ctx->stats.n_candidates = ps.n_cands;
  ctx->stats.n_rows = ps.n_rows;
  ctx->stats.algorithmic_bytes = ps.algorithmic_bytes;
  for (int k = 0; k < 4; k++)
    ctx->stats.lattice_caps[k] = ctx->plan.compressed(k) ? (int32_t)ctx->plan.cap_code[k] : -1;
}

// One upload + fill + check of the lattice compression. Returns 1 when some optimal peak
// exceeded its cap (caps in ctx->caps have then been raised), 0 when the tables are exact.
int fill_once(mrl_ctx* ctx) {
  double t0 = now_s();
  if (ctx->dev.upload(ctx->plan) != 0) return fail(ctx, -2, ctx->dev.error());
  ctx->uploaded = true;
  ctx->stats.upload_seconds += now_s() - t0;
  ctx->stats.h2d_bytes += ctx->dev.h2d_bytes();
  float ms = 0;
  uint64_t launches = 0;
  if (ctx->dev.run(ctx->plan, &ms, &launches) != 0) return fail(ctx, -2, ctx->dev.error());
  ctx->stats.fill_ms_total += ms;
  ctx->stats.fill_ms = ms;
  ctx->stats.n_launches = launches;
  ctx->stats.n_launches_total += launches;
  ctx->stats.fill_attempts++;
  uint32_t pk[4];
  if (ctx->dev.max_peaks(pk) != 0) return fail(ctx, -2, ctx->dev.error());
  bool violated = false;
  for (int k = 0; k < 4; k++)
    if (ctx->plan.compressed(k) && pk[k] > ctx->plan.cap_code[k]) {
      violated = true;
      ctx->caps[k] = (int)pk[k];
    }
  return violated ? 1 : 0;
}

// Fills the planned tables, raising the lattice caps until the compression is exact.
int fill_verified(mrl_ctx* ctx) {
  if (ctx->device < 0) return fail(ctx, -2, "planning-only context: no device to fill on");
  ctx->stats.upload_seconds = 0;
  ctx->stats.h2d_bytes = 0;
  ctx->stats.fill_ms_total = 0;
  ctx->stats.n_launches_total = 0;
  ctx->stats.fill_attempts = 0;
  ctx->filled = false;
  for (int attempt = 0; attempt < 16; attempt++) {
    int rc = fill_once(ctx);
    if (rc < 0) return rc;
    if (rc == 0) {
      ctx->filled = true;
      return 0;
    }
    ctx->caps_chosen = true;  // raised caps are kept for later plans on this context
    if (!ctx->auto_raise) return fail(ctx, -5, "an optimal peak exceeds the lattice caps; raise them (mrl_set_lattice_caps)");
    double t0 = now_s();
    relayout_plan(ctx->plan, ctx->caps);
    copy_plan_stats(ctx);
    ctx->stats.plan_seconds += now_s() - t0;
  }
  return fail(ctx, -5, "lattice caps did not converge");
}

// Starting caps by the largest Spec dimension among the goals: the values earlier fills of that
// size ended with. Only a starting point - every fill is checked and the caps raised if needed.
void choose_initial_caps(mrl_ctx* ctx, const std::vector<LogicalSpec>& goals) {
  if (ctx->caps_chosen) return;
  u32 maxdim = 1;
  for (const LogicalSpec& g : goals)
    for (int i = 0; i < g.spec_shape.n; i++) maxdim = std::max(maxdim, g.spec_shape[i]);
  static const int table[4][4] = {{0, 0, 3, 0}, {8, 2, 5, 0}, {-1, 12, 7, 4}, {-1, -1, 9, 6}};
  int row = maxdim <= 1 ? 0 : (maxdim <= 2 ? 1 : (maxdim <= 4 ? 2 : 3));
  for (int k = 0; k < 4; k++) ctx->caps[k] = table[row][k];
}

int set_plan(mrl_ctx* ctx, const std::vector<LogicalSpec>& goals) {
  double t0 = now_s();
  choose_initial_caps(ctx, goals);
  ctx->plan = build_plan(goals, ctx->n_threads, nullptr, ctx->caps, ctx->rank, ctx->world);
  ctx->planned = true;
  ctx->uploaded = ctx->filled = false;
  copy_plan_stats(ctx);
  const PlanStats& ps = ctx->plan.stats;
  ctx->stats.n_specs = ps.n_specs;
  ctx->stats.n_goal_specs = ps.n_goal_specs;
  ctx->stats.n_candidates = ps.n_cands;
  ctx->stats.n_rows = ps.n_rows;
  ctx->stats.algorithmic_bytes = ps.algorithmic_bytes;
  ctx->stats.plan_seconds = now_s() - t0;
  return 0;
}

int parse_goals(const uint8_t* blobs, const uint64_t* off, size_t n, std::vector<LogicalSpec>& out) {
  for (size_t i = 0; i < n; i++) {
    LogicalSpec ls = LogicalSpec::from_key(std::string((const char*)blobs + off[i], off[i + 1] - off[i]));
    if (logicalspec_canonicalize(ls) != CANON_OK) return -1;
    out.push_back(ls);
  }
  return 0;
}

}  // namespace

extern "C" {

int mrl_ctx_create(int device, int n_threads, mrl_ctx** out) {
  if (!out) return -1;
  mrl_ctx* ctx = new mrl_ctx();
  ctx->device = device;
  if (n_threads <= 0) n_threads = (int)std::thread::hardware_concurrency();
  if (n_threads <= 0) n_threads = 1;
  ctx->n_threads = n_threads;
  memset(&ctx->stats, 0, sizeof(ctx->stats));
  *out = ctx;
  // device < 0: a planning-only context (closure, candidate tables, shard ownership can be
  // inspected; nothing can be filled or looked up). Otherwise a usable GPU is required:
  // there is no CPU path.
  if (device < 0) return 0;
  if (ctx->dev.init(device) != 0) {
    ctx->err = std::string("no usable CUDA device: ") + ctx->dev.error();
    return -2;
  }
  return 0;
}

void mrl_ctx_destroy(mrl_ctx* ctx) { delete ctx; }

const char* mrl_last_error(const mrl_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }

int mrl_spec_simple(int kind, int dtype, const uint32_t* spec_shape, int rank, int memory, uint8_t* out, size_t cap) {
  try {
    if (kind < 0 || kind > K_MATMUL || rank < 1 || rank > MAX_RANK || memory < 0 || memory > GL) return -1;
    LogicalSpec l;
    l.kind = (SpecKind)kind;
    l.dtype = (Dtype)dtype;
    l.serial_only = true;
    l.spec_shape.n = (u8)rank;
    for (int i = 0; i < rank; i++) l.spec_shape.d[i] = spec_shape[i];
    if ((l.kind == K_MATMUL || l.kind == K_MATMUL_ACCUM) && rank != 4) return -1;
    for (int i = 0; i < l.nops(); i++) {
      l.aux[i].mem = (Mem)memory;
      l.aux[i].vector_size = 0;
      if (mem_is_vector((Mem)memory)) return -1;
      l.aux[i].layout = mem_has_layout((Mem)memory) ? layout_row_major(l.operand_shape(i)) : Layout();
    }
    if (logicalspec_canonicalize(l) != CANON_OK) return -2;
    std::string k = l.key();
    if (k.size() > cap) return -3;
    memcpy(out, k.data(), k.size());
    return (int)k.size();
  } catch (const std::exception&) {
    return -1;
  }
}

int mrl_spec_canonicalize(const uint8_t* blob, size_t len, uint8_t* out, size_t cap) {
  try {
    LogicalSpec l = LogicalSpec::from_key(std::string((const char*)blob, len));
    if (logicalspec_canonicalize(l) != CANON_OK) return -2;
    std::string k = l.key();
    if (k.size() > cap) return -3;
    memcpy(out, k.data(), k.size());
    return (int)k.size();
  } catch (const std::exception&) {
    return -1;
  }
}

int mrl_spec_describe(const uint8_t* blob, size_t len, char* out, size_t cap) {
  try {
    std::string s = LogicalSpec::from_key(std::string((const char*)blob, len)).str();
    if (s.size() + 1 > cap) return -3;
    memcpy(out, s.c_str(), s.size() + 1);
    return (int)s.size();
  } catch (const std::exception&) {
    return -1;
  }
}

void mrl_max_mem(uint64_t limits[4]) { for (int i = 0; i < 4; i++) limits[i] = AVX2_MAX_MEM[i]; }

int mrl_plan_precompute(mrl_ctx* ctx, uint32_t size, int through, int dtype_mask) {
  if (!ctx) return -1;
  try {
    if (size == 0 || !is_pow2(size)) return fail(ctx, -1, "size must be a power of two");
    if (through < 0 || through > THROUGH_MATMUL) return fail(ctx, -1, "bad `through`");
    std::vector<Dtype> dts = dtypes_of(dtype_mask);
    if (dts.empty()) return fail(ctx, -1, "empty dtype mask");
    double t0 = now_s();
    std::vector<LogicalSpec> goals = precompute_goals(size, (Through)through, dts, ctx->n_threads);
    int rc = set_plan(ctx, goals);
    ctx->stats.plan_seconds = now_s() - t0;
    return rc;
  } catch (const std::exception& e) {
    return fail(ctx, -1, e.what());
  }
}

int mrl_plan_goals(mrl_ctx* ctx, const uint8_t* blobs, const uint64_t* blob_off, size_t n) {
  if (!ctx) return -1;
  try {
    std::vector<LogicalSpec> goals;
    if (parse_goals(blobs, blob_off, n, goals) != 0) return fail(ctx, -4, "goal Spec is not canonicalizable");
    return set_plan(ctx, goals);
  } catch (const std::exception& e) {
    return fail(ctx, -1, e.what());
  }
}

int mrl_upload(mrl_ctx* ctx) {
  if (!ctx) return -1;
  if (ctx->device < 0) return fail(ctx, -2, "planning-only context: no device to fill on");
  if (!ctx->planned) return fail(ctx, -1, "nothing planned");
  double t0 = now_s();
  if (ctx->dev.upload(ctx->plan) != 0) return fail(ctx, -2, ctx->dev.error());
  ctx->uploaded = true;
  ctx->filled = false;
  ctx->stats.upload_seconds = now_s() - t0;
  ctx->stats.h2d_bytes = ctx->dev.h2d_bytes();
  return 0;
}

int mrl_fill(mrl_ctx* ctx) {
  if (!ctx) return -1;
  if (!ctx->uploaded) return fail(ctx, -1, "plan not uploaded");
  float ms = 0;
  uint64_t launches = 0;
  if (ctx->dev.run(ctx->plan, &ms, &launches) != 0) return fail(ctx, -2, ctx->dev.error());
  ctx->stats.fill_ms = ms;
  ctx->stats.n_launches = launches;
  uint32_t pk[4];
  if (ctx->dev.max_peaks(pk) != 0) return fail(ctx, -2, ctx->dev.error());
  for (int k = 0; k < 4; k++)
    if (ctx->plan.compressed(k) && pk[k] > ctx->plan.cap_code[k]) {
      ctx->filled = false;
      return fail(ctx, -5, "an optimal peak exceeds the lattice caps of this plan; use mrl_precompute / "
                           "mrl_top_down_many (they raise the caps) or mrl_set_lattice_caps");
    }
  ctx->filled = true;
  return 0;
}

int mrl_set_lattice_caps(mrl_ctx* ctx, const int32_t caps[4], int auto_raise) {
  if (!ctx || !caps) return -1;
  for (int k = 0; k < 4; k++) ctx->caps[k] = caps[k];
  ctx->caps_chosen = true;
  ctx->auto_raise = auto_raise != 0;
  if (ctx->planned) {
    relayout_plan(ctx->plan, ctx->caps);
    copy_plan_stats(ctx);
    ctx->uploaded = ctx->filled = false;
  }
  return 0;
}

int mrl_get_many(mrl_ctx* ctx, const uint8_t* blobs, const uint64_t* blob_off, size_t n, const uint64_t* limits,
                 mrl_decision* out) {
  if (!ctx) return -1;
  if (!ctx->filled) return fail(ctx, -1, "tables are not filled");
  try {
    std::vector<uint64_t> idx;
    std::vector<size_t> where;
    for (size_t i = 0; i < n; i++) {
      memset(&out[i], 0, sizeof(out[i]));
      out[i].found = -1;
      LogicalSpec ls = LogicalSpec::from_key(std::string((const char*)blobs + blob_off[i], blob_off[i + 1] - blob_off[i]));
      if (logicalspec_canonicalize(ls) != CANON_OK) continue;
      long id = ctx->plan.find(ls);
      if (id < 0) continue;
      long row = ctx->plan.row_of((u32)id, limits + 4 * i);
      if (row < 0) continue;
      idx.push_back((uint64_t)row);
      where.push_back(i);
    }
    std::vector<MrlRow> rows(idx.size());
    if (ctx->dev.read_rows(idx.data(), idx.size(), rows.data()) != 0) return fail(ctx, -2, ctx->dev.error());
    for (size_t j = 0; j < idx.size(); j++) decode_row(rows[j], &out[where[j]]);
    ctx->stats.d2h_bytes = idx.size() * sizeof(MrlRow);
    return 0;
  } catch (const std::exception& e) {
    return fail(ctx, -1, e.what());
  }
}

int mrl_top_down_many(mrl_ctx* ctx, const uint8_t* blobs, const uint64_t* blob_off, size_t n, const uint64_t* limits,
                      mrl_decision* out) {
  int rc = mrl_plan_goals(ctx, blobs, blob_off, n);
  if (rc) return rc;
  if ((rc = fill_verified(ctx))) return rc;
  return mrl_get_many(ctx, blobs, blob_off, n, limits, out);
}

int mrl_top_down_many_noalloc(mrl_ctx* ctx, const uint8_t* blobs, const uint64_t* blob_off, size_t n,
                              const uint64_t* limits, mrl_decision* out) {
  if (!ctx) return -1;
  try {
    std::vector<LogicalSpec> goals;
    if (parse_goals(blobs, blob_off, n, goals) != 0) return fail(ctx, -4, "goal Spec is not canonicalizable");
    // A plan of its own: the context's tables (and their device memory) are left as they are.
    // Every lattice code is kept here (no caps): the fill is small by construction and one
    // pass must be final.
    const int no_caps[4] = {-1, -1, -1, -1};
    Plan plan = build_plan(goals, ctx->n_threads, nullptr, no_caps);
    std::vector<uint64_t> idx;
    std::vector<size_t> where;
    for (size_t i = 0; i < n; i++) {
      memset(&out[i], 0, sizeof(out[i]));
      out[i].found = -1;
      long id = plan.find(goals[i]);
      if (id < 0) continue;
      long row = plan.row_of((u32)id, limits + 4 * i);
      if (row < 0) continue;
      idx.push_back((uint64_t)row);
      where.push_back(i);
    }
    std::vector<MrlRow> rows(idx.size());
    char err[256] = {0};
    int rc = fill_static(ctx->dev.device(), ctx->dev.stream(), plan, idx.data(), idx.size(), rows.data(), err, sizeof(err));
    if (rc != 0) return fail(ctx, rc, err);
    for (size_t j = 0; j < idx.size(); j++) decode_row(rows[j], &out[where[j]]);
    return 0;
  } catch (const std::exception& e) {
    return fail(ctx, -1, e.what());
  }
}

int mrl_precompute(mrl_ctx* ctx, uint32_t size, int through, int dtype_mask) {
  int rc = mrl_plan_precompute(ctx, size, through, dtype_mask);
  if (rc) return rc;
  return fill_verified(ctx);
}

int mrl_set_shard(mrl_ctx* ctx, uint32_t rank, uint32_t world) {
  if (!ctx) return -1;
  if (world < 1 || rank >= world) return fail(ctx, -1, "bad shard rank / world size");
  ctx->rank = rank;
  ctx->world = world;
  ctx->planned = ctx->uploaded = ctx->filled = false;
  return 0;
}

int mrl_set_stream(mrl_ctx* ctx, void* cuda_stream) {
  if (!ctx) return -1;
  return ctx->dev.set_stream((cudaStream_t)cuda_stream);
}

uint64_t mrl_num_groups(const mrl_ctx* ctx) { return ctx && ctx->planned ? ctx->plan.groups.size() : 0; }
uint64_t mrl_num_families(const mrl_ctx* ctx) { return ctx && ctx->planned ? ctx->plan.families.size() : 0; }

int mrl_family_info(const mrl_ctx* ctx, uint64_t family, uint32_t* group, uint32_t* owner, uint64_t* row_lo,
                    uint64_t* row_hi) {
  if (!ctx || !ctx->planned || family >= ctx->plan.families.size()) return -1;
  const Family& f = ctx->plan.families[family];
  if (group) *group = f.group;
  if (owner) *owner = f.owner;
  if (row_lo) *row_lo = f.row_lo;
  if (row_hi) *row_hi = f.row_hi;
  return 0;
}

uint32_t mrl_row_bytes(void) { return (uint32_t)sizeof(MrlRow); }

int mrl_device_rows(const mrl_ctx* ctx, void** ptr, uint64_t* n_rows) {
  if (!ctx || !ctx->uploaded) return -1;
  if (ptr) *ptr = ctx->dev.device_rows();
  if (n_rows) *n_rows = ctx->dev.n_rows();
  return 0;
}

int mrl_fill_begin(mrl_ctx* ctx) {
  if (!ctx) return -1;
  if (!ctx->uploaded) return fail(ctx, -1, "plan not uploaded");
  ctx->filled = false;
  if (ctx->dev.begin_fill() != 0) return fail(ctx, -2, ctx->dev.error());
  return 0;
}

int mrl_fill_group(mrl_ctx* ctx, uint64_t group) {
  if (!ctx || !ctx->uploaded) return -1;
  if (ctx->dev.run_group(ctx->plan, (uint32_t)group) != 0) return fail(ctx, -2, ctx->dev.error());
  return 0;
}

int mrl_fill_end(mrl_ctx* ctx, int32_t raised_caps[4]) {
  if (!ctx || !ctx->uploaded) return -1;
  float ms = 0;
  uint64_t launches = 0;
  if (ctx->dev.end_fill(&ms, &launches) != 0) return fail(ctx, -2, ctx->dev.error());
  ctx->stats.fill_ms = ms;
  ctx->stats.n_launches = launches;
  uint32_t pk[4];
  if (ctx->dev.max_peaks(pk) != 0) return fail(ctx, -2, ctx->dev.error());
  bool violated = false;
  for (int k = 0; k < 4; k++) {
    if (raised_caps) raised_caps[k] = ctx->caps[k];
    if (ctx->plan.compressed(k) && pk[k] > ctx->plan.cap_code[k]) {
      violated = true;
      if (raised_caps) raised_caps[k] = (int32_t)pk[k];
    }
  }
  if (violated) return 1;  // not an error: the caller raises the caps on every rank and refills
  ctx->filled = true;
  return 0;
}

int mrl_get_stats(const mrl_ctx* ctx, mrl_stats* out) {
  if (!ctx || !out) return -1;
  *out = ctx->stats;
  return 0;
}

uint64_t mrl_num_specs(const mrl_ctx* ctx) { return ctx && ctx->planned ? ctx->plan.specs.size() : 0; }

int mrl_spec_blob(const mrl_ctx* ctx, uint64_t spec_id, uint8_t* out, size_t cap) {
  if (!ctx || !ctx->planned || spec_id >= ctx->plan.specs.size()) return -1;
  std::string k = ctx->plan.specs[spec_id].key();
  if (k.size() > cap) return -3;
  memcpy(out, k.data(), k.size());
  return (int)k.size();
}

int mrl_spec_grid(const mrl_ctx* ctx, uint64_t spec_id, uint32_t masks[4], uint64_t* n_cells) {
  if (!ctx || !ctx->planned || spec_id >= ctx->plan.specs.size()) return -1;
  const SpecHdr& h = ctx->plan.hdrs[spec_id];
  uint64_t n = 1;
  for (int k = 0; k < 4; k++) { masks[k] = h.mask[k]; n *= (uint64_t)__builtin_popcount(h.mask[k]); }
  if (n_cells) *n_cells = n;
  return 0;
}

int mrl_export_rows(mrl_ctx* ctx, uint64_t spec_id, mrl_decision* out, size_t cap) {
  if (!ctx || !ctx->filled || spec_id >= ctx->plan.specs.size()) return -1;
  const SpecHdr& h = ctx->plan.hdrs[spec_id];
  uint64_t n = 1;
  for (int k = 0; k < 4; k++) n *= (uint64_t)__builtin_popcount(h.mask[k]);
  if (n > cap) return fail(ctx, -3, "export buffer too small");
  std::vector<uint64_t> idx(n);
  for (uint64_t i = 0; i < n; i++) idx[i] = h.row_base + i;
  std::vector<MrlRow> rows(n);
  if (ctx->dev.read_rows(idx.data(), n, rows.data()) != 0) return fail(ctx, -2, ctx->dev.error());
  for (uint64_t i = 0; i < n; i++) decode_row(rows[i], &out[i]);
  return 0;
}

}  // extern "C"

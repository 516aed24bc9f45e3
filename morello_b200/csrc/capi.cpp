// C ABI of the B200 synthesis-database fill (declared in include/morello_b200.h).
#include "../../include/morello_b200.h"
#include "fill.hpp"
#include "model/impl_text.hpp"
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
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
  uint32_t rank = 0, world = 1;
  uint32_t plan_flags = 0;        // PLAN_NO_TWINS | PLAN_NO_MEMO
  bool cands_elsewhere = false;   // adopted plan whose candidate records only exist on the planning rank
  bool table_only = false;        // loaded from a file without a matching plan: lookups only
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

void copy_fill_stats(mrl_ctx* ctx) {
  const FillStats& fs = ctx->dev.stats();
  ctx->stats.n_rows = fs.n_rows;
  ctx->stats.n_cells_solved = fs.cells_solved;
  ctx->stats.n_candidates_evaluated = fs.cands_evaluated;
  ctx->stats.n_rows_gathered = fs.lookups;
  ctx->stats.n_passes = fs.passes;
  ctx->stats.n_launches = fs.launches;
  ctx->stats.n_grid_syncs = fs.grid_syncs;
  ctx->stats.algorithmic_bytes = fs.alg_bytes;
  ctx->stats.fill_ms = fs.fill_ms;
  ctx->stats.combine_ms = fs.combine_ms;
  ctx->stats.early_ms = fs.early_ms;
  ctx->stats.n_sweeps = fs.sweeps;
  ctx->stats.n_cells_unordered = fs.early_cells;
  ctx->stats.n_candidates_swept = fs.late_cands;
  ctx->stats.n_items_swept = fs.late_items;
  ctx->stats.n_buffer_growths = fs.growths;
  for (int k = 0; k < 8; k++) ctx->stats.phase_ms[k] = fs.phase_ms[k];
}

// Upload + fill of the planned tables.
int upload_and_fill(mrl_ctx* ctx) {
  if (ctx->device < 0) return fail(ctx, -2, "planning-only context: no device to fill on");
  ctx->filled = false;
  double t0 = now_s();
  int rc = ctx->dev.upload(ctx->plan);
  if (rc != 0) return fail(ctx, (rc == -5 || rc == -6 || rc == -3) ? rc : -2, ctx->dev.error());
  ctx->uploaded = true;
  ctx->stats.upload_seconds = now_s() - t0;
  ctx->stats.h2d_bytes = ctx->dev.h2d_bytes();
  rc = ctx->dev.run(ctx->plan);
  copy_fill_stats(ctx);
  if (rc != 0) return fail(ctx, (rc == -5 || rc == -6 || rc == -3) ? rc : -2, ctx->dev.error());
  ctx->filled = true;
  return 0;
}

int set_plan(mrl_ctx* ctx, const std::vector<LogicalSpec>& goals, int mirror_dtype = -1) {
  double t0 = now_s();
  ctx->cands_elsewhere = false;
  ctx->table_only = false;
  ctx->dev.wait_upload();   // a background upload may still be reading the old plan
  ctx->plan = build_plan(goals, ctx->n_threads, nullptr, ctx->rank, ctx->world, mirror_dtype, ctx->plan_flags);
  ctx->planned = true;
  ctx->uploaded = ctx->filled = false;
  const PlanStats& ps = ctx->plan.stats;
  memset(&ctx->stats, 0, sizeof(ctx->stats));
  ctx->stats.n_specs = ps.n_specs;
  ctx->stats.n_goal_specs = ps.n_goal_specs;
  ctx->stats.n_candidates = ps.n_cands;
  ctx->stats.n_stages = ps.n_stages;
  ctx->stats.plan_seconds = now_s() - t0;
  ctx->stats.plan_discover_seconds = ps.seconds_discover;
  ctx->stats.plan_layout_seconds = ps.seconds_layout;
  for (int k = 0; k < 8; k++) ctx->stats.plan_layout_step_seconds[k] = ps.seconds_layout_step[k];
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

long mrl_tabulate(const uint8_t* blob, size_t len, uint8_t* out, size_t cap) {
  try {
    LogicalSpec ls = LogicalSpec::from_key(std::string((const char*)blob, len));
    if (logicalspec_canonicalize(ls) != CANON_OK) return -4;
    std::vector<Candidate> cs;
    tabulate_candidates(ls, cs);
    std::string buf;
    auto put32 = [&](uint32_t v) { for (int k = 0; k < 4; k++) buf.push_back((char)(v >> (8 * k))); };
    for (const Candidate& c : cs) {
      buf.push_back((char)(c.action & 0xff)); buf.push_back((char)(c.action >> 8));
      buf.push_back((char)c.kind); buf.push_back((char)c.nchild);
      put32(c.imm);
      buf.push_back((char)c.level); buf.push_back(0); buf.push_back(0); buf.push_back(0);
      put32(c.units);
      for (int j = 0; j < c.nchild; j++) {
        const std::string k = c.child[j].key();
        buf.push_back((char)(k.size() & 0xff)); buf.push_back((char)(k.size() >> 8));
        buf += k;
      }
    }
    if (buf.size() > cap) return -3;
    memcpy(out, buf.data(), buf.size());
    return (long)buf.size();
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
    // u32 + f32: the goal sets mirror each other by construction, so only the u32 goals are
    // enumerated and the planner derives the f32 half (plan.cpp, "dtype twins")
    int mirror = -1;
    if (dts.size() == 2 && dts[0] == DT_U32 && dts[1] == DT_F32 && !(ctx->plan_flags & PLAN_NO_TWINS)) {
      dts.pop_back();
      mirror = DT_F32;
    }
    std::vector<LogicalSpec> goals = precompute_goals(size, (Through)through, dts, ctx->n_threads);
    const double t_goals = now_s() - t0;
    int rc = set_plan(ctx, goals, mirror);
    ctx->stats.plan_seconds = now_s() - t0;
    ctx->stats.plan_goal_seconds = t_goals;
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

int mrl_set_plan_flags(mrl_ctx* ctx, uint32_t flags) {
  if (!ctx) return -1;
  if (flags & ~(uint32_t)(PLAN_NO_TWINS | PLAN_NO_MEMO)) return fail(ctx, -1, "unknown plan flag");
  ctx->plan_flags = flags;
  return 0;
}

int mrl_upload(mrl_ctx* ctx) {
  if (!ctx) return -1;
  if (ctx->device < 0) return fail(ctx, -2, "planning-only context: no device to fill on");
  if (!ctx->planned) return fail(ctx, -1, "nothing planned");
  if (ctx->table_only) return fail(ctx, -1, "the tables were loaded from a file without their plan: nothing to upload or fill");
  double t0 = now_s();
  int urc = ctx->dev.upload(ctx->plan, ctx->cands_elsewhere);
  if (urc != 0) return fail(ctx, urc == -6 ? -6 : -2, ctx->dev.error());
  ctx->uploaded = true;
  ctx->filled = false;
  ctx->stats.upload_seconds = now_s() - t0;
  ctx->stats.h2d_bytes = ctx->dev.h2d_bytes();
  return 0;
}

int mrl_fill(mrl_ctx* ctx) {
  if (!ctx) return -1;
  if (!ctx->uploaded || ctx->table_only) return fail(ctx, -1, "plan not uploaded");
  ctx->filled = false;
  int rc = ctx->dev.run(ctx->plan);
  copy_fill_stats(ctx);
  if (rc != 0) return fail(ctx, (rc == -5 || rc == -6 || rc == -3) ? rc : -2, ctx->dev.error());
  ctx->filled = true;
  return 0;
}

// Resolves each query to (Spec id, packed limit codes); `where` = its position in the caller's arrays.
static void resolve_queries(const Plan& plan, const uint8_t* blobs, const uint64_t* blob_off, size_t n,
                            const uint64_t* limits, mrl_decision* out, std::vector<uint32_t>& ids,
                            std::vector<uint32_t>& packs, std::vector<size_t>& where) {
  for (size_t i = 0; i < n; i++) {
    memset(&out[i], 0, sizeof(out[i]));
    out[i].found = -1;
    LogicalSpec ls = LogicalSpec::from_key(std::string((const char*)blobs + blob_off[i], blob_off[i + 1] - blob_off[i]));
    if (logicalspec_canonicalize(ls) != CANON_OK) continue;
    long id = plan.find(ls);
    if (id < 0) continue;
    uint32_t pack;
    if (!plan.pack_limits(limits + 4 * i, &pack)) continue;
    ids.push_back((uint32_t)id);
    packs.push_back(pack);
    where.push_back(i);
  }
}

int mrl_get_many(mrl_ctx* ctx, const uint8_t* blobs, const uint64_t* blob_off, size_t n, const uint64_t* limits,
                 mrl_decision* out) {
  if (!ctx) return -1;
  if (!ctx->filled) return fail(ctx, -1, "tables are not filled");
  try {
    std::vector<uint32_t> ids, packs;
    std::vector<size_t> where;
    resolve_queries(ctx->plan, blobs, blob_off, n, limits, out, ids, packs, where);
    std::vector<MrlRow> rows(ids.size());
    if (ctx->dev.lookup(ids.data(), packs.data(), ids.size(), rows.data()) != 0) return fail(ctx, -2, ctx->dev.error());
    for (size_t j = 0; j < ids.size(); j++) decode_row(rows[j], &out[where[j]]);
    ctx->stats.d2h_bytes = ids.size() * sizeof(MrlRow);
    return 0;
  } catch (const std::exception& e) {
    return fail(ctx, -1, e.what());
  }
}

int mrl_top_down_many(mrl_ctx* ctx, const uint8_t* blobs, const uint64_t* blob_off, size_t n, const uint64_t* limits,
                      mrl_decision* out) {
  int rc = mrl_plan_goals(ctx, blobs, blob_off, n);
  if (rc) return rc;
  if ((rc = upload_and_fill(ctx))) return rc;
  return mrl_get_many(ctx, blobs, blob_off, n, limits, out);
}

int mrl_top_down_many_noalloc(mrl_ctx* ctx, const uint8_t* blobs, const uint64_t* blob_off, size_t n,
                              const uint64_t* limits, mrl_decision* out) {
  if (!ctx) return -1;
  if (ctx->device < 0) return fail(ctx, -2, "planning-only context: no device to fill on");
  try {
    std::vector<LogicalSpec> goals;
    if (parse_goals(blobs, blob_off, n, goals) != 0) return fail(ctx, -4, "goal Spec is not canonicalizable");
    // A plan of its own: the context's tables (and their device memory) are left as they are.
    Plan plan = build_plan(goals, ctx->n_threads, nullptr, 0, 1, -1, ctx->plan_flags);
    std::vector<uint32_t> ids, packs;
    std::vector<size_t> where;
    resolve_queries(plan, blobs, blob_off, n, limits, out, ids, packs, where);
    std::vector<MrlRow> rows(ids.size());
    char err[256] = {0};
    int rc = fill_static(ctx->dev.device(), ctx->dev.stream(), plan, ids.data(), packs.data(), ids.size(), rows.data(),
                         err, sizeof(err));
    if (rc != 0) return fail(ctx, rc, err);
    for (size_t j = 0; j < ids.size(); j++) decode_row(rows[j], &out[where[j]]);
    return 0;
  } catch (const std::exception& e) {
    return fail(ctx, -1, e.what());
  }
}

int mrl_precompute(mrl_ctx* ctx, uint32_t size, int through, int dtype_mask) {
  int rc = mrl_plan_precompute(ctx, size, through, dtype_mask);
  if (rc) return rc;
  return upload_and_fill(ctx);
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

int mrl_plan_share(mrl_ctx* ctx, void* ptrs[8], uint64_t sizes[8]) {
  if (!ctx || !ptrs || !sizes) return -1;
  if (!ctx->planned) return fail(ctx, -1, "nothing planned");
  u64 sz[Plan::N_BLOBS];
  ctx->plan.share_blobs(ptrs, sz);
  for (int k = 0; k < Plan::N_BLOBS; k++) sizes[k] = sz[k];
  return 0;
}

int mrl_plan_adopt(mrl_ctx* ctx, const uint64_t sizes[8], void* ptrs[8], int cands_on_device_only) {
  if (!ctx || !sizes || !ptrs) return -1;
  try {
    u64 sz[Plan::N_BLOBS];
    for (int k = 0; k < Plan::N_BLOBS; k++) sz[k] = sizes[k];
    ctx->dev.wait_upload();   // a background upload may still be reading the old plan
    ctx->plan = Plan();
    ctx->planned = ctx->uploaded = ctx->filled = false;
    ctx->table_only = false;
    ctx->plan.adopt_alloc(sz);
    ctx->plan.share_blobs(ptrs, sz);
    ctx->cands_elsewhere = cands_on_device_only != 0;
    if (ctx->cands_elsewhere) ptrs[3] = nullptr;   // never touched on this host
    return 0;
  } catch (const std::exception& e) {
    return fail(ctx, -1, e.what());
  }
}

int mrl_plan_adopt_done(mrl_ctx* ctx, double plan_seconds) {
  if (!ctx) return -1;
  try {
    ctx->plan.adopt_done(ctx->rank, ctx->world, ctx->n_threads, !ctx->cands_elsewhere);
    const PlanStats& ps = ctx->plan.stats;
    memset(&ctx->stats, 0, sizeof(ctx->stats));
    ctx->stats.n_specs = ps.n_specs;
    ctx->stats.n_goal_specs = ps.n_goal_specs;
    ctx->stats.n_candidates = ps.n_cands;
    ctx->stats.n_stages = ps.n_stages;
    ctx->stats.plan_seconds = plan_seconds;
    ctx->planned = true;
    return 0;
  } catch (const std::exception& e) {
    return fail(ctx, -1, e.what());
  }
}

uint64_t mrl_num_stages(const mrl_ctx* ctx) { return ctx && ctx->planned ? ctx->plan.stages.size() : 0; }
uint64_t mrl_num_families(const mrl_ctx* ctx) { return ctx && ctx->planned ? ctx->plan.families.size() : 0; }

int mrl_stage_info(const mrl_ctx* ctx, uint64_t stage, uint32_t* spec_lo, uint32_t* spec_hi, uint32_t* family_lo,
                   uint32_t* family_hi) {
  if (!ctx || !ctx->planned || stage >= ctx->plan.stages.size()) return -1;
  const Stage& st = ctx->plan.stages[stage];
  if (spec_lo) *spec_lo = st.spec_lo;
  if (spec_hi) *spec_hi = st.spec_hi;
  if (family_lo) *family_lo = st.fam_lo;
  if (family_hi) *family_hi = st.fam_hi;
  return 0;
}

int mrl_family_info(const mrl_ctx* ctx, uint64_t family, uint32_t* stage, uint32_t* owner, uint32_t* spec_lo,
                    uint32_t* spec_hi) {
  if (!ctx || !ctx->planned || family >= ctx->plan.families.size()) return -1;
  const Family& f = ctx->plan.families[family];
  if (stage) *stage = f.stage;
  if (owner) *owner = f.owner;
  if (spec_lo) *spec_lo = f.spec_lo;
  if (spec_hi) *spec_hi = f.spec_hi;
  return 0;
}

int mrl_spec_owners(const mrl_ctx* ctx, uint8_t* out, uint64_t n) {
  if (!ctx || !ctx->planned || !out || n != ctx->plan.hdrs.size()) return -1;
  if (ctx->plan.owner.empty()) memset(out, 0, n);
  else memcpy(out, ctx->plan.owner.data(), n);
  return 0;
}

int mrl_device_cands(const mrl_ctx* ctx, void** ptr, uint64_t* bytes) {
  if (!ctx || !ctx->uploaded) return -1;
  if (const_cast<mrl_ctx*>(ctx)->dev.wait_upload()) return -2;   // the caller is about to read them
  if (ptr) *ptr = ctx->dev.device_cands();
  if (bytes) *bytes = ctx->dev.device_cand_bytes();
  return 0;
}

int mrl_cands_arrived(mrl_ctx* ctx) {
  if (!ctx || !ctx->uploaded) return -1;
  int rc = ctx->dev.cands_arrived();
  if (rc != 0) return fail(ctx, rc == -2 ? -2 : -1, ctx->dev.error());
  return 0;
}

uint32_t mrl_row_bytes(void) { return (uint32_t)sizeof(MrlRow); }

int mrl_device_rows(const mrl_ctx* ctx, void** ptr, uint64_t* n_rows) {
  if (!ctx || !ctx->filled) return -1;
  if (ptr) *ptr = ctx->dev.device_rows();
  if (n_rows) *n_rows = ctx->dev.stats().n_rows;
  return 0;
}

int mrl_fill_begin(mrl_ctx* ctx) {
  if (!ctx) return -1;
  if (!ctx->uploaded) return fail(ctx, -1, "plan not uploaded");
  ctx->filled = false;
  int rc = ctx->dev.begin_fill();
  if (rc != 0) return fail(ctx, rc == -3 ? -3 : -2, ctx->dev.error());
  return 0;
}

int mrl_fill_stage_solve(mrl_ctx* ctx, uint64_t stage, void** masks, uint64_t* mask_bytes) {
  if (!ctx || !ctx->uploaded) return -1;
  int rc = ctx->dev.solve_stage(ctx->plan, (uint32_t)stage);
  if (rc != 0) return fail(ctx, (rc == -5 || rc == -6 || rc == -3) ? rc : -2, ctx->dev.error());
  if (ctx->dev.stage_masks(ctx->plan, (uint32_t)stage, masks, mask_bytes) != 0) return fail(ctx, -2, ctx->dev.error());
  return 0;
}

int mrl_fill_stage_place(mrl_ctx* ctx, uint64_t stage, void** rows, uint64_t* row_bytes) {
  if (!ctx || !ctx->uploaded) return -1;
  void* p = nullptr;
  uint64_t b = 0;
  int rc = ctx->dev.place_stage(ctx->plan, (uint32_t)stage, &p, &b);
  if (rc != 0) return fail(ctx, (rc == -5 || rc == -6 || rc == -3) ? rc : -2, ctx->dev.error());
  if (rows) *rows = p;
  if (row_bytes) *row_bytes = b;
  return 0;
}

int mrl_fill_end(mrl_ctx* ctx) {
  if (!ctx || !ctx->uploaded) return -1;
  int rc = ctx->dev.end_fill();
  copy_fill_stats(ctx);
  if (rc != 0) return fail(ctx, -2, ctx->dev.error());
  ctx->filled = true;
  return 0;
}

namespace {
// One node of the reconstruction and, below it, its sub-Specs at the limits the stored action
// leaves them (morello/src/reconstruct.rs:14-80).
void reconstruct(mrl_ctx* ctx, const LogicalSpec& ls, const u64 limits[4], int level, std::string& out) {
  const long id = ctx->plan.find(ls);
  uint32_t pack = 0;
  if (id < 0 || !ctx->plan.pack_limits(limits, &pack)) throw ModelError("not in the tables: " + ls.str());
  const uint32_t id32 = (uint32_t)id;
  MrlRow row;
  if (ctx->dev.lookup(&id32, &pack, 1, &row) != 0) throw ModelError(ctx->dev.error());
  mrl_decision d;
  decode_row(row, &d);
  if (d.found != 1) throw ModelError("no implementation for " + ls.str());
  std::vector<Candidate> cs;
  tabulate_candidates(ls, cs);
  const Candidate* chosen = nullptr;
  for (const Candidate& c : cs) if (c.action == d.action) chosen = &c;
  if (!chosen) throw ModelError("stored action is not among the Spec's actions: " + ls.str());
  out += impl_line(level, ls, limits, d.action, action_text(*chosen), d.main_cost, d.peaks, d.depth);
  u64 child_limits[4] = {limits[0], limits[1], limits[2], limits[3]};
  if (chosen->kind == CK_MOVE) {
    const int m = chosen->level;
    if (limits[m] < chosen->units) throw ModelError("stored Move does not fit its limits");
    const u64 rem = limits[m] - chosen->units;
    child_limits[m] = mem_counts_registers((Mem)m) ? rem : prev_power_of_two(rem);
  }
  for (int j = 0; j < chosen->nchild; j++) reconstruct(ctx, chosen->child[j], child_limits, level + 1, out);
}
}  // namespace

long mrl_get_impl(mrl_ctx* ctx, const uint8_t* blob, size_t len, const uint64_t limits[4], char* out, size_t cap) {
  if (!ctx) return -1;
  if (!ctx->filled) return fail(ctx, -1, "tables are not filled");
  try {
    LogicalSpec ls = LogicalSpec::from_key(std::string((const char*)blob, len));
    if (logicalspec_canonicalize(ls) != CANON_OK) return fail(ctx, -4, "Spec is not canonicalizable");
    std::string text;
    reconstruct(ctx, ls, limits, 0, text);
    if (text.size() + 1 > cap) return fail(ctx, -3, "implementation text needs " + std::to_string(text.size() + 1) + " bytes");
    memcpy(out, text.c_str(), text.size() + 1);
    return (long)text.size();
  } catch (const std::exception& e) {
    return fail(ctx, -1, e.what());
  }
}

int mrl_verify(mrl_ctx* ctx, uint64_t n_samples, uint64_t seed, uint64_t* n_checked, uint64_t* n_mismatch) {
  if (!ctx) return -1;
  if (!ctx->filled) return fail(ctx, -1, "tables are not filled");
  if (ctx->table_only) return fail(ctx, -1, "the tables were loaded from a file without their plan: plan the job, then load, to verify");
  uint64_t first_bad = 0;
  if (ctx->dev.verify(ctx->plan, n_samples, seed, n_checked, n_mismatch, &first_bad) != 0) return fail(ctx, -2, ctx->dev.error());
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

int mrl_spec_grid(mrl_ctx* ctx, uint64_t spec_id, uint32_t masks[4], uint64_t* n_cells) {
  if (!ctx || !ctx->filled || spec_id >= ctx->plan.specs.size()) return -1;
  SpecHdr h;
  if (ctx->dev.read_hdr((uint32_t)spec_id, &h) != 0) return fail(ctx, -2, ctx->dev.error());
  uint64_t n = 1;
  for (int k = 0; k < 4; k++) { masks[k] = h.mask[k]; n *= (uint64_t)__builtin_popcount(h.mask[k]); }
  if (n_cells) *n_cells = n;
  return 0;
}

int mrl_export_rows(mrl_ctx* ctx, uint64_t spec_id, mrl_decision* out, size_t cap) {
  if (!ctx || !ctx->filled || spec_id >= ctx->plan.specs.size()) return -1;
  SpecHdr h;
  if (ctx->dev.read_hdr((uint32_t)spec_id, &h) != 0) return fail(ctx, -2, ctx->dev.error());
  uint64_t n = 1;
  for (int k = 0; k < 4; k++) n *= (uint64_t)__builtin_popcount(h.mask[k]);
  if (n > cap) return fail(ctx, -3, "export buffer too small");
  std::vector<MrlRow> rows(n);
  if (ctx->dev.read_rows(h.row_base, n, rows.data()) != 0) return fail(ctx, -2, ctx->dev.error());
  for (uint64_t i = 0; i < n; i++) decode_row(rows[i], &out[i]);
  return 0;
}

int mrl_checksum(mrl_ctx* ctx, uint64_t* out) {
  if (!ctx || !out) return -1;
  if (!ctx->filled) return fail(ctx, -1, "tables are not filled");
  if (ctx->dev.checksum(out) != 0) return fail(ctx, -2, ctx->dev.error());
  return 0;
}

void mrl_decode_row(const mrl_row* row, mrl_decision* out) {
  MrlRow r;
  r.main = row->main_cost; r.peaks = row->peak_codes; r.tail = row->depth_action; r.aux = 0;
  decode_row(r, out);
}

int mrl_export_all(mrl_ctx* ctx, uint32_t* masks, uint64_t* first_row, mrl_row* rows, uint64_t rows_cap) {
  if (!ctx || !masks || !first_row || !rows) return -1;
  if (!ctx->filled) return fail(ctx, -1, "tables are not filled");
  static_assert(sizeof(mrl_row) == sizeof(MrlRow), "exported rows are the device rows");
  try {
    const uint64_t n = ctx->plan.hdrs.size(), n_rows = ctx->dev.stats().n_rows;
    if (rows_cap < n_rows) return fail(ctx, -3, "export buffer too small");
    std::vector<SpecHdr> h(n);
    if (ctx->dev.read_table(h.data(), reinterpret_cast<MrlRow*>(rows)) != 0) return fail(ctx, -2, ctx->dev.error());
    for (uint64_t i = 0; i < n; i++) {
      for (int k = 0; k < 4; k++) masks[4 * i + k] = h[i].mask[k];
      first_row[i] = h[i].row_base;
    }
    first_row[n] = n_rows;
    ctx->stats.d2h_bytes = n * sizeof(SpecHdr) + n_rows * sizeof(MrlRow);
    return 0;
  } catch (const std::exception& e) {
    return fail(ctx, -1, e.what());
  }
}

long mrl_export_rects(mrl_ctx* ctx, uint64_t spec_id, uint8_t* lo, uint8_t* hi, mrl_decision* out, size_t cap) {
  if (!ctx || !ctx->filled || spec_id >= ctx->plan.specs.size()) return -1;
  try {
    SpecHdr h;
    if (ctx->dev.read_hdr((uint32_t)spec_id, &h) != 0) return fail(ctx, -2, ctx->dev.error());
    uint32_t nn[4], codes[4][32];
    uint64_t n = 1;
    for (int k = 0; k < 4; k++) {
      nn[k] = 0;
      for (uint32_t c = 0; c < 31; c++) if (h.mask[k] >> c & 1u) codes[k][nn[k]++] = c;
      n *= nn[k];
    }
    std::vector<MrlRow> rows(n);
    if (ctx->dev.read_rows(h.row_base, n, rows.data()) != 0) return fail(ctx, -2, ctx->dev.error());
    // One rectangle per cell to begin with: [breakpoint .. next breakpoint - 1] (the last one ends at
    // the top limits); then, axis by axis, neighbours with equal decisions and equal extents in the
    // other axes are merged - what merge-on-insert leaves of a sequence of puts (pagecontents.rs:125-184).
    struct Rect { uint8_t lo[4], hi[4]; uint32_t row; bool dead; };
    std::vector<Rect> rects(n);
    for (uint64_t i = 0; i < n; i++) {
      uint64_t rest = i;
      Rect& r = rects[i];
      for (int k = 0; k < 4; k++) {
        const uint32_t s = (uint32_t)(rest % nn[k]);
        rest /= nn[k];
        r.lo[k] = (uint8_t)codes[k][s];
        r.hi[k] = (uint8_t)(s + 1 < nn[k] ? codes[k][s + 1] - 1 : ctx->plan.top_code[k]);
      }
      r.row = (uint32_t)i;
      r.dead = false;
    }
    auto same_value = [&](const Rect& a, const Rect& b) {
      const MrlRow &x = rows[a.row], &y = rows[b.row];
      return x.main == y.main && x.peaks == y.peaks && x.tail == y.tail;
    };
    for (int k = 0; k < 4; k++) {
      // sort by the other axes' extents, then by lo[k]; merge runs that touch
      std::vector<uint32_t> idx;
      for (uint32_t i = 0; i < rects.size(); i++) if (!rects[i].dead) idx.push_back(i);
      auto key_other = [&](const Rect& r, int q) { return ((uint32_t)r.lo[q] << 8) | r.hi[q]; };
      std::sort(idx.begin(), idx.end(), [&](uint32_t a, uint32_t b) {
        for (int q = 0; q < 4; q++) {
          if (q == k) continue;
          const uint32_t ka = key_other(rects[a], q), kb = key_other(rects[b], q);
          if (ka != kb) return ka < kb;
        }
        return rects[a].lo[k] < rects[b].lo[k];
      });
      for (size_t p = 0; p + 1 < idx.size();) {
        Rect& a = rects[idx[p]];
        size_t q = p + 1;
        while (q < idx.size()) {
          Rect& b = rects[idx[q]];
          bool same_other = true;
          for (int d = 0; d < 4; d++) if (d != k && (a.lo[d] != b.lo[d] || a.hi[d] != b.hi[d])) same_other = false;
          if (!same_other || b.lo[k] != a.hi[k] + 1 || !same_value(a, b)) break;
          a.hi[k] = b.hi[k];
          b.dead = true;
          q++;
        }
        p = q;
      }
    }
    size_t m = 0;
    for (const Rect& r : rects) {
      if (r.dead) continue;
      if (m >= cap) return fail(ctx, -3, "export buffer too small");
      for (int k = 0; k < 4; k++) { lo[4 * m + k] = r.lo[k]; hi[4 * m + k] = r.hi[k]; }
      decode_row(rows[r.row], &out[m]);
      m++;
    }
    return (long)m;
  } catch (const std::exception& e) {
    return fail(ctx, -1, e.what());
  }
}

int mrl_put(mrl_ctx* ctx, const uint8_t* blob, size_t len, const uint64_t limits[4], const mrl_decision* decision) {
  if (!ctx || !blob || !limits || !decision) return -1;
  if (!ctx->filled) return fail(ctx, -1, "tables are not filled");
  const uint64_t off[2] = {0, len};
  mrl_decision have;
  int rc = mrl_get_many(ctx, blob, off, 1, limits, &have);
  if (rc) return rc;
  if (have.found < 0) return fail(ctx, -3, "the Spec (or its limits) is not in the tables; plan a fill that covers it");
  bool same = have.found == (decision->found ? 1 : 0);
  if (same && have.found == 1)
    same = have.action == decision->action && have.main_cost == decision->main_cost && have.depth == decision->depth &&
           memcmp(have.peaks, decision->peaks, sizeof(have.peaks)) == 0;
  if (!same) return fail(ctx, -9, "the tables hold another decision for this Spec and limits; every cell is a direct solve and is not overwritten");
  return 0;
}

namespace {
// File layout of a saved database. All integers little-endian.
struct FileHeader {
  char magic[8];          // "MRLB200\0"
  uint32_t version;       // 1
  uint32_t target;        // 1 = Avx2 (the X86 target's default), the TARGET guard of db/mod.rs:2091-2153
  uint32_t tile_scale;    // 1 = power-of-two tiles, the TILESCALE guard
  uint32_t top_code[4];
  uint32_t reserved;
  uint64_t n_specs, n_rows, blob_bytes;
  uint64_t fingerprint;   // of the Specs in id order
  uint64_t table_checksum;  // mrl_checksum of the contents
};
const char kMagic[8] = {'M', 'R', 'L', 'B', '2', '0', '0', 0};

bool write_all(FILE* f, const void* p, size_t n) { return n == 0 || fwrite(p, 1, n, f) == n; }
bool read_all(FILE* f, void* p, size_t n) { return n == 0 || fread(p, 1, n, f) == n; }
}  // namespace

int mrl_save(mrl_ctx* ctx, const char* path) {
  if (!ctx || !path) return -1;
  if (!ctx->filled) return fail(ctx, -1, "tables are not filled");
  try {
    const uint64_t n = ctx->plan.hdrs.size(), n_rows = ctx->dev.stats().n_rows;
    std::vector<SpecHdr> h(n);
    std::vector<MrlRow> rows(n_rows);
    if (ctx->dev.read_table(h.data(), rows.data()) != 0) return fail(ctx, -2, ctx->dev.error());
    FileHeader fh;
    memset(&fh, 0, sizeof(fh));
    memcpy(fh.magic, kMagic, 8);
    fh.version = 1; fh.target = 1; fh.tile_scale = 1;
    for (int k = 0; k < 4; k++) fh.top_code[k] = ctx->plan.top_code[k];
    fh.n_specs = n; fh.n_rows = n_rows;
    fh.fingerprint = ctx->plan.fingerprint(ctx->n_threads);
    if (ctx->dev.checksum(&fh.table_checksum) != 0) return fail(ctx, -2, ctx->dev.error());
    std::string blobs;
    std::vector<uint32_t> blob_end(n);
    for (uint64_t i = 0; i < n; i++) {
      char kb[LogicalSpec::MAX_KEY];
      const int kl = ctx->plan.specs[i].key_into(kb);
      blobs.append(kb, (size_t)kl);
      blob_end[i] = (uint32_t)blobs.size();
    }
    fh.blob_bytes = blobs.size();
    const std::string tmp = std::string(path) + ".tmp";
    FILE* f = fopen(tmp.c_str(), "wb");
    if (!f) return fail(ctx, -1, "cannot create " + tmp);
    bool ok = write_all(f, &fh, sizeof(fh)) && write_all(f, blob_end.data(), n * sizeof(uint32_t)) &&
              write_all(f, blobs.data(), blobs.size()) && write_all(f, h.data(), n * sizeof(SpecHdr)) &&
              write_all(f, rows.data(), n_rows * sizeof(MrlRow));
    ok = (fflush(f) == 0) && ok;
    ok = (fclose(f) == 0) && ok;
    if (!ok || rename(tmp.c_str(), path) != 0) {
      remove(tmp.c_str());
      return fail(ctx, -1, std::string("cannot write ") + path);
    }
    ctx->stats.d2h_bytes = n * sizeof(SpecHdr) + n_rows * sizeof(MrlRow);
    return 0;
  } catch (const std::exception& e) {
    return fail(ctx, -1, e.what());
  }
}

int mrl_load(mrl_ctx* ctx, const char* path) {
  if (!ctx || !path) return -1;
  FILE* f = fopen(path, "rb");
  if (!f) return fail(ctx, -1, std::string("cannot open ") + path);
  struct Closer { FILE* f; ~Closer() { fclose(f); } } closer{f};
  try {
    FileHeader fh;
    if (!read_all(f, &fh, sizeof(fh)) || memcmp(fh.magic, kMagic, 8) != 0 || fh.version != 1)
      return fail(ctx, -7, "not a database saved by this library");
    if (fh.target != 1 || fh.tile_scale != 1) return fail(ctx, -7, "the database was saved for another target or tile scale");
    // sizes must add up to the file's length before anything is allocated by them
    if (fseek(f, 0, SEEK_END) != 0) return fail(ctx, -8, "cannot size the file");
    const long long file_len = ftell(f);
    const unsigned __int128 want = (unsigned __int128)sizeof(fh) + (unsigned __int128)fh.n_specs * (4 + sizeof(SpecHdr)) + fh.blob_bytes +
                                   (unsigned __int128)fh.n_rows * sizeof(MrlRow);
    if (file_len < 0 || want != (unsigned __int128)file_len || fh.n_specs > 0xFFFFFFF0ull)
      return fail(ctx, -8, "the database file is truncated or its sizes are corrupt");
    for (int k = 0; k < 4; k++) if (fh.top_code[k] > 30) return fail(ctx, -8, "the database file is corrupt (limits)");
    fseek(f, (long)sizeof(fh), SEEK_SET);
    const uint64_t n = fh.n_specs;
    std::vector<uint32_t> blob_end(n);
    std::string blobs(fh.blob_bytes, '\0');
    RawVec<SpecHdr> hdrs;
    hdrs.reset(n);
    std::vector<MrlRow> rows(fh.n_rows);
    if (!read_all(f, blob_end.data(), n * sizeof(uint32_t)) || !read_all(f, &blobs[0], blobs.size()) ||
        !read_all(f, hdrs.data(), n * sizeof(SpecHdr)) || !read_all(f, rows.data(), fh.n_rows * sizeof(MrlRow)))
      return fail(ctx, -8, "the database file is truncated");
    // headers: every Spec's cell block inside the rows
    for (uint64_t i = 0; i < n; i++) {
      uint64_t cells = 1;
      for (int k = 0; k < 4; k++) {
        if (!(hdrs[i].mask[k] & 1u) || (hdrs[i].mask[k] >> (fh.top_code[k] + 1))) return fail(ctx, -8, "the database file is corrupt (masks)");
        cells *= (uint64_t)__builtin_popcount(hdrs[i].mask[k]);
      }
      if (hdrs[i].row_base > fh.n_rows || cells > fh.n_rows - hdrs[i].row_base) return fail(ctx, -8, "the database file is corrupt (rows)");
      if (blob_end[i] > blobs.size() || (i && blob_end[i] < blob_end[i - 1])) return fail(ctx, -8, "the database file is corrupt (Specs)");
    }
    // the file is sound as far as the host can tell; from here on a device is needed
    if (ctx->device < 0) return fail(ctx, -2, "planning-only context: no device to load onto");
    const bool same_job = ctx->planned && !ctx->table_only && ctx->plan.hdrs.size() == n &&
                          ctx->plan.fingerprint(ctx->n_threads) == fh.fingerprint;
    if (!same_job) {
      RawVec<LogicalSpec> specs;
      specs.reset(n);
      for (uint64_t i = 0; i < n; i++) {
        const size_t lo = i ? blob_end[i - 1] : 0;
        new (&specs[i]) LogicalSpec(LogicalSpec::from_key(blobs.substr(lo, blob_end[i] - lo)));
      }
      for (uint64_t i = 0; i < n; i++) { hdrs[i].cand_off = 0; hdrs[i].ncand = 0; }
      ctx->dev.wait_upload();
      ctx->plan = table_only_plan(std::move(specs), std::move(hdrs), fh.top_code, ctx->n_threads);
      if (ctx->plan.fingerprint(ctx->n_threads) != fh.fingerprint) return fail(ctx, -8, "the database file is corrupt (Spec fingerprint)");
      ctx->planned = true;
      ctx->table_only = true;
      ctx->cands_elsewhere = false;
      memset(&ctx->stats, 0, sizeof(ctx->stats));
      ctx->stats.n_specs = n;
      int rc = ctx->dev.upload(ctx->plan);
      if (rc != 0) return fail(ctx, rc == -6 ? -6 : -2, ctx->dev.error());
      ctx->uploaded = true;
      if (ctx->dev.load_table(ctx->plan, ctx->plan.hdrs.data(), rows.data(), fh.n_rows) != 0) return fail(ctx, -2, ctx->dev.error());
    } else {
      if (!ctx->uploaded) {
        int rc = ctx->dev.upload(ctx->plan, ctx->cands_elsewhere);
        if (rc != 0) return fail(ctx, rc == -6 ? -6 : -2, ctx->dev.error());
        ctx->uploaded = true;
      }
      // the plan's own candidate ranges stay; masks and first rows come from the file
      for (uint64_t i = 0; i < n; i++) { hdrs[i].cand_off = ctx->plan.hdrs[i].cand_off; hdrs[i].ncand = ctx->plan.hdrs[i].ncand; }
      if (ctx->dev.load_table(ctx->plan, hdrs.data(), rows.data(), fh.n_rows) != 0) return fail(ctx, -2, ctx->dev.error());
    }
    ctx->filled = true;
    ctx->stats.n_rows = fh.n_rows;
    ctx->stats.h2d_bytes = n * sizeof(SpecHdr) + fh.n_rows * sizeof(MrlRow);
    uint64_t sum = 0;
    if (ctx->dev.checksum(&sum) != 0) return fail(ctx, -2, ctx->dev.error());
    if (sum != fh.table_checksum) {
      ctx->filled = false;
      return fail(ctx, -8, "the database file is corrupt (contents do not match their checksum)");
    }
    return 0;
  } catch (const std::exception& e) {
    ctx->filled = false;
    return fail(ctx, -8, std::string("the database file is corrupt: ") + e.what());
  }
}

}  // extern "C"

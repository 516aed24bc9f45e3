// Host-side planner of the database fill. See plan.hpp.
#include "plan.hpp"
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <chrono>
#include <mutex>
#include <thread>
#include <unordered_map>

namespace mrl {

namespace {

constexpr int NSHARD = 512;

struct Shard {
  std::mutex mu;
  std::unordered_map<std::string, u32> map;
};

struct TempSpec {
  LogicalSpec ls;
  std::string key;
  std::vector<CandRec> cands;  // child[] holds temporary ids
};

double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

template <class F>
void parallel_for(size_t n, int n_threads, F f) {
  if (n_threads <= 1 || n < 64) {
    for (size_t i = 0; i < n; i++) f(i, 0);
    return;
  }
  std::atomic<size_t> next{0};
  std::vector<std::thread> pool;
  std::vector<std::string> errors(n_threads);
  for (int t = 0; t < n_threads; t++) {
    pool.emplace_back([&, t]() {
      try {
        while (true) {
          size_t lo = next.fetch_add(64);
          if (lo >= n) break;
          size_t hi = std::min(n, lo + 64);
          for (size_t i = lo; i < hi; i++) f(i, t);
        }
      } catch (const std::exception& e) {
        errors[t] = e.what();
      }
    });
  }
  for (auto& th : pool) th.join();
  for (auto& e : errors) if (!e.empty()) throw ModelError(e);
}

u32 shape_log_sum(const LogicalSpec& ls) {
  u32 s = 0;
  for (int i = 0; i < ls.spec_shape.n; i++) s += bit_length(ls.spec_shape[i]) - 1;
  return s;
}

// Smallest limit code whose value is >= units, and the code of the peak `units` itself
// leaves behind (registers: raw; caches: rounded to a power of two,
// morello/src/memorylimits.rs:159-170,458-470).
u32 code_ceil(int mem, u64 units) {
  if (mem_counts_registers((Mem)mem)) return (u32)units;
  return bit_length(next_binary_power(units));
}

}  // namespace

std::vector<LogicalSpec> precompute_goals(u32 size, Through through, const std::vector<Dtype>& dtypes, int n_threads) {
  struct Task { Bound b; std::vector<u32> pt; };
  std::vector<Task> tasks;
  for (auto& phase : goal_phases(size, through, dtypes))
    for (const Bound& b : phase)
      for (auto& stage : diagonals(bound_point(b)))
        for (auto& pt : stage) tasks.push_back(Task{b, pt});
  std::vector<std::vector<LogicalSpec>> per_task(tasks.size());
  parallel_for(tasks.size(), n_threads, [&](size_t i, int) { per_task[i] = task_point_specs(tasks[i].b, tasks[i].pt); });
  std::vector<LogicalSpec> goals;
  size_t total = 0;
  for (auto& v : per_task) total += v.size();
  goals.reserve(total);
  for (auto& v : per_task) goals.insert(goals.end(), v.begin(), v.end());
  return goals;
}

long Plan::find(const LogicalSpec& ls) const {
  std::string k = ls.key();
  auto it = std::lower_bound(sorted_keys_.begin(), sorted_keys_.end(), k,
                             [](const std::pair<std::string, u32>& a, const std::string& b) { return a.first < b; });
  if (it == sorted_keys_.end() || it->first != k) return -1;
  return it->second;
}

long Plan::row_of(u32 id, const u64 limits[NMEM]) const {
  const SpecHdr& h = hdrs[id];
  u64 idx = 0, stride = 1;
  for (int k = 0; k < NMEM; k++) {
    u32 code = limit_code(k, limits[k]);
    if (code > top_code[k]) return -1;  // beyond the limits this table was filled for
    code = slot_of_code(k, code);
    u32 below = h.mask[k] & (code >= 31 ? 0xFFFFFFFFu : ((2u << code) - 1u));
    u32 i = (u32)__builtin_popcount(below) - 1;
    idx += stride * i;
    stride *= (u32)__builtin_popcount(h.mask[k]);
  }
  return (long)(h.row_base + idx);
}

Plan build_plan(const std::vector<LogicalSpec>& goals, int n_threads, const u64* top_limits, const int* caps,
                u32 rank, u32 world) {
  if (n_threads < 1) n_threads = 1;
  if (world < 1 || rank >= world) throw ModelError("bad shard rank / world size");
  Plan plan;
  plan.rank = rank;
  plan.world = world;
  plan.n_threads = n_threads;
  if (const char* e = getenv("MRL_LANES_PER_CELL")) {
    int v = atoi(e);
    if (v == 1 || v == 2) plan.lanes_per_cell = v;
  }
  u32 top_code[NMEM];
  for (int k = 0; k < NMEM; k++) {
    u64 v = top_limits ? top_limits[k] : AVX2_MAX_MEM[k];
    if (!mem_counts_registers((Mem)k) && v != 0 && !is_pow2(v)) throw ModelError("cache limits must be powers of two");
    top_code[k] = limit_code(k, v);
    if (top_code[k] > 30) throw ModelError("memory limit too large for the lattice masks");
    plan.top_code[k] = top_code[k];
    plan.cap_code[k] = (caps && caps[k] >= 0 && (u32)caps[k] < top_code[k]) ? (u32)caps[k] : top_code[k];
  }

  // ---- 1. discovery: closure of the goals under "is a sub-Spec of some candidate" ----
  double t0 = now_s();
  std::vector<Shard> shards(NSHARD);
  std::vector<TempSpec> temp;
  std::atomic<u32> next_id{0};
  auto shard_of = [&](const std::string& k) -> Shard& { return shards[std::hash<std::string>()(k) % NSHARD]; };

  std::vector<u32> frontier;
  {
    for (const LogicalSpec& g0 : goals) {
      LogicalSpec g = g0;
      if (logicalspec_canonicalize(g) != CANON_OK) throw ModelError("goal Spec cannot be canonicalized: " + g0.str());
      std::string k = g.key();
      Shard& sh = shard_of(k);
      auto it = sh.map.find(k);
      if (it == sh.map.end()) {
        u32 id = next_id++;
        sh.map.emplace(k, id);
        TempSpec ts;
        ts.ls = g;
        ts.key = k;
        temp.push_back(std::move(ts));
        frontier.push_back(id);
        plan.goal_ids.push_back(id);
      } else {
        plan.goal_ids.push_back(it->second);
      }
    }
  }
  plan.stats.n_goal_specs = frontier.size();

  while (!frontier.empty()) {
    struct NewSpec { u32 id; LogicalSpec ls; std::string key; };
    std::vector<std::vector<NewSpec>> fresh(n_threads);
    parallel_for(frontier.size(), n_threads, [&](size_t fi, int tid) {
      TempSpec& ts = temp[frontier[fi]];
      std::vector<Candidate> cs;
      tabulate_candidates(ts.ls, cs);
      ts.cands.reserve(cs.size());
      for (const Candidate& c : cs) {
        CandRec r;
        memset(&r, 0, sizeof(r));
        r.action = c.action;
        r.kind = c.kind;
        r.nchild = c.nchild;
        r.imm = c.imm;
        r.level = c.level;
        r.units = c.units;
        u32 thr = (c.kind == CK_MOVE || c.kind == CK_LEAF) ? code_ceil(c.level, c.units) : 0;
        if (thr > top_code[c.level]) continue;  // never fits, at any limits in the lattice
        r.thr_code = (u8)thr;
        r.peak_code = (c.kind == CK_LEAF) ? (u8)code_ceil(c.level, c.units) : 0;
        for (int j = 0; j < c.nchild; j++) {
          std::string k = c.child[j].key();
          Shard& sh = shard_of(k);
          u32 id;
          {
            std::lock_guard<std::mutex> g(sh.mu);
            auto it = sh.map.find(k);
            if (it != sh.map.end()) id = it->second;
            else {
              id = next_id++;
              sh.map.emplace(k, id);
              fresh[tid].push_back(NewSpec{id, c.child[j], k});
            }
          }
          r.child[j] = id;
        }
        ts.cands.push_back(r);
      }
    });
    frontier.clear();
    temp.resize(next_id.load());
    for (auto& v : fresh)
      for (auto& ns : v) {
        temp[ns.id].ls = ns.ls;
        temp[ns.id].key = std::move(ns.key);
        frontier.push_back(ns.id);
      }
    std::sort(frontier.begin(), frontier.end());
  }
  const u32 n = (u32)temp.size();
  plan.stats.seconds_discover = now_s() - t0;

  // ---- 2. final ids: group-major (phase, log-shape sum), then key order ----
  double t1 = now_s();
  std::vector<u32> order(n);
  for (u32 i = 0; i < n; i++) order[i] = i;
  std::vector<u32> gkey(n);
  for (u32 i = 0; i < n; i++) gkey[i] = ((u32)temp[i].ls.kind << 8) | shape_log_sum(temp[i].ls);
  std::sort(order.begin(), order.end(), [&](u32 a, u32 b) {
    if (gkey[a] != gkey[b]) return gkey[a] < gkey[b];
    return temp[a].key < temp[b].key;
  });
  if (getenv("MRL_PLAN_TIMING")) fprintf(stderr, "[plan]   sort ids %.2fs\n", now_s() - t1);
  std::vector<u32> new_id(n);
  for (u32 i = 0; i < n; i++) new_id[order[i]] = i;
  for (u32& g : plan.goal_ids) g = new_id[g];

  plan.specs.resize(n);
  plan.hdrs.resize(n);
  u64 ncand = 0;
  for (u32 i = 0; i < n; i++) ncand += temp[order[i]].cands.size();
  if (ncand > 0xFFFFFFFFull) throw ModelError("too many candidate records");
  plan.cands.resize(ncand);
  {
    std::vector<u64> offs(n + 1, 0);
    for (u32 i = 0; i < n; i++) offs[i + 1] = offs[i] + temp[order[i]].cands.size();
    plan.sorted_keys_.resize(n);
    std::vector<u64> kids_t(n_threads, 0);
    parallel_for(n, n_threads, [&](size_t i, int tid) {
      TempSpec& ts = temp[order[i]];
      plan.specs[i] = ts.ls;
      SpecHdr& h = plan.hdrs[i];
      memset(&h, 0, sizeof(h));
      u64 off = offs[i];
      h.cand_off = (u32)off;
      h.ncand = (u32)ts.cands.size();
      // Evaluation order is free (the argmin carries the action number): kernels first, then
      // loops and blocks, then Moves by ascending base cost, so that the kernel's lower-bound
      // test on a Move's base cost cuts as early as possible.
      std::stable_sort(ts.cands.begin(), ts.cands.end(), [](const CandRec& a, const CandRec& b) {
        auto rank = [](const CandRec& c) -> u64 {
          u64 k = c.kind == MRL_CK_LEAF ? 0 : (c.kind == MRL_CK_LOOP ? 1 : (c.kind == MRL_CK_BLOCK ? 2 : 3));
          return (k << 32) | (c.kind == MRL_CK_MOVE ? c.imm : 0u);
        };
        return rank(a) < rank(b);
      });
      for (CandRec r : ts.cands) {
        for (int j = 0; j < r.nchild; j++) r.child[j] = new_id[r.child[j]];
        kids_t[tid] += r.nchild;
        plan.cands[off++] = r;
      }
      plan.sorted_keys_[i] = {std::move(ts.key), (u32)i};
      std::vector<CandRec>().swap(ts.cands);
    });
    for (u64 k : kids_t) plan.stats.n_children += k;
  }
  if (getenv("MRL_PLAN_TIMING")) fprintf(stderr, "[plan]   move specs+cands %.2fs\n", now_s() - t1);
  std::vector<TempSpec>().swap(temp);
  if (getenv("MRL_PLAN_TIMING")) fprintf(stderr, "[plan]   free temp %.2fs\n", now_s() - t1);
  std::sort(plan.sorted_keys_.begin(), plan.sorted_keys_.end());
  if (getenv("MRL_PLAN_TIMING")) fprintf(stderr, "[plan]   sort keys %.2fs\n", now_s() - t1);

  // groups
  for (u32 i = 0; i < n;) {
    u32 gk = ((u32)plan.specs[i].kind << 8) | shape_log_sum(plan.specs[i]);
    u32 j = i;
    while (j < n && ((((u32)plan.specs[j].kind << 8) | shape_log_sum(plan.specs[j])) == gk)) j++;
    Group g;
    g.spec_lo = i;
    g.spec_hi = j;
    g.phase = (u8)(gk >> 8);
    g.shape_sum = (u8)(gk & 0xff);
    plan.groups.push_back(g);
    i = j;
  }
  // families: maximal runs with equal dtype and shape inside a group (ids are key-sorted, and
  // the key starts with kind, dtype, serial flag, rank, shape)
  for (u32 gi = 0; gi < plan.groups.size(); gi++) {
    const Group& g = plan.groups[gi];
    for (u32 i = g.spec_lo; i < g.spec_hi;) {
      u32 j = i;
      while (j < g.spec_hi && plan.specs[j].dtype == plan.specs[i].dtype && plan.specs[j].spec_shape == plan.specs[i].spec_shape) j++;
      Family f;
      f.spec_lo = i;
      f.spec_hi = j;
      f.group = gi;
      plan.families.push_back(f);
      i = j;
    }
  }
  plan.stats.seconds_layout = now_s() - t1;
  if (getenv("MRL_PLAN_TIMING")) fprintf(stderr, "[plan] discover %.2fs, ids/groups/families %.2fs\n", plan.stats.seconds_discover, plan.stats.seconds_layout);

  plan.stats.n_specs = n;
  plan.stats.n_cands = ncand;
  relayout_plan(plan, caps);
  return plan;
}

void relayout_plan(Plan& plan, const int* caps) {
  const u32 n = (u32)plan.hdrs.size();
  const u32* top_code = plan.top_code;
  const int n_threads = plan.n_threads;
  for (int k = 0; k < NMEM; k++)
    plan.cap_code[k] = (caps && caps[k] >= 0 && (u32)caps[k] < top_code[k]) ? (u32)caps[k] : top_code[k];
  plan.steps.clear();
  plan.stats.mask_sweeps = 0;

  // ---- 3. breakpoint masks: least fixpoint of "a parent's result can change wherever one
  //         of its candidates becomes feasible or one of its children's results changes" ----
  double t2 = now_s();
  for (u32 i = 0; i < n; i++) for (int k = 0; k < NMEM; k++) plan.hdrs[i].mask[k] = 1u;
  // Masks live in slot space (Plan::cap_code). A threshold at limit code t sets slot_ceil(t).
  // A Move lowers its children's limit in the destination memory, so their code there is always
  // below the top: only the child's slots 0..cap (real codes) feed the parent's thresholds.
  u32 real_slots[NMEM];   // mask of slots that are plain codes (0..cap, or 0..top when not compressed)
  for (int k = 0; k < NMEM; k++) {
    u32 hi = plan.compressed(k) ? plan.cap_code[k] : top_code[k];
    real_slots[k] = (hi >= 31) ? 0xFFFFFFFFu : ((2u << hi) - 1u);
  }
  // Sweeps run on all threads over disjoint Spec ranges; a thread may read a mask another thread
  // is growing (relaxed atomics). Masks only ever gain bits, so any interleaving reaches the
  // same least fixpoint; the loop ends after a sweep in which nothing changed.
  std::atomic<bool> changed{true};
  while (changed.load()) {
    changed = false;
    plan.stats.mask_sweeps++;
    parallel_for(n, n_threads, [&](size_t i, int) {
      SpecHdr& h = plan.hdrs[i];
      u32 m[NMEM];
      for (int k = 0; k < NMEM; k++) m[k] = __atomic_load_n(&h.mask[k], __ATOMIC_RELAXED);
      const u32 m0[NMEM] = {m[0], m[1], m[2], m[3]};
      for (u32 c = h.cand_off; c < h.cand_off + h.ncand; c++) {
        const CandRec& r = plan.cands[c];
        if (r.kind == MRL_CK_LEAF) {
          m[r.level] |= 1u << plan.slot_ceil(r.level, r.thr_code);
          continue;
        }
        for (int j = 0; j < r.nchild; j++) {
          const SpecHdr& ch = plan.hdrs[r.child[j]];
          for (int k = 0; k < NMEM; k++) {
            u32 cmask = __atomic_load_n(&ch.mask[k], __ATOMIC_RELAXED);
            if (r.kind != MRL_CK_MOVE || k != r.level) { m[k] |= cmask; continue; }
            u32 cm = cmask & real_slots[k];
            if (mem_counts_registers((Mem)k)) {
              // registers: every child breakpoint b becomes b + units
              u32 hi_code = plan.compressed(k) ? plan.cap_code[k] : top_code[k];
              u64 shifted = (r.units >= 32) ? 0 : ((u64)cm << r.units);
              u64 keep = (hi_code >= 63) ? ~0ull : ((2ull << hi_code) - 1ull);
              m[k] |= (u32)(shifted & keep);
              u64 top_keep = (top_code[k] >= 63) ? ~0ull : ((2ull << top_code[k]) - 1ull);
              if (plan.compressed(k) && (shifted & ~keep & top_keep)) m[k] |= 1u << (plan.cap_code[k] + 1);
              continue;
            }
            while (cm) {
              u32 b = (u32)__builtin_ctz(cm);
              cm &= cm - 1;
              u32 code = bit_length(next_binary_power(bit_length_inverse(b) + r.units));
              if (code <= top_code[k]) m[k] |= 1u << plan.slot_ceil(k, code);
            }
          }
        }
      }
      bool ch_any = false;
      for (int k = 0; k < NMEM; k++)
        if (m[k] != m0[k]) { __atomic_fetch_or(&h.mask[k], m[k], __ATOMIC_RELAXED); ch_any = true; }
      if (ch_any) changed = true;
    });
  }
  plan.stats.seconds_masks = now_s() - t2;

  // ---- 4. rows, owners, warps, schedule, byte accounting ----
  double t3 = now_s();
  u64 row = 0;
  for (u32 i = 0; i < n; i++) {
    SpecHdr& h = plan.hdrs[i];
    u64 ncells = 1;
    for (int k = 0; k < NMEM; k++) ncells *= (u64)__builtin_popcount(h.mask[k]);
    h.row_base = row;
    row += ncells;
  }
  // Owners: per group, heaviest family first onto the least loaded rank.
  for (Family& f : plan.families) {
    f.row_lo = plan.hdrs[f.spec_lo].row_base;
    f.row_hi = (f.spec_hi < n) ? plan.hdrs[f.spec_hi].row_base : row;
    f.owner = 0;
  }
  if (plan.world > 1) {
    size_t fi = 0;
    for (u32 gi = 0; gi < plan.groups.size(); gi++) {
      std::vector<u32> fam;
      while (fi < plan.families.size() && plan.families[fi].group == gi) fam.push_back((u32)fi++);
      std::stable_sort(fam.begin(), fam.end(), [&](u32 a, u32 b) {
        return plan.families[a].row_hi - plan.families[a].row_lo > plan.families[b].row_hi - plan.families[b].row_lo;
      });
      std::vector<u64> load(plan.world, 0);
      for (u32 f : fam) {
        u32 best = 0;
        for (u32 r = 1; r < plan.world; r++) if (load[r] < load[best]) best = r;
        plan.families[f].owner = best;
        load[best] += plan.families[f].row_hi - plan.families[f].row_lo;
      }
    }
  }
  std::vector<u8> mine(n, 1);
  if (plan.world > 1)
    for (const Family& f : plan.families)
      for (u32 i = f.spec_lo; i < f.spec_hi; i++) mine[i] = (f.owner == plan.rank);

  // Per Spec: warps, top diagonal and algorithmic bytes (one 12-byte row out; per candidate a
  // 16-byte header; per child of a candidate that fits the cell's limits a 4-byte index and a
  // 12-byte row in). Independent per Spec, so computed on all threads.
  // Per group, the memory with the most slots in total becomes the one the diagonal fixes:
  // a column then has a cell on as many of the group's diagonals as possible.
  std::vector<u8> free_of(n, 3);
  for (Group& g : plan.groups) {
    u64 tot[NMEM] = {0, 0, 0, 0};
    for (u32 i = g.spec_lo; i < g.spec_hi; i++)
      for (int k = 0; k < NMEM; k++) tot[k] += (u64)__builtin_popcount(plan.hdrs[i].mask[k]);
    int best = NMEM - 1;
    for (int k = NMEM - 2; k >= 0; k--) if (tot[k] > tot[best]) best = k;
    if (const char* e = getenv("MRL_FREE_DIM")) { int v = atoi(e); if (v >= 0 && v < NMEM) best = v; }
    g.free_dim = (u8)best;
    for (u32 i = g.spec_lo; i < g.spec_hi; i++) free_of[i] = (u8)best;
  }
  std::vector<u32> warps(n), top_sums(n);
  std::vector<u64> bytes_t(std::max(n_threads, 1), 0), cols_t(std::max(n_threads, 1), 0);
  parallel_for(n, n_threads, [&](size_t i, int tid) {
    const SpecHdr& h = plan.hdrs[i];
    u32 nk[NMEM];
    u32 top_sum = 0;
    for (int k = 0; k < NMEM; k++) {
      nk[k] = (u32)__builtin_popcount(h.mask[k]);
      top_sum += 31 - (u32)__builtin_clz(h.mask[k]);
    }
    u64 ncells = (u64)nk[0] * nk[1] * nk[2] * nk[3];
    u32 ncols = (u32)(ncells / nk[free_of[i]]);  // the slot in the group's free memory is fixed by the diagonal
    u64 bytes = ncells * 12;
    for (u32 c = h.cand_off; c < h.cand_off + h.ncand; c++) {
      const CandRec& r = plan.cands[c];
      bytes += ncells * 16;
      if (r.nchild) {
        u32 feasible_k = (u32)__builtin_popcount(h.mask[r.level] >> plan.slot_ceil(r.level, r.thr_code));
        bytes += ncells / nk[r.level] * feasible_k * r.nchild * 16;
      }
    }
    bytes_t[tid] += bytes;
    cols_t[tid] += ncols;
    const u32 cols_per_warp = 32u / (u32)plan.lanes_per_cell;
    warps[i] = mine[i] ? (ncols + cols_per_warp - 1) / cols_per_warp : 0;
    top_sums[i] = top_sum;
  });
  u64 bytes = 0, cols_total = 0;
  for (u64 b : bytes_t) bytes += b;
  for (u64 c : cols_t) cols_total += c;
  plan.warp_prefix.assign(n + 1, 0);
  u64 wsum = 0;
  for (u32 i = 0; i < n; i++) {
    plan.warp_prefix[i] = (u32)wsum;
    wsum += warps[i];
    if (wsum > 0xFFFFFFFFull) throw ModelError("too many warps in one plan");
  }
  plan.warp_prefix[n] = (u32)wsum;
  for (Group& g : plan.groups) {
    g.chunk_lo = plan.warp_prefix[g.spec_lo];
    g.chunk_hi = plan.warp_prefix[g.spec_hi];
    g.max_diag = 0;
    for (u32 i = g.spec_lo; i < g.spec_hi; i++)
      if (mine[i]) g.max_diag = std::max(g.max_diag, top_sums[i]);
  }
  u32 max_diag = 0;
  for (const Group& g : plan.groups) max_diag = std::max(max_diag, g.max_diag);
  // Group-major: a group only needs earlier groups (any limits) and, inside itself, cells on
  // lower diagonals. Moves keep kind, dtype and shape, so they never leave their group;
  // tile-outs and splits go to a smaller log-shape sum; ToAccum and Move prologues/epilogues
  // go to an earlier phase.
  for (u32 gi = 0; gi < plan.groups.size(); gi++)
    if (plan.groups[gi].chunk_hi > plan.groups[gi].chunk_lo)
      for (u32 d = 0; d <= plan.groups[gi].max_diag; d++) plan.steps.push_back(Step{gi, d});

  plan.stats.n_rows = row;
  plan.stats.n_columns = cols_total;
  plan.stats.n_groups = plan.groups.size();
  plan.stats.n_steps = plan.steps.size();
  plan.stats.max_diag = max_diag;
  plan.stats.algorithmic_bytes = bytes;
  plan.stats.seconds_layout += now_s() - t3;
  if (getenv("MRL_PLAN_TIMING")) fprintf(stderr, "[plan] masks %.2fs (%llu sweeps), rows/owners/warps %.2fs\n", plan.stats.seconds_masks, (unsigned long long)plan.stats.mask_sweeps, now_s() - t3);
}

}  // namespace mrl

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

// Third component of the stage order. Moves to a faster memory lower the sum of the operands'
// memory indices, and the prologue / epilogue Moves of a Matmul or Fill lie in an earlier phase.
// Inside the Move phase they do not: Move(GL -> L1) relayouts its source through
// Move(GL -> GL), whose own destination moves lead back to Move(GL -> L1). There only the
// slowest memory a Spec touches never grows along an action, so it orders the stages.
u32 level_rank(const LogicalSpec& ls) {
  u32 s = 0, mx = 0;
  for (int i = 0; i < ls.nops(); i++) {
    s += (u32)ls.aux[i].mem;
    mx = std::max(mx, (u32)ls.aux[i].mem);
  }
  return ls.kind == K_MOVE ? mx : s;
}

u32 stage_key(const LogicalSpec& ls) { return ((u32)ls.kind << 16) | (shape_log_sum(ls) << 8) | level_rank(ls); }

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

bool Plan::pack_limits(const u64 limits[NMEM], u32* out) const {
  u32 pack = 0;
  for (int k = 0; k < NMEM; k++) {
    if (!mem_counts_registers((Mem)k) && limits[k] != 0 && !is_pow2(limits[k])) return false;
    u32 code = limit_code(k, limits[k]);
    if (code > top_code[k]) return false;  // beyond the limits this table was filled for
    pack |= code << (8 * k);
  }
  *out = pack;
  return true;
}

Plan build_plan(const std::vector<LogicalSpec>& goals, int n_threads, const u64* top_limits, u32 rank, u32 world) {
  if (n_threads < 1) n_threads = 1;
  if (world < 1 || rank >= world) throw ModelError("bad shard rank / world size");
  Plan plan;
  plan.rank = rank;
  plan.world = world;
  plan.n_threads = n_threads;
  u32 top_code[NMEM];
  for (int k = 0; k < NMEM; k++) {
    u64 v = top_limits ? top_limits[k] : AVX2_MAX_MEM[k];
    if (!mem_counts_registers((Mem)k) && v != 0 && !is_pow2(v)) throw ModelError("cache limits must be powers of two");
    top_code[k] = limit_code(k, v);
    if (top_code[k] > 30) throw ModelError("memory limit too large for the lattice masks");
    plan.top_code[k] = top_code[k];
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

  // ---- 2. final ids: stage-major (phase, log-shape sum, memory-level sum), then key order ----
  double t1 = now_s();
  std::vector<u32> order(n);
  for (u32 i = 0; i < n; i++) order[i] = i;
  std::vector<u32> gkey(n);
  for (u32 i = 0; i < n; i++) gkey[i] = stage_key(temp[i].ls);
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

  // stages, and inside them families: maximal runs with equal dtype and shape (ids are
  // key-sorted, and the key starts with kind, dtype, serial flag, rank, shape)
  for (u32 i = 0; i < n;) {
    const u32 sk = stage_key(plan.specs[i]);
    u32 j = i;
    while (j < n && stage_key(plan.specs[j]) == sk) j++;
    Stage st;
    st.spec_lo = i;
    st.spec_hi = j;
    st.phase = (u8)(sk >> 16);
    st.shape_sum = (u8)((sk >> 8) & 0xff);
    st.level_rank = (u8)(sk & 0xff);
    st.fam_lo = (u32)plan.families.size();
    for (u32 a = i; a < j;) {
      u32 b = a;
      u64 w = 0;
      while (b < j && plan.specs[b].dtype == plan.specs[a].dtype && plan.specs[b].spec_shape == plan.specs[a].spec_shape) {
        w += plan.hdrs[b].ncand + 1;
        b++;
      }
      Family f;
      f.spec_lo = a;
      f.spec_hi = b;
      f.stage = (u32)plan.stages.size();
      f.weight = w;
      plan.families.push_back(f);
      a = b;
    }
    st.fam_hi = (u32)plan.families.size();
    plan.stages.push_back(st);
    i = j;
  }

  // The order the device relies on: a child never lies in a later stage; a child inside its
  // parent's stage belongs to a Move that consumes memory (so it sits at strictly lower limits)
  // and to the parent's family.
  {
    std::vector<u32> stage_of(n), fam_of(n);
    for (u32 si = 0; si < plan.stages.size(); si++)
      for (u32 i = plan.stages[si].spec_lo; i < plan.stages[si].spec_hi; i++) stage_of[i] = si;
    for (u32 fi = 0; fi < plan.families.size(); fi++)
      for (u32 i = plan.families[fi].spec_lo; i < plan.families[fi].spec_hi; i++) fam_of[i] = fi;
    std::atomic<int> bad{0};
    std::atomic<u64> bad_pair{0};
    parallel_for(n, n_threads, [&](size_t i, int) {
      const SpecHdr& h = plan.hdrs[i];
      for (u32 c = h.cand_off; c < h.cand_off + h.ncand; c++) {
        const CandRec& r = plan.cands[c];
        for (int j = 0; j < r.nchild; j++) {
          const u32 ch = r.child[j];
          if (stage_of[ch] > stage_of[i]) { bad = 1; bad_pair = ((u64)i << 32) | ch; }
          if (stage_of[ch] == stage_of[i] && (r.kind != MRL_CK_MOVE || r.units == 0 || fam_of[ch] != fam_of[i])) {
            bad = 2;
            bad_pair = ((u64)i << 32) | ch;
          }
        }
      }
    });
    const std::string who = bad.load() ? (": parent " + plan.specs[bad_pair.load() >> 32].str() + ", child " +
                                          plan.specs[bad_pair.load() & 0xFFFFFFFFu].str()) : std::string();
    if (bad.load() == 1) throw ModelError("planner: a child Spec lies in a later stage than its parent" + who);
    if (bad.load() == 2) throw ModelError("planner: a same-stage child is not below its parent in the limits lattice" + who);
  }

  // Owners: per stage, heaviest family first onto the least loaded rank.
  if (plan.world > 1) {
    plan.mine.assign(n, 0);
    for (const Stage& st : plan.stages) {
      std::vector<u32> fam;
      for (u32 f = st.fam_lo; f < st.fam_hi; f++) fam.push_back(f);
      std::stable_sort(fam.begin(), fam.end(), [&](u32 a, u32 b) { return plan.families[a].weight > plan.families[b].weight; });
      std::vector<u64> load(plan.world, 0);
      for (u32 f : fam) {
        u32 best = 0;
        for (u32 r = 1; r < plan.world; r++) if (load[r] < load[best]) best = r;
        plan.families[f].owner = best;
        load[best] += plan.families[f].weight;
      }
    }
    for (const Family& f : plan.families)
      if (f.owner == plan.rank)
        for (u32 i = f.spec_lo; i < f.spec_hi; i++) plan.mine[i] = 1;
  }
  plan.stats.seconds_layout = now_s() - t1;
  if (getenv("MRL_PLAN_TIMING")) fprintf(stderr, "[plan] discover %.2fs, ids/stages/families %.2fs\n", plan.stats.seconds_discover, plan.stats.seconds_layout);

  plan.stats.n_specs = n;
  plan.stats.n_cands = ncand;
  plan.stats.n_stages = plan.stages.size();
  plan.stats.n_families = plan.families.size();
  return plan;
}

}  // namespace mrl

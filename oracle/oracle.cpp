// TEST INFRASTRUCTURE — NOT PART OF THE PRODUCT PATH. See oracle.hpp.
#include "oracle.hpp"
#include "../morello_b200/csrc/model/impl_text.hpp"
#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <set>
#include <thread>

namespace orc {

// action_dominates (db/pagecontents.rs:191-210): lhs wins ties.
static bool dominates(const Decision& a, const Decision& b, std::atomic<u64>& conflicts) {
  if (a.found != b.found) { conflicts++; return a.found; }
  if (!a.found) return true;
  if (a.cost.main != b.cost.main) { conflicts++; return a.cost.main < b.cost.main; }
  int p = lex_cmp(a.cost.peaks, b.cost.peaks);
  if (p) return p < 0;
  if (a.cost.depth != b.cost.depth) return a.cost.depth < b.cost.depth;
  return a.action <= b.action;
}

bool Database::get(const std::string& key, const Codes& pt, Decision& out) {
  gets++;
  Shard& sh = shard_for(key);
  std::lock_guard<std::mutex> g(sh.mu);
  auto it = sh.map.find(key);
  if (it == sh.map.end()) return false;
  const Entry& e = it->second;
  const u32 G = 0x80808080u;
  const u32 p = pack(pt);
  const size_t n = e.lo.size();
  bool any = false;
  for (size_t i = 0; i < n; i++) {
    // every byte of (p - lo) and (hi - p) is non-negative <=> guard bits survive
    u32 ok = ((p | G) - e.lo[i]) & ((e.hi[i] | G) - p) & G;
    if (ok != G) continue;
    if (!any) { out = e.val[i]; any = true; }
    else if (!dominates(out, e.val[i], dominance_conflicts)) out = e.val[i];
  }
  if (any) hits++;
  return any;
}

// put_canon + put_range_to_fill (db/mod.rs:650-766,1782-1819): fill [peaks .. limits];
// an empty decision fills [0 .. limits].
void Database::put(const std::string& key, const Limits& limits, const Decision& d) {
  puts++;
  PutRect r;
  r.hi = limits_to_codes(limits);
  Limits lo = {0, 0, 0, 0};
  if (d.found) lo = d.cost.peaks;
  r.lo = limits_to_codes(lo);
  for (int i = 0; i < NMEM; i++)
    if (r.lo[i] > r.hi[i]) throw ModelError("peak memory exceeds the Spec's limits in put");
  r.value = d;
  Shard& sh = shard_for(key);
  std::lock_guard<std::mutex> g(sh.mu);
  Entry& e = sh.map[key];
  e.lo.push_back(pack(r.lo));
  e.hi.push_back(pack(r.hi));
  e.val.push_back(d);
}

const std::vector<Candidate>& Search::candidates_for(const LogicalSpec& ls, const std::string& key,
                                                     std::vector<Candidate>& scratch) {
  if (!cache_) {
    tabulate_candidates(ls, scratch);
    return scratch;
  }
  auto it = cand_cache_.find(key);
  if (it != cand_cache_.end()) return it->second;
  if (cand_cache_.size() > 200000) cand_cache_.clear();  // bound memory
  std::vector<Candidate>& v = cand_cache_[key];
  tabulate_candidates(ls, v);
  return v;
}

namespace {
struct Partial {
  const Candidate* cand;
  Limits child_limits;
  std::vector<std::optional<Cost>> costs;
  int state = 0;  // 0 constructing, 1 unsat, 2 sat
};
}  // namespace

// algo::solve_node (search/algo.rs:61-95) over SpecTask (search/spectask.rs:55-253).
Decision Search::solve(const LogicalSpec& ls, const Limits& limits) {
  const std::string key = ls.key();
  const Codes pt = limits_to_codes(limits);
  Decision memo;
  if (db_.get(key, pt, memo)) return memo;
  if (out_of_time && (stats.solves & 15) == 0 && out_of_time()) throw OutOfTime();

  stats.solves++;
  std::vector<Candidate> scratch;
  // Copy when cached: recursive solves may rehash or clear the cache.
  std::vector<Candidate> cands = candidates_for(ls, key, scratch);

  Reducer reducer;
  std::vector<Partial> partials;
  size_t max_children = 0;
  for (const Candidate& c : cands) {
    Limits child_limits = limits;
    if (c.kind == CK_MOVE) {  // OutOfMemory check of plan_alloc_shared (moves.rs:354-374)
      Limits consumed = {0, 0, 0, 0};
      consumed[c.level] = c.units;
      if (!checked_sub_snap_down(limits, consumed, child_limits)) continue;
    } else if (c.kind == CK_LEAF) {  // select.rs:34-47
      if (c.units > limits[c.level]) continue;
    }
    stats.candidates_seen++;
    max_children = std::max<size_t>(max_children, c.nchild);
    if (c.nchild == 0) {
      reducer.insert(c.action, combine(c, ls, {}));
    } else {
      Partial p;
      p.cand = &c;
      p.child_limits = child_limits;
      p.costs.resize(c.nchild);
      partials.push_back(std::move(p));
    }
  }
  // SORT_ACTIONS_BY_DEPENDENCY_COUNT (spectask.rs:94-99): stable by child count.
  std::stable_sort(partials.begin(), partials.end(),
                   [](const Partial& a, const Partial& b) { return a.cand->nchild < b.cand->nchild; });

  size_t incomplete = partials.size();
  bool running = incomplete != 0;
  for (size_t batch = 0; running && batch < max_children; batch++) {
    std::vector<size_t> members;  // the batch is materialised before any child is solved
    for (size_t i = 0; i < partials.size(); i++)
      if (partials[i].state == 0 && batch < partials[i].cand->nchild) members.push_back(i);
    for (size_t i : members) {
      Partial& p = partials[i];
      Decision child = solve(p.cand->child[batch], p.child_limits);
      // resolve_request (spectask.rs:167-253)
      if (p.state == 0) {
        bool finished = false;
        if (child.found) {
          p.costs[batch] = child.cost;
          bool all = true;
          for (auto& c : p.costs) if (!c.has_value()) all = false;
          if (all) {
            std::vector<Cost> kids;
            for (auto& c : p.costs) kids.push_back(*c);
            reducer.insert(p.cand->action, combine(*p.cand, ls, kids));
            p.state = 2;
            finished = true;
          }
        } else {
          p.state = 1;
          finished = true;
        }
        if (finished && --incomplete == 0) running = false;
      }
      if (!running) break;  // STOP_BATCH_WHEN_TASK_COMPLETES (algo.rs:10,73-84)
    }
  }
  Decision result = reducer.finalize();
  db_.put(key, limits, result);
  return result;
}

// The driver's schedule (precompute/src/main.rs:221-241,304-385): phases one after another; inside
// a phase every bound Spec runs its own sequence of stages (`phase.into_par_iter()`, :229), and the
// tasks of a stage run in parallel (`stage.into_par_iter()`, :339). One pool of workers serves
// all of it: a bound whose stage is finished queues the tasks of its next stage.
namespace {
struct BoundRun {
  Bound bound;
  std::vector<std::vector<std::vector<u32>>> stages;   // task points by stage
  size_t stage = 0;       // stage whose tasks are queued or running
  size_t open_tasks = 0;  // of that stage, not finished yet
};
struct TaskRef { size_t bound, stage, task; };
}  // namespace

PrecomputeReport precompute(Database& db, u32 size, Through through, const std::vector<Dtype>& dtypes, int threads,
                            double time_budget_s, bool* finished, bool cache_candidates, const double* phase_budget_s,
                            PhaseReport* phase_reports) {
  auto t0 = std::chrono::steady_clock::now();
  auto elapsed = [&]() { return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count(); };
  PrecomputeReport rep;
  Limits top;
  for (int i = 0; i < NMEM; i++) top[i] = AVX2_MAX_MEM[i];
  if (threads < 1) threads = 1;
  std::atomic<u64> solves{0}, lspecs{0};
  std::atomic<u64> busy_ns{0};
  bool all_finished = true;

  auto phases = goal_phases(size, through, dtypes);
  for (size_t pi = 0; pi < phases.size(); pi++) {
    const double phase_start = elapsed();
    const double phase_budget = phase_budget_s ? phase_budget_s[pi] : 0.0;
    auto out_of_time_now = [&]() {
      if (time_budget_s > 0 && elapsed() > time_budget_s) return true;
      return phase_budget > 0 && elapsed() - phase_start > phase_budget;
    };
    std::vector<BoundRun> runs;
    for (const Bound& b : phases[pi]) {
      BoundRun r;
      r.bound = b;
      r.stages = diagonals(bound_point(b));
      runs.push_back(std::move(r));
    }
    std::mutex mu;
    std::condition_variable cv;
    std::deque<TaskRef> queue;
    size_t bounds_open = 0;
    std::atomic<bool> stop{false};
    std::atomic<u64> phase_lspecs{0};
    const u64 puts_before = db.puts.load();
    auto queue_stage = [&](size_t bi) {   // under mu; skips empty stages
      BoundRun& r = runs[bi];
      while (r.stage < r.stages.size() && r.stages[r.stage].empty()) r.stage++;
      if (r.stage >= r.stages.size()) return false;
      r.open_tasks = r.stages[r.stage].size();
      for (size_t t = 0; t < r.open_tasks; t++) queue.push_back(TaskRef{bi, r.stage, t});
      return true;
    };
    {
      std::lock_guard<std::mutex> g(mu);
      for (size_t bi = 0; bi < runs.size(); bi++)
        if (queue_stage(bi)) bounds_open++;
    }
    auto worker = [&]() {
      Search search(db, cache_candidates);
      if (time_budget_s > 0 || phase_budget > 0) search.out_of_time = [&]() { return stop.load() || out_of_time_now(); };
      for (;;) {
        TaskRef ref;
        {
          std::unique_lock<std::mutex> lk(mu);
          cv.wait(lk, [&]() { return !queue.empty() || bounds_open == 0 || stop.load(); });
          if (stop.load() || (queue.empty() && bounds_open == 0)) break;
          ref = queue.front();
          queue.pop_front();
        }
        auto w0 = std::chrono::steady_clock::now();
        const BoundRun& r = runs[ref.bound];
        std::vector<LogicalSpec> task = task_point_specs(r.bound, r.stages[ref.stage][ref.task]);
        bool complete = true;
        // every Spec of the task at the top limits, then the limits worklist (main.rs:340-361)
        std::vector<std::pair<LogicalSpec, Limits>> worklist;
        for (auto& l : task) worklist.push_back({l, top});
        while (!worklist.empty() && complete) {
          std::set<std::pair<std::string, Limits>> next;  // dedup like the HashSet at :346,361
          for (auto& w : worklist) {
            if (stop.load() || out_of_time_now()) { complete = false; break; }
            Decision d;
            try {
              d = search.solve(w.first, w.second);
            } catch (const Search::OutOfTime&) {
              complete = false;
              break;
            }
            if (d.found)
              for (const Limits& l : next_limits(w.second, d.cost.peaks)) next.insert({w.first.key(), l});
          }
          worklist.clear();
          for (auto& n : next) worklist.push_back({LogicalSpec::from_key(n.first), n.second});
        }
        busy_ns += (u64)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - w0).count();
        if (complete) phase_lspecs += task.size();
        {
          std::lock_guard<std::mutex> g(mu);
          if (!complete) stop = true;
          BoundRun& rr = runs[ref.bound];
          if (--rr.open_tasks == 0 && !stop.load()) {
            rr.stage++;
            if (!queue_stage(ref.bound)) bounds_open--;
          }
        }
        cv.notify_all();
      }
      solves += search.stats.solves;
    };
    if (threads == 1) worker();
    else {
      std::vector<std::thread> pool;
      for (int i = 0; i < threads; i++) pool.emplace_back(worker);
      for (auto& th : pool) th.join();
    }
    lspecs += phase_lspecs.load();
    if (phase_reports) {
      phase_reports[pi].seconds = elapsed() - phase_start;
      phase_reports[pi].logical_specs = phase_lspecs.load();
      phase_reports[pi].puts = db.puts.load() - puts_before;
      phase_reports[pi].finished = !stop.load();
    }
    if (stop.load()) {
      all_finished = false;
      if (!phase_budget_s) break;                                     // one budget for the whole run: it is spent
      if (time_budget_s > 0 && elapsed() > time_budget_s) break;
    }
  }
  if (finished) *finished = all_finished;
  rep.seconds = elapsed();
  rep.puts = db.puts.load();
  rep.logical_specs = lspecs.load();
  rep.solves = solves.load();
  rep.busy_seconds = busy_ns.load() * 1e-9;
  return rep;
}

}  // namespace orc

// ---- C interface for the tests (ctypes) ----
using namespace orc;

struct OrcHandle {
  Database db;
};

struct OrcDecision {
  int32_t found;     // 1 found, 0 unsat, -1 miss (get only)
  uint32_t action;
  uint32_t main;
  uint32_t depth;
  uint64_t peaks[4];
};

static void fill_decision(OrcDecision* o, const Decision& d) {
  o->found = d.found ? 1 : 0;
  o->action = d.action;
  o->main = d.cost.main;
  o->depth = d.cost.depth;
  for (int i = 0; i < 4; i++) o->peaks[i] = d.cost.peaks[i];
}

extern "C" {

void* orc_create() { return new OrcHandle(); }
void orc_destroy(void* h) { delete (OrcHandle*)h; }

// Faithful precompute. dtype_mask bit0 = u32, bit1 = f32. Returns 0, or -1 on a model error.
int orc_precompute(void* h, uint32_t size, int through, int dtype_mask, int threads, double time_budget_s,
                   int cache_candidates, double* seconds, uint64_t* puts, uint64_t* logical_specs, uint64_t* solves, int* finished,
                   double* busy_seconds) {
  try {
    std::vector<Dtype> dts;
    if (dtype_mask & 1) dts.push_back(DT_U32);
    if (dtype_mask & 2) dts.push_back(DT_F32);
    bool fin = false;
    PrecomputeReport r = precompute(((OrcHandle*)h)->db, size, (Through)through, dts, threads, time_budget_s, &fin, cache_candidates != 0);
    if (seconds) *seconds = r.seconds;
    if (puts) *puts = r.puts;
    if (logical_specs) *logical_specs = r.logical_specs;
    if (solves) *solves = r.solves;
    if (finished) *finished = fin ? 1 : 0;
    if (busy_seconds) *busy_seconds = r.busy_seconds;
    return 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "oracle error: %s\n", e.what());
    return -1;
  }
}

// The same under one time budget per phase (Move, Zero, Matmul): each phase runs its own stage
// order until its budget is spent, then the next phase starts on what is in the database so far.
// phase_out: per phase seconds, goal Specs completed, puts, finished flag.
int orc_precompute_phases(void* h, uint32_t size, int through, int dtype_mask, int threads, const double* phase_budget_s,
                          double* seconds, double* busy_seconds, uint64_t* puts, uint64_t* logical_specs, double* phase_seconds,
                          uint64_t* phase_specs, uint64_t* phase_puts, int* phase_finished) {
  try {
    std::vector<Dtype> dts;
    if (dtype_mask & 1) dts.push_back(DT_U32);
    if (dtype_mask & 2) dts.push_back(DT_F32);
    PhaseReport pr[3];
    bool fin = false;
    PrecomputeReport r = precompute(((OrcHandle*)h)->db, size, (Through)through, dts, threads, 0.0, &fin, false, phase_budget_s, pr);
    if (seconds) *seconds = r.seconds;
    if (busy_seconds) *busy_seconds = r.busy_seconds;
    if (puts) *puts = r.puts;
    if (logical_specs) *logical_specs = r.logical_specs;
    for (int k = 0; k <= through && k < 3; k++) {
      if (phase_seconds) phase_seconds[k] = pr[k].seconds;
      if (phase_specs) phase_specs[k] = pr[k].logical_specs;
      if (phase_puts) phase_puts[k] = pr[k].puts;
      if (phase_finished) phase_finished[k] = pr[k].finished ? 1 : 0;
    }
    return 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "oracle error: %s\n", e.what());
    return -1;
  }
}

// search::top_down on one goal (morello/src/search/mod.rs:44).
int orc_top_down(void* h, const uint8_t* key, uint32_t key_len, const uint64_t* limits, OrcDecision* out) {
  try {
    LogicalSpec ls = LogicalSpec::from_key(std::string((const char*)key, key_len));
    if (logicalspec_canonicalize(ls) != CANON_OK) return -2;
    Limits l = {limits[0], limits[1], limits[2], limits[3]};
    Search s(((OrcHandle*)h)->db);
    fill_decision(out, s.solve(ls, l));
    return 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "oracle error: %s\n", e.what());
    return -1;
  }
}

// Reconstruction of the optimal implementation from stored actions
// (morello/src/reconstruct.rs:14-80): solve (or look up) the Spec, re-apply the stored action,
// recurse into the sub-Specs at the limits the action leaves them. Appends one line per node.
static void reconstruct(Search& s, const LogicalSpec& ls, const Limits& limits, int level, std::string& out) {
  const Decision d = s.solve(ls, limits);
  if (!d.found) throw ModelError("no implementation for " + ls.str());
  std::vector<Candidate> cs;
  tabulate_candidates(ls, cs);
  const Candidate* chosen = nullptr;
  for (const Candidate& c : cs) if (c.action == d.action) chosen = &c;
  if (!chosen) throw ModelError("stored action is not among the Spec's actions: " + ls.str());
  out += impl_line(level, ls, limits.data(), d.action, action_text(*chosen), d.cost.main, d.cost.peaks.data(), d.cost.depth);
  Limits child_limits = limits;
  if (chosen->kind == CK_MOVE) {
    Limits consumed = {0, 0, 0, 0};
    consumed[chosen->level] = chosen->units;
    if (!checked_sub_snap_down(limits, consumed, child_limits)) throw ModelError("stored Move does not fit its limits");
  }
  for (int j = 0; j < chosen->nchild; j++) reconstruct(s, chosen->child[j], child_limits, level + 1, out);
}

// FilesDatabase::get_impl (morello/src/db/mod.rs:505-516) as text. Returns the length, or < 0.
long orc_get_impl(void* h, const uint8_t* key, uint32_t key_len, const uint64_t* limits, char* out, uint64_t cap) {
  try {
    LogicalSpec ls = LogicalSpec::from_key(std::string((const char*)key, key_len));
    if (logicalspec_canonicalize(ls) != CANON_OK) return -2;
    Limits l = {limits[0], limits[1], limits[2], limits[3]};
    Search s(((OrcHandle*)h)->db);
    std::string text;
    reconstruct(s, ls, l, 0, text);
    if (text.size() + 1 > cap) return -3;
    memcpy(out, text.c_str(), text.size() + 1);
    return (long)text.size();
  } catch (const std::exception& e) {
    fprintf(stderr, "oracle error: %s\n", e.what());
    return -1;
  }
}

int orc_get(void* h, const uint8_t* key, uint32_t key_len, const uint64_t* limits, OrcDecision* out) {
  try {
    Limits l = {limits[0], limits[1], limits[2], limits[3]};
    Decision d;
    if (!((OrcHandle*)h)->db.get(std::string((const char*)key, key_len), limits_to_codes(l), d)) {
      out->found = -1;
      return 0;
    }
    fill_decision(out, d);
    return 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "oracle error: %s\n", e.what());
    return -1;
  }
}

uint64_t orc_num_puts(void* h) { return ((OrcHandle*)h)->db.puts.load(); }
uint64_t orc_num_dominance_conflicts(void* h) { return ((OrcHandle*)h)->db.dominance_conflicts.load(); }

// Dump every put: sizes first (pass nulls), then buffers. Keys are concatenated;
// key_off has n+1 entries. rect is n*8 bytes (lo[4], hi[4] lattice codes); dec is n entries.
int orc_dump(void* h, uint64_t* n_out, uint64_t* key_bytes_out, uint8_t* keys, uint64_t* key_off, uint8_t* rect,
             OrcDecision* dec) {
  Database& db = ((OrcHandle*)h)->db;
  uint64_t n = 0, kb = 0;
  for (auto& sh : db.shards)
    for (auto& kv : sh.map) { n += kv.second.val.size(); kb += kv.first.size() * kv.second.val.size(); }
  if (n_out) *n_out = n;
  if (key_bytes_out) *key_bytes_out = kb;
  if (!keys) return 0;
  // deterministic order: sort keys
  std::vector<const std::pair<const std::string, Database::Entry>*> items;
  for (auto& sh : db.shards) for (auto& kv : sh.map) items.push_back(&kv);
  std::sort(items.begin(), items.end(), [](auto* a, auto* b) { return a->first < b->first; });
  uint64_t i = 0, off = 0;
  for (auto* kv : items) {
    const Database::Entry& e = kv->second;
    for (size_t j = 0; j < e.val.size(); j++) {
      key_off[i] = off;
      memcpy(keys + off, kv->first.data(), kv->first.size());
      off += kv->first.size();
      for (int k = 0; k < 4; k++) {
        rect[i * 8 + k] = (uint8_t)(e.lo[j] >> (8 * k));
        rect[i * 8 + 4 + k] = (uint8_t)(e.hi[j] >> (8 * k));
      }
      fill_decision(&dec[i], e.val[j]);
      i++;
    }
  }
  key_off[i] = off;
  return 0;
}

}  // extern "C"

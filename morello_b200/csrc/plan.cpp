// Host-side planner of the database fill. See plan.hpp.
#include "plan.hpp"
#include <malloc.h>
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <atomic>
#include <chrono>
#include <mutex>
#include <thread>
#include <memory>
#include <unordered_map>

namespace mrl {

namespace {

constexpr int NSHARD = 1024;

// 64-bit hash of a Spec key (8 bytes at a time, multiply-xorshift mixing).
u64 hash_key(const char* p, int len) {
  u64 h = 0x9E3779B97F4A7C15ull ^ (u64)len;
  int i = 0;
  for (; i + 8 <= len; i += 8) {
    u64 w;
    memcpy(&w, p + i, 8);
    h = (h ^ w) * 0xD6E8FEB86659FD93ull;
    h ^= h >> 32;
  }
  u64 w = 0;
  if (i < len) memcpy(&w, p + i, (size_t)(len - i));
  h = (h ^ w) * 0xD6E8FEB86659FD93ull;
  h ^= h >> 32;
  h *= 0xD6E8FEB86659FD93ull;
  h ^= h >> 29;
  return h;
}

// One shard of the key -> id map used during discovery: open addressing over (hash, id) with
// the key bytes kept in a shard-local arena for the equality check.
struct KeyShard {
  struct Entry { u64 h; u32 id; u32 off; u32 len; u32 used; };
  std::mutex mu;
  std::vector<Entry> tab;
  std::string arena;
  size_t count = 0;
  // where the table is, for prefetches from outside the lock (may be stale: a prefetch of
  // memory that has moved on does no harm)
  std::atomic<const Entry*> peek_ptr{nullptr};
  std::atomic<size_t> peek_mask{0};
  KeyShard() : tab(256) {
    for (auto& e : tab) e.used = 0;
    peek_ptr = tab.data();
    peek_mask = tab.size() - 1;
  }
  void prefetch(u64 h) const {
    const Entry* p = peek_ptr.load(std::memory_order_relaxed);
    __builtin_prefetch(p + ((size_t)(h >> 10) & peek_mask.load(std::memory_order_relaxed)));
  }
  // Returns the id stored for the key, or inserts `fresh_id()` and returns it with *inserted.
  template <class F>
  u32 find_or_insert(u64 h, const char* key, int len, F fresh_id, bool* inserted) {
    std::lock_guard<std::mutex> g(mu);
    size_t mask = tab.size() - 1;
    size_t i = (size_t)(h >> 10) & mask;
    while (tab[i].used) {
      const Entry& e = tab[i];
      if (e.h == h && e.len == (u32)len && memcmp(arena.data() + e.off, key, (size_t)len) == 0) {
        *inserted = false;
        return e.id;
      }
      i = (i + 1) & mask;
    }
    if ((count + 1) * 2 > tab.size()) {
      std::vector<Entry> bigger(tab.size() * 2);
      for (auto& e : bigger) e.used = 0;
      const size_t m2 = bigger.size() - 1;
      for (const Entry& e : tab) {
        if (!e.used) continue;
        size_t j = (size_t)(e.h >> 10) & m2;
        while (bigger[j].used) j = (j + 1) & m2;
        bigger[j] = e;
      }
      tab.swap(bigger);
      peek_mask.store(0, std::memory_order_relaxed);
      peek_ptr.store(tab.data(), std::memory_order_relaxed);
      peek_mask.store(tab.size() - 1, std::memory_order_relaxed);
      mask = tab.size() - 1;
      i = (size_t)(h >> 10) & mask;
      while (tab[i].used) i = (i + 1) & mask;
    }
    Entry e;
    e.h = h;
    e.id = fresh_id();
    e.off = (u32)arena.size();
    e.len = (u32)len;
    e.used = 1;
    arena.append(key, (size_t)len);
    tab[i] = e;
    count++;
    *inserted = true;
    return e.id;
  }
};

struct TempSpec {
  LogicalSpec ls;
  std::string key;
  std::vector<CandRec> cands;  // child[] holds temporary ids
  u16 leaf_first = 0, leaf_end = 0;  // action numbers of the leaf-kernel section [first, end)
  u16 n_leaf = 0;                    // leaf records among cands
  u16 twin_leaf_end = 0;             // the dtype twin's leaf_end and leaf records (set when ids are laid out)
  std::vector<CandRec> twin_leaf;
};

// Growing array of TempSpec in fixed blocks: elements never move, blocks are allocated on demand
// from any thread, and an element is constructed by the thread that discovers the Spec.
class TempSpecs {
 public:
  static constexpr u32 BLOCK_BITS = 15, BLOCK = 1u << BLOCK_BITS, MAX_BLOCKS = 1u << 17;
  TempSpecs() : blocks_(MAX_BLOCKS) { for (auto& b : blocks_) b.store(nullptr, std::memory_order_relaxed); }
  ~TempSpecs() { for (auto& b : blocks_) free(b.load(std::memory_order_relaxed)); }
  TempSpec& operator[](u32 id) { return blocks_[id >> BLOCK_BITS].load(std::memory_order_acquire)[id & (BLOCK - 1)]; }
  TempSpec& construct(u32 id) {
    std::atomic<TempSpec*>& slot = blocks_[id >> BLOCK_BITS];
    TempSpec* b = slot.load(std::memory_order_acquire);
    if (!b) {
      TempSpec* fresh = static_cast<TempSpec*>(malloc(sizeof(TempSpec) * BLOCK));
      if (!fresh) throw std::bad_alloc();
      if (slot.compare_exchange_strong(b, fresh, std::memory_order_acq_rel)) b = fresh;
      else free(fresh);
    }
    return *new (&b[id & (BLOCK - 1)]) TempSpec();
  }
  void destroy(u32 id) { (*this)[id].~TempSpec(); }

 private:
  std::vector<std::atomic<TempSpec*>> blocks_;
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
  for (auto& v : per_task) {
    goals.insert(goals.end(), v.begin(), v.end());
    std::vector<LogicalSpec>().swap(v);
  }
  return goals;
}

long Plan::find(const LogicalSpec& ls) const {
  if (find_tab_.empty()) return -1;
  char buf[LogicalSpec::MAX_KEY];
  const int len = ls.key_into(buf);
  const u64 h = hash_key(buf, len);
  const size_t mask = find_tab_.size() - 1;
  for (size_t i = (size_t)h & mask;; i = (i + 1) & mask) {
    const u32 id = find_tab_[i];
    if (id == 0xFFFFFFFFu) return -1;
    if (specs[id] == ls) return id;
  }
}

void Plan::share_blobs(void* ptrs[N_BLOBS], u64 sizes[N_BLOBS]) {
  for (int k = 0; k < NMEM; k++) meta_.top_code[k] = top_code[k];
  meta_.world = world;
  meta_.pad = 0;
  meta_.stats = stats;
  ptrs[0] = &meta_;              sizes[0] = sizeof(Meta);
  ptrs[1] = specs.data();        sizes[1] = specs.size() * sizeof(LogicalSpec);
  ptrs[2] = hdrs.data();         sizes[2] = hdrs.size() * sizeof(SpecHdr);
  ptrs[3] = cands.data();        sizes[3] = cands.size() * sizeof(CandRec);
  ptrs[4] = stages.data();       sizes[4] = stages.size() * sizeof(Stage);
  ptrs[5] = families.data();     sizes[5] = families.size() * sizeof(Family);
  ptrs[6] = goal_ids.data();     sizes[6] = goal_ids.size() * sizeof(u32);
  ptrs[7] = find_tab_.data();    sizes[7] = find_tab_.size() * sizeof(u32);
}

void Plan::adopt_alloc(const u64 sizes[N_BLOBS]) {
  if (sizes[0] != sizeof(Meta) || sizes[1] % sizeof(LogicalSpec) || sizes[2] % sizeof(SpecHdr) ||
      sizes[3] % sizeof(CandRec) || sizes[4] % sizeof(Stage) || sizes[5] % sizeof(Family) || sizes[6] % sizeof(u32) ||
      sizes[7] % sizeof(u32) || sizes[1] / sizeof(LogicalSpec) != sizes[2] / sizeof(SpecHdr))
    throw ModelError("shared plan: sizes do not describe a plan of this library version");
  specs.reset(sizes[1] / sizeof(LogicalSpec));
  hdrs.reset(sizes[2] / sizeof(SpecHdr));
  cands.reset(sizes[3] / sizeof(CandRec));
  stages.assign(sizes[4] / sizeof(Stage), Stage());
  families.assign(sizes[5] / sizeof(Family), Family());
  goal_ids.assign(sizes[6] / sizeof(u32), 0);
  find_tab_.assign(sizes[7] / sizeof(u32), 0xFFFFFFFFu);
  mine.clear();
}

// Unit of work handed to one rank: the Specs of a family whose operands sit in the same
// memories. Relayout Moves (the only same-stage dependency outside the Move phase) keep every
// operand's memory, so such units do not depend on each other; in the Move phase same-stage
// Moves do change memories and the unit is the whole family. Deterministic in (plan, world):
// every rank computes the same owners.
static inline u32 unit_tag(const LogicalSpec& ls) {
  if (ls.kind == K_MOVE) return 0;
  u32 t = 1;
  for (int i = 0; i < ls.nops(); i++) t = t * 4 + (u32)ls.aux[i].mem;
  return t;   // < 256
}

void Plan::assign_owners_() {
  mine.clear();
  owner.clear();
  for (Family& f : families) f.owner = 0;
  if (world <= 1) return;
  const u32 n = (u32)hdrs.size();
  owner.assign(n, 0);
  for (const Stage& st : stages) {
    // weights per (family, tag)
    std::vector<u64> w((size_t)(st.fam_hi - st.fam_lo) * 256, 0);
    for (u32 f = st.fam_lo; f < st.fam_hi; f++)
      for (u32 i = families[f].spec_lo; i < families[f].spec_hi; i++)
        w[(size_t)(f - st.fam_lo) * 256 + unit_tag(specs[i])] += hdrs[i].ncand + 1;
    std::vector<u32> units;
    for (u32 u = 0; u < w.size(); u++) if (w[u]) units.push_back(u);
    std::stable_sort(units.begin(), units.end(), [&](u32 a, u32 b) { return w[a] > w[b]; });
    std::vector<u64> load(world, 0);
    std::vector<u8> unit_owner(w.size(), 0);
    for (u32 u : units) {   // heaviest first onto the least loaded rank
      u32 best = 0;
      for (u32 r = 1; r < world; r++) if (load[r] < load[best]) best = r;
      unit_owner[u] = (u8)best;
      load[best] += w[u];
    }
    for (u32 f = st.fam_lo; f < st.fam_hi; f++) {
      for (u32 i = families[f].spec_lo; i < families[f].spec_hi; i++)
        owner[i] = unit_owner[(size_t)(f - st.fam_lo) * 256 + unit_tag(specs[i])];
      families[f].owner = owner[families[f].spec_lo];
    }
  }
  mine.assign(n, 0);
  for (u32 i = 0; i < n; i++) mine[i] = owner[i] == rank;
}

void Plan::adopt_done(u32 rank_, u32 world_, int n_threads_, bool have_cands) {
  if (meta_.world != world_) throw ModelError("shared plan was made for another world size");
  if (world_ < 1 || rank_ >= world_) throw ModelError("bad shard rank / world size");
  for (int k = 0; k < NMEM; k++) {
    top_code[k] = meta_.top_code[k];
    if (top_code[k] > 30) throw ModelError("shared plan: bad top limits");
  }
  stats = meta_.stats;
  rank = rank_;
  world = world_;
  n_threads = n_threads_;
  const u64 n = hdrs.size();
  if (stats.n_specs != n || stats.n_cands != cands.size() || stats.n_stages != stages.size() ||
      stats.n_families != families.size())
    throw ModelError("shared plan: contents do not match their description");
  // Everything a kernel or a lookup indexes with: stages and families tile the ids in order, every
  // Spec's candidate range lies inside the records, goal ids and the id table point at Specs.
  u32 pos = 0, fam = 0;
  for (size_t si = 0; si < stages.size(); si++) {
    const Stage& st = stages[si];
    if (st.spec_lo != pos || st.spec_hi < st.spec_lo || st.spec_hi > n || st.fam_lo != fam || st.fam_hi < st.fam_lo ||
        st.fam_hi > families.size())
      throw ModelError("shared plan: bad stage");
    for (u32 f = st.fam_lo; f < st.fam_hi; f++) {
      const Family& fm = families[f];
      if (fm.spec_lo != pos || fm.spec_hi <= fm.spec_lo || fm.spec_hi > st.spec_hi || fm.stage != si)
        throw ModelError("shared plan: bad family");
      pos = fm.spec_hi;
    }
    if (pos != st.spec_hi) throw ModelError("shared plan: families do not tile their stage");
    fam = st.fam_hi;
  }
  if (pos != n || fam != families.size()) throw ModelError("shared plan: stages do not cover the Specs");
  for (u32 g : goal_ids)
    if (g >= n) throw ModelError("shared plan: bad goal id");
  if (find_tab_.empty() || (find_tab_.size() & (find_tab_.size() - 1)) || find_tab_.size() < n)
    throw ModelError("shared plan: bad id table");
  for (u32 id : find_tab_)
    if (id != 0xFFFFFFFFu && id >= n) throw ModelError("shared plan: bad id table");
  const u64 ncand = stats.n_cands;
  std::atomic<int> bad{0};
  parallel_for(n, n_threads_, [&](size_t i, int) {
    const SpecHdr& h = hdrs[i];
    if ((u64)h.cand_off + h.ncand > ncand) { bad = 1; return; }
    if (specs[i].kind > K_MATMUL || specs[i].spec_shape.n > MAX_RANK) { bad = 2; return; }
    for (int o = 0; o < specs[i].nops(); o++)
      if (specs[i].aux[o].mem > GL || specs[i].aux[o].layout.n > MAX_PHYS) { bad = 2; return; }
    if (!have_cands) return;
    for (u32 c = h.cand_off; c < h.cand_off + h.ncand; c++) {
      const CandRec& r = cands[c];
      if (r.kind > MRL_CK_BLOCK || r.nchild > 3 || r.level >= NMEM || r.thr_code > 30 || r.late > 1 || (r.kind == MRL_CK_LEAF) != (r.nchild == 0)) { bad = 3; return; }
      for (int j = 0; j < r.nchild; j++)
        if (r.child[j] >= n) { bad = 3; return; }
    }
  });
  if (bad.load() == 1) throw ModelError("shared plan: a Spec's candidate range lies outside the records");
  if (bad.load() == 2) throw ModelError("shared plan: bad Spec");
  if (bad.load() == 3) throw ModelError("shared plan: bad candidate record");
  assign_owners_();
}

u64 Plan::fingerprint(int n_threads_) const {
  const size_t n = specs.size();
  std::vector<u64> hs(n);
  parallel_for(n, n_threads_, [&](size_t i, int) {
    char kb[LogicalSpec::MAX_KEY];
    const int kl = specs[i].key_into(kb);
    hs[i] = hash_key(kb, kl) * (2 * (u64)i + 1);
  });
  u64 h = 0x243F6A8885A308D3ull ^ (u64)n;
  for (size_t i = 0; i < n; i++) h = (h ^ hs[i]) * 0x9E3779B97F4A7C15ull + (h >> 29);
  for (int k = 0; k < NMEM; k++) h = (h ^ top_code[k]) * 0xD6E8FEB86659FD93ull;
  return h ^ (h >> 31);
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

namespace {

// The limits-independent record of one candidate, without child ids. False: the candidate never
// fits, at any limits in the lattice.
bool make_rec(const Candidate& c, const u32* top_code, CandRec& r) {
  memset(&r, 0, sizeof(r));
  r.action = c.action;
  r.kind = c.kind;
  r.nchild = c.nchild;
  r.imm = c.imm;
  r.level = c.level;
  r.units = c.units;
  const u32 thr = (c.kind == CK_MOVE || c.kind == CK_LEAF) ? code_ceil(c.level, c.units) : 0;
  if (thr > top_code[c.level]) return false;
  r.thr_code = (u8)thr;
  r.peak_code = (c.kind == CK_LEAF) ? (u8)code_ceil(c.level, c.units) : 0;
  return true;
}

// Evaluation order of a Spec's records is free (the argmin carries the action number). Records
// whose children all lie in earlier stages come first: kernels, then loops and blocks, then Moves
// by ascending base cost. Records with a child in the Spec's own stage (relayout Moves) come
// last, dearest first: the device walks them from the end, cheapest first, and stops at the first
// one whose base cost alone exceeds the cell's optimum so far.
u64 cand_rank(const CandRec& c) {
  if (c.late) return (u64(1) << 40) | (0xFFFFFFFFu - c.imm);
  const u64 k = c.kind == MRL_CK_LEAF ? 0 : (c.kind == MRL_CK_LOOP ? 1 : (c.kind == MRL_CK_BLOCK ? 2 : 3));
  return (k << 32) | (c.kind == MRL_CK_MOVE ? c.imm : 0u);
}
// Whether a candidate of `parent` has a child in the parent's own stage.
bool has_same_stage_child(const LogicalSpec& parent, const Candidate& c) {
  const u32 sk = stage_key(parent);
  for (int j = 0; j < c.nchild; j++)
    if (stage_key(c.child[j]) == sk) return true;
  return false;
}
bool cand_before(const CandRec& a, const CandRec& b) { return cand_rank(a) < cand_rank(b); }

// Two 64-bit hashes of a goal's canonical key with the dtype byte forced to `as`.
std::pair<u64, u64> twin_hash(const LogicalSpec& g0, Dtype as) {
  LogicalSpec g = g0;
  g.dtype = as;
  if (logicalspec_canonicalize(g) != CANON_OK) return {0, 0};
  char kb[LogicalSpec::MAX_KEY + 8];
  const int kl = g.key_into(kb);
  const u64 h1 = hash_key(kb, kl);
  kb[kl] = (char)0x5a;
  return {h1, hash_key(kb, kl + 1)};
}

}  // namespace

Plan build_plan(const std::vector<LogicalSpec>& goals, int n_threads, const u64* top_limits, u32 rank, u32 world,
                int mirror_dtype, u32 flags) {
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

  // ---- 0. dtype twins ----
  // When the goals come in two dtypes of one byte size (u32 and f32) and the two goal sets are
  // each other's images under swapping the dtype, only the first dtype is discovered and
  // tabulated: a Spec's Moves, tile-outs and splits depend on the dtype's size only, so the twin's
  // records are the same with its own leaf kernels put in (step 2). A sample of the twins is
  // tabulated directly afterwards and compared. PLAN_NO_TWINS disables this.
  bool twin = false;
  Dtype dt_a = DT_U8, dt_b = DT_U8;
  const bool mirrored = mirror_dtype >= 0 && !goals.empty();   // the caller vouches: goals come in one dtype, mirror them
  if (mirrored) {
    dt_a = goals[0].dtype;
    dt_b = (Dtype)mirror_dtype;
    for (const LogicalSpec& g : goals)
      if (g.dtype != dt_a) throw ModelError("mirrored goals must come in one dtype");
    if (dt_b <= dt_a || dtype_size(dt_a) != dtype_size(dt_b)) throw ModelError("cannot mirror goals into this dtype");
    twin = true;
  } else {
    int seen[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (const LogicalSpec& g : goals) seen[g.dtype & 7] = 1;
    int n_dt = 0;
    for (int d = 0; d < 8; d++)
      if (seen[d]) { if (n_dt == 0) dt_a = (Dtype)d; else dt_b = (Dtype)d; n_dt++; }
    if (n_dt == 2 && dtype_size(dt_a) == dtype_size(dt_b) && !(flags & PLAN_NO_TWINS)) {
      std::vector<std::pair<u64, u64>> ha, hb;
      std::vector<std::pair<u64, u64>> all(goals.size());
      parallel_for(goals.size(), n_threads, [&](size_t i, int) { all[i] = twin_hash(goals[i], dt_a); });
      for (size_t i = 0; i < goals.size(); i++) (goals[i].dtype == dt_a ? ha : hb).push_back(all[i]);
      std::sort(ha.begin(), ha.end());
      std::sort(hb.begin(), hb.end());
      ha.erase(std::unique(ha.begin(), ha.end()), ha.end());
      hb.erase(std::unique(hb.begin(), hb.end()), hb.end());
      twin = ha == hb && !ha.empty() && ha.front() != std::pair<u64, u64>{0, 0};
    }
  }

  // ---- 1. discovery: closure of the goals under "is a sub-Spec of some candidate" ----
  double t0 = now_s();
  std::vector<KeyShard> shards(NSHARD);
  std::shared_ptr<TempSpecs> temp_owner = std::make_shared<TempSpecs>();
  TempSpecs& temp = *temp_owner;
  std::atomic<u32> next_id{0};

  plan.goal_ids.assign(goals.size(), 0);
  parallel_for(goals.size(), n_threads, [&](size_t gi, int) {
    LogicalSpec g = goals[gi];
    if (twin) g.dtype = dt_a;   // the twin's id is derived from this one in step 2
    if (logicalspec_canonicalize(g) != CANON_OK) throw ModelError("goal Spec cannot be canonicalized: " + goals[gi].str());
    char kb[LogicalSpec::MAX_KEY];
    const int kl = g.key_into(kb);
    const u64 h = hash_key(kb, kl);
    bool inserted = false;
    const u32 id = shards[h % NSHARD].find_or_insert(h, kb, kl, [&]() { return next_id++; }, &inserted);
    if (inserted) {
      TempSpec& ts = temp.construct(id);
      ts.ls = g;
      ts.key.assign(kb, (size_t)kl);
    }
    plan.goal_ids[gi] = id;
  });
  plan.stats.n_goal_specs = (u64)next_id.load() * (twin ? 2 : 1);

  // Per thread: the Moves of an operand, and the ids of their prologue / epilogue Move Specs, are
  // worked out once and reused by every Spec that has the operand.
  std::vector<std::unique_ptr<MoveMemo>> move_memos(n_threads);
  if (!(flags & PLAN_NO_MEMO))   // without: every Spec is tabulated from scratch (for cross-checks)
    for (auto& mm : move_memos) mm.reset(new MoveMemo());
  // Breadth-first: the Specs found in one round (a range of ids) are tabulated in the next.
  for (u32 round_lo = 0, round_hi = next_id.load(); round_lo < round_hi; round_lo = round_hi, round_hi = next_id.load()) {
    struct ChildKey { u64 h; int len; char bytes[LogicalSpec::MAX_KEY]; };
    struct alignas(128) PerThread { std::vector<Candidate> scratch; std::vector<ChildKey> keys; std::vector<int> key_of;
                                   std::vector<std::pair<u64, u32>> ranks; std::vector<CandRec> sorted; };
    // (the Move memos live across rounds: see move_memos below)
    std::vector<PerThread> per_thread(n_threads);
    parallel_for(round_hi - round_lo, n_threads, [&](size_t fi, int tid) {
      TempSpec& ts = temp[round_lo + (u32)fi];
      std::vector<Candidate>& cs = per_thread[tid].scratch;
      cs.clear();
      u32 leaf_first = 0, leaf_end = 0;
      tabulate_candidates(ts.ls, cs, &leaf_first, &leaf_end, move_memos[tid].get());
      ts.leaf_first = (u16)leaf_first;
      ts.leaf_end = (u16)leaf_end;
      ts.cands.reserve(cs.size());
      // Keys and hashes of the children first, with a prefetch of each one's table slot: the
      // probes below then find their cache lines on the way instead of missing one by one.
      std::vector<ChildKey>& keys = per_thread[tid].keys;
      std::vector<int>& key_of = per_thread[tid].key_of;   // per (candidate, child) in order: index into keys, or -1
      keys.clear();
      key_of.clear();
      for (const Candidate& c : cs)
        for (int j = 0; j < c.nchild; j++) {
          if (c.child_id_slot[j] && *c.child_id_slot[j] != 0xFFFFFFFFu) { key_of.push_back(-1); continue; }
          key_of.push_back((int)keys.size());
          keys.emplace_back();
          ChildKey& k = keys.back();
          k.len = c.child[j].key_into(k.bytes);
          k.h = hash_key(k.bytes, k.len);
          shards[k.h % NSHARD].prefetch(k.h);
        }
      size_t next_child = 0;
      for (const Candidate& c : cs) {
        CandRec r;
        const bool keep = make_rec(c, top_code, r);
        if (keep) r.late = has_same_stage_child(ts.ls, c) ? 1 : 0;
        for (int j = 0; j < c.nchild; j++) {
          const int ki = key_of[next_child++];
          if (!keep) continue;   // the candidate never fits: its children are not part of the closure
          if (c.child_id_slot[j] && *c.child_id_slot[j] != 0xFFFFFFFFu) {
            r.child[j] = *c.child_id_slot[j];   // this thread met the Move Spec before (maybe a moment ago)
            continue;
          }
          const ChildKey& k = keys[ki];
          bool inserted = false;
          const u32 id = shards[k.h % NSHARD].find_or_insert(k.h, k.bytes, k.len, [&]() { return next_id++; }, &inserted);
          if (inserted) {
            TempSpec& fresh = temp.construct(id);
            fresh.ls = c.child[j];
            fresh.key.assign(k.bytes, (size_t)k.len);
          }
          r.child[j] = id;
          if (c.child_id_slot[j]) *c.child_id_slot[j] = id;
        }
        if (!keep) continue;
        ts.n_leaf += r.kind == MRL_CK_LEAF;
        ts.cands.push_back(r);
      }
      // final record order, while the records are still in cache: a stable sort by rank; a few
      // tens of records, so by insertion on (rank, position) pairs
      {
        std::vector<std::pair<u64, u32>>& rk = per_thread[tid].ranks;
        const size_t nr = ts.cands.size();
        if (nr > 96) {
          std::stable_sort(ts.cands.begin(), ts.cands.end(), cand_before);
        } else if (nr > 1) {
          rk.resize(nr);
          for (size_t k = 0; k < nr; k++) {
            const std::pair<u64, u32> me(cand_rank(ts.cands[k]), (u32)k);
            size_t at = k;
            while (at > 0 && rk[at - 1].first > me.first) { rk[at] = rk[at - 1]; at--; }
            rk[at] = me;
          }
          std::vector<CandRec>& tmp = per_thread[tid].sorted;
          tmp.resize(nr);
          for (size_t k = 0; k < nr; k++) tmp[k] = ts.cands[rk[k].second];
          memcpy(ts.cands.data(), tmp.data(), nr * sizeof(CandRec));
        }
      }
    });
  }
  { std::vector<KeyShard>().swap(shards); }
  const u32 n = next_id.load();
  plan.stats.seconds_discover = now_s() - t0;

  // ---- 2. final ids: stage-major (phase, log-shape sum, memory-level sum), then key order ----
  double t1 = now_s();
  double t_step = t1;
  auto step_done = [&](int k) { const double t = now_s(); plan.stats.seconds_layout_step[k] += t - t_step; t_step = t; };
  std::vector<u32> order(n);
  std::vector<u32> gkey(n);
  parallel_for(n, n_threads, [&](size_t i, int) { gkey[i] = stage_key(temp[(u32)i].ls); });
  {
    // bucket by stage key, then sort every bucket by Spec key on all threads
    std::vector<u32> uniq(gkey);
    std::sort(uniq.begin(), uniq.end());
    uniq.erase(std::unique(uniq.begin(), uniq.end()), uniq.end());
    std::vector<u32> start(uniq.size() + 1, 0);
    std::vector<u32> bucket(n);
    parallel_for(n, n_threads, [&](size_t i, int) {
      bucket[i] = (u32)(std::lower_bound(uniq.begin(), uniq.end(), gkey[i]) - uniq.begin());
    });
    for (u32 i = 0; i < n; i++) start[bucket[i] + 1]++;
    for (size_t b = 0; b < uniq.size(); b++) start[b + 1] += start[b];
    std::vector<u32> cur(start.begin(), start.end() - 1);
    for (u32 i = 0; i < n; i++) order[cur[bucket[i]]++] = i;
    std::vector<u32> by_size(uniq.size());
    for (u32 b = 0; b < uniq.size(); b++) by_size[b] = b;
    std::sort(by_size.begin(), by_size.end(), [&](u32 a, u32 b) { return start[a + 1] - start[a] > start[b + 1] - start[b]; });
    std::atomic<size_t> nextb{0};
    std::vector<std::thread> pool;
    for (int t = 0; t < n_threads; t++)
      pool.emplace_back([&]() {
        for (;;) {
          const size_t k = nextb.fetch_add(1);
          if (k >= by_size.size()) break;
          const u32 b = by_size[k];
          std::sort(order.begin() + start[b], order.begin() + start[b + 1],
                    [&](u32 x, u32 y) { return temp[x].key < temp[y].key; });
        }
      });
    for (auto& th : pool) th.join();
  }
  step_done(0);   // stage keys, buckets, key sort
  // Final ids. Without twins: the sorted position. With twins every stage holds its discovered
  // Specs followed by their twins (the key orders by dtype right after the kind, and dt_a < dt_b):
  // position i of a stage that starts at sorted position lo and has cnt Specs becomes id i + lo,
  // its twin id i + lo + cnt.
  const u32 mult = twin ? 2u : 1u;
  if ((u64)n * mult > 0xFFFFFFF0ull) throw ModelError("too many Specs");
  const u32 N = n * mult;
  std::vector<u32> id_a(n), id_b(twin ? n : 0);   // by temporary id
  std::vector<u32> pos_a(n), pos_b(twin ? n : 0); // by sorted position
  for (u32 i = 0; i < n;) {
    u32 j = i;
    while (j < n && gkey[order[j]] == gkey[order[i]]) j++;
    for (u32 k = i; k < j; k++) {
      pos_a[k] = twin ? k + i : k;
      id_a[order[k]] = pos_a[k];
      if (twin) { pos_b[k] = pos_a[k] + (j - i); id_b[order[k]] = pos_b[k]; }
    }
    i = j;
  }
  if (mirrored) {   // goals, then their mirror images
    const size_t ng = goals.size();
    plan.goal_ids.resize(2 * ng);
    for (size_t gi = 0; gi < ng; gi++) {
      const u32 t = plan.goal_ids[gi];
      plan.goal_ids[gi] = id_a[t];
      plan.goal_ids[ng + gi] = id_b[t];
    }
  } else {
    for (size_t gi = 0; gi < goals.size(); gi++)
      plan.goal_ids[gi] = (twin && goals[gi].dtype == dt_b) ? id_b[plan.goal_ids[gi]] : id_a[plan.goal_ids[gi]];
  }

  step_done(1);   // final ids
  plan.specs.reset(N);
  plan.hdrs.reset(N);
  // candidate records per final id; a twin swaps the leaf records for its own
  std::vector<u64> offs((size_t)N + 1, 0);
  parallel_for(n, n_threads, [&](size_t i, int) {
    TempSpec& ts = temp[order[i]];
    offs[pos_a[i] + 1] = ts.cands.size();
    if (twin) {
      // the twin's own leaf kernels, kept for the pass that writes the records
      LogicalSpec sb = ts.ls;
      sb.dtype = dt_b;
      std::vector<Candidate> lv;
      ts.twin_leaf_end = (u16)tabulate_leaves(sb, ts.leaf_first, lv);
      CandRec r;
      for (const Candidate& c : lv)
        if (make_rec(c, top_code, r)) ts.twin_leaf.push_back(r);
      offs[pos_b[i] + 1] = ts.cands.size() - ts.n_leaf + ts.twin_leaf.size();
    }
  });
  for (u32 i = 0; i < N; i++) offs[i + 1] += offs[i];
  const u64 ncand = offs[N];
  if (ncand > 0xFFFFFFFFull) throw ModelError("too many candidate records");
  plan.cands.reset(ncand);
  step_done(2);   // twin leaf kernels, record offsets
  {
    // Written in the order the Specs were discovered - the order their temporary records were
    // allocated in - and each Spec's temporary records are released as soon as they are copied. A
    // large job does this in slices and hands the freed pages back to the system after each, so
    // that the final arrays grow as the temporaries shrink instead of on top of them.
    std::vector<u64> kids_t(1, 0);
    const u32 n_slices = n > (8u << 20) ? 24 : 1;
    for (u32 sl = 0; sl < n_slices; sl++) {
      const u32 t_lo = (u32)((u64)n * sl / n_slices), t_hi = (u32)((u64)n * (sl + 1) / n_slices);
      parallel_for(t_hi - t_lo, n_threads, [&](size_t k, int) {
        const u32 t = t_lo + (u32)k;
        TempSpec& ts = temp[t];
        u64 kids = 0;
        // the children's final ids are scattered reads: ask for all of them before any is needed
        for (const CandRec& r : ts.cands)
          for (int j = 0; j < r.nchild; j++) {
            __builtin_prefetch(&id_a[r.child[j]]);
            if (twin) __builtin_prefetch(&id_b[r.child[j]]);
          }
        {
          const u32 id = id_a[t];
          plan.specs[id] = ts.ls;
          SpecHdr& h = plan.hdrs[id];
          memset(&h, 0, sizeof(h));
          u64 off = offs[id];
          h.cand_off = (u32)off;
          h.ncand = (u32)ts.cands.size();
          for (CandRec r : ts.cands) {
            for (int j = 0; j < r.nchild; j++) r.child[j] = id_a[r.child[j]];
            kids += r.nchild;
            plan.cands[off++] = r;
          }
        }
        if (twin) {
          const u32 id = id_b[t];
          LogicalSpec sb = ts.ls;
          sb.dtype = dt_b;
          plan.specs[id] = sb;
          SpecHdr& h = plan.hdrs[id];
          memset(&h, 0, sizeof(h));
          u64 off = offs[id];
          h.cand_off = (u32)off;
          h.ncand = (u32)(offs[id + 1] - offs[id]);
          // its own leaf kernels, numbered from where the leaf section starts ...
          const u32 leaf_end_b = ts.twin_leaf_end;
          for (const CandRec& r : ts.twin_leaf) plan.cands[off++] = r;
          // ... then the first dtype's other records; what is numbered after the leaf section
          // (ToAccum, splits) moves by the difference in applicable kernels
          const int shift = (int)leaf_end_b - (int)ts.leaf_end;
          for (CandRec r : ts.cands) {
            if (r.kind == MRL_CK_LEAF) continue;
            if (r.kind == MRL_CK_BLOCK || (r.kind == MRL_CK_LOOP && r.action >= ts.leaf_end)) r.action = (u16)((int)r.action + shift);
            for (int j = 0; j < r.nchild; j++) r.child[j] = id_b[r.child[j]];
            kids += r.nchild;
            plan.cands[off++] = r;
          }
          if (off != offs[id + 1]) throw ModelError("planner: twin record count mismatch");
        }
        std::vector<CandRec>().swap(ts.cands);
        std::vector<CandRec>().swap(ts.twin_leaf);
        std::string().swap(ts.key);
        __atomic_fetch_add(&kids_t[0], kids, __ATOMIC_RELAXED);
      });
      if (n_slices > 1) malloc_trim(0);
    }
    plan.stats.n_children += kids_t[0];
  }
  step_done(3);   // record array
  // The temporary Specs are taken apart by a few threads of their own while the rest of the
  // plan is built; whoever drops the plan's handle last (normally the end of this function)
  // waits for them.
  {
    TempSpecs* tp = temp_owner.get();
    const int nt = std::max(1, n_threads / 3);
    std::thread* bg = new std::thread([tp, n, nt]() { parallel_for(n, nt, [tp](size_t i, int) { tp->destroy((u32)i); }); });
    plan.cleanup_ = std::shared_ptr<void>(nullptr, [bg, temp_owner](void*) mutable {
      bg->join();
      delete bg;
      temp_owner.reset();
    });
  }
  // from here on everything is about the final arrays (N Specs)
  // id lookup table for find(): open addressing over the Spec key hash, ids only (equality is
  // checked on the Spec itself)
  {
    size_t cap = 64;
    while (cap < (size_t)N * 2) cap *= 2;
    plan.find_tab_.assign(cap, 0xFFFFFFFFu);
    std::vector<u64> hs(N);
    parallel_for(N, n_threads, [&](size_t i, int) {
      char kb[LogicalSpec::MAX_KEY];
      const int kl = plan.specs[i].key_into(kb);
      hs[i] = hash_key(kb, kl);
    });
    // claimed slot by slot with compare-and-swap from all threads (which slot of a probe run an
    // id ends up in depends on the race; lookups do not care)
    const size_t mask = cap - 1;
    u32* tab = plan.find_tab_.data();
    parallel_for(N, n_threads, [&](size_t i, int) {
      size_t j = (size_t)hs[i] & mask;
      for (;;) {
        u32 expect = 0xFFFFFFFFu;
        if (__atomic_load_n(&tab[j], __ATOMIC_RELAXED) == expect &&
            __atomic_compare_exchange_n(&tab[j], &expect, (u32)i, false, __ATOMIC_RELAXED, __ATOMIC_RELAXED))
          break;
        j = (j + 1) & mask;
      }
    });
  }

  step_done(4);   // id table
  // stages, and inside them families: maximal runs with equal dtype and shape (ids are
  // key-sorted, and the key starts with kind, dtype, serial flag, rank, shape)
  {
    std::vector<u32> skey(N);
    std::vector<u8> fam_start(N);   // dtype or shape differs from the Spec before
    parallel_for(N, n_threads, [&](size_t i, int) {
      skey[i] = stage_key(plan.specs[i]);
      fam_start[i] = i == 0 || plan.specs[i].dtype != plan.specs[i - 1].dtype || plan.specs[i].spec_shape != plan.specs[i - 1].spec_shape;
    });
    for (u32 i = 0; i < N;) {
      const u32 sk = skey[i];
      u32 j = i;
      while (j < N && skey[j] == sk) j++;
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
        do {
          w += plan.hdrs[b].ncand + 1;
          b++;
        } while (b < j && !fam_start[b]);
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
  }

  step_done(5);   // stages and families
  // The order the device relies on: a child never lies in a later stage; a child inside its
  // parent's stage belongs to a Move that consumes memory (so it sits at strictly lower limits),
  // to the parent's family and - when the fill is sharded - to the rank that solves the parent.
  if (plan.world > 255) throw ModelError("at most 255 ranks");
  plan.assign_owners_();
  {
    std::vector<u32> stage_of(N), fam_of(N);
    for (u32 si = 0; si < plan.stages.size(); si++)
      for (u32 i = plan.stages[si].spec_lo; i < plan.stages[si].spec_hi; i++) stage_of[i] = si;
    for (u32 fi = 0; fi < plan.families.size(); fi++)
      for (u32 i = plan.families[fi].spec_lo; i < plan.families[fi].spec_hi; i++) fam_of[i] = fi;
    std::atomic<int> bad{0};
    std::atomic<u64> bad_pair{0};
    const bool sharded = !plan.owner.empty();
    parallel_for(N, n_threads, [&](size_t i, int) {
      const SpecHdr& h = plan.hdrs[i];
      for (u32 c = h.cand_off; c < h.cand_off + h.ncand; c++) {
        const CandRec& r = plan.cands[c];
        if (c > h.cand_off && plan.cands[c - 1].late && (!r.late || r.imm > plan.cands[c - 1].imm)) { bad = 4; bad_pair = ((u64)i << 32) | i; }
        bool any_same = false;
        for (int j = 0; j < r.nchild; j++) any_same |= stage_of[r.child[j]] == stage_of[i];
        if (any_same != (r.late != 0)) { bad = 4; bad_pair = ((u64)i << 32) | i; }
        for (int j = 0; j < r.nchild; j++) {
          const u32 ch = r.child[j];
          int what = 0;
          if (stage_of[ch] > stage_of[i]) what = 1;
          else if (stage_of[ch] < stage_of[i]) { /* finished before the parent's stage starts */ }
          else if (stage_of[ch] == stage_of[i]) {
            if (r.kind != MRL_CK_MOVE || r.units == 0 || fam_of[ch] != fam_of[i] || !r.late) what = 2;
            else if (sharded && plan.owner[ch] != plan.owner[i]) what = 3;
          }
          if (what) { bad = what; bad_pair = ((u64)i << 32) | ch; }
        }
      }
    });
    const std::string who = bad.load() ? (": parent " + plan.specs[bad_pair.load() >> 32].str() + ", child " +
                                          plan.specs[bad_pair.load() & 0xFFFFFFFFu].str()) : std::string();
    if (bad.load() == 1) throw ModelError("planner: a child Spec lies in a later stage than its parent" + who);
    if (bad.load() == 2) throw ModelError("planner: a same-stage child is not below its parent in the limits lattice" + who);
    if (bad.load() == 3) throw ModelError("planner: a same-stage child belongs to another rank than its parent" + who);
    if (bad.load() == 4) throw ModelError("planner: records with a same-stage child are not flagged or not stored last, dearest first" + who);
  }
  if (twin) {
    // Sample check of the twin derivation: tabulate every 2039th Spec (originals and twins alike)
    // directly and compare with the records built above, byte for byte.
    const u32 step = 2039;
    std::atomic<long> bad{-1};
    parallel_for((N + step - 1) / step, n_threads, [&](size_t k, int) {
      const u32 id = (u32)k * step;
      std::vector<Candidate> cs;
      tabulate_candidates(plan.specs[id], cs);
      std::vector<CandRec> recs;
      for (const Candidate& c : cs) {
        CandRec r;
        if (!make_rec(c, top_code, r)) continue;
        r.late = has_same_stage_child(plan.specs[id], c) ? 1 : 0;
        for (int j = 0; j < c.nchild; j++) {
          const long ch = plan.find(c.child[j]);
          if (ch < 0) { bad = id; return; }
          r.child[j] = (u32)ch;
        }
        recs.push_back(r);
      }
      std::stable_sort(recs.begin(), recs.end(), cand_before);
      const SpecHdr& h = plan.hdrs[id];
      if (recs.size() != h.ncand || (h.ncand && memcmp(recs.data(), &plan.cands[h.cand_off], h.ncand * sizeof(CandRec)) != 0)) bad = id;
    });
    if (bad.load() >= 0)
      throw ModelError("planner: records derived for a dtype twin differ from direct tabulation: " + plan.specs[(u32)bad.load()].str());
  }
  step_done(6);   // owners, order check, twin spot check
  plan.cleanup_.reset();   // waits for the release of the temporaries
  step_done(7);   // waiting for the temporaries' release
  plan.stats.seconds_layout = now_s() - t1;

  plan.stats.n_specs = N;
  plan.stats.n_cands = ncand;
  plan.stats.n_stages = plan.stages.size();
  plan.stats.n_families = plan.families.size();
  return plan;
}

Plan table_only_plan(RawVec<LogicalSpec>&& specs, RawVec<SpecHdr>&& hdrs, const u32* top_code, int n_threads) {
  if (specs.size() != hdrs.size()) throw ModelError("saved table: Specs and headers differ in number");
  if (n_threads < 1) n_threads = 1;
  Plan plan;
  plan.n_threads = n_threads;
  for (int k = 0; k < NMEM; k++) {
    if (top_code[k] > 30) throw ModelError("saved table: bad top limits");
    plan.top_code[k] = top_code[k];
  }
  plan.specs = std::move(specs);
  plan.hdrs = std::move(hdrs);
  const u32 N = (u32)plan.specs.size();
  size_t cap = 64;
  while (cap < (size_t)N * 2) cap *= 2;
  plan.find_tab_.assign(cap, 0xFFFFFFFFu);
  const size_t mask = cap - 1;
  u32* tab = plan.find_tab_.data();
  parallel_for(N, n_threads, [&](size_t i, int) {
    char kb[LogicalSpec::MAX_KEY];
    const int kl = plan.specs[i].key_into(kb);
    size_t j = (size_t)hash_key(kb, kl) & mask;
    for (;;) {
      u32 expect = 0xFFFFFFFFu;
      if (__atomic_load_n(&tab[j], __ATOMIC_RELAXED) == expect &&
          __atomic_compare_exchange_n(&tab[j], &expect, (u32)i, false, __ATOMIC_RELAXED, __ATOMIC_RELAXED))
        break;
      j = (j + 1) & mask;
    }
  });
  plan.stats.n_specs = N;
  return plan;
}

}  // namespace mrl

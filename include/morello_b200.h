/*
 * morello_b200 — C ABI of the B200 synthesis-database fill.
 *
 * Drop-in boundary for ONE path of Morello: the search/database calls its `precompute`
 * binary and `top_down` make. Plain pointers and sizes only; the library owns every device
 * allocation; no call throws or aborts across this boundary (int status, 0 = success,
 * negative = error, text from mrl_last_error).
 *
 * Spec blobs. A logical Spec crosses the boundary as the byte string produced by
 * mrl_spec_* helpers (or built by hand): kind, dtype, serial flag, rank, dims (u16 LE each),
 * then per operand: memory, vector size, physical-dim count, contiguous count and 4 bytes per
 * physical dim (logical dim, kind, size u16 LE). Memory limits are four u64 in the order
 * RF, VRF, L1, GL: registers, and cache lines (powers of two), exactly the decoded MemVec of
 * morello/src/memorylimits.rs:51.
 */
#ifndef MORELLO_B200_H
#define MORELLO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mrl_ctx mrl_ctx;

/* One ActionCostVec with k = 1 (morello/src/db/mod.rs:54,171): found = 1 with the optimal
 * (ActionNum, Cost{main, peaks, depth}) (morello/src/cost.rs:13-17), found = 0 when the Spec
 * has no implementation under its limits, found = -1 for a Spec the tables do not hold. */
typedef struct mrl_decision {
  int32_t found;
  uint32_t action;
  uint32_t main_cost;
  uint32_t depth;
  uint64_t peaks[4]; /* decoded: RF, VRF registers; L1, GL cache lines */
} mrl_decision;

typedef struct mrl_stats {
  uint64_t n_specs;            /* logical Specs in the tables (goals and their closure) */
  uint64_t n_goal_specs;
  uint64_t n_candidates;       /* candidate records */
  uint64_t n_stages;           /* stages of the fill (plan order) */
  uint64_t n_rows;             /* rows of the finished tables: cells of the Specs' final limits grids */
  uint64_t n_cells_solved;     /* working-grid cells the last fill solved (all passes) */
  uint64_t n_candidates_evaluated; /* candidate records evaluated by those solves */
  uint64_t n_rows_gathered;    /* child rows they read */
  uint64_t n_passes;           /* solve passes of the last fill, summed over stages */
  uint64_t n_launches;         /* kernel launches of the last fill (one cooperative launch per stage) */
  uint64_t n_grid_syncs;       /* grid-wide barriers inside those launches */
  uint64_t algorithmic_bytes;  /* of the finished table: per final row 12 bytes out, 16 per candidate record of
                                * its Spec, 16 per child of each candidate that fits the row's limits */
  uint64_t h2d_bytes;          /* bytes copied host->device by the last upload */
  uint64_t d2h_bytes;          /* bytes copied device->host by the last query */
  double plan_seconds;         /* host: closure, candidate tabulation, stage order */
  double upload_seconds;
  double fill_ms;              /* device time of the last fill (CUDA events on the launch stream) */
  double combine_ms;           /* of which inside the solve phases (device timer) */
  double early_ms;             /* of which the phase that needs no order: candidates whose children lie in earlier stages */
  uint64_t n_sweeps;           /* relaxation sweeps over the candidates with a same-stage child, all passes */
  double plan_goal_seconds;    /* of plan_seconds: enumerating the goal Specs */
  double plan_discover_seconds;/* of plan_seconds: closure of the goals and their candidate records */
  double plan_layout_seconds;  /* of plan_seconds: stage order, final ids, record array */
  double plan_layout_step_seconds[8]; /* of that: key sort, final ids, twin leaf kernels and offsets, record array, id table,
                                       * stages and families, order and twin checks, release of temporaries */
  uint64_t n_cells_unordered;  /* of n_cells_solved: cells of the grids of the unordered phase */
  uint64_t n_candidates_swept; /* of n_candidates_evaluated: by the relaxation sweeps */
  uint64_t n_items_swept;      /* work items (pieces of one Spec's working grid) the sweeps evaluated */
  uint64_t n_buffer_growths;   /* times the last fill had to enlarge a device buffer and solve a stage again */
  double phase_ms[8];          /* device time of the last fill by part of the stage kernels: setup, unordered phase, its real
                                * breakpoints, per-pass setup, cell initialisation, first sweeps, later sweeps, real breakpoints */
} mrl_stats;

/* One row of the device table as mrl_export_all hands it out: main cost; peak memory as lattice
 * codes, RF in the top byte .. GL in the low byte (registers raw, caches as bit length of the
 * line count: MemoryLimitsBimap, morello/src/memorylimits.rs:696-734); depth << 16 | ActionNum,
 * all ones when the cell has no implementation. */
typedef struct mrl_row {
  uint32_t main_cost;
  uint32_t peak_codes;
  uint32_t depth_action;
  uint32_t reserved;
} mrl_row;

enum { MRL_KIND_MOVE = 0, MRL_KIND_FILL_ZERO = 1, MRL_KIND_MATMUL_ACCUM = 2, MRL_KIND_MATMUL = 3 };
enum { MRL_DTYPE_U32 = 4, MRL_DTYPE_F32 = 6 };
enum { MRL_MEM_RF = 0, MRL_MEM_VRF = 1, MRL_MEM_L1 = 2, MRL_MEM_GL = 3 };
enum { MRL_THROUGH_MOVE = 0, MRL_THROUGH_ZERO = 1, MRL_THROUGH_MATMUL = 2 };

/* Replaces FilesDatabase::new (morello/src/db/mod.rs:350-380): one context = one in-memory
 * database on one GPU. n_threads = host threads for planning (0 = all cores). */
int mrl_ctx_create(int device, int n_threads, mrl_ctx** out);
/* Replaces Drop for FilesDatabase (morello/src/db/mod.rs:1154-1167); frees device memory. */
void mrl_ctx_destroy(mrl_ctx* ctx);
const char* mrl_last_error(const mrl_ctx* ctx);

/* Builds the blob of a Spec whose operands are all row-major in one memory: the goal Specs of
 * frontend/src/main.rs:192-204 and the bound Specs of precompute/src/main.rs:651-736.
 * Returns the blob length, or a negative status. */
int mrl_spec_simple(int kind, int dtype, const uint32_t* spec_shape, int rank, int memory, uint8_t* out,
                    size_t cap);
/* Spec::canonicalize (morello/src/spec.rs:1704-1747). Returns the new blob length. */
int mrl_spec_canonicalize(const uint8_t* blob, size_t len, uint8_t* out, size_t cap);
/* Display form of a Spec blob (debugging aid). Returns the string length. */
int mrl_spec_describe(const uint8_t* blob, size_t len, char* out, size_t cap);
/* Avx2Target::max_mem() (morello/src/target/avx2.rs:59-65). */
void mrl_max_mem(uint64_t limits[4]);

/* The applicable actions of a Spec as the fill tabulates them (Target::actions,
 * morello/src/target/cpu.rs:455-823, with each action's solver, morello/src/scheduling/mod.rs:148-167):
 * per action, in enumeration order, 16 bytes - ActionNum u16, combine kind u8 (0 kernel, 1 loop,
 * 2 move, 3 block), number of sub-Specs u8, immediate u32 (kernel cost / loop iterations / base move
 * cost), memory u8 and 3 bytes of padding, units u32 - followed per sub-Spec by its blob length (u16)
 * and its canonical blob. Host only; for inspection and cross-checks. Returns the number of bytes
 * written, or a negative status (-3: `cap` too small). */
long mrl_tabulate(const uint8_t* blob, size_t len, uint8_t* out, size_t cap);

/* Replaces search::top_down_many (morello/src/search/mod.rs:21-42) as called from
 * precompute/src/main.rs:419 and frontend/src/main.rs:296: canonicalises each goal, fills the
 * tables for the goals' whole dependency closure on the GPU and returns each goal's decision
 * at its limits. Host buffers in, host buffers out. blob_off has n+1 entries. */
int mrl_top_down_many(mrl_ctx* ctx, const uint8_t* blobs, const uint64_t* blob_off, size_t n, const uint64_t* limits,
                      mrl_decision* out);

/* Cross-check modes of the host planner (tests): same plan, built the slow way. Bit 0: tabulate
 * both dtypes of a mirrored goal set instead of deriving f32 records from u32 ones; bit 1:
 * tabulate every Spec from scratch instead of re-using per-operand results. */
int mrl_set_plan_flags(mrl_ctx* ctx, uint32_t flags);

/* No counterpart in the reference. Same inputs, outputs and results as mrl_top_down_many, for
 * callers that must not allocate device memory: a process that handed all of HBM to its tables
 * at start-up has none left to give, and worker threads that call in concurrently would be
 * serialised by the device-wide synchronisation of every cudaMalloc / cudaFree. This call makes
 * neither; the device working set of the fill (plan arrays, working grids, row table, lookup staging) lives in
 * one fixed array of MRL_NOALLOC_MAX_BYTES that each GPU loading the library holds until the
 * process exits. A goal set whose fill needs more is refused with status -5 and a message; use
 * mrl_top_down_many for it (a goal that cannot be canonicalised is status -4, as in mrl_plan_goals).
 * The context's own tables are not touched.
 * The first call on a device resolves the array's device address; make that call before any
 * stream capture. All calls share the array, so calls that overlap on one GPU race - issue them
 * one at a time per device. */
#define MRL_NOALLOC_MAX_BYTES (32u << 20)
int mrl_top_down_many_noalloc(mrl_ctx* ctx, const uint8_t* blobs, const uint64_t* blob_off, size_t n,
                              const uint64_t* limits, mrl_decision* out);

/* Replaces the precompute driver (precompute/src/main.rs:172-386) for the Move, Zero and Matmul
 * phases: fills the tables of every canonical Spec up to `size` (and their closure).
 * dtype_mask: bit 0 = u32, bit 1 = f32 (DTYPES, precompute/src/main.rs:55). */
int mrl_precompute(mrl_ctx* ctx, uint32_t size, int through, int dtype_mask);

/* The three steps of the two calls above, exposed separately for measurement: plan on the
 * host, copy the plan to the device, fill (may be repeated). Gigabytes of candidate records keep
 * going up in the background after mrl_upload has returned, in stage order; a fill waits stage by
 * stage for the records it needs, so its first stages overlap the copy. Calls that replace the
 * plan or read the device records (mrl_plan_*, mrl_verify, mrl_device_cands) wait for the copy. */
int mrl_plan_precompute(mrl_ctx* ctx, uint32_t size, int through, int dtype_mask);
int mrl_plan_goals(mrl_ctx* ctx, const uint8_t* blobs, const uint64_t* blob_off, size_t n);
int mrl_upload(mrl_ctx* ctx);
int mrl_fill(mrl_ctx* ctx);

/* Multi-GPU (one process per GPU; no counterpart in the reference, whose workers are threads
 * sharing one database, precompute/src/main.rs:229-240,339). Every rank plans the same job and
 * keeps the whole table. The plan orders Specs into stages; inside a stage the "families"
 * (Specs with equal dtype and shape - Moves change neither) are independent, and outside the Move
 * phase so are the Specs of a family whose operands sit in different memories; rank r computes
 * the Specs it owns (mrl_spec_owners). Per stage the caller sums two device buffers over all ranks on the
 * stream given to mrl_set_stream (e.g. ncclAllReduce, sum of int32, in place; a Spec's words are
 * zero on every rank but its owner):
 *   mrl_set_shard, mrl_plan_*, mrl_upload, then per fill: mrl_fill_begin;
 *   for s in stages { mrl_fill_stage_solve(s, &masks, &n); sum masks;
 *                     mrl_fill_stage_place(s, &rows, &n); sum rows }; mrl_fill_end.
 * masks: the limits-grid breakpoints of the stage's Specs; rows: their finished table rows.
 * Both stage calls wait for the stream: mrl_fill_stage_solve until the masks are final (a rank
 * whose solve ran out of working room enlarges its own buffers and solves the stage again there,
 * while the others wait in the sum), mrl_fill_stage_place until the size of the row slice is known. */
int mrl_set_shard(mrl_ctx* ctx, uint32_t rank, uint32_t world);
/* The ranks of one node share its host cores, so only one of them should plan: it exposes its
 * plan as eight flat host byte ranges (mrl_plan_share), the caller carries the bytes to the other
 * ranks (e.g. ncclBroadcast through device staging), which receive them into ranges of the same
 * sizes (mrl_plan_adopt gives the pointers) and finish with mrl_plan_adopt_done. The planning rank
 * must have called mrl_set_shard with the same world size before planning. */
int mrl_plan_share(mrl_ctx* ctx, void* ptrs[8], uint64_t sizes[8]);
int mrl_plan_adopt(mrl_ctx* ctx, const uint64_t sizes[8], void* ptrs[8], int cands_on_device_only);
/* The candidate records (range 3, by far the largest) are only ever read on the device. With
 * cands_on_device_only the adopting rank gets no host pointer for them (ptrs[3] = NULL): after
 * mrl_upload on every rank the caller copies the planning rank's device records into
 * mrl_device_cands of the others (e.g. ncclBroadcast over NVLink) and then calls mrl_cands_arrived
 * on every rank: it checks on the device that every record the kernels will index with is in
 * range; until it has succeeded a fill is refused with a status. */
int mrl_device_cands(const mrl_ctx* ctx, void** ptr, uint64_t* bytes);
int mrl_cands_arrived(mrl_ctx* ctx);
int mrl_plan_adopt_done(mrl_ctx* ctx, double plan_seconds);
int mrl_set_stream(mrl_ctx* ctx, void* cuda_stream);
uint64_t mrl_num_stages(const mrl_ctx* ctx);
uint64_t mrl_num_families(const mrl_ctx* ctx);
int mrl_stage_info(const mrl_ctx* ctx, uint64_t stage, uint32_t* spec_lo, uint32_t* spec_hi, uint32_t* family_lo,
                   uint32_t* family_hi);
int mrl_family_info(const mrl_ctx* ctx, uint64_t family, uint32_t* stage, uint32_t* owner, uint32_t* spec_lo,
                    uint32_t* spec_hi);
int mrl_spec_owners(const mrl_ctx* ctx, uint8_t* out, uint64_t n); /* rank that computes each Spec; n = mrl_num_specs */
int mrl_device_rows(const mrl_ctx* ctx, void** ptr, uint64_t* n_rows); /* the finished table on the device */
uint32_t mrl_row_bytes(void); /* bytes per row of the device table */
int mrl_fill_begin(mrl_ctx* ctx);
int mrl_fill_stage_solve(mrl_ctx* ctx, uint64_t stage, void** masks, uint64_t* mask_bytes);
int mrl_fill_stage_place(mrl_ctx* ctx, uint64_t stage, void** rows, uint64_t* row_bytes);
int mrl_fill_end(mrl_ctx* ctx);

/* Replaces FilesDatabase::get (morello/src/db/mod.rs:481-503, 538-573): point lookups in the
 * filled tables; found = -1 for Specs outside the tables. */
int mrl_get_many(mrl_ctx* ctx, const uint8_t* blobs, const uint64_t* blob_off, size_t n, const uint64_t* limits,
                 mrl_decision* out);

/* Replaces FilesDatabase::get_impl (morello/src/db/mod.rs:505-516; morello/src/reconstruct.rs:14-80)
 * as called from frontend/src/main.rs:299-304: re-applies, from the given Spec down, the action the
 * tables store for each (Spec, limits) and writes the resulting tree as text, one line per node:
 *   <2 spaces per level><Spec> @ [rf, vrf, l1, gl]: #<action> <what> cost <main> peaks [..] depth <d>
 * Returns the text length (NUL not counted) or a negative status (-3: `cap` too small). */
long mrl_get_impl(mrl_ctx* ctx, const uint8_t* blob, size_t len, const uint64_t limits[4], char* out, size_t cap);

/* Self-check of the filled tables, no counterpart in the reference (its closest relative is the
 * proptest that synthesis at peak memory yields the same decision, morello/src/search/mod.rs:152-199):
 * at n_samples pseudo-random points of (Spec x limits lattice) - every point when n_samples is 0 -
 * the decision recomputed on the GPU from the children's tables (morello/src/scheduling/mod.rs:286-368)
 * must equal what the Spec's own table returns there. n_mismatch == 0 means the tables satisfy the
 * recurrence that defines the database at every checked point. */
int mrl_verify(mrl_ctx* ctx, uint64_t n_samples, uint64_t seed, uint64_t* n_checked, uint64_t* n_mismatch);

/* 64-bit checksum of the filled tables, no counterpart in the reference: a sum over all Specs of a
 * hash of (Spec id, breakpoint masks, rows in cell order). Independent of where rows lie in device
 * memory, so a sharded fill and a single-GPU fill of one plan must agree. */
int mrl_checksum(mrl_ctx* ctx, uint64_t* out);

int mrl_get_stats(const mrl_ctx* ctx, mrl_stats* out);

/* Table export (the data a FilesDatabase::put stream would have produced,
 * morello/src/db/mod.rs:637-766): number of Specs, a Spec's blob, its lattice breakpoint masks
 * and its dense cell block (n0*n1*n2*n3 decisions, RF index fastest). */
uint64_t mrl_num_specs(const mrl_ctx* ctx);
int mrl_spec_blob(const mrl_ctx* ctx, uint64_t spec_id, uint8_t* out, size_t cap);
int mrl_spec_grid(mrl_ctx* ctx, uint64_t spec_id, uint32_t masks[4], uint64_t* n_cells);
int mrl_export_rows(mrl_ctx* ctx, uint64_t spec_id, mrl_decision* out, size_t cap);
/* The whole table in two device-to-host copies: per Spec its four masks (masks, 4 * n_specs words)
 * and the index of its first row (first_row, n_specs + 1 entries), and all rows (rows, n_rows
 * entries: mrl_get_stats.n_rows). mrl_decode_row turns a row into a decision. */
int mrl_export_all(mrl_ctx* ctx, uint32_t* masks, uint64_t* first_row, mrl_row* rows, uint64_t rows_cap);
void mrl_decode_row(const mrl_row* row, mrl_decision* out);
/* The reference's logical table contents for one Spec (what FilesDatabase::put leaves behind,
 * morello/src/db/mod.rs:650-766, morello/src/db/pagecontents.rs:125-184): rectangles over the four
 * limit dimensions, each with one decision. Neighbouring cells of the Spec's grid with equal
 * decisions are merged along RF, then VRF, L1, GL. lo / hi: 4 lattice codes per rectangle,
 * inclusive. Returns the number of rectangles (-3: cap too small). */
long mrl_export_rects(mrl_ctx* ctx, uint64_t spec_id, uint8_t* lo, uint8_t* hi, mrl_decision* out, size_t cap);

/* Replaces FilesDatabase::save (morello/src/db/mod.rs:769-775) and the reopening of a database
 * directory (FilesDatabase::new on an existing path, :350-380, with its TARGET / TILESCALE guards,
 * :2091-2153). One file: target and tile-scale tags, the top limits, every Spec blob, the masks
 * and rows. Written to `path`.tmp and renamed. mrl_load checks tags, sizes and a checksum of the
 * contents and answers lookups afterwards; when the context already holds the plan of the same job
 * (same Specs in the same order) its candidate records stay usable (mrl_verify, mrl_fill).
 * Status -7: not a database of this library / target; -8: truncated or corrupt. */
int mrl_save(mrl_ctx* ctx, const char* path);
int mrl_load(mrl_ctx* ctx, const char* path);

/* FilesDatabase::put (morello/src/db/mod.rs:637-766) has no writing counterpart here: every cell of
 * these tables is a direct solve from the children's cells, so a decision from elsewhere cannot be
 * stored without breaking that. What the reference debug-asserts on overlapping puts (equal cost,
 * morello/src/db/pagecontents.rs:194-198) is what this checks: 0 when the tables hold exactly this
 * decision at (Spec, limits), -9 when they hold another one, -3 when the Spec is not in the tables. */
int mrl_put(mrl_ctx* ctx, const uint8_t* blob, size_t len, const uint64_t limits[4], const mrl_decision* decision);

#ifdef __cplusplus
}
#endif
#endif /* MORELLO_B200_H */

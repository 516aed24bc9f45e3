// Plain-data records shared by the host planner and the CUDA fill kernels.
//
// Limits lattice: one integer "code" per memory, in the reference's own database
// coordinates (MemoryLimitsBimap, morello/src/memorylimits.rs:696-734): registers (RF, VRF)
// use the raw count, caches (L1, GL) use the bit length of the line count (0 -> 0,
// 2^(c-1) lines -> c).
#pragma once
#include <stdint.h>

// One table row = the optimum of one (logical Spec, limits cell): the reference's
// (ActionNum, Cost{main, peaks, depth}) (morello/src/db/mod.rs:54,171; morello/src/cost.rs:13-17).
// Compared as the 96-bit big-endian number (main, peaks, tail) it orders exactly like
// (Cost, ActionNum) (morello/src/cost.rs:87-104, morello/src/search/reducer.rs:41-48);
// an unsatisfiable cell is all ones, which sorts after everything.
struct MrlRow {
  uint32_t main;   // saturating u32 main cost
  uint32_t peaks;  // RF<<24 | VRF<<16 | L1 code<<8 | GL code   (peak memory, as lattice codes)
  uint32_t tail;   // depth<<16 | action number; 0xFFFFFFFF = no implementation
  uint32_t aux;    // finished table: 0. Working rows of the stage being solved: index of the winning
                   // candidate record within its Spec (0xFFFFFFFF when there is none).
                   // 12 bytes of payload in a 16-byte slot: one aligned vector load per gather.
};
#define MRL_UNSAT 0xFFFFFFFFu

// Per logical Spec: breakpoint masks of its limits grid (bit c set = code c starts a new
// cell; bit 0 always set), the first row of its dense cell block and its candidates.
// Cell (i0,i1,i2,i3) has row ((i3*n2 + i2)*n1 + i1)*n0 + i0 with n_k = popcount(mask[k]).
// While a stage is being solved its Specs point at a working grid in the working-row buffer;
// once the stage is consistent they point at the compacted final grid.
struct SpecHdr {
  uint32_t mask[4];
  uint64_t row_base;
  uint32_t cand_off;
  uint32_t ncand;
};

enum { MRL_CK_LEAF = 0, MRL_CK_LOOP = 1, MRL_CK_MOVE = 2, MRL_CK_BLOCK = 3 };

// One applicable action of a Spec, reduced to what the limits-dependent combine needs
// (morello/src/scheduling/mod.rs:286-368).
struct CandRec {
  uint16_t action;   // ActionNum in the reference's enumeration order
  uint8_t kind;      // MRL_CK_*
  uint8_t nchild;    // 0..3
  uint32_t imm;      // LEAF: kernel main cost; LOOP: iterations; MOVE: base move cost
  uint8_t level;     // memory the action allocates in (MOVE, LEAF)
  uint8_t thr_code;  // smallest limit code in `level` at which the action applies
  uint8_t peak_code; // LEAF: the kernel's own peak in `level`, as a code
  uint8_t late;      // 1: a child lies in the Spec's own stage (a relayout Move); such records come last
  uint32_t units;    // MOVE: units consumed in `level` (registers or cache lines)
  uint32_t child[3]; // Spec ids, in request order
  uint32_t pad1;
};

// A warp-sized slice of one Spec's "columns": cells with the slot of one memory (the Spec's
// free memory F, the one with the most slots) left open; the column index runs over the other
// three memories, lowest first. col_start = first column | F << 30.
struct Chunk {
  uint32_t spec;
  uint32_t col_start;
};

// A piece of one Spec's grid for a solve phase: consecutive cells from
// first_cell on, at most MRL_ITEM_CELLS of them (a pass picks the size). Warps take items as they
// finish others.
#define MRL_ITEM_CELLS 1024u
struct WorkItem {
  uint32_t spec;
  uint32_t first_cell;
};

// Error bits a fill kernel can raise (sticky until the host clears them).
enum {
  MRL_ERR_CHILD = 1,      // a candidate record names a Spec id outside the plan
  MRL_ERR_WORKING = 2,    // a working buffer (rows, chunks, work items) is too small
  MRL_ERR_TABLE = 4,      // the row table is too small
  MRL_ERR_PASSES = 8,     // a stage did not reach a consistent limits grid
};

// Parts of a stage kernel whose device time is accounted separately.
enum {
  MRL_PH_SETUP = 0,       // corners, grids of the unordered phase, their placement
  MRL_PH_EARLY = 1,       // the unordered phase
  MRL_PH_EARLY_MASKS = 2, // real breakpoints of its result
  MRL_PH_PASS_SETUP = 3,  // per pass: working grids, marks, placement
  MRL_PH_INIT = 4,        // per pass: cells start from the unordered phase's result
  MRL_PH_SWEEP_FIRST = 5, // per pass: the first relaxation sweep
  MRL_PH_SWEEP_MORE = 6,  // per pass: the sweeps after it
  MRL_PH_PASS_MASKS = 7,  // per pass: real breakpoints of the working grids
};

// Control block of a fill, in device memory. The stage kernels read their sizes and cursors
// here and leave the host nothing to decide between launches; the host reads it once per fill
// (once per stage when the fill is sharded).
struct FillCtl {
  // -- one solve pass (zeroed by the kernel before every pass)
  unsigned long long cells;          // working cells of the Specs solved in this pass
  unsigned long long warps;          // chunks those cells need
  unsigned long long row_cursor;     // placement cursors of the pass
  uint32_t chunk_cursor;
  uint32_t item_cursor;
  uint32_t item_next;                // next work item to hand out
  uint32_t spread_epoch;             // closure of the re-solve marks: last round that marked a Spec
  uint32_t sweep_next[2];            // work hand-out of the relaxation sweeps, alternating
  uint32_t late_changed;             // last relaxation sweep that improved a cell
  uint32_t pad0;
  // -- one stage
  unsigned long long temp_top;       // working rows handed out so far in this stage
  // -- sticky over a fill
  uint32_t error;                    // MRL_ERR_* bits
  uint32_t failed_stage;             // first stage that raised one
  unsigned long long need_temp, need_chunks, need_items, need_rows;   // what it would have taken
  unsigned long long final_top;      // rows of the finished table
  unsigned long long stage_first_row, stage_rows;   // the last placed stage's slice of the table
  // -- statistics of a fill
  unsigned long long st_cells;       // working cells solved, all passes
  unsigned long long st_cands;       // candidate records evaluated
  unsigned long long st_lookups;     // child rows gathered
  unsigned long long st_passes;
  unsigned long long st_final_bytes; // algorithmic bytes of the finished rows (see fill.hpp)
  unsigned long long st_syncs;       // grid-wide barriers executed
  unsigned long long st_sweeps;      // relaxation sweeps, all passes
  unsigned long long st_early_cells; // of st_cells: cells of the grids of the unordered phase
  unsigned long long st_late_cands;  // of st_cands: evaluated by the sweeps
  unsigned long long st_late_items;  // work items the sweeps evaluated
  unsigned long long st_phase_ns[8]; // device time by part of the stage kernel (see MRL_PH_*)
  // -- scratch of verify and checksum
  unsigned long long scratch[4];
};

#ifdef __cplusplus
static_assert(sizeof(MrlRow) == 16, "row slot is 16 bytes");
static_assert(sizeof(SpecHdr) == 32, "spec header is 32 bytes");
static_assert(sizeof(CandRec) == 32, "candidate record is 32 bytes");
static_assert(sizeof(FillCtl) % 8 == 0 && sizeof(FillCtl) <= 512, "control block");
#endif

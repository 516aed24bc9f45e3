// Plain-data records shared by the host planner and the CUDA combine kernel.
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
  uint32_t pad;    // 12 bytes of payload kept in a 16-byte slot: one aligned vector load per gather
};
#define MRL_UNSAT 0xFFFFFFFFu

// Per logical Spec: breakpoint masks of its limits grid (bit c set = code c starts a new
// cell; bit 0 always set), the first row of its dense cell block and its candidates.
// Cell (i0,i1,i2,i3) has row ((i3*n2 + i2)*n1 + i1)*n0 + i0 with n_k = popcount(mask[k]).
// While a stage is being solved its Specs point at a working grid in the scratch end of the
// row arena; once the stage is consistent they point at the compacted final grid.
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
  uint8_t pad0;
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

// Counters one solve pass of a stage leaves for the host (zeroed before every pass).
struct PassCounters {
  uint32_t changed;             // a Spec was marked for solving by totals_kernel itself (marks were not closed)
  uint32_t n_chunks;            // chunk cursor (place kernel)
  unsigned long long cells;     // working cells of the Specs to solve in this pass
  unsigned long long warps;     // chunks those cells need
  unsigned long long temp_rows; // row cursor (place kernel)
  unsigned long long alg_bytes; // algorithmic bytes of one solve of those cells
  unsigned long long all_cells; // working cells of all the stage's Specs under the current masks
  uint32_t pad0[2];
  uint32_t error;               // bad child index / capacity overrun seen by a kernel (sticky over a fill)
  uint32_t pad;
};

// Per limits diagonal (sum of the four codes, < 128) of the stage being solved: how many working
// cells lie on it, and where their descriptors start in the cell list.
#define MRL_MAX_DIAG 128
struct DiagTable {
  uint32_t count[MRL_MAX_DIAG];
  uint32_t cursor[MRL_MAX_DIAG];
  unsigned long long base[MRL_MAX_DIAG];
};

// One working cell: Spec id and the cell's limits as lattice codes, one per byte (RF in byte 0
// .. GL in byte 3). Its place in the Spec's working grid follows from the masks by popcounts.
struct CellRef {
  uint32_t spec;
  uint32_t cpack;
};

#ifdef __cplusplus
static_assert(sizeof(MrlRow) == 16, "row slot is 16 bytes");
static_assert(sizeof(SpecHdr) == 32, "spec header is 32 bytes");
static_assert(sizeof(CandRec) == 32, "candidate record is 32 bytes");
static_assert(sizeof(PassCounters) == 64, "pass counters are 64 bytes");
#endif

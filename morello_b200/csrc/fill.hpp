// Device side of the fill: owns the device copies of a Plan and the row arena, and runs the
// stages. Callers hand in host data only.
#pragma once
#include "plan.hpp"
#include <cuda_runtime.h>
#include <atomic>
#include <memory>
#include <mutex>
#include <thread>

namespace mrl {

struct FillStats {
  uint64_t n_rows = 0;          // final table rows
  uint64_t cells_solved = 0;    // working-grid cells solved, all passes
  uint64_t alg_bytes = 0;       // algorithmic bytes of those solves
  uint64_t passes = 0;          // solve passes over all stages
  uint64_t launches = 0;        // kernel launches
  uint64_t combine_launches = 0;
  float fill_ms = 0;            // device time of the whole fill (CUDA events on the launch stream)
  float combine_ms = 0;         // device time inside the combine launches only
};

class DeviceFill {
 public:
  ~DeviceFill();
  int init(int device);
  int init_events();   // the part of init a caller with its own stream and buffer needs
  // Memory from cudaMalloc (the default), or carved out of one caller-supplied device buffer
  // that is never grown or freed (attach_buffer before upload).
  void attach_buffer(void* base, size_t bytes, cudaStream_t stream, int device);
  // Copies headers and candidate records to the device and sets up the arena.
  // Gigabytes of candidate records keep going up in the background, in id order, after upload()
  // has returned: the plan must stay as it is until wait_upload() (a fill waits stage by stage
  // for the records it is about to read, so its first stages overlap the copy).
  // skip_cands: the candidate records are not on this host; the caller fills device_cands()
  // itself (e.g. a broadcast from the rank that planned) before the first fill.
  int upload(const Plan& plan, bool skip_cands = false);
  // Blocks until every candidate record is on the device.
  int wait_upload();
  void* device_cands() const { return d_cands_; }
  uint64_t device_cand_bytes() const { return n_cand_bytes_; }
  // Runs every stage.
  int run(const Plan& plan);
  // The same one stage at a time, for callers that exchange tables between stages (multi-GPU):
  // begin_fill; per stage solve_stage, [exchange stage_masks], place_stage, [exchange rows];
  // end_fill. All work is enqueued on the stream; solve_stage and place_stage synchronise it.
  int begin_fill();
  int solve_stage(const Plan& plan, uint32_t stage);
  int stage_masks(const Plan& plan, uint32_t stage, void** ptr, uint64_t* bytes);
  int place_stage(const Plan& plan, uint32_t stage, void** rows_ptr, uint64_t* bytes);
  int end_fill();
  // Run on a caller-owned stream (e.g. the one a collective library orders against).
  int set_stream(cudaStream_t s);
  // Point lookups: rows of (Spec id, packed limit codes).
  int lookup(const uint32_t* spec_ids, const uint32_t* cpacks, size_t n, MrlRow* out);
  int verify(const Plan& plan, uint64_t n_samples, uint64_t seed, uint64_t* checked, uint64_t* mismatches,
             uint64_t* first_bad);
  int read_hdr(uint32_t spec, SpecHdr* out);
  int read_rows(uint64_t first, uint64_t n, MrlRow* out);
  void release();
  const char* error() const { return err_; }
  const FillStats& stats() const { return stats_; }
  uint64_t h2d_bytes() const { return h2d_bytes_; }
  MrlRow* device_rows() const { return d_rows_; }
  cudaStream_t stream() const { return stream_; }
  int device() const { return device_; }

 private:
  int alloc_(void** p, size_t bytes);
  void free_(void* p);
  int ensure_rows_(uint64_t need, bool refresh);
  int ensure_temp_(uint64_t need, uint64_t keep);
  int ensure_chunks_(uint64_t need);
  int ensure_cells_(uint64_t need);
  int read_counters_(PassCounters* out);
  int wait_cands_(uint64_t upto_bytes);   // until the candidate bytes [0, upto_bytes) are on the device

  int device_ = 0;
  bool fixed_ = false;            // carved from an attached buffer: no growth
  unsigned char* buf_ = nullptr;  // attached buffer
  size_t buf_bytes_ = 0, buf_off_ = 0;
  SpecHdr* d_hdrs_ = nullptr;
  CandRec* d_cands_ = nullptr;
  uint4* d_rmask_ = nullptr;
  uint8_t* d_mine_ = nullptr;
  uint8_t* d_dirty_ = nullptr;   // by Spec id: to be solved (again) in the coming pass
  Chunk* d_chunks_ = nullptr;
  CellRef* d_cells_ = nullptr;   // working cells of the pass, listed diagonal by diagonal
  DiagTable* d_diag_ = nullptr;
  DiagTable* h_diag_ = nullptr;  // pinned
  DiagTable diag_pageable_;      // used instead when nothing may be allocated
  MrlRow* d_rows_ = nullptr;   // the table
  MrlRow* d_temp_ = nullptr;   // working grids of the stage being solved
  uint32_t* d_fcount_ = nullptr;
  unsigned long long* d_block_sums_ = nullptr;
  PassCounters* d_ctr_ = nullptr;       // [0]: pass counters; then final_top, stage_info[2]
  unsigned long long* d_final_top_ = nullptr;
  unsigned long long* d_stage_info_ = nullptr;
  void* d_stage_ = nullptr;             // lookup staging
  size_t stage_bytes_ = 0;
  PassCounters* h_ctr_ = nullptr;       // pinned
  uint32_t n_specs_ = 0;
  uint64_t row_cap_ = 0, temp_cap_ = 0, chunk_cap_ = 0, cell_cap_ = 0;
  uint64_t final_bound_ = 0;            // upper bound of the final rows placed so far
  unsigned long long final_top_seen_ = 0, stage_info_seen_[2] = {0, 0};  // last values read back
  uint64_t last_cells_ = 0;             // working cells of the last pass of the stage being solved
  uint64_t h2d_bytes_ = 0;
  uint64_t n_cand_bytes_ = 0;
  bool filling_ = false;
  // Before the first solve of a stage a Spec's working masks also take the first masks of its
  // same-stage children (shifted), this many hops deep: one hop saves a third of the solve
  // passes at size 8 for 9 % more cells; two hops cost more cells than they save. MRL_SEED_HOPS
  // overrides (0..8); any value gives the same tables.
  int seed_hops_ = 1;
  uint32_t profile_min_cells_ = 0;      // MRL_PROFILE_MIN_CELLS
  bool stage_log_ = false;              // MRL_STAGE_LOG: one line per solve pass on stderr
  FillStats stats_;
  cudaStream_t stream_ = nullptr;
  bool own_stream_ = false;
  cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
  std::vector<cudaEvent_t> ev_pool_;
  size_t ev_used_ = 0;
  std::mutex lookup_mu_;
  // background candidate upload: pieces handed out in order to a few copying threads
  std::vector<std::thread> up_threads_;
  std::unique_ptr<std::atomic<uint8_t>[]> up_done_;   // by piece
  std::atomic<size_t> up_next_{0};
  std::atomic<int> up_err_{0};                        // cudaError_t of the first failed copy
  size_t up_pieces_ = 0, up_piece_bytes_ = 0, up_ready_ = 0;   // up_ready_: pieces known complete, a prefix
  char err_[256] = {0};
};

// Size of the fixed device array behind the no-allocation entry point (32 MiB per GPU).
#define MRL_STATIC_SCRATCH_BYTES (32u << 20)

// One whole small fill inside the fixed device array: plan arrays, row arena and lookup
// staging; no device allocation. See combine.cu.
int fill_static(int device, cudaStream_t stream, const Plan& plan, const uint32_t* spec_ids, const uint32_t* cpacks,
                size_t n, MrlRow* out, char* err, size_t err_len);

}  // namespace mrl

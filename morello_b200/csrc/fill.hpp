// Device side of the fill: owns the device copies of a Plan and the row table, and runs the
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
  uint64_t cands_evaluated = 0; // candidate records evaluated
  uint64_t lookups = 0;         // child rows gathered
  // Algorithmic bytes of the finished table: per final row 12 bytes out, 16 per candidate record
  // of its Spec and 16 (index + row) per child of every candidate that fits the row's limits.
  // Working cells that do not survive compaction do not count.
  uint64_t alg_bytes = 0;
  uint64_t passes = 0;          // solve passes over all stages
  uint64_t launches = 0;        // kernel launches
  uint64_t early_cells = 0;     // of cells_solved: cells of the grids of the unordered phase
  uint64_t late_cands = 0;      // of cands_evaluated: by the relaxation sweeps
  uint64_t late_items = 0;      // work items the sweeps evaluated
  uint64_t growths = 0;         // times a buffer had to be enlarged (the stage that asked is solved again)
  uint64_t sweeps = 0;          // relaxation sweeps of the candidates with a same-stage child
  uint64_t grid_syncs = 0;      // grid-wide barriers inside the stage kernels
  float fill_ms = 0;            // device time of the whole fill (CUDA events on the launch stream)
  float combine_ms = 0;         // device time inside the solve phases (device timer)
  float early_ms = 0;           // of which the unordered phase
  float phase_ms[8] = {};       // device time by part of the stage kernels (MRL_PH_*)
};

class DeviceFill {
 public:
  ~DeviceFill();
  int init(int device);
  int init_events();   // the part of init a caller with its own stream and buffer needs
  // Memory from cudaMalloc (the default), or carved out of one caller-supplied device buffer
  // that is never grown or freed (attach_buffer before upload).
  void attach_buffer(void* base, size_t bytes, cudaStream_t stream, int device);
  // Copies headers and candidate records to the device and sets up the buffers.
  // Gigabytes of candidate records keep going up in the background, in id order, after upload()
  // has returned: the plan must stay as it is until wait_upload() (a fill waits stage by stage
  // for the records it is about to read, so its first stages overlap the copy).
  // skip_cands: the candidate records are not on this host; the caller fills device_cands()
  // itself (e.g. a broadcast from the rank that planned) and then calls cands_arrived().
  int upload(const Plan& plan, bool skip_cands = false);
  // Blocks until every candidate record is on the device.
  int wait_upload();
  void* device_cands() const { return d_cands_; }
  uint64_t device_cand_bytes() const { return n_cand_bytes_; }
  // After the caller has written device_cands(): checks every record on the device (child ids
  // inside the plan, kinds and levels in range) and lets fills run.
  int cands_arrived();
  // Runs every stage: two launches per stage, no host synchronisation before the end.
  int run(const Plan& plan);
  // The same one stage at a time, for callers that exchange tables between stages (multi-GPU):
  // begin_fill; per stage solve_stage, [exchange stage_masks], place_stage, [exchange rows];
  // end_fill. All work is enqueued on the stream; place_stage synchronises it once.
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
  // Order-independent 64-bit checksum of the logical table: per Spec its id, masks and rows in
  // cell order; where the rows lie in the table does not enter.
  int checksum(uint64_t* out);
  // The whole finished table in two copies: headers (masks, first row) and rows.
  int read_table(SpecHdr* hdrs_out, MrlRow* rows_out);
  // Replaces the table by a saved one (hdrs as read_table gave them).
  int load_table(const Plan& plan, const SpecHdr* hdrs, const MrlRow* rows, uint64_t n_rows);
  int read_hdr(uint32_t spec, SpecHdr* out);
  int read_rows(uint64_t first, uint64_t n, MrlRow* out);
  void release();
  const char* error() const { return err_; }
  const FillStats& stats() const { return stats_; }
  uint64_t h2d_bytes() const { return h2d_bytes_; }
  MrlRow* device_rows() const { return d_rows_; }
  cudaStream_t stream() const { return stream_; }
  int device() const { return device_; }
  uint32_t n_specs() const { return n_specs_; }

 private:
  int alloc_(void** p, size_t bytes);
  void free_(void* p);
  int launch_solve_(const Plan& plan, uint32_t stage, bool place_too);
  int launch_place_(const Plan& plan, uint32_t stage);
  int read_ctl_();                       // device control block -> h_ctl_ (synchronises the stream)
  int grow_after_error_(uint32_t bits);  // enlarges the buffers a failed stage asked for
  int wait_cands_(uint64_t upto_bytes);  // until the candidate bytes [0, upto_bytes) are on the device
  void take_stats_();
  int too_large_();

  int device_ = 0;
  bool fixed_ = false;            // carved from an attached buffer: no growth
  unsigned char* buf_ = nullptr;  // attached buffer
  size_t buf_bytes_ = 0, buf_off_ = 0;
  SpecHdr* d_hdrs_ = nullptr;
  CandRec* d_cands_ = nullptr;
  uint4* d_rmask_ = nullptr;
  uint8_t* d_mine_ = nullptr;
  uint8_t* d_dirty_ = nullptr;   // by Spec id: to be solved (again) in the coming pass
  uint32_t* d_minsat_ = nullptr; // by Spec id: lower corner of the satisfiable region
  SpecHdr* d_ehdr_ = nullptr;    // by position in the stage being solved: the Spec's grid of the unordered phase
  uint32_t* d_stamp_ = nullptr;  // by position in the stage being solved: last relaxation sweep that improved the Spec
  uint32_t* d_corner_ = nullptr; // by position in the stage being solved: where its working grids are clipped
  Chunk* d_chunks_ = nullptr;
  WorkItem* d_items_ = nullptr;  // pieces of grids, handed out to warps by the solve phases
  MrlRow* d_rows_ = nullptr;     // the table
  MrlRow* d_temp_ = nullptr;     // working grids of the stage being solved (temp_cap_ rows), then as many rows for the grids of the unordered phase
  uint32_t* d_fcount_ = nullptr;
  unsigned long long* d_block_sums_ = nullptr;
  FillCtl* d_ctl_ = nullptr;
  void* d_stage_ = nullptr;      // lookup staging
  size_t stage_bytes_ = 0;
  FillCtl* h_ctl_ = nullptr;     // pinned, or &ctl_pageable_ when nothing may be allocated
  FillCtl ctl_pageable_;
  uint32_t n_specs_ = 0, max_stage_ = 1;
  uint64_t row_cap_ = 0, temp_cap_ = 0, chunk_cap_ = 0, item_cap_ = 0;
  uint64_t h2d_bytes_ = 0;
  uint64_t n_cand_bytes_ = 0;
  bool cands_present_ = false;   // the device candidate records are complete and checked
  bool filling_ = false;
  int coop_blocks_ = 0;          // co-resident blocks of the stage kernel on this device
  int n_sm_ = 0;
  FillStats stats_;
  cudaStream_t stream_ = nullptr;
  bool own_stream_ = false;
  cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
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

// One whole small fill inside the fixed device array: plan arrays, working buffers, row table
// and lookup staging; no device allocation. See combine.cu.
int fill_static(int device, cudaStream_t stream, const Plan& plan, const uint32_t* spec_ids, const uint32_t* cpacks,
                size_t n, MrlRow* out, char* err, size_t err_len);

}  // namespace mrl

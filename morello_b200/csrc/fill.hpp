// Device side of the fill: owns the device copies of a Plan and the row table, and runs
// the launch schedule. All device memory is allocated here with cudaMalloc; callers hand
// in host data only.
#pragma once
#include "plan.hpp"
#include <cuda_runtime.h>

namespace mrl {

class DeviceFill {
 public:
  ~DeviceFill();
  int init(int device);
  // Copies headers, candidate records and chunk lists to the device and allocates the rows.
  int upload(const Plan& plan);
  // Runs every (group, diagonal) step. ms_out: device time of the whole schedule, measured
  // with CUDA events on the launching stream.
  int run(const Plan& plan, float* ms_out, uint64_t* launches_out);
  // The same schedule one group at a time, for callers that exchange rows between groups
  // (multi-GPU): begin_fill, then run_group for every group in order with the exchange in
  // between on the same stream, then end_fill.
  int begin_fill();
  int run_group(const Plan& plan, uint32_t group);
  int end_fill(float* ms_out, uint64_t* launches_out);
  // Run on a caller-owned stream (e.g. the one a collective library orders against).
  int set_stream(cudaStream_t s);
  // Largest peak (lattice code) per memory over the filled table: the check that a compressed
  // lattice lost nothing (every peak must stay at or below its memory's cap).
  int max_peaks(uint32_t out[4]);
  int read_rows(const uint64_t* row_idx, size_t n, MrlRow* out);
  int download(std::vector<MrlRow>& out);
  void release();
  const char* error() const { return err_; }
  uint64_t n_rows() const { return n_rows_; }
  uint64_t h2d_bytes() const { return h2d_bytes_; }
  MrlRow* device_rows() const { return d_rows_; }
  cudaStream_t stream() const { return stream_; }
  int device() const { return device_; }

 private:
  int device_ = 0;
  SpecHdr* d_hdrs_ = nullptr;
  CandRec* d_cands_ = nullptr;
  Chunk* d_chunks_ = nullptr;
  MrlRow* d_rows_ = nullptr;
  int* d_err_ = nullptr;
  uint32_t* d_peaks_ = nullptr;
  uint32_t n_specs_ = 0;
  uint64_t n_rows_ = 0;
  uint64_t h2d_bytes_ = 0;
  uint64_t launches_ = 0;
  cudaStream_t stream_ = nullptr;
  bool own_stream_ = false;
  cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
  char err_[256] = {0};
};

// Size of the fixed device array behind the no-allocation entry point (32 MiB per GPU).
#define MRL_STATIC_SCRATCH_BYTES (32u << 20)

// One whole small fill inside the fixed device array: plan arrays, row table and lookup
// staging; no device allocation. See combine.cu.
int fill_static(int device, cudaStream_t stream, const Plan& plan, const uint64_t* row_idx, size_t n, MrlRow* out,
                char* err, size_t err_len);

}  // namespace mrl

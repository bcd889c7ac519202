// Tensor-parallel communicator: one symmetric device buffer per rank, mapped into every peer through CUDA IPC,
// and an all-reduce kernel that sums over plain peer loads (no multicast, no library collective).
//
// The reference has no multi-GPU path; this is the exchange step of the tensor-parallel Llama plan: the partial
// products of the row-sharded o_proj / down_proj (llama.rs:303-347, 349-385 split over heads / FFN columns) are
// summed across ranks and added to the residual stream.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "tensor.h"

struct cg_ctx;

namespace cg {
constexpr int TP_MAX_RANKS = 8;
constexpr size_t TP_HEADER_BYTES = 4096;  // flag words in front of the data area
}  // namespace cg

struct cg_comm {
  cg_ctx* ctx = nullptr;
  int rank = 0, size = 1, device = 0;
  size_t data_bytes = 0;                  // bytes after the header
  unsigned char* local = nullptr;         // cudaMalloc'd: header + data
  unsigned char* peer[cg::TP_MAX_RANKS];  // base of every rank's buffer in this process (peer[rank] == local)
  bool attached = false;
  bool local_peers = false;               // peers are buffers of this process (no IPC mapping to close)
  uint64_t wait_ms = 5000;                // limit of every device-side wait
  cudaIpcMemHandle_t handle;

  unsigned char* data() const { return local + cg::TP_HEADER_BYTES; }
  // x[0:n] (+)= sum over ranks of part[0:n]; both are byte offsets into the data area, the same on every rank.
  // residual: x = round(x + round(sum)); otherwise x = round(sum).  Enqueued on `st`; waits are bounded and report
  // through the device error word `err`.
  void allreduce(cg::Dtype dt, size_t x_off, size_t part_off, int64_t n, bool residual, int sm_count, cudaStream_t st,
                 unsigned* err);
};

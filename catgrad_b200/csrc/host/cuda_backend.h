// The CUDA implementation of cg::Backend: device tensors, a caching allocator, one stream.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <mutex>
#include <vector>

#include "../kernels/common.cuh"
#include "backend.h"

namespace cg {

#define CG_CUDA(call)                                                                                      \
  do {                                                                                                     \
    cudaError_t e_ = (call);                                                                               \
    if (e_ != cudaSuccess)                                                                                 \
      throw ::cg::Error(e_ == cudaErrorMemoryAllocation ? ::cg::ERR_OOM : ::cg::ERR_CUDA,                  \
                        std::string(#call) + ": " + cudaGetErrorString(e_));                               \
  } while (0)

// Size-bucketed caching allocator.  All work of a context runs on one stream, so a block freed by the host
// can be handed out again at once: the next kernel that writes it is ordered after the last one that read it.
// Blocks are returned from any thread (tensor handles may be released anywhere), hence the mutex.
class CachingAllocator {
 public:
  explicit CachingAllocator(int device);
  ~CachingAllocator();
  void* alloc(size_t bytes);
  void free(void* p, size_t bytes);
  void trim();  // cudaFree everything cached
  // Refuses allocations that would take live+cached bytes above `cap` (0 = no cap).  Host-side fault
  // injection for out-of-memory handling; also settable with the environment variable CATGRAD_B200_MEM_CAP.
  void set_cap(size_t cap) { cap_ = cap; }
  size_t live_bytes() const { return live_; }
  size_t cached_bytes() const { return cached_; }
  size_t cuda_mallocs() const { return mallocs_; }
  static size_t round_size(size_t bytes);

 private:
  int device_;
  std::mutex mu_;
  std::map<size_t, std::vector<void*>> free_;
  size_t live_ = 0, cached_ = 0, mallocs_ = 0, cap_ = 0;
};

class CudaBackend : public Backend {
 public:
  explicit CudaBackend(int device);
  ~CudaBackend() override;
  const char* name() const override { return "b200"; }

  Tensor zeros(const Shape& shape, Dtype dt) override;
  Tensor from_vec(const void* data, int64_t n, const Shape& shape, Dtype dt) override;
  Tensor arange(int64_t end) override;
  Tensor cast(const Tensor& x, Dtype target) override;
  Tensor matmul(const Tensor& a, const Tensor& b) override;
  Tensor binary(BinOp op, const Tensor& a, const Tensor& b) override;
  Tensor where_cond(const Tensor& mask, const Tensor& x, const Tensor& y) override;
  Tensor unary(UnOp op, const Tensor& x) override;
  Tensor broadcast(const Tensor& x, const Shape& shape) override;
  Tensor reshape(const Tensor& x, const Shape& shape) override;
  Tensor transpose(const Tensor& x, int64_t d0, int64_t d1) override;
  Tensor max(const Tensor& x) override;
  Tensor sum(const Tensor& x) override;
  Tensor argmax(const Tensor& x) override;
  std::pair<Tensor, Tensor> topk(const Tensor& x, int64_t k) override;
  bool compare(const Tensor& a, const Tensor& b) override;
  Tensor concat(const Tensor& a, const Tensor& b, int64_t dim) override;
  Tensor index(const Tensor& x, int64_t dim, const Tensor& indices) override;
  Tensor slice(const Tensor& x, int64_t dim, int64_t start, int64_t len) override;
  bool to_bool(const Tensor& x) override;
  void to_vec(const Tensor& x, void* dst, size_t cap_bytes) override;
  void synchronize() override;

  // ---- used by the fused runner and the timing entry points ----
  void guard() const;  // makes this context's device current
  Tensor empty(const Shape& shape, Dtype dt);
  Tensor contiguous(const Tensor& x);
  Tensor softmax(const Tensor& x);   // not in the trait: stdlib nn::softmax (nn/mod.rs:168-179) fused, last axis
  void check_launch(const char* what);
  void check_device_errors();  // reads the sticky error word; call only at synchronising points
  cudaStream_t stream() const { return stream_; }
  int sm_count() const { return sm_count_; }
  int device() const { return device_; }
  unsigned* dev_err() const { return dev_words_; }
  CachingAllocator& allocator() { return *alloc_; }
  cudaEvent_t event(int slot);
  uint64_t launches = 0;

 private:
  Tensor reduce(int kind, const Tensor& x);
  void copy_into(const Tensor& src, const Tensor& dst_view);
  unsigned read_flag_and_clear();

  int device_;
  int sm_count_ = 148;
  cudaStream_t stream_ = nullptr;
  std::shared_ptr<CachingAllocator> alloc_;
  unsigned* dev_words_ = nullptr;   // [0] sticky error bits, [1] predicate flag
  unsigned* host_words_ = nullptr;  // pinned mirror
  std::vector<cudaEvent_t> events_;
};

}  // namespace cg

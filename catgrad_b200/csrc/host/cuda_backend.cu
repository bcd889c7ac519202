// CudaBackend: one method per `Backend` trait method (catgrad/src/interpreter/backend/mod.rs:24-122),
// each a shape/dtype check on the host plus at most a few kernel launches on the context's stream.
// View-producing ops (broadcast, transpose, slice, reshape of a contiguous tensor) launch nothing.
// Only to_vec, to_bool, compare and synchronize wait for the device.
#include "cuda_backend.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "../kernels/elementwise.h"
#include "../kernels/gemm_tcgen05.h"
#include "../kernels/matmul.h"

namespace cg {

// ---------------------------------------------------------------------------------------------
CachingAllocator::CachingAllocator(int device) : device_(device) {
  if (const char* e = std::getenv("CATGRAD_B200_MEM_CAP")) cap_ = (size_t)std::strtoull(e, nullptr, 10);
}
CachingAllocator::~CachingAllocator() { trim(); }

// Size classes: 512 B granules up to 4 KiB; above that four classes per power of two (a request is rounded up by at
// most 25 %, and by at most 16 MiB).  Few classes matter more than tight fits: a tensor that grows a little
// every step (the KV cache an op-by-op evaluation re-concatenates per token) then reuses cached blocks instead of asking
// cudaMalloc - a synchronising call of 0.1-1 ms in a process that holds many allocations - for a new size every step.
size_t CachingAllocator::round_size(size_t bytes) {
  if (bytes == 0) bytes = 1;
  if (bytes <= 4096) return (bytes + 511) & ~(size_t)511;
  int p = 63;
  while (!((bytes >> p) & 1)) --p;                 // 2^p <= bytes
  size_t step = (size_t)1 << (p - 2);              // a quarter of that power of two
  if (step > ((size_t)16 << 20)) step = (size_t)16 << 20;   // large, long-lived buffers: at most 16 MiB of slack
  return (bytes + step - 1) / step * step;
}

void* CachingAllocator::alloc(size_t bytes) {
  size_t sz = round_size(bytes);
  std::lock_guard<std::mutex> lk(mu_);
  auto it = free_.find(sz);
  if (it != free_.end() && !it->second.empty()) {
    void* p = it->second.back();
    it->second.pop_back();
    cached_ -= sz;
    live_ += sz;
    return p;
  }
  if (cap_ && live_ + cached_ + sz > cap_) {
    // give cached blocks back before refusing
    for (auto& kv : free_) {
      for (void* p : kv.second) cudaFree(p);
      kv.second.clear();
    }
    cached_ = 0;
    if (live_ + sz > cap_)
      throw Error(ERR_OOM, "device allocation of " + std::to_string(sz) + " bytes exceeds the memory cap");
  }
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, sz);
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    for (auto& kv : free_) {
      for (void* q : kv.second) cudaFree(q);
      kv.second.clear();
    }
    cached_ = 0;
    e = cudaMalloc(&p, sz);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    throw Error(e == cudaErrorMemoryAllocation ? ERR_OOM : ERR_CUDA,
                std::string("cudaMalloc of ") + std::to_string(sz) + " bytes: " + cudaGetErrorString(e));
  }
  ++mallocs_;
  live_ += sz;
  return p;
}

void CachingAllocator::free(void* p, size_t bytes) {
  size_t sz = round_size(bytes);
  std::lock_guard<std::mutex> lk(mu_);
  free_[sz].push_back(p);
  live_ -= sz;
  cached_ += sz;
}

void CachingAllocator::trim() {
  std::lock_guard<std::mutex> lk(mu_);
  int prev = -1;
  cudaGetDevice(&prev);
  cudaSetDevice(device_);
  for (auto& kv : free_) {
    for (void* p : kv.second) cudaFree(p);
    kv.second.clear();
  }
  cached_ = 0;
  if (prev >= 0) cudaSetDevice(prev);
}

// ---------------------------------------------------------------------------------------------
namespace {
__global__ void set_word_kernel(unsigned* p, unsigned v) { *p = v; }
__global__ void set_half_kernel(unsigned short* p, unsigned short v) { *p = v; }

// Collapsed common index space of up to three inputs and one output.  Strides of absent operands are 0.
cgk::View4 make_view(const Shape& shape, const Shape* sa, const Shape* sb, const Shape* sc, const Shape* so) {
  cgk::View4 v;
  std::memset(&v, 0, sizeof(v));
  std::vector<int64_t> sh, a, b, c, o;
  for (size_t i = 0; i < shape.size(); ++i) {
    if (shape[i] == 1) continue;
    sh.push_back(shape[i]);
    a.push_back(sa ? (*sa)[i] : 0);
    b.push_back(sb ? (*sb)[i] : 0);
    c.push_back(sc ? (*sc)[i] : 0);
    o.push_back(so ? (*so)[i] : 0);
  }
  // merge adjacent axes that every operand walks as one
  for (int i = (int)sh.size() - 2; i >= 0; --i) {
    int64_t n = sh[i + 1];
    if (a[i] == a[i + 1] * n && b[i] == b[i + 1] * n && c[i] == c[i + 1] * n && o[i] == o[i + 1] * n) {
      sh[i] *= n;
      a[i] = a[i + 1];
      b[i] = b[i + 1];
      c[i] = c[i + 1];
      o[i] = o[i + 1];
      sh.erase(sh.begin() + i + 1);
      a.erase(a.begin() + i + 1);
      b.erase(b.begin() + i + 1);
      c.erase(c.begin() + i + 1);
      o.erase(o.begin() + i + 1);
    }
  }
  if (sh.empty()) {
    sh.push_back(1);
    a.push_back(0);
    b.push_back(0);
    c.push_back(0);
    o.push_back(0);
  }
  v.rank = (int)sh.size();
  v.total = 1;
  for (int i = 0; i < v.rank; ++i) {
    v.shape[i] = sh[i];
    v.sa[i] = a[i];
    v.sb[i] = b[i];
    v.sc[i] = c[i];
    v.so[i] = o[i];
    v.total *= sh[i];
  }
  return v;
}

// Can operand with strides s / base pointer p use VEC-wide vector access along the innermost axis?
bool vec_ok_in(const cgk::View4& v, const long long* s, const void* p, int vec, size_t elem) {
  long long inner = s[v.rank - 1];
  if (inner == 0) return true;  // splat
  if (inner != 1) return false;
  if ((uintptr_t)p % (vec * elem) != 0) return false;
  for (int d = 0; d < v.rank - 1; ++d)
    if (s[d] % vec != 0) return false;
  return true;
}
bool vec_ok_out(const cgk::View4& v, const long long* s, const void* p, int vec, size_t elem) {
  if (s[v.rank - 1] != 1) return false;
  return vec_ok_in(v, s, p, vec, elem);
}
}  // namespace

CudaBackend::CudaBackend(int device) : device_(device) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n <= 0) {
    cudaGetLastError();
    throw Error(ERR_CUDA, std::string("no usable CUDA device (") + (e != cudaSuccess ? cudaGetErrorString(e) : "count 0") +
                              "); this backend has no CPU fallback");
  }
  CG_CHECK(device >= 0 && device < n, ERR_INVALID_ARG, "device index out of range");
  CG_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  CG_CUDA(cudaGetDeviceProperties(&prop, device));
  CG_CHECK(prop.major == 10, ERR_CUDA,
           std::string("this library holds sm_100a code only; device is ") + prop.name + " (sm_" +
               std::to_string(prop.major) + std::to_string(prop.minor) + ")");
  sm_count_ = prop.multiProcessorCount;
  CG_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
  alloc_ = std::make_shared<CachingAllocator>(device);
  CG_CUDA(cudaMalloc(&dev_words_, 64));
  CG_CUDA(cudaMemset(dev_words_, 0, 64));
  CG_CUDA(cudaMallocHost(&host_words_, 64));
  events_.assign(64, nullptr);
}

CudaBackend::~CudaBackend() {
  cudaSetDevice(device_);
  if (stream_) cudaStreamSynchronize(stream_);
  for (auto ev : events_)
    if (ev) cudaEventDestroy(ev);
  if (dev_words_) cudaFree(dev_words_);
  if (host_words_) cudaFreeHost(host_words_);
  if (stream_) cudaStreamDestroy(stream_);
  // alloc_ is shared with live tensors' deleters; cached blocks are freed when the last one goes.
}

void CudaBackend::guard() const { cudaSetDevice(device_); }

cudaEvent_t CudaBackend::event(int slot) {
  CG_CHECK(slot >= 0 && slot < (int)events_.size(), ERR_INVALID_ARG, "event slot out of range");
  if (!events_[slot]) CG_CUDA(cudaEventCreate(&events_[slot]));
  return events_[slot];
}

void CudaBackend::check_launch(const char* what) {
  ++launches;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw Error(ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}

void CudaBackend::synchronize() {
  guard();
  CG_CUDA(cudaStreamSynchronize(stream_));
  check_device_errors();
}

void CudaBackend::check_device_errors() {
  CG_CUDA(cudaMemcpyAsync(host_words_, dev_words_, 4, cudaMemcpyDeviceToHost, stream_));
  CG_CUDA(cudaStreamSynchronize(stream_));
  unsigned bits = host_words_[0];
  if (!bits) return;
  CG_CUDA(cudaMemsetAsync(dev_words_, 0, 4, stream_));
  std::string msg;
  if (bits & cgk::DEV_ERR_DIV_ZERO) msg += "attempt to divide by zero (u32 div); ";
  if (bits & cgk::DEV_ERR_INDEX_OOB) msg += "index out of bounds (index); ";
  if (bits & cgk::DEV_ERR_WAIT_TIMEOUT) msg += "a bounded device-side wait timed out; ";
  throw Error((bits & cgk::DEV_ERR_WAIT_TIMEOUT) ? ERR_TIMEOUT : ERR_INVALID_ARG, msg);
}

unsigned CudaBackend::read_flag_and_clear() {
  CG_CUDA(cudaMemcpyAsync(host_words_ + 1, dev_words_ + 1, 4, cudaMemcpyDeviceToHost, stream_));
  CG_CUDA(cudaMemsetAsync(dev_words_ + 1, 0, 4, stream_));
  CG_CUDA(cudaStreamSynchronize(stream_));
  return host_words_[1];
}

Tensor CudaBackend::empty(const Shape& shape, Dtype dt) {
  CG_CHECK(shape.size() <= 8, ERR_INVALID_ARG, "rank above 8 is not supported");
  for (auto d : shape) CG_CHECK(d >= 0, ERR_INVALID_ARG, "negative extent");
  guard();
  size_t bytes = (size_t)numel(shape) * dtype_size(dt);
  void* p = alloc_->alloc(bytes);
  std::shared_ptr<CachingAllocator> al = alloc_;
  Tensor t;
  t.st = std::make_shared<Storage>(p, bytes, [al](void* q, size_t b) { al->free(q, b); });
  t.dt = dt;
  t.shape = shape;
  t.strides = contiguous_strides(shape);
  return t;
}

// mod.rs:28 / ndarray.rs:72-87
Tensor CudaBackend::zeros(const Shape& shape, Dtype dt) {
  Tensor t = empty(shape, dt);
  if (t.st->bytes) CG_CUDA(cudaMemsetAsync(t.st->ptr, 0, t.st->bytes, stream_));
  return t;
}

// mod.rs:30-58 / ndarray.rs:89-132
Tensor CudaBackend::from_vec(const void* data, int64_t n, const Shape& shape, Dtype dt) {
  CG_CHECK(n == numel(shape), ERR_SHAPE,
           "ShapeError: " + std::to_string(n) + " elements for shape " + shape_str(shape));
  Tensor t = empty(shape, dt);
  if (n == 0) return t;
  size_t es = dtype_size(dt);
  if (n == 1 && es == 4) {  // literals: the value travels as a kernel argument, no staging copy
    unsigned v;
    std::memcpy(&v, data, 4);
    set_word_kernel<<<1, 1, 0, stream_>>>((unsigned*)t.st->ptr, v);
    check_launch("from_vec");
  } else if (n == 1 && es == 2) {
    unsigned short v;
    std::memcpy(&v, data, 2);
    set_half_kernel<<<1, 1, 0, stream_>>>((unsigned short*)t.st->ptr, v);
    check_launch("from_vec");
  } else {
    // pageable source: the call returns once the data is staged, the caller may free `data` at once
    CG_CUDA(cudaMemcpyAsync(t.st->ptr, data, (size_t)n * es, cudaMemcpyHostToDevice, stream_));
  }
  return t;
}

// mod.rs:111 / ndarray.rs:134-138
Tensor CudaBackend::arange(int64_t end) {
  CG_CHECK(end >= 0 && end <= 0xffffffffLL, ERR_INVALID_ARG, "arange: end out of range");
  Tensor t = empty({end}, Dtype::U32);
  if (end) {
    cgk::launch_arange((unsigned*)t.st->ptr, end, sm_count_, stream_);
    check_launch("arange");
  }
  return t;
}

// Strided copy src -> dst view (same shape and dtype).
void CudaBackend::copy_into(const Tensor& src, const Tensor& dst) {
  if (src.size() == 0) return;
  cgk::View4 v = make_view(src.shape, &src.strides, nullptr, nullptr, &dst.strides);
  int es = (int)dtype_size(src.dt);
  int vec = 16 / es;
  bool ok = v.shape[v.rank - 1] % vec == 0 && vec_ok_in(v, v.sa, src.raw(), vec, es) &&
            vec_ok_out(v, v.so, dst.raw(), vec, es);
  cgk::launch_copy(es, v, ok ? vec : 1, src.raw(), dst.raw(), sm_count_, stream_);
  check_launch("copy");
}

Tensor CudaBackend::contiguous(const Tensor& x) {
  if (x.is_contiguous()) return x;
  Tensor t = empty(x.shape, x.dt);
  copy_into(x, t);
  return t;
}

// mod.rs:60 / ndarray.rs:151-174; reduced-precision targets as in candle.rs:575-599
Tensor CudaBackend::cast(const Tensor& x, Dtype target) {
  if (x.dt == target) return x;
  Tensor t = empty(x.shape, target);
  if (x.size() == 0) return t;
  cgk::View4 v = make_view(x.shape, &x.strides, nullptr, nullptr, &t.strides);
  int vec = cgk::vector_width((int)dtype_size(x.dt), (int)dtype_size(target));
  bool ok = v.shape[v.rank - 1] % vec == 0 && vec_ok_in(v, v.sa, x.raw(), vec, dtype_size(x.dt)) &&
            vec_ok_out(v, v.so, t.raw(), vec, dtype_size(target));
  cgk::launch_cast((int)x.dt, (int)target, v, ok ? vec : 1, x.raw(), t.raw(), sm_count_, stream_);
  check_launch("cast");
  return t;
}

// mod.rs:62-71 / ndarray.rs:185-323
Tensor CudaBackend::binary(BinOp op, const Tensor& a, const Tensor& b) {
  check_same(a, b, "binary");
  CG_CHECK(a.dt != Dtype::F8, ERR_UNSUPPORTED_DTYPE, "fp8 tensors support cast and data movement only");
  Tensor t = empty(a.shape, a.dt);
  if (a.size() == 0) return t;
  cgk::View4 v = make_view(a.shape, &a.strides, &b.strides, nullptr, &t.strides);
  int es = (int)dtype_size(a.dt), vec = 16 / es;
  bool ok = v.shape[v.rank - 1] % vec == 0 && vec_ok_in(v, v.sa, a.raw(), vec, es) &&
            vec_ok_in(v, v.sb, b.raw(), vec, es) && vec_ok_out(v, v.so, t.raw(), vec, es);
  cgk::launch_binary((int)op, (int)a.dt, v, ok ? vec : 1, a.raw(), b.raw(), t.raw(), dev_words_, sm_count_, stream_);
  check_launch("binary");
  return t;
}

// mod.rs:72 / ndarray.rs:325-350
Tensor CudaBackend::where_cond(const Tensor& m, const Tensor& x, const Tensor& y) {
  check_same(m, x, "where");
  check_same(x, y, "where");
  CG_CHECK(x.dt != Dtype::F8, ERR_UNSUPPORTED_DTYPE, "fp8 tensors support cast and data movement only");
  Tensor t = empty(x.shape, x.dt);
  if (x.size() == 0) return t;
  cgk::View4 v = make_view(x.shape, &m.strides, &x.strides, &y.strides, &t.strides);
  int es = (int)dtype_size(x.dt), vec = 16 / es;
  bool ok = v.shape[v.rank - 1] % vec == 0 && vec_ok_in(v, v.sa, m.raw(), vec, es) &&
            vec_ok_in(v, v.sb, x.raw(), vec, es) && vec_ok_in(v, v.sc, y.raw(), vec, es) &&
            vec_ok_out(v, v.so, t.raw(), vec, es);
  cgk::launch_where((int)x.dt, v, ok ? vec : 1, m.raw(), x.raw(), y.raw(), t.raw(), sm_count_, stream_);
  check_launch("where");
  return t;
}

// mod.rs:73-79 / ndarray.rs:352-407
Tensor CudaBackend::unary(UnOp op, const Tensor& x) {
  static const char* names[] = {"neg", "sin", "cos", "exp", "log", "floor", "round"};
  CG_CHECK(x.dt != Dtype::F8, ERR_UNSUPPORTED_DTYPE, "fp8 tensors support cast and data movement only");
  CG_CHECK(x.dt != Dtype::U32 || op == UnOp::Neg, ERR_UNSUPPORTED_DTYPE,
           std::string("Invalid input types for ") + names[(int)op]);
  Tensor t = empty(x.shape, x.dt);
  if (x.size() == 0) return t;
  cgk::View4 v = make_view(x.shape, &x.strides, nullptr, nullptr, &t.strides);
  int es = (int)dtype_size(x.dt), vec = 16 / es;
  bool ok = v.shape[v.rank - 1] % vec == 0 && vec_ok_in(v, v.sa, x.raw(), vec, es) &&
            vec_ok_out(v, v.so, t.raw(), vec, es);
  cgk::launch_unary((int)op, (int)x.dt, v, ok ? vec : 1, x.raw(), t.raw(), sm_count_, stream_);
  check_launch("unary");
  return t;
}

// mod.rs:61 / ndarray.rs:176-183, 732-816
Tensor CudaBackend::matmul(const Tensor& a, const Tensor& b) {
  Shape out = matmul_shape(a, b);
  CG_CHECK(a.dt != Dtype::F8, ERR_UNSUPPORTED_DTYPE, "fp8 matmul is not supported");
  int r = a.rank();
  int64_t M = a.shape[r - 2], K = a.shape[r - 1], N = b.shape[r - 1];
  // the kernels index rows, columns and output tiles with 32-bit integers
  CG_CHECK(M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31) && ((M + 63) / 64) * ((N + 63) / 64) < (1ll << 31), ERR_INVALID_ARG,
           "matmul: a dimension (or the number of 64 x 64 output tiles) reaches 2^31");
  Tensor t = empty(out, a.dt);
  if (t.size() == 0) return t;
  if (K == 0) {
    CG_CUDA(cudaMemsetAsync(t.st->ptr, 0, t.st->bytes, stream_));
    return t;
  }
  Shape bshape(a.shape.begin(), a.shape.end() - 2);
  Shape sa(a.strides.begin(), a.strides.end() - 2), sb(b.strides.begin(), b.strides.end() - 2);
  cgk::View4 bt = make_view(bshape, &sa, &sb, nullptr, nullptr);
  int64_t batch = numel(bshape);
  if (bshape.empty()) {
    bt.rank = 0;
    bt.total = 1;
  }
  CG_CHECK(batch <= 65535, ERR_INVALID_ARG, "matmul: more than 65535 batch entries");

  int64_t sam = a.strides[r - 2], sak = a.strides[r - 1], sbk = b.strides[r - 2], sbn = b.strides[r - 1];
  // bf16 products with K-contiguous A go to the tensor cores; the right operand may be K-contiguous (x @ W^T) or
  // N-contiguous (the trait's row-major [.., K, N])
  const bool b_n_contig = sbk != 1 && sbn == 1;
  if (a.dt == Dtype::BF16 && cgk::tcgen05_gemm_applicable(bt, batch, a.raw(), b.raw(), M, N, K, sam, sak, sbk, sbn) &&
      cgk::launch_tcgen05_gemm(bt, batch, a.raw(), b.raw(), t.raw(), M, N, K, sam, b_n_contig ? sbk : sbn, dev_words_,
                               sm_count_, stream_, b_n_contig)) {
    check_launch("matmul(tcgen05)");
    return t;
  }
  // large f32 products with plain layouts: exact-f32 result from three-way bf16 splits on the tensor cores
  if (a.dt == Dtype::F32 && cgk::matmul_f32x3_applicable(M, N, K, batch) && sak == 1 && sam == K &&
      ((uintptr_t)a.raw() % 16 == 0) && ((uintptr_t)b.raw() % 16 == 0)) {
    const bool b_row_major = sbn == 1 && sbk == N, b_k_major = sbk == 1 && sbn == K;
    bool a_ok = batch == 1, b_ok = batch == 1, b_shared = false;
    if (batch > 1 && bt.rank == 1) {
      a_ok = bt.sa[0] == M * K;
      b_shared = bt.sb[0] == 0;
      b_ok = b_shared || bt.sb[0] == K * N;
    }
    if ((b_row_major || b_k_major) && a_ok && b_ok) {
      Tensor a3 = empty({(int64_t)cgk::matmul_f32x3_scratch_elems(M * batch, K)}, Dtype::BF16);
      Tensor b3 = empty({(int64_t)cgk::matmul_f32x3_scratch_elems(N * (b_shared ? 1 : batch), K)}, Dtype::BF16);
      if (cgk::launch_matmul_f32x3((const float*)a.raw(), (const float*)b.raw(), (float*)t.raw(), a3.raw(), b3.raw(), M, N, K,
                                   batch, b_row_major, b_shared, dev_words_, sm_count_, stream_)) {
        check_launch("matmul(f32 via bf16x3)");
        return t;
      }
    }
  }
  cgk::launch_matmul((int)a.dt, bt, batch, a.raw(), b.raw(), t.raw(), M, N, K, sam, sak, sbk, sbn, sm_count_, stream_);
  check_launch("matmul");
  return t;
}

// mod.rs:80-82: views (the reference materialises broadcast and reshape, ndarray.rs:545-559)
Tensor CudaBackend::broadcast(const Tensor& x, const Shape& shape) {
  CG_CHECK(shape.size() <= 8, ERR_INVALID_ARG, "rank above 8 is not supported");
  return view_broadcast(x, shape);
}
Tensor CudaBackend::reshape(const Tensor& x, const Shape& shape) {
  CG_CHECK(shape.size() <= 8, ERR_INVALID_ARG, "rank above 8 is not supported");
  CG_CHECK(numel(shape) == x.size(), ERR_SHAPE_MISMATCH, "reshape: " + shape_str(x.shape) + " -> " + shape_str(shape));
  Tensor c = contiguous(x);
  Tensor r;
  view_reshape(c, shape, &r);
  return r;
}
Tensor CudaBackend::transpose(const Tensor& x, int64_t d0, int64_t d1) { return view_transpose(x, d0, d1); }
Tensor CudaBackend::slice(const Tensor& x, int64_t dim, int64_t start, int64_t len) {
  return view_slice(x, dim, start, len);
}

Tensor CudaBackend::reduce(int kind, const Tensor& x) {
  CG_CHECK(x.rank() >= 1, ERR_SHAPE_MISMATCH, "reduction needs rank >= 1");
  CG_CHECK(x.dt != Dtype::F8, ERR_UNSUPPORTED_DTYPE, "fp8 tensors support cast and data movement only");
  Shape os = x.shape;
  int64_t n = os.back();
  os.back() = 1;
  CG_CHECK(kind != cgk::R_ARGMAX || n > 0, ERR_INVALID_ARG, "argmax over an empty axis");
  Tensor t = empty(os, kind == cgk::R_ARGMAX ? Dtype::U32 : x.dt);
  int64_t rows = t.size();
  if (rows == 0) return t;
  Shape oshape(x.shape.begin(), x.shape.end() - 1), ostr(x.strides.begin(), x.strides.end() - 1);
  // a pick over few, long float rows (logits): one CTA per row would leave most SMs idle, so the row is cut into
  // 4096-element chunks first (two launches, scratch from the allocator)
  if (kind == cgk::R_ARGMAX && x.dt != Dtype::U32 && x.strides.back() == 1 && n >= 8192 && n < (1ll << 31) && rows <= 65535 &&
      rows < 4 * (int64_t)sm_count_ && (x.rank() <= 2 || x.is_contiguous())) {
    const int64_t row_stride = x.rank() == 1 ? n : (x.rank() == 2 ? x.strides[0] : n);
    const int64_t chunks = (n + 4095) / 4096;
    Tensor scratch = empty({rows * chunks * 2}, Dtype::U32);
    cgk::launch_argmax_two_stage((int)x.dt, x.raw(), row_stride, rows, n, scratch.raw(), (unsigned*)t.raw(), stream_);
    check_launch("argmax");
    return t;
  }
  cgk::View4 outer = make_view(oshape, &ostr, nullptr, nullptr, nullptr);
  cgk::launch_reduce(kind, (int)x.dt, outer, rows, n, x.strides.back(), x.raw(), t.raw(), sm_count_, stream_);
  check_launch("reduce");
  return t;
}
Tensor CudaBackend::softmax(const Tensor& x) {
  CG_CHECK(x.rank() >= 1, ERR_SHAPE_MISMATCH, "softmax needs rank >= 1");
  CG_CHECK(x.dt == Dtype::F32 || x.dt == Dtype::BF16 || x.dt == Dtype::F16, ERR_UNSUPPORTED_DTYPE,
           "softmax is defined for f32, f16 and bf16");
  Tensor c = contiguous(x);
  Tensor t = empty(x.shape, x.dt);
  const int64_t n = x.shape.back();
  if (t.size() == 0) return t;
  CG_CHECK(t.size() / n <= 0x7fffffffll, ERR_INVALID_ARG, "softmax: too many rows");
  cgk::launch_softmax((int)x.dt, c.raw(), t.raw(), t.size() / n, n, stream_);
  check_launch("softmax");
  return t;
}
Tensor CudaBackend::max(const Tensor& x) { return reduce(cgk::R_MAX, x); }        // mod.rs:83
Tensor CudaBackend::sum(const Tensor& x) { return reduce(cgk::R_SUM, x); }        // mod.rs:84
Tensor CudaBackend::argmax(const Tensor& x) { return reduce(cgk::R_ARGMAX, x); }  // mod.rs:85

// mod.rs:86 / ndarray.rs:696-721
std::pair<Tensor, Tensor> CudaBackend::topk(const Tensor& x, int64_t k) {
  CG_CHECK(x.dt == Dtype::F32 || x.dt == Dtype::BF16 || x.dt == Dtype::F16, ERR_UNSUPPORTED_DTYPE,
           "Unsupported type for topk");
  CG_CHECK(x.rank() >= 1 && k >= 0 && k <= x.shape.back(), ERR_INVALID_ARG, "topk: k exceeds the last axis");
  Shape os = x.shape;
  int64_t n = os.back();
  os.back() = k;
  Tensor vals = empty(os, x.dt), idx = empty(os, Dtype::U32);
  if (vals.size() == 0) return {vals, idx};
  Tensor c = contiguous(x);
  int64_t rows = c.size() / n;
  CG_CHECK(rows <= 0x7fffffff, ERR_INVALID_ARG, "topk: too many rows");
  cgk::launch_topk((int)x.dt, c.raw(), vals.raw(), (unsigned*)idx.raw(), rows, n, k, stream_);
  check_launch("topk");
  return {vals, idx};
}

// mod.rs:87 / ndarray.rs:534-541
bool CudaBackend::compare(const Tensor& a, const Tensor& b) {
  CG_CHECK(a.dt == b.dt, ERR_DTYPE_MISMATCH, "compare: operand dtypes differ");
  if (a.shape != b.shape) return false;
  if (a.size() == 0) return true;
  Tensor ca = contiguous(a), cb = contiguous(b);
  if (a.dt == Dtype::F8) {
    // bit equality, except that NaN patterns never compare equal: widen to f16 first
    ca = cast(ca, Dtype::F16);
    cb = cast(cb, Dtype::F16);
  }
  cgk::launch_any_diff((int)ca.dt, ca.raw(), cb.raw(), ca.size(), dev_words_ + 1, sm_count_, stream_);
  check_launch("compare");
  return read_flag_and_clear() == 0;
}

// mod.rs:88-93 / ndarray.rs:513-532
Tensor CudaBackend::concat(const Tensor& a, const Tensor& b, int64_t dim) {
  CG_CHECK(a.dt == b.dt, ERR_DTYPE_MISMATCH, "Incompatible types for concatenation");
  CG_CHECK(a.rank() == b.rank() && dim >= 0 && dim < a.rank(), ERR_SHAPE_MISMATCH, "concat: rank/axis mismatch");
  for (int i = 0; i < a.rank(); ++i)
    CG_CHECK(i == dim || a.shape[i] == b.shape[i], ERR_SHAPE_MISMATCH,
             "concat: shapes differ off the concatenation axis: " + shape_str(a.shape) + " vs " + shape_str(b.shape));
  Shape os = a.shape;
  os[dim] += b.shape[dim];
  Tensor t = empty(os, a.dt);
  copy_into(a, view_slice(t, dim, 0, a.shape[dim]));
  copy_into(b, view_slice(t, dim, a.shape[dim], b.shape[dim]));
  return t;
}

// mod.rs:94-99 / ndarray.rs:466-487, 571-579
Tensor CudaBackend::index(const Tensor& x, int64_t dim, const Tensor& indices) {
  CG_CHECK(indices.dt == Dtype::U32, ERR_DTYPE_MISMATCH, "Invalid input types for indexing");
  CG_CHECK(dim >= 0 && dim < x.rank(), ERR_INVALID_ARG, "index: axis out of range");
  Tensor ci = contiguous(indices);
  int64_t n_idx = ci.size();
  Shape os = x.shape;
  os[dim] = n_idx;
  Tensor t = empty(os, x.dt);
  if (t.size() == 0) return t;
  Tensor cx = contiguous(x);
  int64_t outer = 1, inner = 1;
  for (int i = 0; i < dim; ++i) outer *= x.shape[i];
  for (int i = (int)dim + 1; i < x.rank(); ++i) inner *= x.shape[i];
  cgk::launch_gather((int)dtype_size(x.dt), cx.raw(), (const unsigned*)ci.raw(), 1, t.raw(), outer, x.shape[dim],
                     n_idx, inner, dev_words_, sm_count_, stream_);
  check_launch("index");
  return t;
}

// mod.rs:113 / ndarray.rs:140-149
bool CudaBackend::to_bool(const Tensor& x) {
  if (x.size() == 0) return false;
  Tensor c = contiguous(x);
  if (c.dt == Dtype::F8) c = cast(c, Dtype::F16);
  cgk::launch_any_positive((int)c.dt, c.raw(), c.size(), dev_words_ + 1, sm_count_, stream_);
  check_launch("to_bool");
  return read_flag_and_clear() != 0;
}

// mod.rs:115 / ndarray.rs:50-59
void CudaBackend::to_vec(const Tensor& x, void* dst, size_t cap) {
  size_t need = (size_t)x.size() * dtype_size(x.dt);
  CG_CHECK(cap >= need, ERR_INVALID_ARG, "to_vec: destination too small");
  guard();
  Tensor c = contiguous(x);
  if (need) CG_CUDA(cudaMemcpyAsync(dst, c.raw(), need, cudaMemcpyDeviceToHost, stream_));
  CG_CUDA(cudaStreamSynchronize(stream_));
  check_device_errors();
}

Backend* make_backend(int device) { return new CudaBackend(device); }

}  // namespace cg

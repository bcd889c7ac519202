// Tensor handle shared by every backend implementation behind the C ABI.
//
// A Tensor is a strided view (offset + shape + strides, in elements) over a
// reference-counted Storage.  Transpose, slice, broadcast and contiguous
// reshape never copy; the reference interpreter's ndarray backend materialises
// most of them (catgrad/src/interpreter/backend/ndarray.rs:545-596), its
// transpose is a stride swap like ours (ndarray.rs:561-569).
#pragma once
#include <cstddef>
#include <cstdint>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace cg {

// Same order as `enum Dtype` in catgrad/src/category/core.rs:23-29.
enum class Dtype : int { F32 = 0, F16 = 1, BF16 = 2, F8 = 3, U32 = 4 };

inline size_t dtype_size(Dtype d) {
  switch (d) {
    case Dtype::F32: return 4;
    case Dtype::U32: return 4;
    case Dtype::F16: return 2;
    case Dtype::BF16: return 2;
    case Dtype::F8: return 1;
  }
  return 0;
}
inline const char* dtype_name(Dtype d) {
  switch (d) {
    case Dtype::F32: return "f32";
    case Dtype::F16: return "f16";
    case Dtype::BF16: return "bf16";
    case Dtype::F8: return "fp8";
    case Dtype::U32: return "u32";
  }
  return "?";
}

// Status codes returned through the C ABI (include/catgrad_b200.h mirrors them).
enum Status : int {
  OK = 0,
  ERR_SHAPE_MISMATCH = 1,   // operands of a pointwise op differ in shape ("Shape mismatch in operation")
  ERR_DTYPE_MISMATCH = 2,   // operands of one op differ in dtype (interpreter TypeError)
  ERR_UNSUPPORTED_DTYPE = 3,
  ERR_OOM = 4,
  ERR_CUDA = 5,
  ERR_TIMEOUT = 6,
  ERR_BAD_HANDLE = 7,
  ERR_SHAPE = 8,            // constructor: element count != product(shape) (BackendError::ShapeError)
  ERR_INVALID_ARG = 9,
  ERR_INTERP = 10,          // evaluator errors (arity, multiple read/write, missing parameter)
};

struct Error : std::runtime_error {
  Status status;
  Error(Status s, const std::string& m) : std::runtime_error(m), status(s) {}
};

#define CG_CHECK(cond, status, msg)                   \
  do {                                                \
    if (!(cond)) throw ::cg::Error((status), (msg));  \
  } while (0)

using Shape = std::vector<int64_t>;

inline int64_t numel(const Shape& s) {
  int64_t n = 1;
  for (auto d : s) n *= d;
  return n;
}
inline Shape contiguous_strides(const Shape& s) {
  Shape st(s.size());
  int64_t acc = 1;
  for (int i = (int)s.size() - 1; i >= 0; --i) {
    st[i] = acc;
    acc *= s[i];
  }
  return st;
}

struct Storage {
  void* ptr = nullptr;
  size_t bytes = 0;
  std::function<void(void*, size_t)> deleter;
  Storage(void* p, size_t b, std::function<void(void*, size_t)> d) : ptr(p), bytes(b), deleter(std::move(d)) {}
  Storage(const Storage&) = delete;
  Storage& operator=(const Storage&) = delete;
  ~Storage() {
    if (ptr && deleter) deleter(ptr, bytes);
  }
};

struct Tensor {
  std::shared_ptr<Storage> st;
  int64_t offset = 0;  // elements
  Dtype dt = Dtype::F32;
  Shape shape;
  Shape strides;  // elements; 0 on broadcast axes

  int rank() const { return (int)shape.size(); }
  int64_t size() const { return numel(shape); }
  bool defined() const { return (bool)st; }
  bool is_contiguous() const {
    int64_t acc = 1;
    for (int i = rank() - 1; i >= 0; --i) {
      if (shape[i] != 1 && strides[i] != acc) return false;
      acc *= shape[i];
    }
    return true;
  }
  template <class T>
  T* data() const {
    return reinterpret_cast<T*>(static_cast<char*>(st->ptr) + (size_t)offset * dtype_size(dt));
  }
  void* raw() const { return static_cast<char*>(st->ptr) + (size_t)offset * dtype_size(dt); }
};

inline std::string shape_str(const Shape& s) {
  std::string r = "[";
  for (size_t i = 0; i < s.size(); ++i) {
    if (i) r += ",";
    r += std::to_string(s[i]);
  }
  return r + "]";
}

// ---- view constructors shared by all backends (pure metadata) -------------------------------

// numpy-style right-aligned broadcast; size-1 or missing axes expand with stride 0
// (semantics of ndarray.rs:553-559; legality as in typecheck/tensor_op.rs:284-307).
inline Tensor view_broadcast(const Tensor& x, const Shape& shape) {
  CG_CHECK(shape.size() >= x.shape.size(), ERR_SHAPE_MISMATCH,
           "broadcast: cannot broadcast " + shape_str(x.shape) + " to " + shape_str(shape));
  Tensor r = x;
  r.shape = shape;
  r.strides.assign(shape.size(), 0);
  size_t lead = shape.size() - x.shape.size();
  for (size_t i = 0; i < x.shape.size(); ++i) {
    int64_t sd = x.shape[i], td = shape[lead + i];
    if (sd == td)
      r.strides[lead + i] = (sd == 1) ? 0 : x.strides[i];
    else if (sd == 1)
      r.strides[lead + i] = 0;
    else
      throw Error(ERR_SHAPE_MISMATCH,
                  "broadcast: cannot broadcast " + shape_str(x.shape) + " to " + shape_str(shape));
  }
  return r;
}

inline Tensor view_transpose(const Tensor& x, int64_t d0, int64_t d1) {
  CG_CHECK(d0 >= 0 && d1 >= 0 && d0 < x.rank() && d1 < x.rank(), ERR_INVALID_ARG, "transpose: axis out of range");
  Tensor r = x;
  std::swap(r.shape[d0], r.shape[d1]);
  std::swap(r.strides[d0], r.strides[d1]);
  return r;
}

inline Tensor view_slice(const Tensor& x, int64_t dim, int64_t start, int64_t len) {
  CG_CHECK(dim >= 0 && dim < x.rank(), ERR_INVALID_ARG, "slice: axis out of range");
  CG_CHECK(start >= 0 && len >= 0 && start + len <= x.shape[dim], ERR_INVALID_ARG,
           "slice: range [" + std::to_string(start) + "," + std::to_string(start + len) + ") exceeds axis of size " +
               std::to_string(x.shape[dim]));
  Tensor r = x;
  r.offset += start * x.strides[dim];
  r.shape[dim] = len;
  return r;
}

// Reshape of a contiguous tensor is a view.  Returns false if x must be copied first.
inline bool view_reshape(const Tensor& x, const Shape& shape, Tensor* out) {
  if (!x.is_contiguous()) return false;
  *out = x;
  out->shape = shape;
  out->strides = contiguous_strides(shape);
  return true;
}

}  // namespace cg

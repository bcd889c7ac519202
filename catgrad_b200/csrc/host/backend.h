// The operator surface every backend implements: one virtual method per method of
// `trait Backend` (catgrad/src/interpreter/backend/mod.rs:24-122), same names,
// same argument meaning.  Conventions kept from the trait's doc comment
// (mod.rs:18-23): operands of one op share a dtype, nothing broadcasts
// implicitly, reductions keep the rank.
//
// Methods throw cg::Error; the C ABI turns that into a status + message.
#pragma once
#include <cstdint>
#include <string>
#include <utility>
#include <vector>

#include "tensor.h"

namespace cg {

enum class BinOp : int { Add, Sub, Mul, Div, Pow, LT, GT, GTE, LTE, EQ };
enum class UnOp : int { Neg, Sin, Cos, Exp, Log, Floor, Round };

class Backend {
 public:
  virtual ~Backend() {}
  virtual const char* name() const = 0;

  // constructors (mod.rs:28-58).  `data` is host memory of n elements of dtype dt.
  virtual Tensor zeros(const Shape& shape, Dtype dt) = 0;
  virtual Tensor from_vec(const void* data, int64_t n, const Shape& shape, Dtype dt) = 0;
  virtual Tensor arange(int64_t end) = 0;

  virtual Tensor cast(const Tensor& x, Dtype target) = 0;
  virtual Tensor matmul(const Tensor& a, const Tensor& b) = 0;
  virtual Tensor binary(BinOp op, const Tensor& a, const Tensor& b) = 0;
  virtual Tensor where_cond(const Tensor& mask, const Tensor& x, const Tensor& y) = 0;
  virtual Tensor unary(UnOp op, const Tensor& x) = 0;

  virtual Tensor broadcast(const Tensor& x, const Shape& shape) = 0;
  virtual Tensor reshape(const Tensor& x, const Shape& shape) = 0;
  virtual Tensor transpose(const Tensor& x, int64_t d0, int64_t d1) = 0;
  virtual Tensor max(const Tensor& x) = 0;
  virtual Tensor sum(const Tensor& x) = 0;
  virtual Tensor argmax(const Tensor& x) = 0;
  virtual std::pair<Tensor, Tensor> topk(const Tensor& x, int64_t k) = 0;
  virtual bool compare(const Tensor& a, const Tensor& b) = 0;
  virtual Tensor concat(const Tensor& a, const Tensor& b, int64_t dim) = 0;
  virtual Tensor index(const Tensor& x, int64_t dim, const Tensor& indices) = 0;
  virtual Tensor slice(const Tensor& x, int64_t dim, int64_t start, int64_t len) = 0;

  virtual bool to_bool(const Tensor& x) = 0;
  // Copies the logical (row-major) contents to host memory; synchronises.
  virtual void to_vec(const Tensor& x, void* dst, size_t cap_bytes) = 0;
  virtual std::string format_tensor(const Tensor& x);

  virtual void synchronize() {}

  // Shared argument checks (same rules for every implementation).
  static void check_same(const Tensor& a, const Tensor& b, const char* what) {
    CG_CHECK(a.dt == b.dt, ERR_DTYPE_MISMATCH, std::string(what) + ": operand dtypes differ");
    // Message pinned by the reference's should_panic tests (tests/test_interpreter_candle.rs:726-862).
    CG_CHECK(a.shape == b.shape, ERR_SHAPE_MISMATCH,
             std::string("Shape mismatch in operation: ") + what + " " + shape_str(a.shape) + " vs " +
                 shape_str(b.shape));
  }
};

// Shape rule of matmul (ndarray.rs:732-816): ranks >= 2 and equal, batch dims equal, inner dims agree.
inline Shape matmul_shape(const Tensor& a, const Tensor& b) {
  CG_CHECK(a.dt == b.dt, ERR_DTYPE_MISMATCH, "matmul: operand dtypes differ");
  CG_CHECK(a.rank() >= 2 && b.rank() >= 2, ERR_SHAPE_MISMATCH, "batched_matmul: operands must be at least rank 2");
  CG_CHECK(a.rank() == b.rank(), ERR_SHAPE_MISMATCH, "batched_matmul: batch dimensions must match");
  int r = a.rank();
  for (int i = 0; i < r - 2; ++i)
    CG_CHECK(a.shape[i] == b.shape[i], ERR_SHAPE_MISMATCH, "batched_matmul: batch dimensions must match");
  CG_CHECK(a.shape[r - 1] == b.shape[r - 2], ERR_SHAPE_MISMATCH, "batched_matmul: incompatible matrix dimensions");
  Shape out(a.shape.begin(), a.shape.end() - 1);
  out.push_back(b.shape[r - 1]);
  return out;
}

}  // namespace cg

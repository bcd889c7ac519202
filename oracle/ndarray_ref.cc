// TEST INFRASTRUCTURE ONLY.  CPU restatement of the reference interpreter's ndarray backend
// (catgrad/src/interpreter/backend/ndarray.rs), used as the parity oracle by tests/, by
// __graft_entry__.smoke() and by bench.py's CPU-baseline leg.  Nothing in the shipped library links,
// loads or calls this file.
//
// Parity status: the reference cannot be compiled in this environment (no Rust toolchain) and its
// arithmetic lives in un-vendored crates (ndarray 0.17.1 -> matrixmultiply 0.3.10, Rust std f32
// functions, half 2.7.1).  This file restates the algorithm of every `Backend` method from
// ndarray.rs and is pinned against the literal vectors of the reference's own tests
// (ndarray.rs:831-1022, tests/test_interpreter*.rs, helpers_tests.rs; see tests/golden/).  What those
// vectors do not reach is "parity unpinned" and follows the source: argmax tie-break (last index under
// total_cmp, ndarray.rs:670-694), `max` folding from f32::MIN (ndarray.rs:656-661), index/slice/concat/
// arange/where at the trait level, u32 wrap-around, and everything in bf16/f16/fp8.
//
// Single-threaded on purpose: the reference's tensor ops are (ndarray without rayon/blas, matrixmultiply
// without its `threading` feature).
//
// f32 and u32 follow ndarray.rs.  ndarray.rs has no reduced-precision floats (ndarray.rs:7-9); for bf16
// and f16 this file follows the candle backend's rule (candle.rs:1165-1192, 575-610): an op runs in the
// operands' dtype, i.e. here: computed in f32 from the stored values and rounded to nearest-even once,
// at the op's output; matmul and sum accumulate in f32.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <numeric>
#include <sstream>

#include "../catgrad_b200/csrc/host/backend.h"

namespace cg {
namespace {

// ---- scalar conversions ------------------------------------------------------------------------
inline uint32_t f2u(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float u2f(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

inline float bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }
inline uint16_t f32_to_bf16(float f) {  // round to nearest even; NaN stays NaN
  uint32_t u = f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
inline float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return u2f(sign);
    float v = std::ldexp((float)man, -24);
    return sign ? -v : v;
  }
  if (exp == 31) return u2f(sign | 0x7f800000u | (man << 13));
  return u2f(sign | ((exp + 112) << 23) | (man << 13));
}
inline uint16_t f32_to_f16(float f) {  // round to nearest even
  uint32_t u = f2u(f), sign = (u >> 16) & 0x8000u, a = u & 0x7fffffffu;
  if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
  if (a >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);  // >= 65536 -> inf (65520 rounds to inf below)
  if (a < 0x33000000u) return (uint16_t)sign;                // < 2^-25 -> 0
  int e = (int)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u;
  int shift = (e < -14) ? (13 + (-14 - e)) : 13;
  uint32_t half_bit = 1u << (shift - 1), rest = m & ((1u << shift) - 1), q = m >> shift;
  if (rest > half_bit || (rest == half_bit && (q & 1))) q++;
  uint32_t r = (e < -14) ? q : (((uint32_t)(e + 15) << 10) + (q - 0x400u));
  return (uint16_t)(sign | r);  // a carry into the exponent is already right, incl. overflow to inf
}
// fp8 e4m3 ("fn" flavour: no infinities, 0x7f/0xff are NaN, max finite 448).  Parity unpinned.
inline float f8_to_f32(uint8_t v) {
  uint32_t sign = v & 0x80u, exp = (v >> 3) & 0xf, man = v & 7u;
  float r;
  if (exp == 15 && man == 7) r = std::numeric_limits<float>::quiet_NaN();
  else if (exp == 0) r = std::ldexp((float)man, -9);
  else r = std::ldexp((float)(8 + man), (int)exp - 10);
  return sign ? -r : r;
}
inline uint8_t f32_to_f8(float f) {  // round to nearest even, saturate to +-448
  uint8_t sign = (f2u(f) >> 24) & 0x80u;
  if (std::isnan(f)) return sign | 0x7f;
  float a = std::fabs(f);
  if (a >= 448.f) return sign | 0x7e;
  uint8_t best = 0;
  // 127 candidates: scan is fine for test infrastructure
  float bd = a;
  for (int c = 1; c < 0x7f; ++c) {
    float d = std::fabs(f8_to_f32((uint8_t)c) - a);
    if (d < bd || (d == bd && !(c & 1))) { bd = d; best = (uint8_t)c; }
  }
  return sign | best;
}

inline bool is_float(Dtype d) { return d != Dtype::U32; }

Tensor alloc(const Shape& shape, Dtype dt, bool zero = false) {
  size_t bytes = (size_t)numel(shape) * dtype_size(dt);
  void* p = zero ? std::calloc(std::max<size_t>(bytes, 1), 1) : std::malloc(std::max<size_t>(bytes, 1));
  CG_CHECK(p, ERR_OOM, "host allocation failed");
  Tensor t;
  t.st = std::make_shared<Storage>(p, bytes, [](void* q, size_t) { std::free(q); });
  t.dt = dt;
  t.shape = shape;
  t.strides = contiguous_strides(shape);
  return t;
}

// Calls f(element offset) for every element in logical (row-major) order.
template <class F>
void for_each_offset(const Tensor& t, F f) {
  int r = t.rank();
  int64_t n = t.size();
  if (n == 0) return;
  if (r == 0) { f(t.offset); return; }
  std::vector<int64_t> idx(r, 0);
  int64_t inner = t.shape[r - 1], istr = t.strides[r - 1];
  int64_t outer = n / inner;
  int64_t base = t.offset;
  for (int64_t o = 0; o < outer; ++o) {
    for (int64_t i = 0; i < inner; ++i) f(base + i * istr);
    for (int d = r - 2; d >= 0; --d) {
      idx[d]++;
      base += t.strides[d];
      if (idx[d] < t.shape[d]) break;
      base -= t.strides[d] * t.shape[d];
      idx[d] = 0;
    }
  }
}

// f32 tensor whose last two axes are a transposed contiguous matrix (stride 1 on the second-to-last axis):
// copied in 32x32 tiles so both sides stay in cache.  Same result as the element-wise walk.
bool load_f32_transposed(const Tensor& t, std::vector<float>& v) {
  int r = t.rank();
  if (t.dt != Dtype::F32 || r < 2 || t.strides[r - 2] != 1 || t.strides[r - 1] == 1) return false;
  int64_t R = t.shape[r - 2], C = t.shape[r - 1], cs = t.strides[r - 1];
  if (R < 32 || C < 32) return false;
  Tensor outer = t;
  outer.shape.resize(r - 2);
  outer.strides.resize(r - 2);
  v.resize((size_t)t.size());
  const float* p = (const float*)t.st->ptr;
  float* dst = v.data();
  for_each_offset(outer, [&](int64_t base) {
    for (int64_t i0 = 0; i0 < R; i0 += 32)
      for (int64_t j0 = 0; j0 < C; j0 += 32) {
        int64_t i1 = std::min(R, i0 + 32), j1 = std::min(C, j0 + 32);
        for (int64_t j = j0; j < j1; ++j)
          for (int64_t i = i0; i < i1; ++i) dst[i * C + j] = p[base + i + j * cs];
      }
    dst += R * C;
  });
  return true;
}

// Logical contents as f32 (float dtypes) or u32.
std::vector<float> load_f(const Tensor& t) {
  std::vector<float> v;
  if (load_f32_transposed(t, v)) return v;
  v.reserve((size_t)t.size());
  const char* p = (const char*)t.st->ptr;
  switch (t.dt) {
    case Dtype::F32: for_each_offset(t, [&](int64_t o) { v.push_back(((const float*)p)[o]); }); break;
    case Dtype::BF16: for_each_offset(t, [&](int64_t o) { v.push_back(bf16_to_f32(((const uint16_t*)p)[o])); }); break;
    case Dtype::F16: for_each_offset(t, [&](int64_t o) { v.push_back(f16_to_f32(((const uint16_t*)p)[o])); }); break;
    case Dtype::F8: for_each_offset(t, [&](int64_t o) { v.push_back(f8_to_f32(((const uint8_t*)p)[o])); }); break;
    case Dtype::U32: throw Error(ERR_DTYPE_MISMATCH, "expected a float tensor");
  }
  return v;
}
std::vector<uint32_t> load_u(const Tensor& t) {
  CG_CHECK(t.dt == Dtype::U32, ERR_DTYPE_MISMATCH, "expected a u32 tensor");
  std::vector<uint32_t> v;
  v.reserve((size_t)t.size());
  const uint32_t* p = (const uint32_t*)t.st->ptr;
  for_each_offset(t, [&](int64_t o) { v.push_back(p[o]); });
  return v;
}
Tensor store_f(const std::vector<float>& v, const Shape& shape, Dtype dt) {
  Tensor t = alloc(shape, dt);
  CG_CHECK((int64_t)v.size() == t.size(), ERR_SHAPE, "internal: element count");
  switch (dt) {
    case Dtype::F32: if (!v.empty()) std::memcpy(t.st->ptr, v.data(), v.size() * 4); break;
    case Dtype::BF16: { auto* p = (uint16_t*)t.st->ptr; for (size_t i = 0; i < v.size(); ++i) p[i] = f32_to_bf16(v[i]); break; }
    case Dtype::F16: { auto* p = (uint16_t*)t.st->ptr; for (size_t i = 0; i < v.size(); ++i) p[i] = f32_to_f16(v[i]); break; }
    case Dtype::F8: { auto* p = (uint8_t*)t.st->ptr; for (size_t i = 0; i < v.size(); ++i) p[i] = f32_to_f8(v[i]); break; }
    case Dtype::U32: throw Error(ERR_DTYPE_MISMATCH, "internal: store_f to u32");
  }
  return t;
}
Tensor store_u(const std::vector<uint32_t>& v, const Shape& shape) {
  Tensor t = alloc(shape, Dtype::U32);
  CG_CHECK((int64_t)v.size() == t.size(), ERR_SHAPE, "internal: element count");
  if (!v.empty()) std::memcpy(t.st->ptr, v.data(), v.size() * 4);
  return t;
}
// Raw copy of logical contents (any dtype), contiguous result.
Tensor materialize(const Tensor& x, const Shape& shape) {
  Tensor t = alloc(shape, x.dt);
  size_t es = dtype_size(x.dt);
  const char* src = (const char*)x.st->ptr;
  char* dst = (char*)t.st->ptr;
  int64_t i = 0;
  switch (es) {
    case 4: for_each_offset(x, [&](int64_t o) { ((uint32_t*)dst)[i++] = ((const uint32_t*)src)[o]; }); break;
    case 2: for_each_offset(x, [&](int64_t o) { ((uint16_t*)dst)[i++] = ((const uint16_t*)src)[o]; }); break;
    default: for_each_offset(x, [&](int64_t o) { ((uint8_t*)dst)[i++] = ((const uint8_t*)src)[o]; }); break;
  }
  return t;
}

// Rust `f32 as u32`: truncate toward zero, saturate, NaN -> 0.
inline uint32_t f32_as_u32(float v) {
  if (!(v == v)) return 0;
  if (v <= 0.f) return 0;
  if (v >= 4294967296.f) return 0xffffffffu;
  return (uint32_t)v;
}
// f32::total_cmp key: monotone map of the bit pattern to a signed integer.
inline int32_t total_key(float v) {
  int32_t b = (int32_t)f2u(v);
  return b ^ (int32_t)(((uint32_t)(b >> 31)) >> 1);
}
// Rust f32::max: if one operand is NaN the other is returned.
inline float rust_max(float a, float b) {
  if (a != a) return b;
  if (b != b) return a;
  return a > b ? a : b;
}
inline uint32_t u32_pow(uint32_t base, uint32_t exp) {  // u32::pow with wrap-around (release build)
  uint32_t r = 1;
  while (exp) {
    if (exp & 1) r *= base;
    base *= base;
    exp >>= 1;
  }
  return r;
}

// C[m,n] += A[m,k] * B[k,n], row-major contiguous, f32, k ascending per output element.
void sgemm_acc(const float* A, const float* B, float* C, int64_t M, int64_t K, int64_t N) {
  const int64_t KB = 256;
  for (int64_t k0 = 0; k0 < K; k0 += KB) {
    int64_t k1 = std::min(K, k0 + KB);
    for (int64_t i = 0; i < M; ++i) {
      float* c = C + i * N;
      for (int64_t k = k0; k < k1; ++k) {
        float a = A[i * K + k];
        const float* b = B + k * N;
        for (int64_t j = 0; j < N; ++j) c[j] = __builtin_fmaf(a, b[j], c[j]);
      }
    }
  }
}

class NdArrayRef : public Backend {
 public:
  const char* name() const override { return "ndarray_ref"; }

  // ndarray.rs:72-87
  Tensor zeros(const Shape& shape, Dtype dt) override { return alloc(shape, dt, true); }

  // ndarray.rs:89-132: element count must equal the shape's product, else ShapeError
  Tensor from_vec(const void* data, int64_t n, const Shape& shape, Dtype dt) override {
    CG_CHECK(n == numel(shape), ERR_SHAPE, "ShapeError: " + std::to_string(n) + " elements for shape " + shape_str(shape));
    Tensor t = alloc(shape, dt);
    if (n) std::memcpy(t.st->ptr, data, (size_t)n * dtype_size(dt));
    return t;
  }

  // ndarray.rs:134-138
  Tensor arange(int64_t end) override {
    std::vector<uint32_t> v((size_t)end);
    for (int64_t i = 0; i < end; ++i) v[i] = f32_as_u32((float)i);  // built as an f32 range, then cast
    return store_u(v, {end});
  }

  // ndarray.rs:151-174
  Tensor cast(const Tensor& x, Dtype target) override {
    if (x.dt == target) return x;
    if (x.dt == Dtype::U32) {
      auto u = load_u(x);
      std::vector<float> f(u.size());
      for (size_t i = 0; i < u.size(); ++i) f[i] = (float)u[i];
      return store_f(f, x.shape, target);
    }
    auto f = load_f(x);
    if (target == Dtype::U32) {
      std::vector<uint32_t> u(f.size());
      for (size_t i = 0; i < f.size(); ++i) u[i] = f32_as_u32(f[i]);
      return store_u(u, x.shape);
    }
    return store_f(f, x.shape, target);
  }

  // ndarray.rs:176-183, 732-816
  Tensor matmul(const Tensor& a, const Tensor& b) override {
    Shape out = matmul_shape(a, b);
    int r = a.rank();
    int64_t M = a.shape[r - 2], K = a.shape[r - 1], N = b.shape[r - 1];
    int64_t batch = 1;
    for (int i = 0; i < r - 2; ++i) batch *= a.shape[i];
    if (a.dt == Dtype::U32) {
      auto A = load_u(a), B = load_u(b);
      std::vector<uint32_t> C((size_t)(batch * M * N), 0);
      for (int64_t bi = 0; bi < batch; ++bi)
        for (int64_t i = 0; i < M; ++i)
          for (int64_t k = 0; k < K; ++k) {
            uint32_t av = A[(bi * M + i) * K + k];
            for (int64_t j = 0; j < N; ++j) C[(bi * M + i) * N + j] += av * B[(bi * K + k) * N + j];
          }
      return store_u(C, out);
    }
    auto A = load_f(a), B = load_f(b);  // the reference copies strided operands too (to_shape, ndarray.rs:797-798)
    std::vector<float> C((size_t)(batch * M * N), 0.f);
    for (int64_t bi = 0; bi < batch; ++bi)
      sgemm_acc(A.data() + bi * M * K, B.data() + bi * K * N, C.data() + bi * M * N, M, K, N);
    return store_f(C, out, a.dt);
  }

  // ndarray.rs:185-323, 598-654
  Tensor binary(BinOp op, const Tensor& a, const Tensor& b) override {
    check_same(a, b, "binary");
    if (a.dt == Dtype::U32) {
      auto x = load_u(a), y = load_u(b);
      std::vector<uint32_t> r(x.size());
      for (size_t i = 0; i < x.size(); ++i) {
        uint32_t p = x[i], q = y[i], o = 0;
        switch (op) {
          case BinOp::Add: o = p + q; break;
          case BinOp::Sub: o = p - q; break;
          case BinOp::Mul: o = p * q; break;
          case BinOp::Div:
            CG_CHECK(q != 0, ERR_INVALID_ARG, "attempt to divide by zero");  // the reference panics
            o = p / q;
            break;
          case BinOp::Pow: o = u32_pow(p, q); break;
          case BinOp::LT: o = p < q; break;
          case BinOp::GT: o = p > q; break;
          case BinOp::GTE: o = p >= q; break;
          case BinOp::LTE: o = p <= q; break;
          case BinOp::EQ: o = p == q; break;
        }
        r[i] = o;
      }
      return store_u(r, a.shape);
    }
    auto x = load_f(a), y = load_f(b);
    std::vector<float> r(x.size());
    for (size_t i = 0; i < x.size(); ++i) {
      float p = x[i], q = y[i], o = 0;
      switch (op) {
        case BinOp::Add: o = p + q; break;
        case BinOp::Sub: o = p - q; break;
        case BinOp::Mul: o = p * q; break;
        case BinOp::Div: o = p / q; break;
        case BinOp::Pow: o = powf(p, q); break;
        case BinOp::LT: o = p < q ? 1.f : 0.f; break;
        case BinOp::GT: o = p > q ? 1.f : 0.f; break;
        case BinOp::GTE: o = p >= q ? 1.f : 0.f; break;
        case BinOp::LTE: o = p <= q ? 1.f : 0.f; break;
        case BinOp::EQ: o = p == q ? 1.f : 0.f; break;
      }
      r[i] = o;
    }
    return store_f(r, a.shape, a.dt);
  }

  // ndarray.rs:325-350: float mask selects x where mask > 0 (NaN selects y); u32 where mask != 0
  Tensor where_cond(const Tensor& m, const Tensor& x, const Tensor& y) override {
    check_same(m, x, "where");
    check_same(x, y, "where");
    if (m.dt == Dtype::U32) {
      auto mm = load_u(m), xx = load_u(x), yy = load_u(y);
      for (size_t i = 0; i < mm.size(); ++i) xx[i] = mm[i] != 0 ? xx[i] : yy[i];
      return store_u(xx, x.shape);
    }
    auto mm = load_f(m), xx = load_f(x), yy = load_f(y);
    for (size_t i = 0; i < mm.size(); ++i) xx[i] = mm[i] > 0.f ? xx[i] : yy[i];
    return store_f(xx, x.shape, x.dt);
  }

  // ndarray.rs:352-407, 630-648
  Tensor unary(UnOp op, const Tensor& x) override {
    if (x.dt == Dtype::U32) {
      CG_CHECK(op == UnOp::Neg, ERR_UNSUPPORTED_DTYPE, "Invalid input types for unary float op");
      auto v = load_u(x);
      for (auto& e : v) e = 0u - e;  // wrapping_neg
      return store_u(v, x.shape);
    }
    auto v = load_f(x);
    for (auto& e : v) {
      switch (op) {
        case UnOp::Neg: e = -e; break;
        case UnOp::Sin: e = sinf(e); break;
        case UnOp::Cos: e = cosf(e); break;
        case UnOp::Exp: e = expf(e); break;
        case UnOp::Log: e = logf(e); break;
        case UnOp::Floor: e = floorf(e); break;
        case UnOp::Round: e = nearbyintf(e); break;  // round_ties_even under the default rounding mode
      }
    }
    return store_f(v, x.shape, x.dt);
  }

  // ndarray.rs:553-559 (materialised there; a stride-0 view here has the same logical contents)
  Tensor broadcast(const Tensor& x, const Shape& shape) override { return view_broadcast(x, shape); }
  // ndarray.rs:545-551
  Tensor reshape(const Tensor& x, const Shape& shape) override {
    CG_CHECK(numel(shape) == x.size(), ERR_SHAPE_MISMATCH,
             "reshape: " + shape_str(x.shape) + " -> " + shape_str(shape));
    return materialize(x, shape);
  }
  // ndarray.rs:561-569
  Tensor transpose(const Tensor& x, int64_t d0, int64_t d1) override { return view_transpose(x, d0, d1); }

  static Shape reduced(const Tensor& x) {
    CG_CHECK(x.rank() >= 1, ERR_SHAPE_MISMATCH, "reduction needs rank >= 1");
    Shape s = x.shape;
    s.back() = 1;
    return s;
  }

  // ndarray.rs:656-668
  Tensor max(const Tensor& x) override {
    Shape os = reduced(x);
    int64_t n = x.shape.back(), rows = numel(os);
    if (x.dt == Dtype::U32) {
      auto v = load_u(x);
      std::vector<uint32_t> r((size_t)rows);
      for (int64_t i = 0; i < rows; ++i) {
        uint32_t acc = 0;
        for (int64_t j = 0; j < n; ++j) acc = std::max(acc, v[i * n + j]);
        r[i] = acc;
      }
      return store_u(r, os);
    }
    auto v = load_f(x);
    std::vector<float> r((size_t)rows);
    for (int64_t i = 0; i < rows; ++i) {
      float acc = std::numeric_limits<float>::lowest();  // f32::MIN, not -inf
      for (int64_t j = 0; j < n; ++j) acc = rust_max(acc, v[i * n + j]);
      r[i] = acc;
    }
    return store_f(r, os, x.dt);
  }

  // ndarray.rs:723-730
  Tensor sum(const Tensor& x) override {
    Shape os = reduced(x);
    int64_t n = x.shape.back(), rows = numel(os);
    if (x.dt == Dtype::U32) {
      auto v = load_u(x);
      std::vector<uint32_t> r((size_t)rows);
      for (int64_t i = 0; i < rows; ++i) {
        uint32_t acc = 0;
        for (int64_t j = 0; j < n; ++j) acc += v[i * n + j];
        r[i] = acc;
      }
      return store_u(r, os);
    }
    auto v = load_f(x);
    std::vector<float> r((size_t)rows);
    for (int64_t i = 0; i < rows; ++i) {
      float acc = 0.f;
      for (int64_t j = 0; j < n; ++j) acc += v[i * n + j];
      r[i] = acc;
    }
    return store_f(r, os, x.dt);
  }

  // ndarray.rs:670-694: Iterator::max_by keeps the LAST of equal maxima; floats order by total_cmp
  Tensor argmax(const Tensor& x) override {
    Shape os = reduced(x);
    int64_t n = x.shape.back(), rows = numel(os);
    CG_CHECK(n > 0, ERR_INVALID_ARG, "argmax over an empty axis");
    std::vector<uint32_t> r((size_t)rows);
    if (x.dt == Dtype::U32) {
      auto v = load_u(x);
      for (int64_t i = 0; i < rows; ++i) {
        int64_t best = 0;
        for (int64_t j = 1; j < n; ++j)
          if (v[i * n + j] >= v[i * n + best]) best = j;
        r[i] = (uint32_t)best;
      }
    } else {
      auto v = load_f(x);
      for (int64_t i = 0; i < rows; ++i) {
        int64_t best = 0;
        for (int64_t j = 1; j < n; ++j)
          if (total_key(v[i * n + j]) >= total_key(v[i * n + best])) best = j;
        r[i] = (uint32_t)best;
      }
    }
    return store_u(r, os);
  }

  // ndarray.rs:696-721: stable sort, descending by total_cmp; equal values keep their original order
  std::pair<Tensor, Tensor> topk(const Tensor& x, int64_t k) override {
    CG_CHECK(x.dt != Dtype::U32, ERR_UNSUPPORTED_DTYPE, "Unsupported type for topk");
    CG_CHECK(x.rank() >= 1 && k <= x.shape.back(), ERR_INVALID_ARG, "topk: k exceeds the last axis");
    Shape os = x.shape;
    int64_t n = x.shape.back();
    os.back() = k;
    int64_t rows = n ? x.size() / n : 0;
    auto v = load_f(x);
    std::vector<float> vals;
    std::vector<uint32_t> idx;
    std::vector<int64_t> order((size_t)n);
    for (int64_t i = 0; i < rows; ++i) {
      std::iota(order.begin(), order.end(), 0);
      const float* lane = v.data() + i * n;
      std::stable_sort(order.begin(), order.end(),
                       [&](int64_t p, int64_t q) { return total_key(lane[p]) > total_key(lane[q]); });
      for (int64_t j = 0; j < k; ++j) {
        vals.push_back(lane[order[j]]);
        idx.push_back((uint32_t)order[j]);
      }
    }
    return {store_f(vals, os, x.dt), store_u(idx, os)};
  }

  // ndarray.rs:534-541: equal shapes and equal elements (NaN != NaN)
  bool compare(const Tensor& a, const Tensor& b) override {
    CG_CHECK(a.dt == b.dt, ERR_DTYPE_MISMATCH, "compare: operand dtypes differ");
    if (a.shape != b.shape) return false;
    if (a.dt == Dtype::U32) return load_u(a) == load_u(b);
    auto x = load_f(a), y = load_f(b);
    for (size_t i = 0; i < x.size(); ++i)
      if (!(x[i] == y[i])) return false;
    return true;
  }

  // ndarray.rs:513-532, 590-596
  Tensor concat(const Tensor& a, const Tensor& b, int64_t dim) override {
    CG_CHECK(a.dt == b.dt, ERR_DTYPE_MISMATCH, "Incompatible types for concatenation");
    CG_CHECK(a.rank() == b.rank() && dim >= 0 && dim < a.rank(), ERR_SHAPE_MISMATCH, "concat: rank/axis mismatch");
    for (int i = 0; i < a.rank(); ++i)
      CG_CHECK(i == dim || a.shape[i] == b.shape[i], ERR_SHAPE_MISMATCH,
               "concat: shapes differ off the concatenation axis: " + shape_str(a.shape) + " vs " + shape_str(b.shape));
    Shape os = a.shape;
    os[dim] += b.shape[dim];
    Tensor am = materialize(a, a.shape), bm = materialize(b, b.shape);
    Tensor t = alloc(os, a.dt);
    size_t es = dtype_size(a.dt);
    int64_t outer = 1, inner = 1;
    for (int i = 0; i < dim; ++i) outer *= os[i];
    for (int i = (int)dim + 1; i < a.rank(); ++i) inner *= os[i];
    size_t ca = (size_t)(a.shape[dim] * inner) * es, cb = (size_t)(b.shape[dim] * inner) * es;
    char* dst = (char*)t.st->ptr;
    for (int64_t o = 0; o < outer; ++o) {
      if (ca) std::memcpy(dst, (char*)am.st->ptr + o * ca, ca);
      dst += ca;
      if (cb) std::memcpy(dst, (char*)bm.st->ptr + o * cb, cb);
      dst += cb;
    }
    return t;
  }

  // ndarray.rs:466-487, 571-579: select(Axis(dim), indices flattened)
  Tensor index(const Tensor& x, int64_t dim, const Tensor& indices) override {
    CG_CHECK(indices.dt == Dtype::U32, ERR_DTYPE_MISMATCH, "Invalid input types for indexing");
    CG_CHECK(dim >= 0 && dim < x.rank(), ERR_INVALID_ARG, "index: axis out of range");
    auto idx = load_u(indices);
    Shape os = x.shape;
    os[dim] = (int64_t)idx.size();
    Tensor xm = materialize(x, x.shape);
    Tensor t = alloc(os, x.dt);
    size_t es = dtype_size(x.dt);
    int64_t outer = 1, inner = 1;
    for (int i = 0; i < dim; ++i) outer *= x.shape[i];
    for (int i = (int)dim + 1; i < x.rank(); ++i) inner *= x.shape[i];
    size_t chunk = (size_t)inner * es;
    for (int64_t o = 0; o < outer; ++o)
      for (size_t j = 0; j < idx.size(); ++j) {
        CG_CHECK((int64_t)idx[j] < x.shape[dim], ERR_INVALID_ARG, "index out of bounds");
        if (chunk)
          std::memcpy((char*)t.st->ptr + ((size_t)o * idx.size() + j) * chunk,
                      (char*)xm.st->ptr + ((size_t)o * x.shape[dim] + idx[j]) * chunk, chunk);
      }
    return t;
  }

  // ndarray.rs:489-502, 581-588
  Tensor slice(const Tensor& x, int64_t dim, int64_t start, int64_t len) override {
    return view_slice(x, dim, start, len);
  }

  // ndarray.rs:140-149
  bool to_bool(const Tensor& x) override {
    if (x.dt == Dtype::U32) {
      for (auto v : load_u(x))
        if (v != 0) return true;
      return false;
    }
    for (auto v : load_f(x))
      if (v > 0.f) return true;
    return false;
  }

  // ndarray.rs:50-59
  void to_vec(const Tensor& x, void* dst, size_t cap) override {
    size_t need = (size_t)x.size() * dtype_size(x.dt);
    CG_CHECK(cap >= need, ERR_INVALID_ARG, "to_vec: destination too small");
    Tensor m = materialize(x, x.shape);
    if (need) std::memcpy(dst, m.st->ptr, need);
  }
};
}  // namespace

Backend* make_backend(int /*device*/) { return new NdArrayRef(); }

}  // namespace cg

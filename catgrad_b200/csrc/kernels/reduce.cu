// Last-axis reductions (sum, max, argmax), gather along an axis, top-k, and the two host-visible
// predicates (`to_bool`, `compare`).
//
// Reference semantics (catgrad/src/interpreter/backend/ndarray.rs):
//   sum     :723-730  last axis, rank kept; f32 accumulate for float dtypes, wrapping for u32
//   max     :656-668  fold from f32::MIN (not -inf) with a NaN-ignoring max; u32 folds from 0
//   argmax  :670-694  u32 index of the LAST maximum under f32::total_cmp (u32: plain order)
//   index   :571-579  select(Axis(dim), indices)
//   topk    :696-721  stable descending sort by total_cmp, first k
//   to_bool :140-149  any element > 0 (u32: != 0);  compare :534-541  all elements equal
//
// HBM-bound: each input element is read once (algorithmic bytes = n x sizeof(T) per row + one output
// element).  Rows up to 1024 elements are reduced by one warp with shuffles; longer rows by one CTA
// (warp shuffles, then one shared-memory pass).  Reduction order is fixed, results are deterministic.
#include <cfloat>

#include <type_traits>

#include "argmax_two_stage.cuh"
#include "elementwise.h"

namespace cgk {
namespace {

template <class T> struct Acc;  // per-kind accumulators over values widened to f32 / u32

// Combined argmax key: high word orders by value (total_cmp image, biased to unsigned), low word by index,
// so the maximum picks the greatest value and, among equals, the greatest index.
template <class T> __device__ __forceinline__ unsigned long long arg_key(T v, unsigned idx) {
  unsigned hi;
  if constexpr (std::is_same<T, unsigned>::value) hi = v;
  else hi = (unsigned)total_key(Elem<T>::load(v)) ^ 0x80000000u;
  return ((unsigned long long)hi << 32) | idx;
}

template <class T, int KIND> struct Red {
  // value type carried through the reduction
  using V = typename std::conditional<KIND == R_ARGMAX, unsigned long long,
                                      typename std::conditional<std::is_same<T, unsigned>::value, unsigned, float>::type>::type;
  static __device__ __forceinline__ V init() {
    if constexpr (KIND == R_ARGMAX) return 0ull;
    else if constexpr (std::is_same<T, unsigned>::value) return 0u;
    else return KIND == R_SUM ? 0.f : -FLT_MAX;
  }
  static __device__ __forceinline__ V lift(T v, unsigned idx) {
    if constexpr (KIND == R_ARGMAX) return arg_key<T>(v, idx);
    else if constexpr (std::is_same<T, unsigned>::value) return v;
    else return Elem<T>::load(v);
  }
  static __device__ __forceinline__ V comb(V a, V b) {
    if constexpr (KIND == R_SUM) return a + b;
    else if constexpr (KIND == R_ARGMAX) return a > b ? a : b;
    else if constexpr (std::is_same<T, unsigned>::value) return a > b ? a : b;
    else return fmaxf(a, b);  // returns the non-NaN operand, like Rust's f32::max
  }
  using O = typename std::conditional<KIND == R_ARGMAX, unsigned, T>::type;
  static __device__ __forceinline__ O finish(V v) {
    if constexpr (KIND == R_ARGMAX) return (unsigned)(v & 0xffffffffull);
    else if constexpr (std::is_same<T, unsigned>::value) return v;
    else return Elem<T>::store(v);
  }
};

template <class V> __device__ __forceinline__ V shfl_xor(V v, int o) { return __shfl_xor_sync(0xffffffffu, v, o); }

template <class R, class V> __device__ __forceinline__ V warp_reduce(V v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = R::comb(v, shfl_xor(v, o));
  return v;
}

__device__ __forceinline__ long long row_offset(const View4& outer, long long row) {
  long long off = 0;
#pragma unroll 1
  for (int d = outer.rank - 1; d >= 0; --d) {
    long long s = outer.shape[d];
    long long q = row / s;
    off += (row - q * s) * outer.sa[d];
    row = q;
  }
  return off;
}

template <class T, int N> struct alignas(sizeof(T) * N) Vec { T v[N]; };

// Accumulates elements [lane_start, n) step `step` of one row.
template <class T, int KIND, int VEC>
__device__ __forceinline__ typename Red<T, KIND>::V row_partial(const T* p, long long n, long long stride, int tid,
                                                                 int nthreads) {
  using R = Red<T, KIND>;
  typename R::V acc = R::init();
  if (VEC > 1) {
    const long long nv = n / VEC;
    for (long long v = tid; v < nv; v += nthreads) {
      Vec<T, VEC> x = *reinterpret_cast<const Vec<T, VEC>*>(p + v * VEC);
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc = R::comb(acc, R::lift(x.v[i], (unsigned)(v * VEC + i)));
    }
  } else {
    for (long long i = tid; i < n; i += nthreads) acc = R::comb(acc, R::lift(p[i * stride], (unsigned)i));
  }
  return acc;
}

template <class T, int KIND, int VEC>
__global__ void __launch_bounds__(256) reduce_warp_kernel(View4 outer, long long rows, long long n, long long stride,
                                                          const T* __restrict__ a,
                                                          typename Red<T, KIND>::O* __restrict__ o) {
  using R = Red<T, KIND>;
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
    const T* p = a + row_offset(outer, row);
    auto acc = row_partial<T, KIND, VEC>(p, n, stride, lane, 32);
    acc = warp_reduce<R>(acc);
    if (lane == 0) o[row] = R::finish(acc);
  }
}

template <class T, int KIND, int VEC>
__global__ void __launch_bounds__(256) reduce_block_kernel(View4 outer, long long rows, long long n, long long stride,
                                                           const T* __restrict__ a,
                                                           typename Red<T, KIND>::O* __restrict__ o) {
  using R = Red<T, KIND>;
  __shared__ typename R::V part[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* p = a + row_offset(outer, row);
    auto acc = row_partial<T, KIND, VEC>(p, n, stride, threadIdx.x, 256);
    acc = warp_reduce<R>(acc);
    if (lane == 0) part[warp] = acc;
    __syncthreads();
    if (warp == 0) {
      auto v = lane < 8 ? part[lane] : R::init();
      v = warp_reduce<R>(v);
      if (lane == 0) o[row] = R::finish(v);
    }
    __syncthreads();
  }
}

template <class T, int KIND>
void launch_reduce_t(const View4& outer, long long rows, long long n, long long stride, const void* a, void* o,
                     int sm, cudaStream_t st) {
  using O = typename Red<T, KIND>::O;
  constexpr int VEC = 16 / sizeof(T);
  // vector path: unit inner stride, rows start on 16-byte boundaries
  bool vec = stride == 1 && n % VEC == 0 && ((uintptr_t)a % 16 == 0);
  for (int d = 0; d < outer.rank && vec; ++d) vec = outer.sa[d] % VEC == 0;
  if (n <= 1024) {
    long long blocks = (rows + 7) / 8;
    long long cap = (long long)sm * 8;
    int grid = (int)(blocks < cap ? (blocks < 1 ? 1 : blocks) : cap);
    if (vec) reduce_warp_kernel<T, KIND, VEC><<<grid, 256, 0, st>>>(outer, rows, n, stride, (const T*)a, (O*)o);
    else reduce_warp_kernel<T, KIND, 1><<<grid, 256, 0, st>>>(outer, rows, n, stride, (const T*)a, (O*)o);
  } else {
    long long cap = (long long)sm * 8;
    int grid = (int)(rows < cap ? rows : cap);
    if (vec) reduce_block_kernel<T, KIND, VEC><<<grid, 256, 0, st>>>(outer, rows, n, stride, (const T*)a, (O*)o);
    else reduce_block_kernel<T, KIND, 1><<<grid, 256, 0, st>>>(outer, rows, n, stride, (const T*)a, (O*)o);
  }
}

template <int KIND>
void launch_reduce_k(int dtype, const View4& outer, long long rows, long long n, long long stride, const void* a,
                     void* o, int sm, cudaStream_t st) {
  switch (dtype) {
    case DT_F32: launch_reduce_t<float, KIND>(outer, rows, n, stride, a, o, sm, st); break;
    case DT_BF16: launch_reduce_t<__nv_bfloat16, KIND>(outer, rows, n, stride, a, o, sm, st); break;
    case DT_F16: launch_reduce_t<__half, KIND>(outer, rows, n, stride, a, o, sm, st); break;
    case DT_U32: launch_reduce_t<unsigned, KIND>(outer, rows, n, stride, a, o, sm, st); break;
    default: break;
  }
}

// ---- gather -----------------------------------------------------------------------------------
// One "unit" = W bytes; a source/destination row is `row_units` units.
template <class U>
__global__ void __launch_bounds__(256) gather_kernel(const U* __restrict__ x, const unsigned* __restrict__ idx,
                                                     long long idx_stride, U* __restrict__ out, long long outer,
                                                     long long dim, long long n_idx, long long row_units,
                                                     unsigned* err) {
  const long long total = outer * n_idx * row_units;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    long long u = t % row_units;
    long long r = t / row_units;
    long long j = r % n_idx;
    long long o = r / n_idx;
    unsigned src = idx[j * idx_stride];
    if (src >= (unsigned long long)dim) {  // the reference panics; record and write zeros
      if (u == 0) atomicOr(err, DEV_ERR_INDEX_OOB);
      U z;
      memset(&z, 0, sizeof(U));
      out[t] = z;
      continue;
    }
    out[t] = x[(o * dim + src) * row_units + u];
  }
}

// ---- top-k ------------------------------------------------------------------------------------
// Selection j picks the greatest (value, lowest index) key strictly below selection j-1's key.
template <class T>
__global__ void __launch_bounds__(256) topk_kernel(const T* __restrict__ x, T* __restrict__ values,
                                                   unsigned* __restrict__ indices, long long n, long long k) {
  __shared__ unsigned long long part[8];
  __shared__ unsigned long long prev_s;
  const T* row = x + (long long)blockIdx.x * n;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned long long prev = ~0ull;
  for (long long j = 0; j < k; ++j) {
    unsigned long long best = 0ull;
    bool any = false;
    for (long long i = threadIdx.x; i < n; i += 256) {
      unsigned hi = (unsigned)total_key(Elem<T>::load(row[i])) ^ 0x80000000u;
      unsigned long long key = ((unsigned long long)hi << 32) | (0xffffffffu - (unsigned)i);
      if ((j == 0 || key < prev) && (!any || key > best)) {
        best = key;
        any = true;
      }
    }
    // keys are unique per element and never 0 for a valid candidate within a row of < 2^32 - 1 elements
    if (!any) best = 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    if (lane == 0) part[warp] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long b = part[0];
      for (int w = 1; w < 8; ++w) b = part[w] > b ? part[w] : b;
      prev_s = b;
      unsigned i = 0xffffffffu - (unsigned)(b & 0xffffffffull);
      values[(long long)blockIdx.x * k + j] = row[i];
      indices[(long long)blockIdx.x * k + j] = i;
    }
    __syncthreads();
    prev = prev_s;
  }
}

template <class T>
__global__ void __launch_bounds__(256) any_positive_kernel(const T* __restrict__ x, long long n, unsigned* flag) {
  bool hit = false;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    if constexpr (std::is_same<T, unsigned>::value) hit |= x[i] != 0u;
    else hit |= Elem<T>::load(x[i]) > 0.f;
  }
  if (__any_sync(0xffffffffu, hit) && (threadIdx.x & 31) == 0) atomicOr(flag, 1u);
}

template <class T>
__global__ void __launch_bounds__(256) any_diff_kernel(const T* __restrict__ a, const T* __restrict__ b, long long n,
                                                       unsigned* flag) {
  bool hit = false;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    if constexpr (std::is_same<T, unsigned>::value) hit |= a[i] != b[i];
    else hit |= !(Elem<T>::load(a[i]) == Elem<T>::load(b[i]));
  }
  if (__any_sync(0xffffffffu, hit) && (threadIdx.x & 31) == 0) atomicOr(flag, 1u);
}

inline int grid_for(long long items, int sm) {
  long long blocks = (items + 255) / 256, cap = (long long)sm * 8;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}
}  // namespace

// ---- fused last-axis softmax: the graph of stdlib nn::softmax (nn/mod.rs:168-179) in one pass --------------
// cast to f32, subtract the row maximum (folded from f32::MIN like `max`, ndarray.rs:656-661), exp, divide by the row
// sum, cast back.  One CTA per row, the row kept in registers (up to 256 x ITEMS x VEC elements); rows longer than
// that are re-read from global memory (L2) for the second and third pass.
template <class T, int ITEMS>
__global__ void __launch_bounds__(256) softmax_rows_kernel(const T* __restrict__ x, T* __restrict__ out, long long n) {
  constexpr int VEC = 16 / sizeof(T);
  __shared__ float red[8];
  const T* xr = x + (long long)blockIdx.x * n;
  T* orow = out + (long long)blockIdx.x * n;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float v[ITEMS][VEC];
  float mx = -FLT_MAX;
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    const long long t0 = ((long long)j * 256 + threadIdx.x) * VEC;
    if (t0 < n) {
      const Vec<T, VEC> in = *reinterpret_cast<const Vec<T, VEC>*>(xr + t0);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        v[j][i] = Elem<T>::load(in.v[i]);
        mx = fmaxf(mx, v[j][i]);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    const long long t0 = ((long long)j * 256 + threadIdx.x) * VEC;
    if (t0 < n) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        v[j][i] = expf(v[j][i] - mx);
        sum += v[j][i];
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = ((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]));
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    const long long t0 = ((long long)j * 256 + threadIdx.x) * VEC;
    if (t0 < n) {
      Vec<T, VEC> o;
#pragma unroll
      for (int i = 0; i < VEC; ++i) o.v[i] = Elem<T>::store(v[j][i] / sum);
      *reinterpret_cast<Vec<T, VEC>*>(orow + t0) = o;
    }
  }
}

// any row length and alignment: three passes over global memory (the row stays in L2)
template <class T>
__global__ void __launch_bounds__(256) softmax_rows_generic_kernel(const T* __restrict__ x, T* __restrict__ out, long long n) {
  __shared__ float red[8];
  const T* xr = x + (long long)blockIdx.x * n;
  T* orow = out + (long long)blockIdx.x * n;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float mx = -FLT_MAX;
  for (long long t = threadIdx.x; t < n; t += 256) mx = fmaxf(mx, Elem<T>::load(xr[t]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  float sum = 0.f;
  for (long long t = threadIdx.x; t < n; t += 256) sum += expf(Elem<T>::load(xr[t]) - mx);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  sum = ((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]));
  for (long long t = threadIdx.x; t < n; t += 256) orow[t] = Elem<T>::store(expf(Elem<T>::load(xr[t]) - mx) / sum);
}

template <class T>
void launch_softmax_t(const void* x, void* out, long long rows, long long n, cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(T);
  const bool vec = n % VEC == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)out % 16 == 0);
  const long long per_item = 256ll * VEC;
  if (vec && n <= per_item * 1)
    softmax_rows_kernel<T, 1><<<(unsigned)rows, 256, 0, st>>>((const T*)x, (T*)out, n);
  else if (vec && n <= per_item * 2)
    softmax_rows_kernel<T, 2><<<(unsigned)rows, 256, 0, st>>>((const T*)x, (T*)out, n);
  else if (vec && n <= per_item * 4)
    softmax_rows_kernel<T, 4><<<(unsigned)rows, 256, 0, st>>>((const T*)x, (T*)out, n);
  else if (vec && n <= per_item * 8)
    softmax_rows_kernel<T, 8><<<(unsigned)rows, 256, 0, st>>>((const T*)x, (T*)out, n);
  else
    softmax_rows_generic_kernel<T><<<(unsigned)rows, 256, 0, st>>>((const T*)x, (T*)out, n);
}

void launch_softmax(int dtype, const void* x, void* out, long long rows, long long n, cudaStream_t st) {
  switch (dtype) {
    case DT_F32: launch_softmax_t<float>(x, out, rows, n, st); break;
    case DT_BF16: launch_softmax_t<__nv_bfloat16>(x, out, rows, n, st); break;
    default: launch_softmax_t<__half>(x, out, rows, n, st); break;
  }
}

void launch_reduce(int kind, int dtype, const View4& outer, long long rows, long long n, long long inner_stride,
                   const void* a, void* o, int sm, cudaStream_t st) {
  if (rows <= 0) return;
  switch (kind) {
    case R_SUM: launch_reduce_k<R_SUM>(dtype, outer, rows, n, inner_stride, a, o, sm, st); break;
    case R_MAX: launch_reduce_k<R_MAX>(dtype, outer, rows, n, inner_stride, a, o, sm, st); break;
    case R_ARGMAX: launch_reduce_k<R_ARGMAX>(dtype, outer, rows, n, inner_stride, a, o, sm, st); break;
  }
}

// Few long rows of a float dtype (rows start `row_stride` elements apart, unit inner stride): the two-stage pick.
// `scratch` holds rows * ceil(n / 4096) 64-bit keys.
void launch_argmax_two_stage(int dtype, const void* x, long long row_stride, long long rows, long long n, void* scratch,
                             unsigned* out, cudaStream_t st) {
  const unsigned chunks = (unsigned)((n + ARGMAX_STAGE_CHUNK - 1) / ARGMAX_STAGE_CHUNK);
  dim3 grid(chunks, (unsigned)rows);
  unsigned long long* part = (unsigned long long*)scratch;
  switch (dtype) {
    case DT_F32: argmax_stage1_kernel<float><<<grid, 256, 0, st>>>((const float*)x, row_stride, (int)n, part); break;
    case DT_BF16: argmax_stage1_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, row_stride, (int)n, part); break;
    default: argmax_stage1_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, row_stride, (int)n, part); break;
  }
  argmax_finish_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(part, (int)chunks, (int)rows, out);
}

void launch_gather(int elem_size, const void* x, const unsigned* idx, long long idx_stride, void* out, long long outer,
                   long long dim, long long n_idx, long long inner, unsigned* err, int sm, cudaStream_t st) {
  long long row_bytes = inner * elem_size;
  long long total_rows = outer * n_idx;
  if (total_rows <= 0 || row_bytes <= 0) return;
  bool a16 = row_bytes % 16 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0;
  if (a16) {
    long long units = row_bytes / 16;
    gather_kernel<uint4><<<grid_for(total_rows * units, sm), 256, 0, st>>>((const uint4*)x, idx, idx_stride, (uint4*)out,
                                                                          outer, dim, n_idx, units, err);
  } else if (elem_size == 4) {
    gather_kernel<unsigned><<<grid_for(total_rows * inner, sm), 256, 0, st>>>((const unsigned*)x, idx, idx_stride,
                                                                              (unsigned*)out, outer, dim, n_idx, inner, err);
  } else if (elem_size == 2) {
    gather_kernel<unsigned short><<<grid_for(total_rows * inner, sm), 256, 0, st>>>(
        (const unsigned short*)x, idx, idx_stride, (unsigned short*)out, outer, dim, n_idx, inner, err);
  } else {
    gather_kernel<unsigned char><<<grid_for(total_rows * inner, sm), 256, 0, st>>>(
        (const unsigned char*)x, idx, idx_stride, (unsigned char*)out, outer, dim, n_idx, inner, err);
  }
}

void launch_topk(int dtype, const void* x, void* values, unsigned* indices, long long rows, long long n, long long k,
                 cudaStream_t st) {
  if (rows <= 0 || k <= 0) return;
  switch (dtype) {
    case DT_F32: topk_kernel<float><<<(int)rows, 256, 0, st>>>((const float*)x, (float*)values, indices, n, k); break;
    case DT_BF16:
      topk_kernel<__nv_bfloat16><<<(int)rows, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)values, indices, n, k);
      break;
    case DT_F16: topk_kernel<__half><<<(int)rows, 256, 0, st>>>((const __half*)x, (__half*)values, indices, n, k); break;
    default: break;
  }
}

void launch_any_positive(int dtype, const void* x, long long n, unsigned* flag, int sm, cudaStream_t st) {
  if (n <= 0) return;
  int g = grid_for(n, sm);
  switch (dtype) {
    case DT_F32: any_positive_kernel<float><<<g, 256, 0, st>>>((const float*)x, n, flag); break;
    case DT_BF16: any_positive_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)x, n, flag); break;
    case DT_F16: any_positive_kernel<__half><<<g, 256, 0, st>>>((const __half*)x, n, flag); break;
    case DT_U32: any_positive_kernel<unsigned><<<g, 256, 0, st>>>((const unsigned*)x, n, flag); break;
    default: break;
  }
}
void launch_any_diff(int dtype, const void* a, const void* b, long long n, unsigned* flag, int sm, cudaStream_t st) {
  if (n <= 0) return;
  int g = grid_for(n, sm);
  switch (dtype) {
    case DT_F32: any_diff_kernel<float><<<g, 256, 0, st>>>((const float*)a, (const float*)b, n, flag); break;
    case DT_BF16:
      any_diff_kernel<__nv_bfloat16><<<g, 256, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, n, flag);
      break;
    case DT_F16: any_diff_kernel<__half><<<g, 256, 0, st>>>((const __half*)a, (const __half*)b, n, flag); break;
    case DT_U32: any_diff_kernel<unsigned><<<g, 256, 0, st>>>((const unsigned*)a, (const unsigned*)b, n, flag); break;
    default: break;
  }
}

}  // namespace cgk

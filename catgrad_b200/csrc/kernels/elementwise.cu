// Pointwise kernels over strided/broadcast views: binary and unary maps, where, cast, strided copy.
//
// Replaces the ndarray backend's pointwise methods (catgrad/src/interpreter/backend/ndarray.rs:185-407,
// 598-654) and its cast (ndarray.rs:151-174).  Broadcast operands stay stride-0 views and are expanded
// in registers; the reference materialises them first (ndarray.rs:553-559).
//
// HBM-bound.  Fast path: 16-byte vector loads/stores along the innermost collapsed axis (each operand's
// inner stride is 1 or 0), grid-stride over vectors; the grid is sized in whole waves of 148 SMs.
// Algorithmic bytes per element: (inputs read + 1 written) x sizeof(T); a broadcast operand adds none.
//
// Float dtypes compute in f32 and round once at the output (bf16/f16: candle.rs:1165-1192).  No FMA
// contraction (file is compiled with -fmad=false): add/sub/mul/div/neg/floor/round/compare/where/cast are
// bit-exact against the CPU restatement.
#include <type_traits>

#include "elementwise.h"

namespace cgk {
namespace {

// ---- op functors -------------------------------------------------------------------------------
__device__ __forceinline__ unsigned u32_pow(unsigned base, unsigned exp) {
  unsigned r = 1;
  while (exp) {
    if (exp & 1u) r *= base;
    base *= base;
    exp >>= 1;
  }
  return r;
}

template <int OP> struct Bin {
  static __device__ __forceinline__ float f(float a, float b) {
    if (OP == B_ADD) return a + b;
    if (OP == B_SUB) return a - b;
    if (OP == B_MUL) return a * b;
    if (OP == B_DIV) return a / b;
    if (OP == B_POW) return powf(a, b);
    if (OP == B_LT) return a < b ? 1.f : 0.f;
    if (OP == B_GT) return a > b ? 1.f : 0.f;
    if (OP == B_GTE) return a >= b ? 1.f : 0.f;
    if (OP == B_LTE) return a <= b ? 1.f : 0.f;
    return a == b ? 1.f : 0.f;
  }
  static __device__ __forceinline__ unsigned u(unsigned a, unsigned b, unsigned* err) {
    if (OP == B_ADD) return a + b;
    if (OP == B_SUB) return a - b;
    if (OP == B_MUL) return a * b;
    if (OP == B_DIV) {
      if (b == 0u) {
        atomicOr(err, DEV_ERR_DIV_ZERO);
        return 0xffffffffu;
      }
      return a / b;
    }
    if (OP == B_POW) return u32_pow(a, b);
    if (OP == B_LT) return a < b;
    if (OP == B_GT) return a > b;
    if (OP == B_GTE) return a >= b;
    if (OP == B_LTE) return a <= b;
    return a == b;
  }
};

template <int OP> struct Un {
  static __device__ __forceinline__ float f(float a) {
    if (OP == U_NEG) return -a;
    if (OP == U_SIN) return sinf(a);
    if (OP == U_COS) return cosf(a);
    if (OP == U_EXP) return expf(a);
    if (OP == U_LOG) return logf(a);
    if (OP == U_FLOOR) return floorf(a);
    return rintf(a);  // ties to even
  }
};

template <class T, int N> struct alignas(sizeof(T) * N) Vec { T v[N]; };

template <class I>
struct Offs { I a, b, c, o; };

// Decomposes the linear element index e over the collapsed shape; accumulates per-operand offsets.
template <class I>
__device__ __forceinline__ Offs<I> decompose(const View4& vw, I e) {
  Offs<I> r{0, 0, 0, 0};
#pragma unroll 1
  for (int d = vw.rank - 1; d >= 0; --d) {
    I s = (I)vw.shape[d];
    I q = e / s;
    I c = e - q * s;
    e = q;
    r.a += c * (I)vw.sa[d];
    r.b += c * (I)vw.sb[d];
    r.c += c * (I)vw.sc[d];
    r.o += c * (I)vw.so[d];
  }
  return r;
}

// Loads VEC elements of one operand: vector load if its inner stride is 1, a splat if it is 0.
template <class T, int VEC, class I>
__device__ __forceinline__ Vec<T, VEC> load_vec(const T* p, I off, long long inner_stride) {
  Vec<T, VEC> r;
  if (inner_stride == 1) {
    r = *reinterpret_cast<const Vec<T, VEC>*>(p + off);
  } else {
    T s = p[off];
#pragma unroll
    for (int i = 0; i < VEC; ++i) r.v[i] = s;
  }
  return r;
}

enum { K_BIN = 0, K_UN = 1, K_WHERE = 2, K_COPY = 3 };

// One kernel body for all pointwise maps over one element type.  KIND/OP select the arithmetic.
template <class T, int KIND, int OP, int VEC, class I>
__global__ void __launch_bounds__(256) ew_kernel(View4 vw, const T* __restrict__ a, const T* __restrict__ b,
                                                 const T* __restrict__ c, T* __restrict__ o, unsigned* err) {
  const int last = vw.rank - 1;
  const long long nvec = vw.total / VEC;
  const long long ia = vw.sa[last], ib = vw.sb[last], ic = vw.sc[last];
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    Offs<I> of = decompose<I>(vw, (I)(v * VEC));
    Vec<T, VEC> va = load_vec<T, VEC, I>(a, of.a, VEC == 1 ? 1 : ia), vb, vc, vo;
    if (KIND == K_BIN || KIND == K_WHERE) vb = load_vec<T, VEC, I>(b, of.b, VEC == 1 ? 1 : ib);
    if (KIND == K_WHERE) vc = load_vec<T, VEC, I>(c, of.c, VEC == 1 ? 1 : ic);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      if constexpr (KIND == K_COPY) {
        vo.v[i] = va.v[i];
      } else if constexpr (sizeof(T) == 4 && !std::is_same<T, float>::value) {  // uint32_t
        if (KIND == K_BIN) vo.v[i] = Bin<OP>::u(va.v[i], vb.v[i], err);
        if (KIND == K_UN) vo.v[i] = 0u - va.v[i];  // wrapping neg (ndarray.rs:634-638)
        if (KIND == K_WHERE) vo.v[i] = va.v[i] != 0u ? vb.v[i] : vc.v[i];
      } else {
        float fa = Elem<T>::load(va.v[i]);
        if (KIND == K_BIN) vo.v[i] = Elem<T>::store(Bin<OP>::f(fa, Elem<T>::load(vb.v[i])));
        if (KIND == K_UN) vo.v[i] = Elem<T>::store(Un<OP>::f(fa));
        if (KIND == K_WHERE) vo.v[i] = fa > 0.f ? vb.v[i] : vc.v[i];  // NaN mask selects y (ndarray.rs:325-336)
      }
    }
    if (VEC == 1)
      o[of.o] = vo.v[0];
    else
      *reinterpret_cast<Vec<T, VEC>*>(o + of.o) = vo;
  }
}

template <class TI, class TO> __device__ __forceinline__ TO cast_one(TI v) {
  if constexpr (std::is_same<TI, unsigned>::value) {
    if constexpr (std::is_same<TO, unsigned>::value) return v;
    else return Elem<TO>::store(__uint2float_rn(v));
  } else {
    float f = Elem<TI>::load(v);
    if constexpr (std::is_same<TO, unsigned>::value) return __float2uint_rz(f);  // truncates, saturates, NaN -> 0
    else return Elem<TO>::store(f);
  }
}

// Cast: strided input, contiguous output.
template <class TI, class TO, int VEC, class I>
__global__ void __launch_bounds__(256) cast_kernel(View4 vw, const TI* __restrict__ a, TO* __restrict__ o) {
  const long long nvec = vw.total / VEC;
  const long long ia = vw.sa[vw.rank - 1];
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long long)gridDim.x * blockDim.x) {
    Offs<I> of = decompose<I>(vw, (I)(v * VEC));
    Vec<TI, VEC> va = load_vec<TI, VEC, I>(a, of.a, VEC == 1 ? 1 : ia);
    Vec<TO, VEC> vo;
#pragma unroll
    for (int i = 0; i < VEC; ++i) vo.v[i] = cast_one<TI, TO>(va.v[i]);
    if (VEC == 1)
      o[of.o] = vo.v[0];
    else
      *reinterpret_cast<Vec<TO, VEC>*>(o + of.o) = vo;
  }
}

__global__ void arange_kernel(unsigned* o, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    o[i] = (unsigned)i;
}

inline int grid_for(long long work_items, int block, int sm_count) {
  long long blocks = (work_items + block - 1) / block;
  long long cap = (long long)sm_count * 8;  // whole waves: 8 resident CTAs of 256 threads per SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

inline bool fits_i32(const View4& vw) {
  if (vw.total >= (1ll << 31)) return false;
  long long m[4] = {0, 0, 0, 0};
  for (int d = 0; d < vw.rank; ++d) {
    m[0] += (vw.shape[d] - 1) * vw.sa[d];
    m[1] += (vw.shape[d] - 1) * vw.sb[d];
    m[2] += (vw.shape[d] - 1) * vw.sc[d];
    m[3] += (vw.shape[d] - 1) * vw.so[d];
  }
  for (long long x : m)
    if (x >= (1ll << 31)) return false;
  return true;
}

template <class T, int KIND, int OP>
void launch_ew_t(const View4& vw, int vec, const void* a, const void* b, const void* c, void* o, unsigned* err,
                 int sm_count, cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(T);
  bool i32 = fits_i32(vw);
  long long items = vec > 1 ? vw.total / VEC : vw.total;
  int grid = grid_for(items, 256, sm_count);
#define GO(V, I) ew_kernel<T, KIND, OP, V, I><<<grid, 256, 0, st>>>(vw, (const T*)a, (const T*)b, (const T*)c, (T*)o, err)
  if (vec > 1) {
    if (i32) GO(VEC, int); else GO(VEC, long long);
  } else {
    if (i32) GO(1, int); else GO(1, long long);
  }
#undef GO
}

template <int KIND, int OP>
void launch_ew(int dtype, const View4& vw, int vec, const void* a, const void* b, const void* c, void* o,
               unsigned* err, int sm_count, cudaStream_t st) {
  switch (dtype) {
    case DT_F32: launch_ew_t<float, KIND, OP>(vw, vec, a, b, c, o, err, sm_count, st); break;
    case DT_BF16: launch_ew_t<__nv_bfloat16, KIND, OP>(vw, vec, a, b, c, o, err, sm_count, st); break;
    case DT_F16: launch_ew_t<__half, KIND, OP>(vw, vec, a, b, c, o, err, sm_count, st); break;
    case DT_U32: launch_ew_t<unsigned, KIND, OP>(vw, vec, a, b, c, o, err, sm_count, st); break;
    default: break;
  }
}

template <class TI, class TO>
void launch_cast_t(const View4& vw, int vec, const void* a, void* o, int sm_count, cudaStream_t st) {
  constexpr int VEC = 16 / (sizeof(TI) > sizeof(TO) ? sizeof(TI) : sizeof(TO));
  bool i32 = fits_i32(vw);
  long long items = vec > 1 ? vw.total / VEC : vw.total;
  int grid = grid_for(items, 256, sm_count);
  if (vec > 1) {
    if (i32) cast_kernel<TI, TO, VEC, int><<<grid, 256, 0, st>>>(vw, (const TI*)a, (TO*)o);
    else cast_kernel<TI, TO, VEC, long long><<<grid, 256, 0, st>>>(vw, (const TI*)a, (TO*)o);
  } else {
    if (i32) cast_kernel<TI, TO, 1, int><<<grid, 256, 0, st>>>(vw, (const TI*)a, (TO*)o);
    else cast_kernel<TI, TO, 1, long long><<<grid, 256, 0, st>>>(vw, (const TI*)a, (TO*)o);
  }
}

template <class TI>
void launch_cast_from(int dt_out, const View4& vw, int vec, const void* a, void* o, int sm, cudaStream_t st) {
  switch (dt_out) {
    case DT_F32: launch_cast_t<TI, float>(vw, vec, a, o, sm, st); break;
    case DT_BF16: launch_cast_t<TI, __nv_bfloat16>(vw, vec, a, o, sm, st); break;
    case DT_F16: launch_cast_t<TI, __half>(vw, vec, a, o, sm, st); break;
    case DT_F8: launch_cast_t<TI, fp8_t>(vw, vec, a, o, sm, st); break;
    case DT_U32: launch_cast_t<TI, unsigned>(vw, vec, a, o, sm, st); break;
  }
}
}  // namespace

int vector_width(int elem_size_in, int elem_size_out) {
  int m = elem_size_in > elem_size_out ? elem_size_in : elem_size_out;
  return 16 / m;
}

void launch_binary(int op, int dtype, const View4& vw, int vec, const void* a, const void* b, void* o,
                   unsigned* err, int sm, cudaStream_t st) {
  switch (op) {
#define C(OPC) case OPC: launch_ew<K_BIN, OPC>(dtype, vw, vec, a, b, nullptr, o, err, sm, st); break;
    C(B_ADD) C(B_SUB) C(B_MUL) C(B_DIV) C(B_POW) C(B_LT) C(B_GT) C(B_GTE) C(B_LTE) C(B_EQ)
#undef C
  }
}
void launch_unary(int op, int dtype, const View4& vw, int vec, const void* a, void* o, int sm, cudaStream_t st) {
  switch (op) {
#define C(OPC) case OPC: launch_ew<K_UN, OPC>(dtype, vw, vec, a, nullptr, nullptr, o, nullptr, sm, st); break;
    C(U_NEG) C(U_SIN) C(U_COS) C(U_EXP) C(U_LOG) C(U_FLOOR) C(U_ROUND)
#undef C
  }
}
void launch_where(int dtype, const View4& vw, int vec, const void* m, const void* x, const void* y, void* o, int sm,
                  cudaStream_t st) {
  launch_ew<K_WHERE, 0>(dtype, vw, vec, m, x, y, o, nullptr, sm, st);
}
// Raw strided copy by element size (any dtype); output may be a strided view too (used by concat).
void launch_copy(int elem_size, const View4& vw, int vec, const void* a, void* o, int sm, cudaStream_t st) {
  switch (elem_size) {
    case 4: launch_ew_t<unsigned, K_COPY, 0>(vw, vec, a, nullptr, nullptr, o, nullptr, sm, st); break;
    case 2: launch_ew_t<unsigned short, K_COPY, 0>(vw, vec, a, nullptr, nullptr, o, nullptr, sm, st); break;
    default: launch_ew_t<unsigned char, K_COPY, 0>(vw, vec, a, nullptr, nullptr, o, nullptr, sm, st); break;
  }
}
void launch_cast(int dt_in, int dt_out, const View4& vw, int vec, const void* a, void* o, int sm, cudaStream_t st) {
  switch (dt_in) {
    case DT_F32: launch_cast_from<float>(dt_out, vw, vec, a, o, sm, st); break;
    case DT_BF16: launch_cast_from<__nv_bfloat16>(dt_out, vw, vec, a, o, sm, st); break;
    case DT_F16: launch_cast_from<__half>(dt_out, vw, vec, a, o, sm, st); break;
    case DT_F8: launch_cast_from<fp8_t>(dt_out, vw, vec, a, o, sm, st); break;
    case DT_U32: launch_cast_from<unsigned>(dt_out, vw, vec, a, o, sm, st); break;
  }
}
void launch_arange(unsigned* o, long long n, int sm, cudaStream_t st) {
  if (n <= 0) return;
  arange_kernel<<<grid_for(n, 256, sm), 256, 0, st>>>(o, n);
}

}  // namespace cgk

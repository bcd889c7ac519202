// Device helpers shared by all kernels: element conversions, strided-view descriptors, error word.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cgk {

constexpr int MAX_RANK = 8;

// Sticky device-side error bits, read by the host at the next synchronising call.  Kernels never trap:
// a bad index records a bit and skips the access.
enum DevError : unsigned int {
  DEV_ERR_DIV_ZERO = 1u,       // u32 division by zero (the reference panics)
  DEV_ERR_INDEX_OOB = 2u,      // gather index outside the axis (the reference panics)
  DEV_ERR_WAIT_TIMEOUT = 4u,   // a bounded device-side wait gave up
};

// ---- element <-> f32 -----------------------------------------------------------------------
template <class T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float load(float v) { return v; }
  static __device__ __forceinline__ float store(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
  // bf16 -> f32 is a 16-bit shift: exact, and NaN payloads/signs pass through unchanged
  static __device__ __forceinline__ float load(__nv_bfloat16 v) {
    return __uint_as_float(((unsigned)__bfloat16_as_ushort(v)) << 16);
  }
  static __device__ __forceinline__ __nv_bfloat16 store(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float load(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half store(float v) { return __float2half_rn(v); }
};
struct fp8_t { uint8_t bits; };
template <> struct Elem<fp8_t> {
  static __device__ __forceinline__ float load(fp8_t v) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(v.bits, __NV_E4M3);
    return __half2float(__half(h));
  }
  static __device__ __forceinline__ fp8_t store(float v) {
    fp8_t r;
    r.bits = (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
    return r;
  }
};

// Up to three operands (a, b, c) and one output (o) over a common collapsed index space.
struct View4 {
  int rank;
  long long total;
  long long shape[MAX_RANK];
  long long sa[MAX_RANK], sb[MAX_RANK], sc[MAX_RANK], so[MAX_RANK];
};

// f32::total_cmp key (monotone signed integer image of the bit pattern).
__device__ __forceinline__ int total_key(float v) {
  int b = __float_as_int(v);
  return b ^ (int)(((unsigned)(b >> 31)) >> 1);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace cgk

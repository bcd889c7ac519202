// f32 matmul on the bf16 tensor cores without TF32: every f32 operand is split into three bf16 pieces
// (x = hi + mid + lo up to 2^-24 relative), and the six products whose pieces' orders sum to at most two
//   lo*hi, mid*mid, hi*lo, mid*hi, hi*mid, hi*hi
// are accumulated in f32 by ONE tensor-core GEMM whose K axis is the six segments side by side, smallest first:
//   A' [M, 6K] = [lo | mid | hi | mid | hi | hi],   B' [N, 6K] = [hi | mid | lo | hi | mid | hi].
// bf16 x bf16 products are exact in f32, so what is left is the dropped third-order terms (~2^-24 relative to
// |a||b|) and the accumulation: the tensor core adds into its f32 accumulator with truncation, which costs up to one
// ulp of the running sum per 16-deep MMA step.  Measured against float64: ~5e-6 of the largest entry at K = 256..1024,
// some 50x above an f32 FMA chain and 1000x below a TF32 or single-bf16 product; the small products go first so that
// they meet a small accumulator.  This is the `matmul` of the
// trait (catgrad/src/interpreter/backend/mod.rs:61; ndarray.rs:732-816) for f32 tensors large enough to pay for the
// two split passes; small or oddly laid out products stay on the SIMT kernel of matmul.cu.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>

#include "gemm_tcgen05.h"
#include "matmul.h"

namespace cgk {
namespace {

__device__ __forceinline__ void split3(float x, __nv_bfloat16& hi, __nv_bfloat16& mid, __nv_bfloat16& lo) {
  hi = __float2bfloat16_rn(x);
  const float r1 = x - __bfloat162float(hi);
  mid = __float2bfloat16_rn(r1);
  const float r2 = r1 - __bfloat162float(mid);
  lo = __float2bfloat16_rn(r2);
}

// piece index (0 hi, 1 mid, 2 lo) of segment s for the left / right operand
__device__ __forceinline__ int piece_of(int seg, int is_b) {
  // A: 2 1 0 1 0 0   B: 0 1 2 0 1 0  (smallest products first, see the header)
  const unsigned code = is_b ? 0x010210u : 0x001012u;  // nibble s (from the low end) = piece of segment s
  return (code >> (4 * seg)) & 3;
}

// x [rows, K] row-major -> out [rows, 6K]; one thread per 4 consecutive k of a row
__global__ void __launch_bounds__(256) split_rows_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                         long long rows, int K, int is_b) {
  const long long total = rows * (K / 4);
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long r = t / (K / 4);
    const int k = (int)(t - r * (K / 4)) * 4;
    const float4 v = *reinterpret_cast<const float4*>(x + r * K + k);
    const float in[4] = {v.x, v.y, v.z, v.w};
    __nv_bfloat16 p[3][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) split3(in[i], p[0][i], p[1][i], p[2][i]);
    __nv_bfloat16* o = out + r * 6 * K + k;
#pragma unroll
    for (int s = 0; s < 6; ++s) {
      const int pc = piece_of(s, is_b);
      const __nv_bfloat162 a = __halves2bfloat162(p[pc][0], p[pc][1]), b = __halves2bfloat162(p[pc][2], p[pc][3]);
      *reinterpret_cast<uint2*>(o + (long long)s * K) =
          make_uint2(*reinterpret_cast<const unsigned*>(&a), *reinterpret_cast<const unsigned*>(&b));
    }
  }
}

// x [batch, K, N] row-major -> out [batch, N, 6K] (the right operand made K-contiguous while it is split);
// 32 x 32 tiles through shared memory so that both sides are coalesced.  grid (N/32, K/32, batch), 256 threads.
__global__ void __launch_bounds__(256) split_transpose_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                              int K, int N) {
  __shared__ float tile[32][33];
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  const float* xb = x + (long long)blockIdx.z * K * N;
  __nv_bfloat16* ob = out + (long long)blockIdx.z * N * 6 * K;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int i = ty; i < 32; i += 8) {
    const int k = k0 + i, n = n0 + tx;
    tile[i][tx] = (k < K && n < N) ? xb[(long long)k * N + n] : 0.f;
  }
  __syncthreads();
  for (int i = ty; i < 32; i += 8) {
    const int n = n0 + i, k = k0 + tx;
    if (n < N && k < K) {
      __nv_bfloat16 p[3];
      split3(tile[tx][i], p[0], p[1], p[2]);
      __nv_bfloat16* o = ob + (long long)n * 6 * K + k;
#pragma unroll
      for (int s = 0; s < 6; ++s) o[(long long)s * K] = p[piece_of(s, 1)];
    }
  }
}

}  // namespace

bool matmul_f32x3_applicable(long long M, long long N, long long K, long long batch) {
  if (!tcgen05_available()) return false;
  if (K % 8 != 0 || K < 64 || N < 64 || M * batch < 128 || batch > 65535) return false;
  return 2.0 * (double)M * (double)N * (double)K * (double)batch >= 2.68e8;   // ~2^28 flop: below that the split passes dominate
}

size_t matmul_f32x3_scratch_elems(long long rows, long long K) { return (size_t)rows * 6 * (size_t)K; }

bool launch_matmul_f32x3(const float* A, const float* B, float* C, void* a3, void* b3, long long M, long long N,
                         long long K, long long batch, bool b_row_major, bool b_shared, unsigned* err, int sm_count,
                         cudaStream_t st) {
  __nv_bfloat16* A3 = (__nv_bfloat16*)a3;
  __nv_bfloat16* B3 = (__nv_bfloat16*)b3;
  const long long a_rows = M * batch, b_batches = b_shared ? 1 : batch;
  const int grid = (int)std::min<long long>((a_rows * (K / 4) + 255) / 256, (long long)sm_count * 16);
  split_rows_kernel<<<grid, 256, 0, st>>>(A, A3, a_rows, (int)K, 0);
  if (b_row_major) {
    dim3 g((unsigned)((N + 31) / 32), (unsigned)((K + 31) / 32), (unsigned)b_batches);
    split_transpose_kernel<<<g, 256, 0, st>>>(B, B3, (int)K, (int)N);
  } else {
    const long long b_rows = N * b_batches;
    const int gb = (int)std::min<long long>((b_rows * (K / 4) + 255) / 256, (long long)sm_count * 16);
    split_rows_kernel<<<gb, 256, 0, st>>>(B, B3, b_rows, (int)K, 1);
  }
  if (cudaGetLastError() != cudaSuccess) return false;
  // a shared right operand: the batch is just more rows of A
  const long long Mg = b_shared ? M * batch : M, bg = b_shared ? 1 : batch;
  return launch_tcgen05_gemm_f32out(A3, B3, C, Mg, N, 6 * K, bg, Mg * 6 * K, N * 6 * K, err, sm_count, st);
}

}  // namespace cgk

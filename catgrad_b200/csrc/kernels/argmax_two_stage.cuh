// Two-stage last-axis argmax for few, long rows (a vocabulary-wide pick): one CTA per 4096-element chunk of a row, then
// one warp per row over the chunk results.  Shared by cg_argmax (scratch from the context's allocator) and
// cg_argmax_rows_noalloc (scratch in a fixed array of the library).
#pragma once
#include "common.cuh"

namespace cgk {

constexpr int ARGMAX_STAGE_CHUNK = 4096;  // elements of one row reduced by one CTA in stage 1

// Stage 1: CTA (chunk, row) reduces 4096 elements of one row to a 64-bit key: the value's image under
// f32::total_cmp in the high word, the index in the low word, so the greatest key is the LAST index among the
// greatest values (the rule of the reference's argmax, ndarray.rs:670-694).  Writes scratch[row * chunks + chunk].
template <class T>
__global__ void __launch_bounds__(256) argmax_stage1_kernel(const T* __restrict__ x, long long row_stride, int n,
                                                            unsigned long long* __restrict__ scratch) {
  __shared__ unsigned long long wbest[8];
  const int chunk = blockIdx.x, row = blockIdx.y, chunks = gridDim.x;
  const T* r = x + (long long)row * row_stride;
  const int lo = chunk * ARGMAX_STAGE_CHUNK, hi = min(n, lo + ARGMAX_STAGE_CHUNK);
  unsigned long long best = 0ull;
  for (int i = lo + threadIdx.x; i < hi; i += 256) {
    unsigned hiw = (unsigned)total_key(Elem<T>::load(r[i])) ^ 0x80000000u;
    unsigned long long key = ((unsigned long long)hiw << 32) | (unsigned)i;
    best = key > best ? key : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) wbest[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) best = wbest[w] > best ? wbest[w] : best;
    scratch[(long long)row * chunks + chunk] = best;
  }
}

// Stage 2: one warp per row reduces that row's partial keys; the low word of the greatest key is the index.
static __global__ void __launch_bounds__(256) argmax_finish_kernel(const unsigned long long* __restrict__ partials, int chunks,
                                                            int rows, unsigned* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  unsigned long long best = 0ull;
  for (int c = lane; c < chunks; c += 32) {
    unsigned long long k = partials[(long long)row * chunks + c];
    best = k > best ? k : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if (lane == 0) out[row] = (unsigned)(best & 0xffffffffull);
}

}  // namespace cgk

// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, TMEM accumulators, TMA-fed operands).
#pragma once
#include "common.cuh"

namespace cgk {
// True when the product can run on the tensor-core kernel: bf16, A rows K-contiguous, B either K-contiguous
// ("x @ W^T" layout, sbk == 1) or N-contiguous (a row-major [K, N] right operand, sbn == 1), 16-byte aligned
// bases and row pitches, more than 16 rows in total.
bool tcgen05_gemm_applicable(const View4& bt, long long batch, const void* A, const void* B, long long M, long long N,
                             long long K, long long sam, long long sak, long long sbk, long long sbn);
// C[batch, M, N] (contiguous bf16) = A x B^T-layout; f32 accumulation in TMEM, one rounding to bf16.
// Device-side waits are bounded; a timeout sets DEV_ERR_WAIT_TIMEOUT in *err and the kernel returns.
// Returns false (nothing launched) if the tensor maps cannot be made; the caller then uses the SIMT kernel.
// residual (optional, C's layout, may alias C; K-major B and a single product only): C = bf16(residual + bf16(A x B)).
// static_b: no earlier kernel of the stream writes B (it is a weight); the kernel is then launched with programmatic
// stream serialization and fetches its first B tiles while the preceding kernel drains.
// silu_pairs: B's rows come in blocks of 64 = 32 `gate` rows then the 32 `up` rows of the same features; C is then
// [M, N / 2] = bf16(bf16(g * sigmoid(g)) * u) with g, u the bf16-rounded products (the MLP's SiLU-and-multiply in the
// epilogue).  K-major B, single product, no residual, N a multiple of 64, more output tiles than SMs (the persistent
// kernel, where the epilogue's exponentials run under the next tile's MMAs); otherwise nothing is launched.
bool launch_tcgen05_gemm(const View4& bt, long long batch, const void* A, const void* B, void* C, long long M,
                         long long N, long long K, long long lda, long long ldb, unsigned* err, int sm_count,
                         cudaStream_t st, bool b_n_contiguous = false, const void* residual = nullptr,
                         bool static_b = false, bool silu_pairs = false);
// C[batch, M, N] (contiguous f32) = A[batch, M, K] x B[batch, N, K]^T with bf16 operands (both K-contiguous, rows K
// apart, batch strides a_bs / b_bs in elements) and the f32 accumulator stored unrounded.
bool launch_tcgen05_gemm_f32out(const void* A, const void* B, float* C, long long M, long long N, long long K,
                                long long batch, long long a_bs, long long b_bs, unsigned* err, int sm_count,
                                cudaStream_t st);
// False when the tensor-core kernels are switched off (CATGRAD_B200_NO_TCGEN05) or the driver entry point is missing.
bool tcgen05_available();
// A batch of products laid out as outer x heads (attention): product (o, h) multiplies
//   A + o*a_outer + h*a_head           rows a_row apart, K contiguous, M rows
//   B + o*b_outer + (h/b_div)*b_head   K-major: N rows b_row apart, K contiguous; or, with b_n_contiguous, K rows
//                                      b_row apart with N contiguous.  Grouped heads (b_div > 1) share it.
// into C + o*c_outer + h*c_head, rows ldc apart.  Strides are in elements and must be multiples of 8 (16 bytes).
// Rows/columns outside M, N, K are zero-filled on the way in, so K need not be a multiple of the tile.
struct GroupedGemm {
  const void* A; long long a_row, a_head, a_outer;
  const void* B; long long b_row, b_head, b_outer; bool b_n_contiguous;
  void* C; long long ldc, c_head, c_outer;
  long long M, N, K, heads, outer, b_div;
};
// Returns false (nothing launched) when the layout does not fit the tensor-core kernel.
bool launch_tcgen05_gemm_grouped(const GroupedGemm& p, unsigned* err, cudaStream_t st);
}  // namespace cgk

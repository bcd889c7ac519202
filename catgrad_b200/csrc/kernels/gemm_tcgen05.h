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
bool launch_tcgen05_gemm(const View4& bt, long long batch, const void* A, const void* B, void* C, long long M,
                         long long N, long long K, long long lda, long long ldb, unsigned* err, int sm_count,
                         cudaStream_t st, bool b_n_contiguous = false);
}  // namespace cgk

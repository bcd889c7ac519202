// Launcher of the strided batched matmul kernels (matmul.cu).
#pragma once
#include "common.cuh"

namespace cgk {
// C (contiguous [batch, M, N]) = A x B.  `bt` enumerates the batch index space (rank may be 0) with A's batch
// strides in bt.sa and B's in bt.sb; sam/sak and sbk/sbn are the matrix strides, all in elements.
void launch_matmul(int dtype, const View4& bt, long long batch, const void* A, const void* B, void* C, long long M,
                   long long N, long long K, long long sam, long long sak, long long sbk, long long sbn, int sm_count,
                   cudaStream_t st);

// f32 product on the bf16 tensor cores from three-way split operands (gemm_f32x3.cu).  A: contiguous [batch, M, K];
// B: contiguous [batch, K, N] (b_row_major) or [batch, N, K], or one such matrix shared by the whole batch
// (b_shared); C: contiguous [batch, M, N].  a3 / b3: caller-provided bf16 scratch of
// matmul_f32x3_scratch_elems(batch*M, K) and (batch or 1)*N rows.  Returns false if nothing could be launched.
bool matmul_f32x3_applicable(long long M, long long N, long long K, long long batch);
size_t matmul_f32x3_scratch_elems(long long rows, long long K);
bool launch_matmul_f32x3(const float* A, const float* B, float* C, void* a3, void* b3, long long M, long long N,
                         long long K, long long batch, bool b_row_major, bool b_shared, unsigned* err, int sm_count,
                         cudaStream_t st);
}  // namespace cgk

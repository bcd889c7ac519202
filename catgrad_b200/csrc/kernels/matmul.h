// Launcher of the strided batched matmul kernels (matmul.cu).
#pragma once
#include "common.cuh"

namespace cgk {
// C (contiguous [batch, M, N]) = A x B.  `bt` enumerates the batch index space (rank may be 0) with A's batch
// strides in bt.sa and B's in bt.sb; sam/sak and sbk/sbn are the matrix strides, all in elements.
void launch_matmul(int dtype, const View4& bt, long long batch, const void* A, const void* B, void* C, long long M,
                   long long N, long long K, long long sam, long long sak, long long sbk, long long sbn, int sm_count,
                   cudaStream_t st);
}  // namespace cgk

// Batched matmul over strided views: C[..,M,N] = A[..,M,K] x B[..,K,N], f32 accumulate.
//
// Replaces `batched_matmul` of the reference (catgrad/src/interpreter/backend/ndarray.rs:732-816).  The
// reference copies strided operands to contiguous buffers first (`to_shape`, ndarray.rs:797-798) and the
// graph materialises the broadcast of every weight (stdlib/nn/mod.rs:182-204 + ndarray.rs:553-559); here
// A and B are read in place through their strides, a stride-0 batch axis on B (one weight shared by the
// whole batch) costs nothing.
//
// Two SIMT kernels (the tensor-core kernel for large bf16 products is in gemm_tcgen05.cu):
//  * gemm_simt: 64x64x16 tiles, 4x4 register micro-tile per thread, FFMA with explicit fmaf.  This is the
//    exact-f32 path (no TF32): products and sums are IEEE f32, only the summation order differs from the
//    reference's sgemm.  Bound by the FP32 pipe.
//  * gemv_nt: M <= 16 rows against a K-contiguous B ("x @ W^T" with W[N,K] row-major, the layout of every
//    linear layer).  One warp per output column streams W with 16-byte loads; the A rows sit in shared
//    memory.  HBM-bound: algorithmic bytes = N*K*sizeof(T) (+ M*K + M*N, negligible).
#include <type_traits>

#include "elementwise.h"
#include "matmul.h"

namespace cgk {
namespace {

__device__ __forceinline__ void batch_offsets(const View4& bt, long long b, long long& oa, long long& ob) {
  oa = 0;
  ob = 0;
#pragma unroll 1
  for (int d = bt.rank - 1; d >= 0; --d) {
    long long s = bt.shape[d];
    long long q = b / s;
    long long c = b - q * s;
    oa += c * bt.sa[d];
    ob += c * bt.sb[d];
    b = q;
  }
}

template <class T> __device__ __forceinline__ float ldf(const T* p) { return Elem<T>::load(*p); }

constexpr int BM = 64, BN = 64, BK = 16;

template <class T>
__global__ void __launch_bounds__(256) gemm_simt_kernel(View4 bt, const T* __restrict__ A, const T* __restrict__ B,
                                                        T* __restrict__ C, int M, int N, int K, long long sam,
                                                        long long sak, long long sbk, long long sbn) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  long long oa, ob;
  batch_offsets(bt, blockIdx.z, oa, ob);
  A += oa;
  B += ob;
  C += (long long)blockIdx.z * M * N;
  // output tiles are flattened onto grid.x (grid.y stops at 65535 tiles: 4 M rows)
  const int ntn = (N + BN - 1) / BN;
  const int m0 = (int)(blockIdx.x / ntn) * BM, n0 = (int)(blockIdx.x % ntn) * BN;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each 4 x 4 outputs
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // Thread -> tile element mapping for the global loads: consecutive threads walk the contiguous axis.
  const bool a_k_fast = (sak == 1);
  const bool b_n_fast = (sbn == 1);
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int r = 0; r < (BM * BK) / 256; ++r) {
      int e = tid + r * 256;
      int mm, kk;
      if (a_k_fast) { kk = e % BK; mm = e / BK; } else { mm = e % BM; kk = e / BM; }
      int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < M && gk < K) ? ldf(A + gm * sam + gk * sak) : 0.f;
    }
#pragma unroll
    for (int r = 0; r < (BN * BK) / 256; ++r) {
      int e = tid + r * 256;
      int nn, kk;
      if (b_n_fast) { nn = e % BN; kk = e / BN; } else { kk = e % BK; nn = e / BK; }
      int gn = n0 + nn, gk = k0 + kk;
      Bs[kk][nn] = (gn < N && gk < K) ? ldf(B + gk * sbk + gn * sbn) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tx * 4 + j;
      if (gn < N) C[(long long)gm * N + gn] = Elem<T>::store(acc[i][j]);
    }
  }
}

// u32 matmul (wrapping), naive: the trait defines it (ndarray.rs:181) but no model uses it.
__global__ void __launch_bounds__(256) gemm_u32_kernel(View4 bt, const unsigned* __restrict__ A,
                                                       const unsigned* __restrict__ B, unsigned* __restrict__ C, int M,
                                                       int N, int K, long long sam, long long sak, long long sbk,
                                                       long long sbn) {
  long long oa, ob;
  batch_offsets(bt, blockIdx.z, oa, ob);
  A += oa;
  B += ob;
  C += (long long)blockIdx.z * M * N;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < (long long)M * N;
       t += (long long)gridDim.x * blockDim.x) {
    int m = (int)(t / N), n = (int)(t % N);
    unsigned acc = 0;
    for (int k = 0; k < K; ++k) acc += A[m * sam + k * sak] * B[k * sbk + n * sbn];
    C[t] = acc;
  }
}

// ---- skinny: M <= 16, B K-contiguous -------------------------------------------------------------
template <class T, int N> struct alignas(sizeof(T) * N) Vec { T v[N]; };

// grid: (column groups, 1, batch); block: 256 threads = 8 warps, each warp owns COLS columns at a time.
// A rows [MT][K] are staged in shared memory as f32 (dynamic smem: MT*K floats).
template <class T, int MT>
__global__ void __launch_bounds__(256) gemv_nt_kernel(View4 bt, const T* __restrict__ A, const T* __restrict__ B,
                                                      T* __restrict__ C, int M, int N, int K, long long sam,
                                                      long long sak, long long sbn) {
  extern __shared__ float xs[];  // [MT][K]
  constexpr int VEC = 16 / sizeof(T);
  long long oa, ob;
  batch_offsets(bt, blockIdx.z, oa, ob);
  A += oa;
  B += ob;
  C += (long long)blockIdx.z * M * N;
  for (int e = threadIdx.x; e < MT * K; e += 256) {
    int m = e / K, k = e - m * K;
    xs[e] = m < M ? ldf(A + m * sam + k * sak) : 0.f;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps_total = gridDim.x * 8;
  const int nvec = K / VEC;
  for (int n = blockIdx.x * 8 + warp; n < N; n += warps_total) {
    const T* w = B + (long long)n * sbn;
    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[m] = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      Vec<T, VEC> wv = *reinterpret_cast<const Vec<T, VEC>*>(w + v * VEC);
      float wf[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) wf[i] = Elem<T>::load(wv.v[i]);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float* x = xs + m * K + v * VEC;
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[m] = fmaf(x[i], wf[i], acc[m]);
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      float s = warp_sum(acc[m]);
      if (lane == 0 && m < M) C[(long long)m * N + n] = Elem<T>::store(s);
    }
  }
}

template <class T, int MT>
void launch_gemv_mt(const View4& bt, long long batch, const void* A, const void* B, void* C, int M, int N, int K,
                    long long sam, long long sak, long long sbn, int sm, cudaStream_t st) {
  size_t smem = (size_t)MT * K * sizeof(float);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(gemv_nt_kernel<T, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int gx = (N + 7) / 8;
  int cap = sm * 4;  // whole waves
  if (batch == 1 && gx > cap) gx = cap;
  dim3 grid(gx, 1, (unsigned)batch);
  gemv_nt_kernel<T, MT><<<grid, 256, smem, st>>>(bt, (const T*)A, (const T*)B, (T*)C, M, N, K, sam, sak, sbn);
}

template <class T>
bool launch_gemv_t(const View4& bt, long long batch, const void* A, const void* B, void* C, int M, int N, int K,
                   long long sam, long long sak, long long sbn, int sm, cudaStream_t st) {
  int mt = M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : 16;
  if ((size_t)mt * K * sizeof(float) > 200 * 1024) return false;
  switch (mt) {
    case 1: launch_gemv_mt<T, 1>(bt, batch, A, B, C, M, N, K, sam, sak, sbn, sm, st); break;
    case 2: launch_gemv_mt<T, 2>(bt, batch, A, B, C, M, N, K, sam, sak, sbn, sm, st); break;
    case 4: launch_gemv_mt<T, 4>(bt, batch, A, B, C, M, N, K, sam, sak, sbn, sm, st); break;
    case 8: launch_gemv_mt<T, 8>(bt, batch, A, B, C, M, N, K, sam, sak, sbn, sm, st); break;
    default: launch_gemv_mt<T, 16>(bt, batch, A, B, C, M, N, K, sam, sak, sbn, sm, st); break;
  }
  return true;
}

template <class T>
void launch_simt_t(const View4& bt, long long batch, const void* A, const void* B, void* C, int M, int N, int K,
                   long long sam, long long sak, long long sbk, long long sbn, cudaStream_t st) {
  dim3 grid((unsigned)((long long)((N + BN - 1) / BN) * ((M + BM - 1) / BM)), 1, (unsigned)batch);   // < 2^31 tiles: checked by the caller
  gemm_simt_kernel<T><<<grid, 256, 0, st>>>(bt, (const T*)A, (const T*)B, (T*)C, M, N, K, sam, sak, sbk, sbn);
}
}  // namespace

void launch_matmul(int dtype, const View4& bt, long long batch, const void* A, const void* B, void* C, long long M,
                   long long N, long long K, long long sam, long long sak, long long sbk, long long sbn, int sm,
                   cudaStream_t st) {
  if (batch <= 0 || M <= 0 || N <= 0) return;
  if (dtype == DT_U32) {
    long long blocks = (M * N + 255) / 256;
    dim3 grid((unsigned)(blocks > 65535 ? 65535 : blocks), 1, (unsigned)batch);
    gemm_u32_kernel<<<grid, 256, 0, st>>>(bt, (const unsigned*)A, (const unsigned*)B, (unsigned*)C, (int)M, (int)N,
                                          (int)K, sam, sak, sbk, sbn);
    return;
  }
  int es = dtype == DT_F32 ? 4 : 2;
  int vec = 16 / es;
  // skinny path: few rows, B rows contiguous along K and 16-byte aligned
  bool skinny = M <= 16 && sbk == 1 && K % vec == 0 && sbn % vec == 0 && ((uintptr_t)B % 16 == 0) && K >= 64 && N >= 8;
  for (int d = 0; d < bt.rank && skinny; ++d) skinny = bt.sb[d] % vec == 0;
  if (skinny) {
    bool ok = false;
    switch (dtype) {
      case DT_F32: ok = launch_gemv_t<float>(bt, batch, A, B, C, (int)M, (int)N, (int)K, sam, sak, sbn, sm, st); break;
      case DT_BF16: ok = launch_gemv_t<__nv_bfloat16>(bt, batch, A, B, C, (int)M, (int)N, (int)K, sam, sak, sbn, sm, st); break;
      case DT_F16: ok = launch_gemv_t<__half>(bt, batch, A, B, C, (int)M, (int)N, (int)K, sam, sak, sbn, sm, st); break;
    }
    if (ok) return;
  }
  switch (dtype) {
    case DT_F32: launch_simt_t<float>(bt, batch, A, B, C, (int)M, (int)N, (int)K, sam, sak, sbk, sbn, st); break;
    case DT_BF16: launch_simt_t<__nv_bfloat16>(bt, batch, A, B, C, (int)M, (int)N, (int)K, sam, sak, sbk, sbn, st); break;
    case DT_F16: launch_simt_t<__half>(bt, batch, A, B, C, (int)M, (int)N, (int)K, sam, sak, sbk, sbn, st); break;
  }
}

}  // namespace cgk

// Fused kernels of the Llama plan.  Each kernel covers a sub-graph of the Llama term
// (catgrad-llm-models/src/models/llama.rs:144-385 and the helpers it expands) and keeps the term's rounding
// points: values the graph types as bf16 are rounded to bf16 exactly where an op of the graph would produce
// them; the f32 islands (rmsnorm, softmax, silu, rope: stdlib/nn/mod.rs:117-179, helpers/tensors.rs:82-111,
// helpers/rope.rs:430-451) run in f32.  Compiled with -fmad=false: products and sums that are separate ops in
// the graph stay separate roundings; dot products use explicit fmaf (accumulation order is free there).
//
// All of them are HBM- or latency-bound; the weight-streaming GEMV dominates a decode step.
#pragma once
#include <cfloat>

#include "common.cuh"

namespace cgk {

template <class T, int N> struct alignas(sizeof(T) * N) VecT { T v[N]; };

template <class T> __device__ __forceinline__ float rt(float v) { return Elem<T>::load(Elem<T>::store(v)); }  // round trip through T

// Deterministic block-wide reductions for 256-thread CTAs (fixed tree).
__device__ __forceinline__ float block_sum_256(float v, float* scratch /* >= 8 floats */) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) r += scratch[w];
  return r;
}
__device__ __forceinline__ float block_max_256(float v, float* scratch) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = -FLT_MAX;
#pragma unroll
  for (int w = 0; w < 8; ++w) r = fmaxf(r, scratch[w]);
  return r;
}

// Programmatic dependent launch: a kernel may be scheduled while its predecessor drains; everything that reads
// the predecessor's results or writes global memory comes after pdl_wait().  Both are no-ops for a kernel
// launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Software pipelining across kernel launches: a kernel asks the L2 to fetch the weights of the launches that follow
// it (fire-and-forget bulk prefetch), so HBM keeps streaming while this kernel works on data that an earlier
// launch prefetched, and across the launch gap.  Each CTA requests its 1/gridDim slice of each region.
struct PrefetchArgs {
  const void* ptr[3];
  long long bytes[3];
};
__device__ __forceinline__ void l2_prefetch_slices(const PrefetchArgs& pf) {
  if (threadIdx.x != 0) return;
  const long long nb = (long long)gridDim.x * gridDim.y, b = (long long)blockIdx.y * gridDim.x + blockIdx.x;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    if (pf.ptr[i] == nullptr || pf.bytes[i] <= 0) continue;
    long long per = ((pf.bytes[i] + nb - 1) / nb + 15) & ~15ll;
    long long lo = b * per, hi = lo + per < pf.bytes[i] ? lo + per : pf.bytes[i];
    const char* base = (const char*)pf.ptr[i];
    for (long long o = lo; o < hi; o += 65536) {
      unsigned sz = (unsigned)((hi - o < 65536 ? hi - o : 65536) & ~15ll);
      if (sz) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + o), "r"(sz) : "memory");
    }
  }
}

// ---- embedding gather (helpers/tensors.rs:255-272) ------------------------------------------------
// x[m, :] = table[ids[m], :].  16-byte copies; an id >= vocab records DEV_ERR_INDEX_OOB and writes zeros.
template <class T>
__global__ void __launch_bounds__(256) embed_kernel(const unsigned* __restrict__ ids, const T* __restrict__ table,
                                                    T* __restrict__ x, int M, int H, int vocab, unsigned* err) {
  constexpr int VEC = 16 / sizeof(T);
  const int per_row = H / VEC;
  pdl_launch_dependents();
  pdl_wait();
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < (long long)M * per_row;
       t += (long long)gridDim.x * blockDim.x) {
    int m = (int)(t / per_row), c = (int)(t - (long long)m * per_row);
    unsigned id = ids[m];
    VecT<T, VEC> v;
    if (id >= (unsigned)vocab) {
      if (c == 0) atomicOr(err, DEV_ERR_INDEX_OOB);
      memset(&v, 0, sizeof(v));
    } else {
      v = *reinterpret_cast<const VecT<T, VEC>*>(table + (long long)id * H + c * VEC);
    }
    *reinterpret_cast<VecT<T, VEC>*>(x + (long long)m * H + c * VEC) = v;
  }
}

// ---- RMSNorm (helpers/tensors.rs:82-111) ------------------------------------------------------------
// y = T( T(x / sqrt(mean(x^2) + eps)) * g ); the reference writes sqrt as pow(.,0.5) (nn/mod.rs:117-122);
// sqrtf is used here, within the logits tolerance.  One CTA per row; source row = in + (m*row_mul+row_off)*H.
template <class T>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const T* __restrict__ in, const T* __restrict__ gain,
                                                      T* __restrict__ out, int H, float eps, long long row_mul,
                                                      long long row_off) {
  __shared__ float scratch[8];
  pdl_launch_dependents();   // a GEMM that follows may start fetching its weight tiles
  pdl_wait();                // no-op unless launched with programmatic stream serialization
  const T* x = in + ((long long)blockIdx.x * row_mul + row_off) * H;
  T* y = out + (long long)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += 256) {
    float v = Elem<T>::load(x[i]);
    ss += v * v;
  }
  ss = block_sum_256(ss, scratch);
  float rms = sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += 256) {
    float n = rt<T>(Elem<T>::load(x[i]) / rms);
    y[i] = Elem<T>::store(n * Elem<T>::load(gain[i]));
  }
}

// Same with the row in registers and 16-byte accesses: thread t of the CTA owns vectors t, t + 256, ... (at most four:
// rows of up to 1024 vectors), one load and one store per vector instead of two passes of scalar loads.
template <class T>
__global__ void __launch_bounds__(256) rmsnorm_vec_kernel(const T* __restrict__ in, const T* __restrict__ gain,
                                                          T* __restrict__ out, int H, float eps, long long row_mul,
                                                          long long row_off) {
  constexpr int VEC = 16 / sizeof(T);
  __shared__ float scratch[8];
  pdl_launch_dependents();
  pdl_wait();
  const T* x = in + ((long long)blockIdx.x * row_mul + row_off) * H;
  T* y = out + (long long)blockIdx.x * H;
  const int nvec = H / VEC;
  VecT<T, VEC> xv[4];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int v = threadIdx.x + j * 256;
    if (v < nvec) {
      xv[j] = *reinterpret_cast<const VecT<T, VEC>*>(x + v * VEC);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float f = Elem<T>::load(xv[j].v[i]);
        ss += f * f;
      }
    }
  }
  ss = block_sum_256(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int v = threadIdx.x + j * 256;
    if (v < nvec) {
      const VecT<T, VEC> g = *reinterpret_cast<const VecT<T, VEC>*>(gain + v * VEC);
      VecT<T, VEC> o;
#pragma unroll
      for (int i = 0; i < VEC; ++i) o.v[i] = Elem<T>::store(rt<T>(Elem<T>::load(xv[j].v[i]) / rms) * Elem<T>::load(g.v[i]));
      *reinterpret_cast<VecT<T, VEC>*>(y + v * VEC) = o;
    }
  }
}

// Same with one warp per row and the row in registers (NV 16-byte vectors per lane, H = 32 * NV * (16 / sizeof(T))):
// one pass over the row, every load of a lane in flight at once, no block-level synchronisation.
template <class T, int NV>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const T* __restrict__ in, const T* __restrict__ gain,
                                                           T* __restrict__ out, long long rows, float eps, long long row_mul,
                                                           long long row_off) {
  constexpr int VEC = 16 / sizeof(T);
  constexpr int H = 32 * NV * VEC;
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* x = in + (row * row_mul + row_off) * H;
  T* y = out + row * H;
  VecT<T, VEC> xv[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) xv[j] = *reinterpret_cast<const VecT<T, VEC>*>(x + (j * 32 + lane) * VEC);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j)
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float v = Elem<T>::load(xv[j].v[i]);
      ss += v * v;
    }
  ss = warp_sum(ss);
  const float rms = sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const VecT<T, VEC> g = *reinterpret_cast<const VecT<T, VEC>*>(gain + (j * 32 + lane) * VEC);
    VecT<T, VEC> o;
#pragma unroll
    for (int i = 0; i < VEC; ++i) o.v[i] = Elem<T>::store(rt<T>(Elem<T>::load(xv[j].v[i]) / rms) * Elem<T>::load(g.v[i]));
    *reinterpret_cast<VecT<T, VEC>*>(y + (j * 32 + lane) * VEC) = o;
  }
}

// ---- weight-streaming GEMV with fused prologue/epilogue --------------------------------------------
// out[m, n] = epilogue( sum_k xin[m, k] * W[n, k] ),  m < M <= MT, W rows K-contiguous (the [out,in] layout of
// every linear layer, nn/mod.rs:182-204: x @ transpose(W) without ever forming the transpose or its broadcast).
enum { PRO_NONE = 0, PRO_NORM = 1 };
enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_SILU_MUL = 2 };

struct GemvArgs {
  const void* w[3];   // up to three weight matrices stacked along N (q,k,v) or paired (gate, up)
  int n_end[3];       // exclusive end row of each segment in the stacked N space
  const void* x;      // [M, K] rows at x + m * x_row_stride
  long long x_row_stride;
  const void* gain;   // PRO_NORM: RMSNorm gain [K]
  float eps;
  void* out;          // [M, N]
  const void* res;    // EPI_RESIDUAL: [M, N], may alias out
  int M, N, K;
  int ks;             // K is split over `ks` warps of a CTA (1, 2, 4 or 8) so that small N still fills the GPU
  PrefetchArgs pf;    // weights of later launches to pull into L2
};

template <class T>
__device__ __forceinline__ const T* gemv_row(const GemvArgs& a, int n) {
  int seg = n < a.n_end[0] ? 0 : (n < a.n_end[1] ? 1 : 2);
  int base = seg == 0 ? 0 : a.n_end[seg - 1];
  return (const T*)a.w[seg] + (long long)(n - base) * a.K;
}

// 256 threads = 8 warps.  A work item is a PAIR of weight rows (two output columns, or gate[n]/up[n] for
// EPI_SILU_MUL); `ks` consecutive warps share one pair, each streaming a 1/ks slice of K with 16-byte loads;
// partial sums meet in shared memory in a fixed order.  The M input rows sit in shared memory as T.
template <class T, int MT, int PRO, int EPI>
__global__ void __launch_bounds__(256, 2) gemv_fused_kernel(GemvArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* xs = reinterpret_cast<T*>(smem_raw);  // [MT][K]
  __shared__ float scratch[8];
  __shared__ float part[8][2 * MT];
  constexpr int VEC = 16 / sizeof(T);
  const int K = a.K;
  const T* xin = (const T*)a.x;
  l2_prefetch_slices(a.pf);

  // ---- this warp's first work item: start streaming its weights before the input vector is even ready ----
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int ks = a.ks, ppc = 8 / ks;            // pairs per CTA per iteration
  const int split = warp % ks, slot = warp / ks;
  const int n_pairs = EPI == EPI_SILU_MUL ? a.N : (a.N + 1) / 2;
  const int nvec = K / VEC;
  const int v_lo = (int)((long long)nvec * split / ks), v_hi = (int)((long long)nvec * (split + 1) / ks);
  const int iters = (n_pairs + gridDim.x * ppc - 1) / (gridDim.x * ppc);
  constexpr int PRE = 4;
  VecT<T, VEC> pre0[PRE], pre1[PRE];
  {
    const int p = blockIdx.x * ppc + slot;
    if (p < n_pairs) {
      const T *w0, *w1;
      if (EPI == EPI_SILU_MUL) {
        w0 = (const T*)a.w[0] + (long long)p * K;
        w1 = (const T*)a.w[1] + (long long)p * K;
      } else {
        w0 = gemv_row<T>(a, 2 * p);
        w1 = gemv_row<T>(a, 2 * p + 1 < a.N ? 2 * p + 1 : 2 * p);
      }
#pragma unroll
      for (int j = 0; j < PRE; ++j) {
        const int v = v_lo + lane + 32 * j;
        if (v < v_hi) {
          pre0[j] = *reinterpret_cast<const VecT<T, VEC>*>(w0 + v * VEC);
          pre1[j] = *reinterpret_cast<const VecT<T, VEC>*>(w1 + v * VEC);
        }
      }
    }
  }

  // weights do not depend on the previous launch; everything below does
  pdl_wait();
  pdl_launch_dependents();

  // ---- input rows into shared memory (as T); PRO_NORM applies RMSNorm (helpers/tensors.rs:82-111) ----
  if (PRO == PRO_NORM && nvec <= 4 * 256) {
    // one pass: every thread keeps its 16-byte groups of x and of the gain in registers across the reduction
    const T* g = (const T*)a.gain;
#pragma unroll 1
    for (int m = 0; m < MT; ++m) {
      VecT<T, VEC> xv[4], gv[4];
      float ss = 0.f;
      if (m < a.M) {
        const T* x = xin + m * a.x_row_stride;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int v = threadIdx.x + 256 * j;
          if (v < nvec) {
            xv[j] = *reinterpret_cast<const VecT<T, VEC>*>(x + v * VEC);
            gv[j] = *reinterpret_cast<const VecT<T, VEC>*>(g + v * VEC);
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
              float f = Elem<T>::load(xv[j].v[i]);
              ss += f * f;
            }
          }
        }
      }
      ss = block_sum_256(ss, scratch);
      const float rms = sqrtf(ss / (float)K + a.eps);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int v = threadIdx.x + 256 * j;
        if (v < nvec) {
          VecT<T, VEC> o;
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            float nrm = m < a.M ? rt<T>(Elem<T>::load(xv[j].v[i]) / rms) : 0.f;
            o.v[i] = Elem<T>::store(m < a.M ? nrm * Elem<T>::load(gv[j].v[i]) : 0.f);
          }
          *reinterpret_cast<VecT<T, VEC>*>(xs + m * K + v * VEC) = o;
        }
      }
    }
  } else if (PRO == PRO_NORM) {
    const T* g = (const T*)a.gain;
    for (int m = 0; m < MT; ++m) {
      if (m < a.M) {
        const T* x = xin + m * a.x_row_stride;
        float ss = 0.f;
        for (int i = threadIdx.x; i < K; i += 256) {
          float v = Elem<T>::load(x[i]);
          ss += v * v;
        }
        ss = block_sum_256(ss, scratch);
        float rms = sqrtf(ss / (float)K + a.eps);
        for (int i = threadIdx.x; i < K; i += 256) {
          float n = rt<T>(Elem<T>::load(x[i]) / rms);
          xs[m * K + i] = Elem<T>::store(n * Elem<T>::load(g[i]));
        }
      } else {
        for (int i = threadIdx.x; i < K; i += 256) xs[m * K + i] = Elem<T>::store(0.f);
      }
    }
  } else {
    for (int e = threadIdx.x; e < MT * (K / VEC); e += 256) {
      int m = e / (K / VEC), c = e - m * (K / VEC);
      VecT<T, VEC> v;
      if (m < a.M) v = *reinterpret_cast<const VecT<T, VEC>*>(xin + m * a.x_row_stride + c * VEC);
      else memset(&v, 0, sizeof(v));
      *reinterpret_cast<VecT<T, VEC>*>(xs + m * K + c * VEC) = v;
    }
  }
  __syncthreads();

  for (int it = 0; it < iters; ++it) {
    const int p = (it * gridDim.x + blockIdx.x) * ppc + slot;
    const bool valid = p < n_pairs;
    int n0 = 0, n1 = 0;
    float acc0[MT], acc1[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) acc0[m] = acc1[m] = 0.f;
    if (valid) {
      const T *w0, *w1;
      if (EPI == EPI_SILU_MUL) {
        n0 = n1 = p;
        w0 = (const T*)a.w[0] + (long long)p * K;
        w1 = (const T*)a.w[1] + (long long)p * K;
      } else {
        n0 = 2 * p;
        n1 = 2 * p + 1 < a.N ? 2 * p + 1 : n0;
        w0 = gemv_row<T>(a, n0);
        w1 = gemv_row<T>(a, n1);
      }
      int vstart = v_lo + lane;
      if (it == 0) {
        // the vectors fetched before the input was ready
#pragma unroll
        for (int j = 0; j < PRE; ++j) {
          const int v = v_lo + lane + 32 * j;
          if (v < v_hi) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
              VecT<T, VEC> xv = *reinterpret_cast<const VecT<T, VEC>*>(xs + m * K + v * VEC);
#pragma unroll
              for (int i = 0; i < VEC; ++i) {
                float xf = Elem<T>::load(xv.v[i]);
                acc0[m] = fmaf(xf, Elem<T>::load(pre0[j].v[i]), acc0[m]);
                acc1[m] = fmaf(xf, Elem<T>::load(pre1[j].v[i]), acc1[m]);
              }
            }
          }
        }
        vstart += 32 * PRE;
      }
#pragma unroll 8
      for (int v = vstart; v < v_hi; v += 32) {
        VecT<T, VEC> a0 = *reinterpret_cast<const VecT<T, VEC>*>(w0 + v * VEC);
        VecT<T, VEC> a1 = *reinterpret_cast<const VecT<T, VEC>*>(w1 + v * VEC);
        float f0[VEC], f1[VEC];
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          f0[i] = Elem<T>::load(a0.v[i]);
          f1[i] = Elem<T>::load(a1.v[i]);
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          VecT<T, VEC> xv = *reinterpret_cast<const VecT<T, VEC>*>(xs + m * K + v * VEC);
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            float xf = Elem<T>::load(xv.v[i]);
            acc0[m] = fmaf(xf, f0[i], acc0[m]);
            acc1[m] = fmaf(xf, f1[i], acc1[m]);
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      acc0[m] = warp_sum(acc0[m]);
      acc1[m] = warp_sum(acc1[m]);
    }
    if (ks > 1) {
      if (lane == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          part[warp][2 * m] = acc0[m];
          part[warp][2 * m + 1] = acc1[m];
        }
      }
      __syncthreads();
      if (split == 0 && lane == 0) {
#pragma unroll
        for (int m = 0; m < MT; ++m) {
          float s0 = 0.f, s1 = 0.f;
          for (int q = 0; q < ks; ++q) {
            s0 += part[warp + q][2 * m];
            s1 += part[warp + q][2 * m + 1];
          }
          acc0[m] = s0;
          acc1[m] = s1;
        }
      }
    }
    if (valid && split == 0 && lane == 0) {
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m >= a.M) continue;
        const float s0 = acc0[m], s1 = acc1[m];
        T* o = (T*)a.out + (long long)m * a.N;
        if (EPI == EPI_STORE) {
          o[n0] = Elem<T>::store(s0);
          if (n1 != n0) o[n1] = Elem<T>::store(s1);
        } else if (EPI == EPI_RESIDUAL) {
          // x = res + linear(.)  (llama.rs:375,384): the linear output is a T tensor, then one add in T
          const T* r = (const T*)a.res + (long long)m * a.N;
          o[n0] = Elem<T>::store(Elem<T>::load(r[n0]) + rt<T>(s0));
          if (n1 != n0) o[n1] = Elem<T>::store(Elem<T>::load(r[n1]) + rt<T>(s1));
        } else {
          // silu(gate) * up  (llama.rs:245; nn/mod.rs:124-148): gate, up are T tensors; silu runs in f32 as
          // x * (1 / (1 + exp(-x))) and is cast back to T before the multiply in T.
          float g = rt<T>(s0), u = rt<T>(s1);
          float sg = 1.f / (1.f + expf(-g));
          float si = rt<T>(g * sg);
          o[n0] = Elem<T>::store(si * u);
        }
      }
    }
    if (ks > 1) __syncthreads();
  }
}

// ---- RoPE + KV append for prefill (helpers/rope.rs:423-451; helpers/cache.rs:30-39) -----------------
// One CTA per token m = (b, s).  q is rotated in place; rotated k and plain v go to the cache row `pos`.
// cos/sin tables are [P, HD/2] f32 (the reference concatenates each with itself, rope.rs:100-101).
struct RopeArgs {
  void* q; long long q_row_stride;        // [M, nh*HD]
  const void* k; long long k_row_stride;  // [M, nkv*HD]
  const void* v; long long v_row_stride;
  void* kc; void* vc;                     // this layer's cache slices [B, nkv, P, HD]
  const float* cos_t; const float* sin_t;
  const int* ctx_len;                     // device scalar: positions already in the cache
  int B, S, nh, nkv, HD, P;
};
template <class T>
__global__ void __launch_bounds__(256) rope_append_kernel(RopeArgs a, unsigned* err) {
  const int m = blockIdx.x, b = m / a.S, s = m - b * a.S;
  const int pos = *a.ctx_len + s;
  if (pos >= a.P) {
    if (threadIdx.x == 0) atomicOr(err, DEV_ERR_INDEX_OOB);
    return;
  }
  const int half = a.HD / 2;
  T* q = (T*)a.q + (long long)m * a.q_row_stride;
  const T* k = (const T*)a.k + (long long)m * a.k_row_stride;
  const T* v = (const T*)a.v + (long long)m * a.v_row_stride;
  const float* ct = a.cos_t + (long long)pos * half;
  const float* st = a.sin_t + (long long)pos * half;
  // 16-byte vectors: a thread rotates VEC pairs (x1 from the first half of a head, x2 from the second)
  constexpr int VEC = 16 / sizeof(T);
  const int gph = half / VEC;  // vector groups per head half
  const int q_groups = a.nh * gph, k_groups = a.nkv * gph;
  for (int e = threadIdx.x; e < q_groups + k_groups; e += 256) {
    const bool is_q = e < q_groups;
    const int ee = is_q ? e : e - q_groups;
    const int h = ee / gph, i = (ee - h * gph) * VEC;
    const T* src = is_q ? q + h * a.HD : k + h * a.HD;
    const VecT<T, VEC> x1 = *reinterpret_cast<const VecT<T, VEC>*>(src + i);
    const VecT<T, VEC> x2 = *reinterpret_cast<const VecT<T, VEC>*>(src + i + half);
    VecT<T, VEC> o1, o2;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float a1 = Elem<T>::load(x1.v[j]), a2 = Elem<T>::load(x2.v[j]);
      const float c = ct[i + j], sn = st[i + j];
      // cos*x + sin*rotate_half(x), rotate_half = cat(-x2, x1): two products and one sum, each rounded
      o1.v[j] = Elem<T>::store(c * a1 + sn * (-a2));
      o2.v[j] = Elem<T>::store(c * a2 + sn * a1);
    }
    T* dst = is_q ? q + h * a.HD : (T*)a.kc + (((long long)b * a.nkv + h) * a.P + pos) * a.HD;
    *reinterpret_cast<VecT<T, VEC>*>(dst + i) = o1;
    *reinterpret_cast<VecT<T, VEC>*>(dst + i + half) = o2;
  }
  const int vph = a.HD / VEC;
  for (int e = threadIdx.x; e < a.nkv * vph; e += 256) {
    const int h = e / vph, i = (e - h * vph) * VEC;
    *reinterpret_cast<VecT<T, VEC>*>((T*)a.vc + (((long long)b * a.nkv + h) * a.P + pos) * a.HD + i) =
        *reinterpret_cast<const VecT<T, VEC>*>(v + h * a.HD + i);
  }
}

// ---- decode attention, S = 1, with RoPE and the KV append fused (llama.rs:296-345) -------------------
// One CTA per (query head, sequence).  It rotates its q and the new k row (rope.rs:430-451), the first head of
// each GQA group stores the rotated k and the v row into the cache (cache.rs:30-39); every head of the group
// uses its own copy of the new row, so no CTA waits for another.  Then scores = T(q.k), T(scores / T(sqrt(HD))),
// softmax in f32 -> T, out = T(P.v).  The causal-mask row of a single new token is all -0.0 and adding it
// changes nothing (helpers/tensors.rs:207-224), so it is skipped.  GQA: head h reads kv head h / rep
// (repeat_kv, tensors.rs:128-151, never materialised).
struct AttnArgs {
  const void* q; long long q_row_stride;  // raw projections [B, ...]: q at [b*stride + h*HD]
  const void* k; long long k_row_stride;  // new k row [b*stride + kvh*HD] (not rotated)
  const void* v; long long v_row_stride;
  void* kc; void* vc;                     // [B, nkv, P, HD]
  void* out; long long out_row_stride;    // [B, nh*HD]
  const float* cos_t; const float* sin_t; // [P, HD/2]
  const int* ctx_len;                     // positions in the cache before this step
  int nh, nkv, P;
  float scale;                            // T(sqrt(HD)) widened
  PrefetchArgs pf;                        // weights of later launches to pull into L2
};
template <class T, int HD>
__global__ void __launch_bounds__(256) attn_decode_kernel(AttnArgs a, unsigned* err) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* sc = reinterpret_cast<float*>(smem_raw);  // [P + 1] scores / probabilities
  __shared__ float scratch[8];
  __shared__ __align__(16) float q_s[HD];
  __shared__ __align__(16) T k_new[HD];
  __shared__ __align__(16) T v_new[HD];
  constexpr int VEC = 16 / sizeof(T);
  constexpr int LPK = HD / VEC;        // lanes per key
  constexpr int KPW = 32 / LPK;        // keys per warp per load round
  constexpr int half = HD / 2;
  const int h = blockIdx.x, b = blockIdx.y;
  const int rep = a.nh / a.nkv, kvh = h / rep;
  l2_prefetch_slices(a.pf);
  pdl_launch_dependents();
  pdl_wait();
  const int pos = *a.ctx_len;          // the new token's position
  if (pos >= a.P) {
    if (threadIdx.x == 0) atomicOr(err, DEV_ERR_INDEX_OOB);
    return;
  }
  const int total = pos + 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LPK, kslot = lane / LPK;
  T* kc = (T*)a.kc + ((long long)b * a.nkv + kvh) * a.P * HD;
  T* vc = (T*)a.vc + ((long long)b * a.nkv + kvh) * a.P * HD;

  // RoPE of q and of the new k row; v row copied
  if (threadIdx.x < HD) {  // threads [0, half): q pair; [half, HD): k pair
    const bool is_q = threadIdx.x < half;
    const int i = is_q ? threadIdx.x : threadIdx.x - half;
    const T* src = is_q ? (const T*)a.q + (long long)b * a.q_row_stride + h * HD
                        : (const T*)a.k + (long long)b * a.k_row_stride + kvh * HD;
    float x1 = Elem<T>::load(src[i]), x2 = Elem<T>::load(src[i + half]);
    float c = a.cos_t[(long long)pos * half + i], sn = a.sin_t[(long long)pos * half + i];
    float o1 = c * x1 + sn * (-x2);
    float o2 = c * x2 + sn * x1;
    if (is_q) {
      q_s[i] = rt<T>(o1);
      q_s[i + half] = rt<T>(o2);
    } else {
      k_new[i] = Elem<T>::store(o1);
      k_new[i + half] = Elem<T>::store(o2);
    }
  } else if (threadIdx.x < 2 * HD) {
    const int i = threadIdx.x - HD;
    v_new[i] = ((const T*)a.v)[(long long)b * a.v_row_stride + kvh * HD + i];
  }
  __syncthreads();
  if (h % rep == 0 && threadIdx.x < HD) {
    kc[(long long)pos * HD + threadIdx.x] = k_new[threadIdx.x];
    vc[(long long)pos * HD + threadIdx.x] = v_new[threadIdx.x];
  }

  float qf[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) qf[i] = q_s[sub * VEC + i];
  // scores over the cached keys: 8 independent 16-byte loads in flight per lane
  constexpr int UN = 8;
  for (int t0 = warp * KPW * UN; t0 < pos; t0 += 8 * KPW * UN) {
    VecT<T, VEC> kv[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      int t = t0 + u * KPW + kslot;
      if (t < pos) kv[u] = *reinterpret_cast<const VecT<T, VEC>*>(kc + (long long)t * HD + sub * VEC);
      else memset(&kv[u], 0, sizeof(kv[u]));
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      int t = t0 + u * KPW + kslot;
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) d = fmaf(qf[i], Elem<T>::load(kv[u].v[i]), d);
#pragma unroll
      for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (sub == 0 && t < pos) sc[t] = rt<T>(rt<T>(d) / a.scale);
    }
  }
  if (warp == 0) {  // the new key, from shared memory
    float d = 0.f;
    for (int i = lane; i < HD; i += 32) d = fmaf(q_s[i], Elem<T>::load(k_new[i]), d);
    d = warp_sum(d);
    if (lane == 0) sc[pos] = rt<T>(rt<T>(d) / a.scale);
  }
  __syncthreads();
  float mx = -FLT_MAX;  // `max` folds from f32::MIN (ndarray.rs:656-661)
  for (int t = threadIdx.x; t < total; t += 256) mx = fmaxf(mx, sc[t]);
  mx = block_max_256(mx, scratch);
  float sum = 0.f;
  for (int t = threadIdx.x; t < total; t += 256) {
    float e = expf(sc[t] - mx);
    sc[t] = e;
    sum += e;
  }
  sum = block_sum_256(sum, scratch);
  for (int t = threadIdx.x; t < total; t += 256) sc[t] = rt<T>(sc[t] / sum);
  __syncthreads();

  // P.v: thread = (16-byte chunk of the head dim, key group); partial sums over its keys, then a fixed-order
  // reduction over the key groups through shared memory.
  constexpr int NCH = HD / VEC, TG = 256 / NCH;
  float* part = sc + a.P + 1;  // [TG][HD]
  const int ch = threadIdx.x % NCH, tg = threadIdx.x / NCH;
  float acc[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
  for (int t0 = tg; t0 < pos; t0 += TG * UN) {
    VecT<T, VEC> vv[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      int t = t0 + u * TG;
      if (t < pos) vv[u] = *reinterpret_cast<const VecT<T, VEC>*>(vc + (long long)t * HD + ch * VEC);
      else memset(&vv[u], 0, sizeof(vv[u]));
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      int t = t0 + u * TG;
      float p = t < pos ? sc[t] : 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = fmaf(p, Elem<T>::load(vv[u].v[i]), acc[i]);
    }
  }
  if (tg == (pos % TG)) {  // the new value row joins the group that would have owned key `pos`
    float p = sc[pos];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = fmaf(p, Elem<T>::load(v_new[ch * VEC + i]), acc[i]);
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i) part[tg * HD + ch * VEC + i] = acc[i];
  __syncthreads();
  if (threadIdx.x < HD) {
    float s = 0.f;
    for (int g = 0; g < TG; ++g) s += part[g * HD + threadIdx.x];
    ((T*)a.out)[(long long)b * a.out_row_stride + h * HD + threadIdx.x] = Elem<T>::store(s);
  }
}

// ---- decode attention for many sequences: one warp per query head, one CTA per (kv head, sequence) ---------
// Same sub-graph and rounding points as attn_decode_kernel; used when batch x heads is large enough to fill the
// GPU with warps.  The `rep` query heads of a GQA group sit in one CTA, so each K/V row is fetched from L2 once
// and served to the other heads by L1.  No block-wide reduction: scores, softmax and P.v of a head stay in its
// warp (lane = key in the score pass, lane = slice of the head dimension in the P.v pass).
template <class T, int HD>
__global__ void __launch_bounds__(256) attn_decode_warp_kernel(AttnArgs a, unsigned* err) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int VEC = 16 / sizeof(T);
  constexpr int half = HD / 2;
  constexpr int DPL = HD / 32;  // head-dim elements per lane in the P.v pass
  const int rep = a.nh / a.nkv;
  const int kvh = blockIdx.x, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = kvh * rep + warp;
  // the new k row is read with 16-byte loads like a cache row, so it sits first (16-byte aligned)
  T* k_new = reinterpret_cast<T*>(smem_raw);                          // [HD]
  T* v_new = k_new + HD;                                              // [HD]
  float* q_all = reinterpret_cast<float*>(v_new + HD);                // [rep][HD]
  float* sc_all = q_all + (size_t)rep * HD;                           // [rep][P + 1]
  float* sc = sc_all + (size_t)warp * (a.P + 1);
  float* q_s = q_all + (size_t)warp * HD;
  pdl_launch_dependents();
  pdl_wait();
  const int pos = *a.ctx_len;
  if (pos >= a.P) {
    if (threadIdx.x == 0) atomicOr(err, DEV_ERR_INDEX_OOB);
    return;
  }
  const int total = pos + 1;
  T* kc = (T*)a.kc + ((long long)b * a.nkv + kvh) * a.P * HD;
  T* vc = (T*)a.vc + ((long long)b * a.nkv + kvh) * a.P * HD;
  const float* ct = a.cos_t + (long long)pos * half;
  const float* st = a.sin_t + (long long)pos * half;

  // RoPE of this warp's q; warp 0 also rotates the new k row and copies the new v row
  {
    const T* qsrc = (const T*)a.q + (long long)b * a.q_row_stride + h * HD;
    for (int i = lane; i < half; i += 32) {
      float x1 = Elem<T>::load(qsrc[i]), x2 = Elem<T>::load(qsrc[i + half]);
      float c = ct[i], sn = st[i];
      q_s[i] = rt<T>(c * x1 + sn * (-x2));
      q_s[i + half] = rt<T>(c * x2 + sn * x1);
    }
    if (warp == 0) {
      const T* ksrc = (const T*)a.k + (long long)b * a.k_row_stride + kvh * HD;
      const T* vsrc = (const T*)a.v + (long long)b * a.v_row_stride + kvh * HD;
      for (int i = lane; i < half; i += 32) {
        float x1 = Elem<T>::load(ksrc[i]), x2 = Elem<T>::load(ksrc[i + half]);
        float c = ct[i], sn = st[i];
        T o1 = Elem<T>::store(c * x1 + sn * (-x2)), o2 = Elem<T>::store(c * x2 + sn * x1);
        k_new[i] = o1;
        k_new[i + half] = o2;
        kc[(long long)pos * HD + i] = o1;
        kc[(long long)pos * HD + i + half] = o2;
      }
      for (int i = lane; i < HD; i += 32) {
        T vv = vsrc[i];
        v_new[i] = vv;
        vc[(long long)pos * HD + i] = vv;
      }
    }
  }
  __syncthreads();

  // scores: lane = key
  float mx = -FLT_MAX;
  for (int t = lane; t < total; t += 32) {
    const T* krow = t == pos ? k_new : kc + (long long)t * HD;
    float d = 0.f;
#pragma unroll
    for (int c = 0; c < HD / VEC; ++c) {
      VecT<T, VEC> kv = *reinterpret_cast<const VecT<T, VEC>*>(krow + c * VEC);
#pragma unroll
      for (int i = 0; i < VEC; ++i) d = fmaf(q_s[c * VEC + i], Elem<T>::load(kv.v[i]), d);
    }
    float sres = rt<T>(rt<T>(d) / a.scale);
    sc[t] = sres;
    mx = fmaxf(mx, sres);
  }
  mx = warp_max(mx);  // `max` folds from f32::MIN (ndarray.rs:656-661): at least one key exists
  float sum = 0.f;
  for (int t = lane; t < total; t += 32) {
    float e = expf(sc[t] - mx);
    sc[t] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  for (int t = lane; t < total; t += 32) sc[t] = rt<T>(sc[t] / sum);
  __syncwarp();

  // P.v: lane = DPL consecutive elements of the head dimension, keys in order
  float acc[DPL];
#pragma unroll
  for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
  const int d0 = lane * DPL;
#pragma unroll 8
  for (int t = 0; t < pos; ++t) {
    const float p = sc[t];
    const VecT<T, DPL> vv = *reinterpret_cast<const VecT<T, DPL>*>(vc + (long long)t * HD + d0);
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = fmaf(p, Elem<T>::load(vv.v[i]), acc[i]);
  }
  {
    const float p = sc[pos];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = fmaf(p, Elem<T>::load(v_new[d0 + i]), acc[i]);
  }
  // `out` is an allocator-aligned buffer whose rows are a multiple of HD elements; h * HD + d0 is a multiple of DPL
  VecT<T, DPL> ov;
#pragma unroll
  for (int i = 0; i < DPL; ++i) ov.v[i] = Elem<T>::store(acc[i]);
  *reinterpret_cast<VecT<T, DPL>*>((T*)a.out + (long long)b * a.out_row_stride + h * HD + d0) = ov;
}

// ---- decode-attention scores on the tensor cores ------------------------------------------------------------------
// scores[h, t] = T(T(q[h] . k[t]) / scale) for the REP (<= 8) query heads of one kv head and the cached keys of the
// 32-key blocks blk0, blk0 + blk_step, ... below `pos`, written to p_s[h * pp + t]; the running maximum per head comes
// back in mx.  mma.sync.m16n8k16: the query heads are rows 0..REP-1 of the A operand (rows up to 15 are zero), eight
// keys are the columns of B, whose fragments are read straight from the key rows in global memory with 16-byte loads.
// The key of the current position (k_new, still in shared memory) is dotted by the whole warp when
// `owns_new`.  Against the FMA form this takes a fifth of the issue slots and has no dependent 64-long FMA chains.
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                               uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <int HD, int REP, int BLKS>
__device__ __forceinline__ void decode_scores_mma(const float* q_s, const __nv_bfloat16* kc, const __nv_bfloat16* k_new, int pos,
                                                  int blk0, int blk_step, bool owns_new, float* p_s, int pp, float scale,
                                                  float (&mx)[REP]) {
  static_assert(REP <= 8, "the query heads of a group are rows 0..7 of the A fragment");
  using T = __nv_bfloat16;
  constexpr int KS = HD / 16;
  constexpr int NBU = HD <= 64 ? 4 : 2;   // 8-key column blocks whose loads are in flight together
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // A dot product does not care in which order the head dimension is walked, as long as both operands agree: lane t of
  // a quad takes the 16-byte chunks t, t + 4, ... of a key row (two 16-byte loads per 64 elements instead of eight
  // 4-byte ones, whole sectors per request), and k-step ks multiplies words 2ks and 2ks + 1 of what it holds.  The
  // query fragment is packed from the same elements: word m = 4j + i of lane t is elements 8t + 32j + 2i, + 1.
  uint32_t qa0[KS], qa2[KS];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    qa0[ks] = 0u;
    qa2[ks] = 0u;
    if (g < REP) {   // q_s holds values already rounded to T: the packing is exact
      const float* qrow = q_s + g * HD + 8 * t + 32 * (ks / 2) + 4 * (ks % 2);
      __nv_bfloat162 lo = __floats2bfloat162_rn(qrow[0], qrow[1]), hi = __floats2bfloat162_rn(qrow[2], qrow[3]);
      qa0[ks] = *reinterpret_cast<uint32_t*>(&lo);
      qa2[ks] = *reinterpret_cast<uint32_t*>(&hi);
    }
  }
  float mxl = -FLT_MAX;
  // BLKS blocks of 32 keys per round, the 16-byte loads of a whole round issued before its first product: the phase
  // is bound by the number of dependent memory round trips, not by arithmetic (measured at 256 sequences, context
  // ~140: two blocks per round -3.5 % of the step with one warp per pair; no gain with two warps per pair)
  for (int blk = blk0; blk * 32 < pos; blk += BLKS * blk_step) {
#pragma unroll
    for (int nb0 = 0; nb0 < 4; nb0 += NBU) {
      uint32_t bf[BLKS][NBU][KS][2];
#pragma unroll
      for (int sb = 0; sb < BLKS; ++sb)
#pragma unroll
        for (int u = 0; u < NBU; ++u) {
          const int key = (blk + sb * blk_step) * 32 + (nb0 + u) * 8 + g;
          const bool valid = key < pos;
          const uint4* row = reinterpret_cast<const uint4*>(kc + (long long)(valid ? key : 0) * HD);
#pragma unroll
          for (int j = 0; j < HD / 32; ++j) {
            const uint4 w = valid ? row[t + 4 * j] : make_uint4(0u, 0u, 0u, 0u);
            bf[sb][u][2 * j][0] = w.x;
            bf[sb][u][2 * j][1] = w.y;
            bf[sb][u][2 * j + 1][0] = w.z;
            bf[sb][u][2 * j + 1][1] = w.w;
          }
        }
#pragma unroll
      for (int sb = 0; sb < BLKS; ++sb)
#pragma unroll
        for (int u = 0; u < NBU; ++u) {
          float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int ks = 0; ks < KS; ++ks) mma_bf16_16816(c, qa0[ks], 0u, qa2[ks], 0u, bf[sb][u][ks][0], bf[sb][u][ks][1]);
          if (g < REP) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int key = (blk + sb * blk_step) * 32 + (nb0 + u) * 8 + t * 2 + e;
              if (key < pos) {
                const float sres = rt<T>(rt<T>(c[e]) / scale);
                p_s[g * pp + key] = sres;
                mxl = fmaxf(mxl, sres);
              }
            }
          }
        }
    }
  }
  mxl = fmaxf(mxl, __shfl_xor_sync(0xffffffffu, mxl, 1));
  mxl = fmaxf(mxl, __shfl_xor_sync(0xffffffffu, mxl, 2));
#pragma unroll
  for (int h = 0; h < REP; ++h) mx[h] = g == h ? mxl : -FLT_MAX;
  if (owns_new) {
#pragma unroll
    for (int h = 0; h < REP; ++h) {
      float d = 0.f;
      for (int i = lane; i < HD; i += 32) d = fmaf(q_s[h * HD + i], __bfloat162float(k_new[i]), d);
      d = warp_sum(d);
      const float sres = rt<T>(rt<T>(d) / scale);
      if (lane == 0) p_s[h * pp + pos] = sres;
      mx[h] = fmaxf(mx[h], sres);
    }
  }
  __syncwarp();   // the scores were written by other lanes than those that read them next
}

// ---- decode attention for very many sequences: one warp per (kv head, sequence), all its query heads --------
// Same sub-graph and rounding points again.  Each K row is loaded once into registers and dotted with the REP query
// heads of the group; in the P.v pass a lane owns 8 head-dim elements of every (32 / (HD/8))-th key, so every load
// is 16 bytes and a warp keeps 4 KB in flight.  No block-level synchronisation: a warp is self-contained.
template <class T, int HD, int REP>
__global__ void __launch_bounds__(128) attn_decode_group_kernel(AttnArgs a, unsigned* err) {
  static_assert(sizeof(T) == 2, "16-byte rows of 8 elements");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int CH = HD / 8;    // 16-byte chunks per K/V row
  constexpr int KG = 32 / CH;   // keys covered by one warp-wide load in the P.v pass
  constexpr int half = HD / 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.x * 4 + warp, b = blockIdx.y;
  // per warp: k_new[HD] T | v_new[HD] T | q[REP][HD] f32 | p[REP][P + 1] f32
  const size_t per_warp = (size_t)2 * HD * sizeof(T) + (size_t)REP * HD * 4 + (size_t)REP * (a.P + 1) * 4;
  unsigned char* base = smem_raw + (size_t)warp * ((per_warp + 15) / 16 * 16);
  T* k_new = reinterpret_cast<T*>(base);
  T* v_new = k_new + HD;
  float* q_s = reinterpret_cast<float*>(v_new + HD);
  float* p_s = q_s + REP * HD;
  const int pp = a.P + 1;
  pdl_launch_dependents();
  pdl_wait();
  if (kvh >= a.nkv) return;
  const int pos = *a.ctx_len;
  if (pos >= a.P) {
    if (lane == 0) atomicOr(err, DEV_ERR_INDEX_OOB);
    return;
  }
  const int total = pos + 1;
  T* kc = (T*)a.kc + ((long long)b * a.nkv + kvh) * a.P * HD;
  T* vc = (T*)a.vc + ((long long)b * a.nkv + kvh) * a.P * HD;
  const float* ct = a.cos_t + (long long)pos * half;
  const float* st = a.sin_t + (long long)pos * half;
  // RoPE of the group's query heads and of the new key; the new value row is copied
  for (int i = lane; i < REP * half; i += 32) {
    const int h = i / half, j = i - h * half;
    const T* qsrc = (const T*)a.q + (long long)b * a.q_row_stride + (kvh * REP + h) * HD;
    float x1 = Elem<T>::load(qsrc[j]), x2 = Elem<T>::load(qsrc[j + half]);
    float c = ct[j], sn = st[j];
    q_s[h * HD + j] = rt<T>(c * x1 + sn * (-x2));
    q_s[h * HD + j + half] = rt<T>(c * x2 + sn * x1);
  }
  {
    const T* ksrc = (const T*)a.k + (long long)b * a.k_row_stride + kvh * HD;
    const T* vsrc = (const T*)a.v + (long long)b * a.v_row_stride + kvh * HD;
    for (int i = lane; i < half; i += 32) {
      float x1 = Elem<T>::load(ksrc[i]), x2 = Elem<T>::load(ksrc[i + half]);
      float c = ct[i], sn = st[i];
      T o1 = Elem<T>::store(c * x1 + sn * (-x2)), o2 = Elem<T>::store(c * x2 + sn * x1);
      k_new[i] = o1;
      k_new[i + half] = o2;
      kc[(long long)pos * HD + i] = o1;
      kc[(long long)pos * HD + i + half] = o2;
    }
    for (int i = lane; i < HD; i += 32) {
      T vv = vsrc[i];
      v_new[i] = vv;
      vc[(long long)pos * HD + i] = vv;
    }
  }
  __syncwarp();

  // scores on the tensor cores (all cached keys, then the new one)
  float mx[REP];
  decode_scores_mma<HD, REP, (HD <= 64 ? 2 : 1)>(q_s, kc, k_new, pos, 0, 1, true, p_s, pp, a.scale, mx);
#pragma unroll
  for (int h = 0; h < REP; ++h) {
    const float m = warp_max(mx[h]);
    float sum = 0.f;
    for (int t = lane; t < total; t += 32) {
      const float e = expf(p_s[h * pp + t] - m);
      p_s[h * pp + t] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    for (int t = lane; t < total; t += 32) p_s[h * pp + t] = rt<T>(p_s[h * pp + t] / sum);
  }
  __syncwarp();

  // P.v: lane = (key group g, chunk c)
  const int g = lane / CH, c = lane % CH;
  float acc[REP][8];
#pragma unroll
  for (int h = 0; h < REP; ++h)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[h][i] = 0.f;
#pragma unroll 16
  for (int t = g; t < pos; t += KG) {
    const uint4 vv = *reinterpret_cast<const uint4*>(vc + (long long)t * HD + c * 8);
    const T* e = reinterpret_cast<const T*>(&vv);
#pragma unroll
    for (int h = 0; h < REP; ++h) {
      const float ph = p_s[h * pp + t];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[h][i] = fmaf(ph, Elem<T>::load(e[i]), acc[h][i]);
    }
  }
  if (g == 0) {
#pragma unroll
    for (int h = 0; h < REP; ++h) {
      const float ph = p_s[h * pp + pos];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[h][i] = fmaf(ph, Elem<T>::load(v_new[c * 8 + i]), acc[h][i]);
    }
  }
#pragma unroll
  for (int h = 0; h < REP; ++h)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float v = acc[h][i];
#pragma unroll
      for (int o = CH; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[h][i] = v;
    }
  if (g == 0) {
#pragma unroll
    for (int h = 0; h < REP; ++h) {
      uint4 ov;
      T* o = reinterpret_cast<T*>(&ov);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = Elem<T>::store(acc[h][i]);
      *reinterpret_cast<uint4*>((T*)a.out + (long long)b * a.out_row_stride + (kvh * REP + h) * HD + c * 8) = ov;
    }
  }
}

// ---- the same with TWO warps per (kv head, sequence): the keys of a pair are interleaved in blocks of 32 between
// its warps (half the dependent load rounds per warp); maxima, sums and the partial P.v meet in shared memory behind
// 64-thread named barriers.  CTA = 2 pairs.  Rounding points unchanged; summation order: warp 0's keys, then warp 1's.
__device__ __forceinline__ void pair_barrier(int pair) { asm volatile("bar.sync %0, 64;" ::"r"(pair + 1) : "memory"); }

template <class T, int HD, int REP>
__global__ void __launch_bounds__(128) attn_decode_pair_kernel(AttnArgs a, unsigned* err) {
  static_assert(sizeof(T) == 2, "16-byte rows of 8 elements");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int CH = HD / 8, KG = 32 / CH, half = HD / 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = warp >> 1, hw = warp & 1, pl = hw * 32 + lane;   // lane index within the pair: 0..63
  const int kvh = blockIdx.x * 2 + pair, b = blockIdx.y;
  // per pair: k_new[HD] T | v_new[HD] T | q[REP][HD] | acc_x[REP][HD] | red[2][2*REP] | p[REP][P + 1]   (f32 after the T rows)
  const size_t per_pair = ((size_t)2 * HD * sizeof(T) + (size_t)(2 * REP * HD + 4 * REP + REP * (a.P + 1)) * 4 + 15) / 16 * 16;
  unsigned char* base = smem_raw + (size_t)pair * per_pair;
  T* k_new = reinterpret_cast<T*>(base);
  T* v_new = k_new + HD;
  float* q_s = reinterpret_cast<float*>(v_new + HD);
  float* acc_x = q_s + REP * HD;
  float* red = acc_x + REP * HD;        // [0..2*REP): maxima of warp 0 / 1, [2*REP..4*REP): sums
  float* p_s = red + 4 * REP;
  const int pp = a.P + 1;
  pdl_launch_dependents();
  pdl_wait();
  const bool live = kvh < a.nkv;
  const int pos = *a.ctx_len;
  if (pos >= a.P) {
    if (threadIdx.x == 0) atomicOr(err, DEV_ERR_INDEX_OOB);
    return;
  }
  const int total = pos + 1;
  const int kv_i = live ? kvh : 0;      // dead pairs (odd nkv) walk pair 0's data and store nothing: barriers stay matched
  T* kc = (T*)a.kc + ((long long)b * a.nkv + kv_i) * a.P * HD;
  T* vc = (T*)a.vc + ((long long)b * a.nkv + kv_i) * a.P * HD;
  const float* ct = a.cos_t + (long long)pos * half;
  const float* st = a.sin_t + (long long)pos * half;
  for (int i = pl; i < REP * half; i += 64) {
    const int h = i / half, j = i - h * half;
    const T* qsrc = (const T*)a.q + (long long)b * a.q_row_stride + (kv_i * REP + h) * HD;
    float x1 = Elem<T>::load(qsrc[j]), x2 = Elem<T>::load(qsrc[j + half]);
    float c = ct[j], sn = st[j];
    q_s[h * HD + j] = rt<T>(c * x1 + sn * (-x2));
    q_s[h * HD + j + half] = rt<T>(c * x2 + sn * x1);
  }
  {
    const T* ksrc = (const T*)a.k + (long long)b * a.k_row_stride + kv_i * HD;
    const T* vsrc = (const T*)a.v + (long long)b * a.v_row_stride + kv_i * HD;
    for (int i = pl; i < half; i += 64) {
      float x1 = Elem<T>::load(ksrc[i]), x2 = Elem<T>::load(ksrc[i + half]);
      float c = ct[i], sn = st[i];
      T o1 = Elem<T>::store(c * x1 + sn * (-x2)), o2 = Elem<T>::store(c * x2 + sn * x1);
      k_new[i] = o1;
      k_new[i + half] = o2;
      if (live) {
        kc[(long long)pos * HD + i] = o1;
        kc[(long long)pos * HD + i + half] = o2;
      }
    }
    for (int i = pl; i < HD; i += 64) {
      T vv = vsrc[i];
      v_new[i] = vv;
      if (live) vc[(long long)pos * HD + i] = vv;
    }
  }
  pair_barrier(pair);
  // scores on the tensor cores: this warp's 32-key blocks hw, hw + 2, ...; the new key goes to the warp whose block holds it
  float mx[REP];
  decode_scores_mma<HD, REP, 1>(q_s, kc, k_new, pos, hw, 2, ((pos >> 5) & 1) == hw, p_s, pp, a.scale, mx);
#pragma unroll
  for (int h = 0; h < REP; ++h) {
    const float m = warp_max(mx[h]);
    if (lane == 0) red[hw * REP + h] = m;
  }
  pair_barrier(pair);
  float sm_[REP];
#pragma unroll
  for (int h = 0; h < REP; ++h) {
    const float m = fmaxf(red[h], red[REP + h]);
    float sum = 0.f;
    for (int t = pl; t < total; t += 64) {
      const float e = expf(p_s[h * pp + t] - m);
      p_s[h * pp + t] = e;
      sum += e;
    }
    sm_[h] = warp_sum(sum);
    if (lane == 0) red[2 * REP + hw * REP + h] = sm_[h];
  }
  pair_barrier(pair);
#pragma unroll
  for (int h = 0; h < REP; ++h) {
    const float sum = red[2 * REP + h] + red[3 * REP + h];
    for (int t = pl; t < total; t += 64) p_s[h * pp + t] = rt<T>(p_s[h * pp + t] / sum);
  }
  pair_barrier(pair);
  // P.v: lane = (key group g, 16-byte chunk c); warp hw takes keys hw*KG + g, + 2*KG, ...
  const int g = lane / CH, c = lane % CH;
  float acc[REP][8];
#pragma unroll
  for (int h = 0; h < REP; ++h)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[h][i] = 0.f;
#pragma unroll 4
  for (int t = hw * KG + g; t < pos; t += 2 * KG) {
    const uint4 vv = *reinterpret_cast<const uint4*>(vc + (long long)t * HD + c * 8);
    const T* e = reinterpret_cast<const T*>(&vv);
#pragma unroll
    for (int h = 0; h < REP; ++h) {
      const float ph = p_s[h * pp + t];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[h][i] = fmaf(ph, Elem<T>::load(e[i]), acc[h][i]);
    }
  }
  if (g == 0 && hw == 1) {   // the new value row
#pragma unroll
    for (int h = 0; h < REP; ++h) {
      const float ph = p_s[h * pp + pos];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[h][i] = fmaf(ph, Elem<T>::load(v_new[c * 8 + i]), acc[h][i]);
    }
  }
#pragma unroll
  for (int h = 0; h < REP; ++h)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float v = acc[h][i];
#pragma unroll
      for (int o = CH; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[h][i] = v;
    }
  if (hw == 1 && g == 0) {
#pragma unroll
    for (int h = 0; h < REP; ++h)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc_x[h * HD + c * 8 + i] = acc[h][i];
  }
  pair_barrier(pair);
  if (hw == 0 && g == 0 && live) {
#pragma unroll
    for (int h = 0; h < REP; ++h) {
      uint4 ov;
      T* o = reinterpret_cast<T*>(&ov);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = Elem<T>::store(acc[h][i] + acc_x[h * HD + c * 8 + i]);
      *reinterpret_cast<uint4*>((T*)a.out + (long long)b * a.out_row_stride + (kvh * REP + h) * HD + c * 8) = ov;
    }
  }
}

// ---- decode attention for long contexts: keys split into chunks of 128 across CTAs ---------------------------
// Two launches per layer, grid (chunk, kv head, sequence), 128 threads.  Same sub-graph and rounding points as
// attn_decode_kernel (scores and probabilities are rounded to T exactly as there; only the f32 summation orders
// differ).  The REP query heads of a kv head share every K/V row that is loaded.
//   attn_split_scores_kernel : RoPE(q), RoPE(k) + cache append (by the CTA whose chunk holds the new position), one
//                              key per thread: scaled scores of the group's heads -> scores[b, h, t] (f32 scratch).
//   attn_split_pv_kernel     : row max and sum over all t (re-read from the scratch, L2-resident), probabilities of
//                              the chunk's keys, partial P.v -> partial[b, h, chunk, :] (f32).  The last CTA of a
//                              (sequence, kv head) to finish - an atomic counter, no waiting - adds the chunks'
//                              partials in chunk order and stores the heads' outputs, so the result is deterministic.
struct AttnSplitArgs {
  AttnArgs a;
  float* scores;      // [B, nh, P]
  float* partial;     // [B, nh, chunks_max, HD]
  unsigned* counters; // [B, nkv], zero between launches
  int chunks_max;
};
constexpr int ATTN_CHUNK = 128;

template <class T, int HD, int REP>
__global__ void __launch_bounds__(128) attn_split_scores_kernel(AttnSplitArgs s, unsigned* err) {
  static_assert(sizeof(T) == 2, "16-byte rows of 8 elements");
  constexpr int CH = HD / 8, half = HD / 2;
  __shared__ __align__(16) float q_s[REP * HD];
  __shared__ __align__(16) T k_new[HD];
  const AttnArgs& a = s.a;
  const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const int pos = *a.ctx_len;
  if (pos >= a.P) {
    if (tid == 0 && chunk == 0) atomicOr(err, DEV_ERR_INDEX_OOB);
    return;
  }
  const int total = pos + 1;
  const int chunks = (total + ATTN_CHUNK - 1) / ATTN_CHUNK;
  if (chunk >= chunks) return;
  T* kc = (T*)a.kc + ((long long)b * a.nkv + kvh) * a.P * HD;
  T* vc = (T*)a.vc + ((long long)b * a.nkv + kvh) * a.P * HD;
  const float* ct = a.cos_t + (long long)pos * half;
  const float* st = a.sin_t + (long long)pos * half;
  for (int i = tid; i < REP * half; i += 128) {
    const int h = i / half, j = i - h * half;
    const T* qsrc = (const T*)a.q + (long long)b * a.q_row_stride + (kvh * REP + h) * HD;
    float x1 = Elem<T>::load(qsrc[j]), x2 = Elem<T>::load(qsrc[j + half]);
    float c = ct[j], sn = st[j];
    q_s[h * HD + j] = rt<T>(c * x1 + sn * (-x2));
    q_s[h * HD + j + half] = rt<T>(c * x2 + sn * x1);
  }
  if (chunk == chunks - 1) {  // this CTA owns position `pos`: it appends the new K/V rows
    const T* ksrc = (const T*)a.k + (long long)b * a.k_row_stride + kvh * HD;
    const T* vsrc = (const T*)a.v + (long long)b * a.v_row_stride + kvh * HD;
    for (int i = tid; i < half; i += 128) {
      float x1 = Elem<T>::load(ksrc[i]), x2 = Elem<T>::load(ksrc[i + half]);
      float c = ct[i], sn = st[i];
      T o1 = Elem<T>::store(c * x1 + sn * (-x2)), o2 = Elem<T>::store(c * x2 + sn * x1);
      k_new[i] = o1;
      k_new[i + half] = o2;
      kc[(long long)pos * HD + i] = o1;
      kc[(long long)pos * HD + i + half] = o2;
    }
    for (int i = tid; i < HD; i += 128) vc[(long long)pos * HD + i] = vsrc[i];
  }
  __syncthreads();
  const int t = chunk * ATTN_CHUNK + tid;
  if (t >= total) return;
  const uint4* krow = reinterpret_cast<const uint4*>(t == pos ? k_new : kc + (long long)t * HD);
  uint4 kr[CH];
#pragma unroll
  for (int c = 0; c < CH; ++c) kr[c] = krow[c];
#pragma unroll
  for (int h = 0; h < REP; ++h) {
    float d = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const T* e = reinterpret_cast<const T*>(&kr[c]);
      const float4 qa = *reinterpret_cast<const float4*>(q_s + h * HD + c * 8);
      const float4 qb = *reinterpret_cast<const float4*>(q_s + h * HD + c * 8 + 4);
      d = fmaf(qa.x, Elem<T>::load(e[0]), d);
      d = fmaf(qa.y, Elem<T>::load(e[1]), d);
      d = fmaf(qa.z, Elem<T>::load(e[2]), d);
      d = fmaf(qa.w, Elem<T>::load(e[3]), d);
      d = fmaf(qb.x, Elem<T>::load(e[4]), d);
      d = fmaf(qb.y, Elem<T>::load(e[5]), d);
      d = fmaf(qb.z, Elem<T>::load(e[6]), d);
      d = fmaf(qb.w, Elem<T>::load(e[7]), d);
    }
    s.scores[((long long)b * a.nh + kvh * REP + h) * a.P + t] = rt<T>(rt<T>(d) / a.scale);
  }
}

template <class T, int HD, int REP>
__global__ void __launch_bounds__(128) attn_split_pv_kernel(AttnSplitArgs s, unsigned* err) {
  static_assert(sizeof(T) == 2, "16-byte rows of 8 elements");
  constexpr int CH = HD / 8, KG = 32 / CH;
  __shared__ float red[4];
  __shared__ float p_s[REP][ATTN_CHUNK];
  __shared__ __align__(16) float accw[4][REP][HD];
  __shared__ int s_last;
  const AttnArgs& a = s.a;
  const int chunk = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  pdl_launch_dependents();
  pdl_wait();
  const int pos = *a.ctx_len;
  if (pos >= a.P) return;
  const int total = pos + 1;
  const int chunks = (total + ATTN_CHUNK - 1) / ATTN_CHUNK;
  if (chunk >= chunks) return;
  const T* vc = (const T*)a.vc + ((long long)b * a.nkv + kvh) * a.P * HD;
  const int t_mine = chunk * ATTN_CHUNK + tid;
  for (int h = 0; h < REP; ++h) {
    const float* sc = s.scores + ((long long)b * a.nh + kvh * REP + h) * a.P;
    float mx = -FLT_MAX;
    for (int t = tid; t < total; t += 128) mx = fmaxf(mx, sc[t]);
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    __syncthreads();
    float sum = 0.f;
    for (int t = tid; t < total; t += 128) sum += expf(sc[t] - mx);
    sum = warp_sum(sum);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = (red[0] + red[1]) + (red[2] + red[3]);
    __syncthreads();
    p_s[h][tid] = t_mine < total ? rt<T>(expf(sc[t_mine] - mx) / sum) : 0.f;
  }
  __syncthreads();
  // P.v over this warp's 32 keys: lane = (key group g, 16-byte chunk c)
  const int g = lane / CH, c = lane % CH;
  float acc[REP][8];
#pragma unroll
  for (int h = 0; h < REP; ++h)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[h][i] = 0.f;
#pragma unroll
  for (int i = 0; i < 32 / KG; ++i) {
    const int j = warp * 32 + g + KG * i;
    const int t = chunk * ATTN_CHUNK + j;
    if (t < total) {
      const uint4 vv = *reinterpret_cast<const uint4*>(vc + (long long)t * HD + c * 8);
      const T* e = reinterpret_cast<const T*>(&vv);
#pragma unroll
      for (int h = 0; h < REP; ++h) {
        const float ph = p_s[h][j];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[h][k] = fmaf(ph, Elem<T>::load(e[k]), acc[h][k]);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < REP; ++h)
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float v = acc[h][k];
#pragma unroll
      for (int o = CH; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (g == 0) accw[warp][h][c * 8 + k] = v;
    }
  __syncthreads();
  for (int i = tid; i < REP * HD; i += 128) {
    const int h = i / HD, d = i - h * HD;
    const float v = (accw[0][h][d] + accw[1][h][d]) + (accw[2][h][d] + accw[3][h][d]);
    s.partial[(((long long)b * a.nh + kvh * REP + h) * s.chunks_max + chunk) * HD + d] = v;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned old = atomicAdd(s.counters + (long long)b * a.nkv + kvh, 1u);
    s_last = old == (unsigned)(chunks - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int i = tid; i < REP * HD; i += 128) {
    const int h = i / HD, d = i - h * HD;
    const float* src = s.partial + (((long long)b * a.nh + kvh * REP + h) * s.chunks_max) * HD + d;
    float v = 0.f;
    for (int cc = 0; cc < chunks; ++cc) v += __ldcg(src + (long long)cc * HD);
    ((T*)a.out)[(long long)b * a.out_row_stride + (kvh * REP + h) * HD + d] = Elem<T>::store(v);
  }
  if (tid == 0) s.counters[(long long)b * a.nkv + kvh] = 0u;
}

// ---- prefill: scale + causal mask + softmax over score rows (llama.rs:330-339) ------------------------
// Row r = ((b*nh + h)*S + s) of scores [.., S, Tt] (T, in place): x = T(x / scale); x = T(x + mask) where the
// mask is T(f32::MIN) for keys after position T0+s (in bf16 that is -inf) and -0.0 otherwise; softmax in f32.
template <class T>
__global__ void __launch_bounds__(256) softmax_mask_kernel(T* __restrict__ scores, int S, int Tt, int pitch, int T0,
                                                           float scale) {
  __shared__ float scratch[8];
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* row = reinterpret_cast<float*>(smem_raw);  // [Tt]
  T* x = scores + (long long)blockIdx.x * pitch;
  const int s = blockIdx.x % S;
  const float masked = rt<T>(-FLT_MAX);
  float mx = -FLT_MAX;
  for (int t = threadIdx.x; t < Tt; t += 256) {
    float v = rt<T>(Elem<T>::load(x[t]) / scale);
    v = rt<T>(v + (t > T0 + s ? masked : -0.0f));
    row[t] = v;
    mx = fmaxf(mx, v);
  }
  mx = block_max_256(mx, scratch);
  float sum = 0.f;
  for (int t = threadIdx.x; t < Tt; t += 256) {
    float e = expf(row[t] - mx);
    row[t] = e;
    sum += e;
  }
  sum = block_sum_256(sum, scratch);
  for (int t = threadIdx.x; t < Tt; t += 256) x[t] = Elem<T>::store(row[t] / sum);
}

// Same for rows that are `pitch` elements apart (pitch a multiple of 16 bytes) and at most 1024 long: one warp per
// row, the row held in registers, 16-byte loads and stores.  Columns [Tt, pitch) are written as zeros.  Used for
// bf16 only: the divisions and the exponential are the fast (~2 ulp of f32) forms, far below the bf16 rounding that
// follows; with the IEEE forms this kernel is bound by the special-function and divide sequences, not by HBM.
template <class T>
__global__ void __launch_bounds__(256) softmax_mask_rows_kernel(T* __restrict__ scores, long long rows, int S, int Tt,
                                                                int pitch, int T0, float scale, int lpr) {
  // lpr = lanes per row (a power of two, 32 / lpr rows per warp): short rows do not leave lanes idle
  constexpr int VEC = 16 / sizeof(T);
  constexpr int MAXV = 1024 / (32 * VEC);
  const int lane = threadIdx.x & 31;
  const int rpw = 32 / lpr, sub = lane / lpr, l = lane % lpr;
  const long long row = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * rpw + sub;
  const bool live = row < rows;
  T* x = scores + (live ? row : 0) * pitch;
  const int s = (int)((live ? row : 0) % S);
  const float masked = rt<T>(-FLT_MAX);
  const int nv = (pitch + lpr * VEC - 1) / (lpr * VEC);
  float v[MAXV][VEC];
  float mx = -FLT_MAX;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int t0 = (j * lpr + l) * VEC;
    if (j < nv && t0 < pitch && live) {
      VecT<T, VEC> in = *reinterpret_cast<const VecT<T, VEC>*>(x + t0);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const int t = t0 + i;
        float y = rt<T>(__fdividef(Elem<T>::load(in.v[i]), scale));
        y = rt<T>(y + (t > T0 + s ? masked : -0.0f));
        y = t < Tt ? y : -FLT_MAX;
        v[j][i] = y;
        mx = fmaxf(mx, y);
      }
    }
  }
  for (int o = lpr >> 1; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int t0 = (j * lpr + l) * VEC;
    if (j < nv && t0 < pitch && live) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        float e = t0 + i < Tt ? __expf(v[j][i] - mx) : 0.f;
        v[j][i] = e;
        sum += e;
      }
    }
  }
  for (int o = lpr >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.0f / sum;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int t0 = (j * lpr + l) * VEC;
    if (j < nv && t0 < pitch && live) {
      VecT<T, VEC> o;
#pragma unroll
      for (int i = 0; i < VEC; ++i) o.v[i] = Elem<T>::store(v[j][i] * inv);
      *reinterpret_cast<VecT<T, VEC>*>(x + t0) = o;
    }
  }
}

// out[b, s, h, :] = in[b, h, s, :]  (the transpose(1,2) + reshape after attention, llama.rs:342-344)
template <class T>
__global__ void __launch_bounds__(256) bhsd_to_bshd_kernel(const T* __restrict__ in, T* __restrict__ out, int B, int nh,
                                                           int S, int HD) {
  constexpr int VEC = 16 / sizeof(T);
  const int per = HD / VEC;
  const long long total = (long long)B * nh * S * per;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    int c = (int)(t % per);
    long long r = t / per;
    int s = (int)(r % S);
    r /= S;
    int h = (int)(r % nh);
    int b = (int)(r / nh);
    VecT<T, VEC> v = *reinterpret_cast<const VecT<T, VEC>*>(in + t * VEC);
    *reinterpret_cast<VecT<T, VEC>*>(out + (((long long)b * S + s) * nh + h) * HD + c * VEC) = v;
  }
}

// h = T( T(silu(gate)) * up )  for the GEMM path (same rounding points as EPI_SILU_MUL)
template <class T>
__global__ void __launch_bounds__(256) silu_mul_kernel(const T* __restrict__ gate, const T* __restrict__ up,
                                                       T* __restrict__ out, long long n) {
  constexpr int VEC = 16 / sizeof(T);
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n / VEC; t += (long long)gridDim.x * blockDim.x) {
    VecT<T, VEC> g = *reinterpret_cast<const VecT<T, VEC>*>(gate + t * VEC);
    VecT<T, VEC> u = *reinterpret_cast<const VecT<T, VEC>*>(up + t * VEC);
    VecT<T, VEC> o;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float gf = Elem<T>::load(g.v[i]);
      float sg = 1.f / (1.f + expf(-gf));
      float si = rt<T>(gf * sg);
      o.v[i] = Elem<T>::store(si * Elem<T>::load(u.v[i]));
    }
    *reinterpret_cast<VecT<T, VEC>*>(out + t * VEC) = o;
  }
}

// Same with gate and up side by side in one [rows, 2F] matrix (the output of one GEMM over the stacked weights):
// gate = gu[r, 0:F], up = gu[r, F:2F]; out is [rows, F].  F is a multiple of 16 bytes.
template <class T>
__global__ void __launch_bounds__(256) silu_mul_packed_kernel(const T* __restrict__ gu, T* __restrict__ out, long long rows,
                                                              int F, int block) {
  constexpr int VEC = 16 / sizeof(T);
  pdl_launch_dependents();   // the down projection that follows may start fetching its weight tiles
  pdl_wait();
  const int per = F / VEC;
  const long long total = rows * per;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long r = t / per;
    const int c = (int)(t - r * per) * VEC;
    // block == 0: row = gate[F] | up[F]; otherwise blocks of `block` gate columns alternate with their up columns
    const long long gi = block ? r * 2 * F + (long long)(c / block) * 2 * block + c % block : r * 2 * F + c;
    const long long ui = block ? gi + block : gi + F;
    VecT<T, VEC> g = *reinterpret_cast<const VecT<T, VEC>*>(gu + gi);
    VecT<T, VEC> u = *reinterpret_cast<const VecT<T, VEC>*>(gu + ui);
    VecT<T, VEC> o;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      float gf = Elem<T>::load(g.v[i]);
      float sg = 1.f / (1.f + expf(-gf));
      float si = rt<T>(gf * sg);
      o.v[i] = Elem<T>::store(si * Elem<T>::load(u.v[i]));
    }
    *reinterpret_cast<VecT<T, VEC>*>(out + r * F + c) = o;
  }
}

// x = T(x + y)  (residual add for the GEMM path)
template <class T>
__global__ void __launch_bounds__(256) add_inplace_kernel(T* __restrict__ x, const T* __restrict__ y, long long n) {
  constexpr int VEC = 16 / sizeof(T);
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < n / VEC; t += (long long)gridDim.x * blockDim.x) {
    VecT<T, VEC> a = *reinterpret_cast<const VecT<T, VEC>*>(x + t * VEC);
    VecT<T, VEC> b = *reinterpret_cast<const VecT<T, VEC>*>(y + t * VEC);
#pragma unroll
    for (int i = 0; i < VEC; ++i) a.v[i] = Elem<T>::store(Elem<T>::load(a.v[i]) + Elem<T>::load(b.v[i]));
    *reinterpret_cast<VecT<T, VEC>*>(x + t * VEC) = a;
  }
}

// RoPE tables, the f32 op sequence of rope_tables_default (helpers/rope.rs:65-104):
// f = i * (2/HD); freq = pow(theta, f); inv = 1/freq; inv = inv / 1.0; ang = pos * inv; cos, sin.
// With llama3 scaling (rope.rs:232-310) inv is rescaled first, again op for op: wavelengths above
// original/low_freq_factor are divided by `factor`, those between the two thresholds blend smoothly.
struct RopeScalingArgs {
  int type;   // 0 none, 1 llama3
  float factor, low_freq_factor, high_freq_factor, original_max_position;
};
__device__ __forceinline__ float rope_inv_freq(int i, float theta, float two_over_d, const RopeScalingArgs& rs) {
  const float f = (float)i * two_over_d;
  float inv = 1.0f / powf(theta, f);
  if (rs.type == 1) {
    const float low_wl = rs.original_max_position / rs.low_freq_factor, high_wl = rs.original_max_position / rs.high_freq_factor;
    const float wavelen = (2.0f * 3.14159265358979323846f) / inv;
    const float low_mask = low_wl < wavelen ? 1.0f : 0.0f;
    inv = low_mask * (inv / rs.factor) + (1.0f - low_mask) * inv;
    const float high_mask = wavelen < high_wl ? 1.0f : 0.0f;
    const float mid_mask = (1.0f - high_mask) * (1.0f - low_mask);
    const float smooth = (rs.original_max_position / wavelen - rs.low_freq_factor) / (rs.high_freq_factor - rs.low_freq_factor);
    const float smoothed = smooth * inv + ((1.0f - smooth) * inv) / rs.factor;
    inv = mid_mask * smoothed + (1.0f - mid_mask) * inv;
  } else {
    inv = inv / 1.0f;
  }
  return inv;
}
__global__ void rope_table_kernel(float* cos_t, float* sin_t, int P, int half, float theta, float two_over_d, RopeScalingArgs rs) {
  for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < P * half; e += gridDim.x * blockDim.x) {
    int pos = e / half, i = e - pos * half;
    float ang = (float)pos * rope_inv_freq(i, theta, two_over_d, rs);
    cos_t[e] = cosf(ang);
    sin_t[e] = sinf(ang);
  }
}

// ---- greedy pick over the logits (llama.rs:225; ndarray.rs:670-694), two stages ----------------------
// Stage 1: every CTA reduces one 4096-wide chunk of one row to a 64-bit key (value image under total_cmp in the
// high word, index in the low word: the maximum key is the LAST index among the greatest values) and writes it
// to the scratch array partials[row * chunks + chunk].  Stage 2 (advance_kernel) reduces the partial keys.
constexpr int ARGMAX_CHUNK = 4096;
template <class T>
__global__ void __launch_bounds__(256) argmax_partial_kernel(const T* __restrict__ logits, long long row_stride, int n,
                                                             unsigned long long* __restrict__ partials) {
  __shared__ unsigned long long wbest[8];
  pdl_launch_dependents();
  pdl_wait();
  const int chunk = blockIdx.x, row = blockIdx.y, chunks = gridDim.x;
  const T* x = logits + (long long)row * row_stride;
  const int lo = chunk * ARGMAX_CHUNK, hi = min(n, lo + ARGMAX_CHUNK);
  unsigned long long best = 0ull;
  constexpr int VEC = 16 / sizeof(T);
  if (((uintptr_t)logits & 15) == 0 && row_stride % VEC == 0) {
    // 16-byte loads over the whole vectors of the chunk (chunk starts are multiples of 4096 elements)
    const int nvec = (hi - lo) / VEC;
    for (int v = threadIdx.x; v < nvec; v += 256) {
      const VecT<T, VEC> in = *reinterpret_cast<const VecT<T, VEC>*>(x + lo + v * VEC);
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        unsigned hiw = (unsigned)total_key(Elem<T>::load(in.v[e])) ^ 0x80000000u;
        unsigned long long key = ((unsigned long long)hiw << 32) | (unsigned)(lo + v * VEC + e);
        best = key > best ? key : best;
      }
    }
    for (int i = lo + nvec * VEC + threadIdx.x; i < hi; i += 256) {
      unsigned hiw = (unsigned)total_key(Elem<T>::load(x[i])) ^ 0x80000000u;
      unsigned long long key = ((unsigned long long)hiw << 32) | (unsigned)i;
      best = key > best ? key : best;
    }
  } else {
    for (int i = lo + threadIdx.x; i < hi; i += 256) {
      unsigned hiw = (unsigned)total_key(Elem<T>::load(x[i])) ^ 0x80000000u;
      unsigned long long key = ((unsigned long long)hiw << 32) | (unsigned)i;
      best = key > best ? key : best;
    }
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
    partials[(long long)row * chunks + chunk] = best;
  }
}

// Stage 2 on its own: one warp per row reduces that row's partial keys to the index (used when the ids of ALL
// positions are wanted, as the term's output is typed: llama.rs:217-225).
__global__ void __launch_bounds__(256) ids_from_partials_kernel(const unsigned long long* __restrict__ partials, int chunks, int rows,
                                                                unsigned* __restrict__ out) {
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

// End of a step: stage 2 of the greedy pick, then the new ids become the next step's input, are recorded for
// the host, and the context length advances.  One CTA of 32 warps (one writer of the two step counters); a warp takes
// rows in groups of eight and issues the loads of a whole group before it reduces any of them, so the kernel costs a
// few dependent memory round trips however many rows there are.
constexpr int ADVANCE_THREADS = 1024;
__global__ void __launch_bounds__(ADVANCE_THREADS) advance_kernel(const unsigned long long* __restrict__ partials, int chunks,
                                                                  unsigned* __restrict__ cur_ids, unsigned* __restrict__ out_ids,
                                                                  int* ctx_len, int* step_no, int B, int S, int out_cap_steps) {
  pdl_launch_dependents();
  pdl_wait();
  const int step = *step_no;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int WARPS = ADVANCE_THREADS / 32, GROUP = 8;
  for (int b0 = warp * GROUP; b0 < B; b0 += WARPS * GROUP) {
    unsigned long long best[GROUP];
#pragma unroll
    for (int j = 0; j < GROUP; ++j) {
      best[j] = 0ull;
      if (b0 + j < B)
        for (int c = lane; c < chunks; c += 32) {
          unsigned long long k = partials[(long long)(b0 + j) * chunks + c];
          best[j] = k > best[j] ? k : best[j];
        }
    }
#pragma unroll
    for (int j = 0; j < GROUP; ++j) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        unsigned long long other = __shfl_xor_sync(0xffffffffu, best[j], o);
        best[j] = other > best[j] ? other : best[j];
      }
      if (lane == 0 && b0 + j < B) {
        unsigned id = (unsigned)(best[j] & 0xffffffffull);
        cur_ids[b0 + j] = id;
        if (step < out_cap_steps) out_ids[(long long)step * B + b0 + j] = id;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    *ctx_len += S;
    *step_no = step + 1;
  }
}

}  // namespace cgk

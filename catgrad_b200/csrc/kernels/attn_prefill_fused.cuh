// Fused causal prefill attention for bf16 (llama.rs:328-344 with stdlib nn::softmax, nn/mod.rs:168-179):
//   scores = bf16(Q K^T) ; y = bf16(scores / scale) ; y = bf16(y + mask) ; p = bf16(softmax_f32(y)) ; out = bf16(p V)
// with every rounding point of the op graph kept, but without the score matrix ever leaving the SM: one CTA owns
// 64 query rows of one head of one sequence, keeps their whole score rows (bf16, as the graph rounds them anyway) in
// shared memory, finds the exact row maximum and sum in f32 from them, rewrites them as bf16 probabilities and
// multiplies by V.  Because the complete row is present, this is the graph's two-pass softmax, not an online
// (rescaling) one.  Key tiles entirely above the causal diagonal are skipped: their probabilities are exactly zero.
// Contexts up to 1024 keys (the score tile must fit in shared memory); longer ones take the unfused kernels.
//
// Tensor cores through mma.sync.m16n8k16 (bf16 in, f32 accumulate): the products are D x 64-sized per tile, too small
// to amortise a tcgen05 pipeline, and the kernel is bound by the softmax arithmetic and the Q / output traffic.
// K and V tiles (64 keys) are staged with cp.async, double-buffered.  Queries of a GQA group read the same K/V rows
// (consecutive CTAs, L2 hits); repeat_kv is an index computation.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cfloat>
#include <cstdint>

namespace cgk {

struct PrefillAttnArgs {
  const __nv_bfloat16* q;   // rotated queries: q[(b * S + s) * q_row + h * HD + d]
  long long q_row;
  const __nv_bfloat16* kc;  // key cache of this layer [B, nkv, P, HD] (rotated keys, positions 0 .. T0 + S - 1 valid)
  const __nv_bfloat16* vc;
  __nv_bfloat16* out;       // [B * S, nh * HD]
  int S, T0, P, nh, nkv;
  float scale;              // bf16(sqrt(HD)) widened
  int pp;                   // row pitch of the score tile in elements: 64 * ceil((T0 + S) / 64) + 8
};

constexpr int PA_ROWS = 64;      // query rows per CTA (4 warps x 16)
constexpr int PA_KEYS = 64;      // keys per staged tile
constexpr int PA_MAX_KEYS = 1024;

__device__ __forceinline__ uint32_t pa_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pa_cp16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;   // src-size 0: the 16 bytes are zero-filled, nothing is read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(pa_smem(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void pa_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void pa_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void pa_ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pa_ldsm4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void pa_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float pa_rt(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float pa_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float pa_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pa_pack(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Stages a tile of 64 rows x HD bf16 (row r from src + r * src_row, rows at or beyond `rows_valid` zero-filled) into
// shared memory with a row pitch of HD + 8 elements (16 bytes of padding: conflict-free ldmatrix).
template <int HD>
__device__ __forceinline__ void pa_stage(__nv_bfloat16* dst, const __nv_bfloat16* src, long long src_row, int rows_valid) {
  constexpr int CPR = HD / 8;   // 16-byte chunks per row
  for (int i = threadIdx.x; i < PA_ROWS * CPR; i += 128) {
    const int r = i / CPR, c = i - r * CPR;
    const bool ok = r < rows_valid;
    pa_cp16(dst + r * (HD + 8) + c * 8, src + (ok ? (long long)r * src_row : 0) + c * 8, ok);
  }
}

template <int HD>
__global__ void __launch_bounds__(128) attn_prefill_fused_kernel(PrefillAttnArgs a) {
  extern __shared__ __align__(16) unsigned char pa_smem_raw[];
  constexpr int TP = HD + 8;                      // tile row pitch (elements)
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(pa_smem_raw);   // [64][TP]
  __nv_bfloat16* kv_s = q_s + PA_ROWS * TP;                             // [2][64][TP]
  __nv_bfloat16* p_s = kv_s + 2 * PA_KEYS * TP;                         // [64][pp]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * PA_ROWS, h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (a.nh / a.nkv);
  const int Tt = a.T0 + a.S;
  int keys = a.T0 + q0 + PA_ROWS;                 // keys any row of this tile may attend to
  if (keys > Tt) keys = Tt;
  const int nkt = (keys + PA_KEYS - 1) / PA_KEYS;
  const __nv_bfloat16* kbase = a.kc + ((long long)b * a.nkv + kvh) * a.P * HD;
  const __nv_bfloat16* vbase = a.vc + ((long long)b * a.nkv + kvh) * a.P * HD;
  const int pp = a.pp;

  // queries of this tile and the first key tile
  pa_stage<HD>(q_s, a.q + ((long long)b * a.S + q0) * a.q_row + (long long)h * HD, a.q_row, a.S - q0);
  pa_stage<HD>(kv_s, kbase, HD, keys);
  pa_commit();
  pa_wait<0>();
  __syncthreads();
  uint32_t qa[HD / 16][4];
  {
    const __nv_bfloat16* qrow = q_s + (warp * 16 + (lane & 15)) * TP + (lane >> 4) * 8;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) pa_ldsm4(qa[ks], pa_smem(qrow + ks * 16));
  }

  // ---- scores: bf16 rows of y into p_s, running row maxima in registers ----
  const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;   // the two tile rows this lane holds in a C fragment
  const int lim_lo = a.T0 + q0 + r_lo, lim_hi = a.T0 + q0 + r_hi;   // last key each row may see
  float mx_lo = -FLT_MAX, mx_hi = -FLT_MAX;
  const float ninf = __int_as_float(0xff800000);
  for (int kt = 0; kt < nkt; ++kt) {
    const __nv_bfloat16* kt_s = kv_s + (kt & 1) * PA_KEYS * TP;
    if (kt + 1 < nkt) {
      pa_stage<HD>(kv_s + ((kt + 1) & 1) * PA_KEYS * TP, kbase + (long long)(kt + 1) * PA_KEYS * HD, HD, keys - (kt + 1) * PA_KEYS);
      pa_commit();
    }
    float acc[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[nb][i] = 0.f;
    // B fragments: K tile rows are keys (n), HD contiguous (k): x4 = two n-blocks x two k-halves
    const __nv_bfloat16* krow = kt_s + ((lane & 7) + ((lane >> 4) << 3)) * TP + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t bf[4];
        pa_ldsm4(bf, pa_smem(krow + np * 16 * TP + ks * 16));
        pa_mma(acc[2 * np], qa[ks], bf[0], bf[1]);
        pa_mma(acc[2 * np + 1], qa[ks], bf[2], bf[3]);
      }
    }
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
      const int t = kt * PA_KEYS + nb * 8 + (lane & 3) * 2;
      float y[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int tt = t + (i & 1);
        const int lim = i < 2 ? lim_lo : lim_hi;
        const float v = pa_rt(__fdividef(pa_rt(acc[nb][i]), a.scale));
        y[i] = tt > lim ? ninf : v;     // bf16(y + bf16(-FLT_MAX)) is -inf for every finite y; bf16(y + -0.0) is y
      }
      mx_lo = fmaxf(mx_lo, fmaxf(y[0], y[1]));
      mx_hi = fmaxf(mx_hi, fmaxf(y[2], y[3]));
      *reinterpret_cast<uint32_t*>(p_s + r_lo * pp + t) = pa_pack(y[0], y[1]);
      *reinterpret_cast<uint32_t*>(p_s + r_hi * pp + t) = pa_pack(y[2], y[3]);
    }
    pa_wait<0>();
    __syncthreads();   // the next tile has landed and nobody still reads the buffer it will replace after that
  }
  // the first V tile travels while the softmax runs (both K buffers are free now)
  pa_stage<HD>(kv_s, vbase, HD, keys);
  pa_commit();
  mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
  mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
  mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
  mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
  __syncwarp();

  // ---- softmax of the warp's 16 rows, exactly two sweeps per row: sum of exp(y - max), then bf16(exp(y - max) / sum) ----
  const int npairs = nkt * PA_KEYS / 2;
  for (int r = 0; r < 16; ++r) {
    const float m = __shfl_sync(0xffffffffu, r < 8 ? mx_lo : mx_hi, (r & 7) * 4);
    uint32_t* row = reinterpret_cast<uint32_t*>(p_s + (warp * 16 + r) * pp);
    float sum = 0.f;
    for (int c = lane; c < npairs; c += 32) {
      const uint32_t w = row[c];
      sum += __expf(pa_lo(w) - m) + __expf(pa_hi(w) - m);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.0f / sum;
    for (int c = lane; c < npairs; c += 32) {
      const uint32_t w = row[c];
      row[c] = pa_pack(__expf(pa_lo(w) - m) * inv, __expf(pa_hi(w) - m) * inv);
    }
  }
  __syncwarp();

  // ---- out = P V ----
  float o[HD / 8][4];
#pragma unroll
  for (int nb = 0; nb < HD / 8; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[nb][i] = 0.f;
  const __nv_bfloat16* prow = p_s + (warp * 16 + (lane & 15)) * pp + (lane >> 4) * 8;
  for (int kt = 0; kt < nkt; ++kt) {
    pa_wait<0>();
    __syncthreads();   // V tile kt is in place; every warp has left the buffer the next one goes to
    if (kt + 1 < nkt) {
      pa_stage<HD>(kv_s + ((kt + 1) & 1) * PA_KEYS * TP, vbase + (long long)(kt + 1) * PA_KEYS * HD, HD, keys - (kt + 1) * PA_KEYS);
      pa_commit();
    }
    const __nv_bfloat16* vt_s = kv_s + (kt & 1) * PA_KEYS * TP;
    // B fragments: V tile rows are keys (k), HD contiguous (n): transposed 8x8 loads, x4 = two k-halves x two n-blocks
    const __nv_bfloat16* vrow = vt_s + ((lane & 7) + ((lane >> 3) & 1) * 8) * TP + (lane >> 4) * 8;
#pragma unroll
    for (int ks = 0; ks < PA_KEYS / 16; ++ks) {
      uint32_t pa[4];
      pa_ldsm4(pa, pa_smem(prow + kt * PA_KEYS + ks * 16));
#pragma unroll
      for (int np = 0; np < HD / 16; ++np) {
        uint32_t bf[4];
        pa_ldsm4_t(bf, pa_smem(vrow + ks * 16 * TP + np * 16));
        pa_mma(o[2 * np], pa, bf[0], bf[1]);
        pa_mma(o[2 * np + 1], pa, bf[2], bf[3]);
      }
    }
  }
  // ---- store: row s of the sequence, columns h * HD + d ----
  const int s_lo = q0 + r_lo, s_hi = q0 + r_hi;
  const long long orow = (long long)a.nh * HD;
  __nv_bfloat16* out_lo = a.out + ((long long)b * a.S + s_lo) * orow + (long long)h * HD + (lane & 3) * 2;
  __nv_bfloat16* out_hi = a.out + ((long long)b * a.S + s_hi) * orow + (long long)h * HD + (lane & 3) * 2;
#pragma unroll
  for (int nb = 0; nb < HD / 8; ++nb) {
    if (s_lo < a.S) *reinterpret_cast<uint32_t*>(out_lo + nb * 8) = pa_pack(o[nb][0], o[nb][1]);
    if (s_hi < a.S) *reinterpret_cast<uint32_t*>(out_hi + nb * 8) = pa_pack(o[nb][2], o[nb][3]);
  }
}

inline size_t prefill_attn_smem(int hd, int total_keys) {
  const int nkt = (total_keys + PA_KEYS - 1) / PA_KEYS;
  return (size_t)(3 * PA_ROWS * (hd + 8) + PA_ROWS * (nkt * PA_KEYS + 8)) * sizeof(__nv_bfloat16);
}

}  // namespace cgk

// Greedy decode steps of the Llama term (llama.rs:144-385, S = 1) as ONE persistent kernel, bf16, batch <= 8.
//
// A decode step of a 1B-parameter model reads ~2.5 GB of weights (0.38 ms at HBM speed) through ~85 dependent
// sub-graphs (per layer: qkv, attention, o_proj, gate/up, down).  As separate launches every sub-graph pays a
// launch, a cold pipeline and a drain.  Here one CTA per SM stays resident for a run of steps and is split in two:
//
//   * the COPY WARP streams this CTA's share of every weight matrix, in the order the step consumes it, into a ring
//     of shared-memory slots with 1-D bulk asynchronous copies (one per weight row, completion counted on the slot's
//     "full" mbarrier).  It waits only for a slot to be released ("empty" mbarrier), never for a grid barrier or an
//     activation: weights depend on nothing, so HBM keeps streaming while the other warps sit in a barrier, load an
//     input vector or run attention, as far ahead as the ring allows;
//   * eight COMPUTE WARPS own the dependent chain: grid barrier -> input vector (RMSNorm fused, helpers/tensors.rs:
//     82-111) -> products -> epilogue of the sub-graph (store / residual add / SiLU-mul / greedy pick).
//
// A ring slot holds a CHUNK: 16 consecutive weight rows x up to 1024 K-columns, rows 2064 bytes apart (the 16 spare
// bytes rotate consecutive rows by four banks, so ldmatrix reads are conflict-free).  The product runs on the tensor
// cores: mma.m16n8k16 with the 16 weight rows as A (ldmatrix.x4 from the slot) and the <= 8 sequences' input vectors
// as the 8 columns of B (f32 accumulate).  The compute warps split the K-steps of a chunk between them, keep their
// partial accumulators across the chunks of a tile, and meet once per tile (named barrier) to add the eight partial
// sums in warp order and run the epilogue.  This is a weight-streaming matrix-vector product; the tensor cores are
// used because they cost one issue slot per 512 bytes of weights, not for their flops.
//
// Attention (llama.rs:296-345) is spread over all CTAs as (sequence, kv head, 128-key chunk) work items.  An item
// rotates q (and the new k row; the item that owns the new position appends k, v to the cache: rope.rs:430-451,
// cache.rs:30-39), computes the bf16-rounded scaled scores of its keys for the query heads of the group, and leaves
// chunk-local softmax statistics (max, sum of exponentials) and the unnormalised P.V partial in global scratch.  The
// loader of the o_proj input combines the chunks (rescale by exp(max_c - max), divide by the total).  Unlike the
// kernel-per-sub-graph plan the probabilities are not rounded to bf16 before P.V; the result differs from it by bf16
// round-off of the attention output and is closer to the f32 evaluation of the term.  Every other rounding point is
// the graph's (bf16 at each op output the graph types as bf16).
//
// Grid barriers (5 per layer, one more for the greedy pick) are taken by the compute warps only.  A launch runs up to
// 64 steps: after a step's last barrier every CTA reduces the per-CTA greedy keys itself, so the next step starts
// without a launch gap and with the weight ring already streaming.  Measured alternatives that were slower on B200
// and are not kept: handing activations over as words tagged with the producing sub-graph's number and re-read until
// current (faster on an idle GPU, slower under the weight stream); an extra L2 prefetch cursor ahead of the ring; a
// polling instead of a blocking copy warp.  Every wait is bounded: on a timeout the CTA
// records DEV_ERR_WAIT_TIMEOUT and raises a device-wide abort word that all other waits poll; the copy warp then
// waits (bounded) for its copies in flight before the CTA returns.  Must be launched cooperatively (all CTAs
// co-resident), 288 threads, one CTA per SM.
//
// HBM-bound; algorithmic bytes per step = every weight once + KV cache read + new KV rows.
#pragma once
#include "llama_kernels.cuh"

namespace cgk {

constexpr int PK_COMPUTE_WARPS = 8;
constexpr int PK_COMPUTE_THREADS = 32 * PK_COMPUTE_WARPS;
constexpr int PK_THREADS = PK_COMPUTE_THREADS + 32;  // + the copy warp
constexpr int PK_TILE_ROWS = 16;                      // weight rows per tile = M of the mma
constexpr int PK_KC = 1024;                           // K-columns per chunk
constexpr int PK_ROW_PITCH = PK_KC * 2 + 16;          // bytes between rows of a slot
constexpr int PK_SLOT_BYTES = PK_TILE_ROWS * PK_ROW_PITCH;
constexpr int PK_MAX_SLOTS = 6;
constexpr int PK_MAX_B = 8;                           // sequences = N of the mma
constexpr int PK_ATT_CHUNK = 128;                     // keys per attention work item
constexpr int PK_XS_PAD = 32;                         // bytes added to an input row so that sequences land on distinct banks
constexpr long long PK_WAIT_CYCLES = 4000000000ll;    // ~2 s
constexpr int PK_PROF_SLOTS = 16;
constexpr int PK_MAX_STEPS = 64;                      // decode steps per launch

struct PkLayer {
  const void *in_norm, *q, *k, *v, *o, *post_norm, *gate, *up, *down;
};

struct PkArgs {
  int L, H, F, NQ, NKV, V, nh, nkv, P, B, G, nslots, xs_pitch, nsteps;
  float eps, scale;
  const void* embed;
  const void* final_norm;
  const void* head;
  const PkLayer* layers;  // device array [L]
  void* x;       // [B, H] residual stream
  void* qkv;     // [B, NQ + 2 NKV]
  void* h;       // [B, F]
  void* logits;  // [B, V]
  float* att;    // [B, nkv, att_chunks, pk_att_item_floats] chunk partials of the attention
  int att_chunks;
  void* kc;      // [L, Bmax, nkv, P, HD]
  void* vc;
  long long kv_layer_stride, kv_seq_stride;
  const float* cos_t;
  const float* sin_t;
  unsigned* ids_cur;            // [B] in: the first step's token ids; out: the ids after the last step
  unsigned* out_ids;            // [steps, B] record
  int* ctx_len;
  int* step_no;
  int out_cap_steps;
  unsigned long long* partials;  // [G * PK_MAX_B] per-CTA greedy-pick keys
  unsigned long long* bar_counter;
  unsigned long long bar_base;   // value of *bar_counter when this launch starts
  unsigned* err;
  unsigned* abort_word;
  unsigned long long* prof;      // optional [G][PK_PROF_SLOTS] cycle counters, or nullptr
};

// Floats of one attention chunk partial: rep x HD accumulators, rep maxima, rep sums; padded to 16 bytes.
__host__ __device__ constexpr int pk_att_item_floats(int HD, int REP) { return (REP * (HD + 2) + 3) & ~3; }

// Number of grid barriers of one step (the host advances bar_base by steps x this x CTAs per launch).
__host__ __device__ inline int pk_barriers_per_step(int L) { return 5 * L + 1; }

__device__ __forceinline__ uint32_t pk_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pk_compute_sync() { asm volatile("bar.sync 1, %0;" ::"n"(PK_COMPUTE_THREADS) : "memory"); }

__device__ __forceinline__ bool pk_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred P1;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n"
      "selp.b32 %0, 1, 0, P1;\n}"
      : "=r"(ok)
      : "r"(pk_smem(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool pk_aborted(const PkArgs& a) { return *(volatile unsigned*)a.abort_word != 0u; }
__device__ __forceinline__ void pk_abort(const PkArgs& a) {
  atomicOr(a.err, DEV_ERR_WAIT_TIMEOUT);
  atomicExch(a.abort_word, 1u);
}
// Bounded mbarrier wait; false = gave up (timeout here, or abort raised elsewhere).
__device__ __forceinline__ bool pk_wait(uint64_t* bar, uint32_t parity, const PkArgs& a) {
  if (pk_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  unsigned spins = 0;
  while (true) {
    if (pk_try_wait(bar, parity)) return true;
    if ((++spins & 255u) == 0u) {
      if (pk_aborted(a)) return false;
      if (clock64() - t0 > PK_WAIT_CYCLES) {
        pk_abort(a);
        return false;
      }
    }
  }
}

// ---- the weight phases and how their tiles are dealt to the CTAs ------------------------------------
// Phases of a layer: 0 qkv (q, k, v stacked), 1 o_proj, 2 gate/up (a tile = 8 gate rows + the same 8 rows of up),
// 3 down; after the last layer: 4 lm_head.  The copy warp and the compute warps walk the same sequence.
enum { PK_QKV = 0, PK_O = 1, PK_GU = 2, PK_DOWN = 3, PK_HEAD = 4 };

struct PkPhase {
  int K, nseg, t_lo, t_hi;
};
__device__ __forceinline__ PkPhase pk_phase(const PkArgs& a, int l, int ph, int cta) {
  PkPhase p;
  int ntiles;
  switch (ph) {
    case PK_QKV: p.K = a.H; ntiles = (a.NQ + 2 * a.NKV) / PK_TILE_ROWS; break;
    case PK_O: p.K = a.NQ; ntiles = a.H / PK_TILE_ROWS; break;
    case PK_GU: p.K = a.H; ntiles = a.F / (PK_TILE_ROWS / 2); break;
    case PK_DOWN: p.K = a.F; ntiles = a.H / PK_TILE_ROWS; break;
    default: p.K = a.H; ntiles = a.V / PK_TILE_ROWS; break;
  }
  p.nseg = (p.K + PK_KC - 1) / PK_KC;
  // contiguous tile ranges, rotated from phase to phase so that the CTAs that get one tile fewer differ
  const unsigned c = (unsigned)(cta + (l * 4 + ph) * 37) % (unsigned)a.G;
  p.t_lo = (int)((unsigned long long)ntiles * c / (unsigned)a.G);
  p.t_hi = (int)((unsigned long long)ntiles * (c + 1) / (unsigned)a.G);
  return p;
}
// Start of weight row r (0..15) of tile t.
__device__ __forceinline__ const __nv_bfloat16* pk_row(const PkArgs& a, int l, int ph, const PkPhase& p, int t, int r) {
  typedef __nv_bfloat16 T;
  if (ph == PK_HEAD) return (const T*)a.head + (long long)(t * PK_TILE_ROWS + r) * p.K;
  const PkLayer& w = a.layers[l];
  if (ph == PK_QKV) {
    const int n = t * PK_TILE_ROWS + r;
    if (n < a.NQ) return (const T*)w.q + (long long)n * p.K;
    if (n < a.NQ + a.NKV) return (const T*)w.k + (long long)(n - a.NQ) * p.K;
    return (const T*)w.v + (long long)(n - a.NQ - a.NKV) * p.K;
  }
  if (ph == PK_O) return (const T*)w.o + (long long)(t * PK_TILE_ROWS + r) * p.K;
  if (ph == PK_GU) {
    const int n = t * (PK_TILE_ROWS / 2) + (r & 7);
    return (const T*)(r < 8 ? w.gate : w.up) + (long long)n * p.K;
  }
  return (const T*)w.down + (long long)(t * PK_TILE_ROWS + r) * p.K;
}

// ---- helpers of the compute warps ----------------------------------------------------------------
__device__ __forceinline__ float pk_block_sum(float v, float* scratch) {
  v = warp_sum(v);
  pk_compute_sync();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  pk_compute_sync();
  float r = 0.f;
#pragma unroll
  for (int w = 0; w < PK_COMPUTE_WARPS; ++w) r += scratch[w];
  return r;
}

// Grid-wide barrier of the compute warps.  Thread 0 publishes the CTA's writes with a release add on the monotonic
// counter and acquires the others' by polling it; the named barrier on both sides extends that to the CTA.
__device__ __forceinline__ bool pk_grid_barrier(const PkArgs& a, unsigned long long& target, int* ok_flag) {
  pk_compute_sync();
  if (threadIdx.x == 0) {
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(a.bar_counter), "l"(1ull) : "memory");
    target += (unsigned long long)a.G;
    int ok = 1;
    const long long t0 = clock64();
    unsigned spins = 0;
    while (true) {
      unsigned long long v;
      asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(a.bar_counter) : "memory");
      if (v >= target) break;
      if ((++spins & 63u) == 0u) {
        if (pk_aborted(a)) { ok = 0; break; }
        if (clock64() - t0 > PK_WAIT_CYCLES) { pk_abort(a); ok = 0; break; }
      }
    }
    *ok_flag = ok;
  }
  pk_compute_sync();
  return *(volatile int*)ok_flag != 0;
}

__device__ __forceinline__ uint4 pk_ldcg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ float pk_bf(unsigned short bits) { return __uint_as_float((unsigned)bits << 16); }
__device__ __forceinline__ unsigned short pk_bits(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float pk_rt(float v) { return pk_bf(pk_bits(v)); }

// Writes the 8 bf16 values of 16-byte group `v` of an input row into shared memory in the order the B fragments of
// mma.m16n8k16 are read: within each 16 K-columns, lane t of a quad reads columns {2t, 2t+1, 2t+8, 2t+9} as one
// 8-byte word.
__device__ __forceinline__ void pk_store_group(unsigned char* xrow, int v, const unsigned short e[8]) {
  unsigned char* g = xrow + (v >> 1) * 32 + (v & 1) * 4;
#pragma unroll
  for (int j = 0; j < 4; ++j) *reinterpret_cast<unsigned*>(g + j * 8) = (unsigned)e[2 * j] | ((unsigned)e[2 * j + 1] << 16);
}

// Input rows of a phase into shared memory: rows[m] (global, bf16, K elements), optionally through RMSNorm.
struct PkRows {
  const __nv_bfloat16* p[PK_MAX_B];
};
__device__ __forceinline__ void pk_load_input(const PkArgs& a, unsigned char* xs, float* scratch, const PkRows& rows, int K,
                                              const __nv_bfloat16* gain) {
  const int nvec = K / 8;
  for (int m = 0; m < a.B; ++m) {
    unsigned char* xrow = xs + (size_t)m * a.xs_pitch;
    if (gain != nullptr) {
      // RMSNorm: y = T( T(x / sqrt(mean(x^2) + eps)) * g ); K / 8 <= 4 * 256 (checked on the host)
      uint4 xv[4], gv[4];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int v = threadIdx.x + j * PK_COMPUTE_THREADS;
        if (v < nvec) {
          xv[j] = pk_ldcg16(rows.p[m] + v * 8);
          gv[j] = *reinterpret_cast<const uint4*>(gain + v * 8);
          const unsigned short* e = reinterpret_cast<const unsigned short*>(&xv[j]);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float f = pk_bf(e[i]);
            ss += f * f;
          }
        }
      }
      ss = pk_block_sum(ss, scratch);
      const float rms = sqrtf(ss / (float)K + a.eps);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int v = threadIdx.x + j * PK_COMPUTE_THREADS;
        if (v < nvec) {
          const unsigned short* e = reinterpret_cast<const unsigned short*>(&xv[j]);
          const unsigned short* g = reinterpret_cast<const unsigned short*>(&gv[j]);
          unsigned short o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = pk_bits(pk_rt(pk_bf(e[i]) / rms) * pk_bf(g[i]));
          pk_store_group(xrow, v, o);
        }
      }
    } else {
      for (int v = threadIdx.x; v < nvec; v += PK_COMPUTE_THREADS) {
        const uint4 u = pk_ldcg16(rows.p[m] + v * 8);
        pk_store_group(xrow, v, reinterpret_cast<const unsigned short*>(&u));
      }
    }
  }
  pk_compute_sync();
}

// Input of o_proj: the attention output [B, NQ], combined from the chunk partials the attention items left behind:
// out[h, :] = sum_c exp(m_c - M) acc_c[h, :] / sum_c exp(m_c - M) l_c with M = max_c m_c, rounded to bf16.
template <int HD, int REP>
__device__ __forceinline__ void pk_load_attention(const PkArgs& a, unsigned char* xs, int nch) {
  constexpr int GPH = HD / 8;  // 16-byte groups per head
  constexpr int item = pk_att_item_floats(HD, REP);
  for (int m = 0; m < a.B; ++m) {
    unsigned char* xrow = xs + (size_t)m * a.xs_pitch;
    for (int v = threadIdx.x; v < a.NQ / 8; v += PK_COMPUTE_THREADS) {
      const int h = v / GPH, d0 = (v - h * GPH) * 8;
      const int kvh = h / REP, r = h - kvh * REP;
      const float* base = a.att + ((long long)(m * a.nkv + kvh) * a.att_chunks) * item;
      float M = -FLT_MAX;
      for (int c = 0; c < nch; ++c) M = fmaxf(M, __ldcg(base + (long long)c * item + REP * HD + r));
      float sum = 0.f, acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int c = 0; c < nch; ++c) {
        const float* it = base + (long long)c * item;
        const float w = expf(__ldcg(it + REP * HD + r) - M);
        sum = fmaf(w, __ldcg(it + REP * HD + REP + r), sum);
        const float4 p0 = __ldcg(reinterpret_cast<const float4*>(it + r * HD + d0));
        const float4 p1 = __ldcg(reinterpret_cast<const float4*>(it + r * HD + d0 + 4));
        acc[0] = fmaf(w, p0.x, acc[0]); acc[1] = fmaf(w, p0.y, acc[1]); acc[2] = fmaf(w, p0.z, acc[2]); acc[3] = fmaf(w, p0.w, acc[3]);
        acc[4] = fmaf(w, p1.x, acc[4]); acc[5] = fmaf(w, p1.y, acc[5]); acc[6] = fmaf(w, p1.z, acc[6]); acc[7] = fmaf(w, p1.w, acc[7]);
      }
      unsigned short o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = pk_bits(acc[i] / sum);
      pk_store_group(xrow, v, o);
    }
  }
  pk_compute_sync();
}

// One attention work item: sequence b, kv head kvh, keys [c * 128, min(pos + 1, (c + 1) * 128)); key `pos` is the new
// token.  256 compute threads.  `smem` needs pk_att_smem_bytes(HD, REP) bytes.
__host__ __device__ constexpr int pk_att_smem_bytes(int HD, int REP) {
  return REP * HD * 4 /*q*/ + REP * PK_ATT_CHUNK * 4 /*scores*/ + PK_COMPUTE_WARPS * REP * HD * 4 /*P.V per warp*/ +
         2 * HD * 2 /*new k, v*/ + 2 * REP * 4 /*max, sum*/ + 64;
}
template <int HD, int REP>
__device__ __forceinline__ void pk_attention_item(const PkArgs& a, int layer, int b, int kvh, int c, int pos,
                                                  unsigned char* smem) {
  typedef __nv_bfloat16 T;
  constexpr int half = HD / 2;
  constexpr int LPK = HD / 8;             // lanes per key (16 bytes each)
  constexpr int KPW = 32 / LPK;           // keys per warp per round
  constexpr int KEYS_W = PK_ATT_CHUNK / PK_COMPUTE_WARPS;  // 16 keys per warp
  constexpr int ROUNDS = KEYS_W / KPW;
  float* q_s = reinterpret_cast<float*>(smem);                 // [REP][HD]
  float* sc = q_s + REP * HD;                                  // [REP][128]
  float* pv_s = sc + REP * PK_ATT_CHUNK;                       // [8][REP][HD]
  unsigned short* k_new = reinterpret_cast<unsigned short*>(pv_s + PK_COMPUTE_WARPS * REP * HD);  // [HD]
  unsigned short* v_new = k_new + HD;                          // [HD]
  float* m_s = reinterpret_cast<float*>(v_new + HD);           // [REP]
  float* l_s = m_s + REP;                                      // [REP]

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LPK, kslot = lane / LPK;
  const int total = pos + 1;
  const int t_base = c * PK_ATT_CHUNK;
  const bool has_new = pos >= t_base && pos < t_base + PK_ATT_CHUNK;
  const long long NQKV = a.NQ + 2 * a.NKV;
  const T* qrow = (const T*)a.qkv + (long long)b * NQKV;
  T* kc = (T*)a.kc + (long long)layer * a.kv_layer_stride + ((long long)b * a.nkv + kvh) * a.kv_seq_stride;
  T* vc = (T*)a.vc + (long long)layer * a.kv_layer_stride + ((long long)b * a.nkv + kvh) * a.kv_seq_stride;

  // ---- cached keys and values of this thread: all loads in flight before anything else ----
  uint4 kv[ROUNDS], vv[ROUNDS];
#pragma unroll
  for (int u = 0; u < ROUNDS; ++u) {
    const int t = t_base + warp * KEYS_W + u * KPW + kslot;
    if (t < pos) {
      kv[u] = *reinterpret_cast<const uint4*>(kc + (long long)t * HD + sub * 8);
      vv[u] = *reinterpret_cast<const uint4*>(vc + (long long)t * HD + sub * 8);
    } else {
      kv[u] = make_uint4(0, 0, 0, 0);
      vv[u] = make_uint4(0, 0, 0, 0);
    }
  }
  // ---- RoPE of the group's query heads and of the new k row (rope.rs:430-451); v row copied ----
  const float* ct = a.cos_t + (long long)pos * half;
  const float* st = a.sin_t + (long long)pos * half;
  for (int e = threadIdx.x; e < REP * half; e += PK_COMPUTE_THREADS) {
    const int r = e / half, i = e - r * half;
    const T* src = qrow + (kvh * REP + r) * HD;
    const float x1 = Elem<T>::load(__ldcg(src + i)), x2 = Elem<T>::load(__ldcg(src + i + half));
    const float cs = ct[i], sn = st[i];
    q_s[r * HD + i] = pk_rt(cs * x1 + sn * (-x2));
    q_s[r * HD + i + half] = pk_rt(cs * x2 + sn * x1);
  }
  if (has_new) {
    for (int i = threadIdx.x; i < half; i += PK_COMPUTE_THREADS) {
      const T* src = qrow + a.NQ + kvh * HD;
      const float x1 = Elem<T>::load(__ldcg(src + i)), x2 = Elem<T>::load(__ldcg(src + i + half));
      const float cs = ct[i], sn = st[i];
      k_new[i] = pk_bits(cs * x1 + sn * (-x2));
      k_new[i + half] = pk_bits(cs * x2 + sn * x1);
    }
    for (int i = threadIdx.x; i < HD; i += PK_COMPUTE_THREADS)
      v_new[i] = __bfloat16_as_ushort(__ldcg(qrow + a.NQ + a.NKV + kvh * HD + i));
  }
  pk_compute_sync();
  if (has_new) {
    // this item owns position `pos`: append to the cache (cache.rs:30-39) and use the rows from shared memory
    for (int i = threadIdx.x; i < HD; i += PK_COMPUTE_THREADS) {
      reinterpret_cast<unsigned short*>(kc)[(long long)pos * HD + i] = k_new[i];
      reinterpret_cast<unsigned short*>(vc)[(long long)pos * HD + i] = v_new[i];
    }
#pragma unroll
    for (int u = 0; u < ROUNDS; ++u) {
      const int t = t_base + warp * KEYS_W + u * KPW + kslot;
      if (t == pos) {
        kv[u] = *reinterpret_cast<const uint4*>(k_new + sub * 8);
        vv[u] = *reinterpret_cast<const uint4*>(v_new + sub * 8);
      }
    }
  }
  // ---- scores = T(T(q.k) / T(sqrt(HD))) (llama.rs:328-333); the mask row of a single new token is all -0.0 ----
  float qf[REP][8];
#pragma unroll
  for (int r = 0; r < REP; ++r)
#pragma unroll
    for (int i = 0; i < 8; ++i) qf[r][i] = q_s[r * HD + sub * 8 + i];
#pragma unroll
  for (int u = 0; u < ROUNDS; ++u) {
    const int tl = warp * KEYS_W + u * KPW + kslot;
    const unsigned short* e = reinterpret_cast<const unsigned short*>(&kv[u]);
    float kf[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) kf[i] = pk_bf(e[i]);
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) d = fmaf(qf[r][i], kf[i], d);
#pragma unroll
      for (int o = LPK / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (sub == 0) sc[r * PK_ATT_CHUNK + tl] = (t_base + tl < total) ? pk_rt(pk_rt(d) / a.scale) : -FLT_MAX;
    }
  }
  pk_compute_sync();
  // ---- chunk-local softmax statistics (nn/mod.rs:168-179 in f32): one warp per query head ----
  for (int r = warp; r < REP; r += PK_COMPUTE_WARPS) {
    float v4[PK_ATT_CHUNK / 32];
    float mx = -FLT_MAX;
#pragma unroll
    for (int j = 0; j < PK_ATT_CHUNK / 32; ++j) {
      v4[j] = sc[r * PK_ATT_CHUNK + lane + 32 * j];
      mx = fmaxf(mx, v4[j]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < PK_ATT_CHUNK / 32; ++j) {
      const int tl = lane + 32 * j;
      const float ev = (t_base + tl < total) ? expf(v4[j] - mx) : 0.f;
      sc[r * PK_ATT_CHUNK + tl] = ev;
      sum += ev;
    }
    sum = warp_sum(sum);
    if (lane == 0) {
      m_s[r] = mx;
      l_s[r] = sum;
    }
  }
  pk_compute_sync();
  // ---- unnormalised P.V partial of this thread's keys, reduced over the warp's key slots, then over the warps ----
  float acc[REP][8];
#pragma unroll
  for (int r = 0; r < REP; ++r)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[r][i] = 0.f;
#pragma unroll
  for (int u = 0; u < ROUNDS; ++u) {
    const int tl = warp * KEYS_W + u * KPW + kslot;
    const unsigned short* e = reinterpret_cast<const unsigned short*>(&vv[u]);
    float vf[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) vf[i] = pk_bf(e[i]);
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      const float p = sc[r * PK_ATT_CHUNK + tl];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[r][i] = fmaf(p, vf[i], acc[r][i]);
    }
  }
#pragma unroll
  for (int r = 0; r < REP; ++r)
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float v = acc[r][i];
#pragma unroll
      for (int o = LPK; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      acc[r][i] = v;
    }
  if (kslot == 0) {
#pragma unroll
    for (int r = 0; r < REP; ++r)
#pragma unroll
      for (int i = 0; i < 8; ++i) pv_s[(warp * REP + r) * HD + sub * 8 + i] = acc[r][i];
  }
  pk_compute_sync();
  float* out = a.att + (((long long)(b * a.nkv + kvh) * a.att_chunks) + c) * pk_att_item_floats(HD, REP);
  for (int e = threadIdx.x; e < REP * HD; e += PK_COMPUTE_THREADS) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < PK_COMPUTE_WARPS; ++w) s += pv_s[w * REP * HD + e];
    out[e] = s;
  }
  if (threadIdx.x < REP) {
    out[REP * HD + threadIdx.x] = m_s[threadIdx.x];
    out[REP * HD + REP + threadIdx.x] = l_s[threadIdx.x];
  }
  pk_compute_sync();   // shared scratch is reused by the next item / the next phase's input
}

// Shared memory: [nslots x slot ring][input rows / attention scratch: xs_bytes][partial sums 2 x 8 x 16 x 8 f32]
//                [mbarriers: full[6], empty[6]][scratch f32[8]][ok flag][best keys u64[128]]
__host__ __device__ constexpr int pk_tail_bytes() { return 2 * PK_COMPUTE_WARPS * PK_TILE_ROWS * PK_MAX_B * 4 + 2 * PK_MAX_SLOTS * 8 + 64 + 16 + 128 * 8 + 32; }

template <int HD, int REP, bool PROF>
__global__ void __launch_bounds__(PK_THREADS, 1) llama_decode_persistent_kernel(PkArgs a, int xs_bytes) {
  typedef __nv_bfloat16 T;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* ring = smem_raw;
  unsigned char* xs = smem_raw + (size_t)a.nslots * PK_SLOT_BYTES;
  float* red = reinterpret_cast<float*>(xs + xs_bytes);                          // [2][8 warps][16 rows][8 cols]
  uint64_t* full = reinterpret_cast<uint64_t*>(red + 2 * PK_COMPUTE_WARPS * PK_TILE_ROWS * PK_MAX_B);
  uint64_t* empty = full + PK_MAX_SLOTS;
  float* scratch = reinterpret_cast<float*>(empty + PK_MAX_SLOTS);               // [16]
  int* ok_flag = reinterpret_cast<int*>(scratch + 16);
  unsigned long long* best_s = reinterpret_cast<unsigned long long*>(ok_flag + 4);  // [128]
  unsigned* ids_s = reinterpret_cast<unsigned*>(best_s + 128);                   // [8] token ids of the current step

  const int cta = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nslots = a.nslots;
  const int B = a.B;

  if (threadIdx.x == 0) {
    for (int s = 0; s < nslots; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pk_smem(&full[s])), "r"(1));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pk_smem(&empty[s])), "r"(PK_COMPUTE_WARPS));
    }
    *ok_flag = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (threadIdx.x < PK_MAX_B) ids_s[threadIdx.x] = threadIdx.x < B ? a.ids_cur[threadIdx.x] : 0u;
  __syncthreads();

  const int pos0 = *a.ctx_len;  // position of the first new token
  if (pos0 + a.nsteps > a.P) {  // cache would overflow: every CTA sees the same value and leaves before anything is issued
    if (threadIdx.x == 0) {
      if (cta == 0) atomicOr(a.err, DEV_ERR_INDEX_OOB);
      // keep the barrier counter in step with the host's bookkeeping (it advances by steps x barriers x CTAs per launch)
      atomicAdd(a.bar_counter, (unsigned long long)a.nsteps * (unsigned long long)pk_barriers_per_step(a.L));
    }
    return;
  }

  // ======================================= the copy warp ===========================================
  if (warp == PK_COMPUTE_WARPS) {
    long long stall = 0;
    int n = 0;
    bool alive = true;
    for (int step = 0; step < a.nsteps && alive; ++step)
    for (int l = 0; l <= a.L && alive; ++l) {
      const int n_ph = l < a.L ? 4 : 1;
      for (int pi = 0; pi < n_ph && alive; ++pi) {
        const int ph = l < a.L ? pi : PK_HEAD;
        const PkPhase p = pk_phase(a, l, ph, cta);
        for (int t = p.t_lo; t < p.t_hi && alive; ++t) {
          const unsigned char* rowp = lane < PK_TILE_ROWS ? reinterpret_cast<const unsigned char*>(pk_row(a, l, ph, p, t, lane)) : nullptr;
          for (int ks = 0; ks < p.nseg; ++ks, ++n) {
            const int slot = n % nslots, use = n / nslots;
            if (use > 0) {
              long long t0 = 0;
              if (PROF) t0 = clock64();
              if (!pk_wait(&empty[slot], (uint32_t)((use - 1) & 1), a)) { alive = false; break; }
              if (PROF) stall += clock64() - t0;
            }
            const int seg = min(PK_KC, p.K - ks * PK_KC);
            const uint32_t bytes = (uint32_t)seg * 2u;
            if (lane == 0)
              asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pk_smem(&full[slot])), "r"(bytes * PK_TILE_ROWS) : "memory");
            __syncwarp();
            if (lane < PK_TILE_ROWS)
              asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                               pk_smem(ring + (size_t)slot * PK_SLOT_BYTES + lane * PK_ROW_PITCH)),
                           "l"(rowp + (size_t)ks * PK_KC * 2), "r"(bytes), "r"(pk_smem(&full[slot]))
                           : "memory");
          }
        }
      }
    }
    if (!alive) {
      // bounded drain of the copies still in flight, so none lands after the CTA has left
      for (int k = n > nslots ? n - nslots : 0; k < n; ++k) {
        const long long t0 = clock64();
        while (!pk_try_wait(&full[k % nslots], (uint32_t)((k / nslots) & 1)) && clock64() - t0 < PK_WAIT_CYCLES) {
        }
      }
    }
    if (PROF && a.prof && lane == 0) a.prof[(long long)cta * PK_PROF_SLOTS + 8] += (unsigned long long)stall;
    asm volatile("bar.sync 2, %0;" ::"n"(PK_THREADS) : "memory");   // leave together with the compute warps
    return;
  }

  // ====================================== the compute warps ========================================
  const long long NQKV = a.NQ + 2 * a.NKV;
  unsigned long long bar_target = a.bar_base;
  // cycle counters of thread 0 (PROF builds): 0 barrier, 1 input, 2 wait for a chunk, 3 products, 4 reduce + epilogue,
  // 5 attention, 6 total, 7 launches; slot 8 is the copy warp's wait for free slots
  long long pc[6] = {0, 0, 0, 0, 0, 0}, pt = 0, pt_start = 0;
  if (PROF) pt = pt_start = clock64();
#define PK_PROF(slot) do { if (PROF) { long long now_ = clock64(); pc[slot] += now_ - pt; pt = now_; } } while (0)

  int n = 0;
  int red_buf = 0;
  bool alive = true;
  const int g = lane >> 2, tq = lane & 3;
  // ldmatrix source of this lane within a slot: rows 0-7 / 8-15 of K-columns 0-7 / 8-15 of a K-step
  const uint32_t lm_off = (uint32_t)(((lane & 7) + ((lane >> 3) & 1) * 8) * PK_ROW_PITCH + (lane >> 4) * 16);
  const uint32_t ring_u32 = pk_smem(ring);
  const uint32_t xfrag_u32 = pk_smem(xs) + (uint32_t)(g * a.xs_pitch + tq * 8);

  for (int step = 0; step < a.nsteps && alive; ++step) {
  const int pos = pos0 + step;              // position of this step's new token
  const int nch = pos / PK_ATT_CHUNK + 1;   // attention chunks in use
  unsigned long long my_best = 0ull;        // greedy pick: thread (row, sequence) keeps the best key of its rows
  // per-sequence embedding rows: the residual stream of layer 0 (helpers/tensors.rs:255-272)
  PkRows emb;
  bool bad_id = false;
#pragma unroll
  for (int m = 0; m < PK_MAX_B; ++m) {
    unsigned id = m < B ? ids_s[m] : 0u;
    if (id >= (unsigned)a.V) {
      bad_id = true;
      id = 0;
    }
    emb.p[m] = (const T*)a.embed + (long long)id * a.H;
  }
  if (bad_id && cta == 0 && threadIdx.x == 0) atomicOr(a.err, DEV_ERR_INDEX_OOB);
  for (int l = 0; l <= a.L && alive; ++l) {
    const int n_ph = l < a.L ? 4 : 1;
    for (int pi = 0; pi < n_ph && alive; ++pi) {
      const int ph = l < a.L ? pi : PK_HEAD;
      // ---- everything the phase reads must be complete: a grid barrier (except before the very first phase) ----
      if (!(l == 0 && ph == PK_QKV)) alive = pk_grid_barrier(a, bar_target, ok_flag);
      if (!alive) break;
      PK_PROF(0);
      if (ph == PK_O) {
        // attention of layer l sits between qkv and o_proj: (sequence, kv head, key chunk) items over the CTAs
        const int items = B * a.nkv * nch;
        for (int it = (int)((unsigned)(cta + l * 61) % (unsigned)a.G); it < items; it += a.G) {
          const int c = it % nch, bk = it / nch;
          pk_attention_item<HD, REP>(a, l, bk / a.nkv, bk % a.nkv, c, pos, xs);
        }
        PK_PROF(5);
        alive = pk_grid_barrier(a, bar_target, ok_flag);
        if (!alive) break;
        PK_PROF(0);
      }
      const PkPhase p = pk_phase(a, l, ph, cta);
      const int K = p.K;
      if (p.t_lo < p.t_hi) {
        // ---- input rows of the phase ----
        if (ph == PK_O) {
          pk_load_attention<HD, REP>(a, xs, nch);
        } else {
          PkRows in;
          const T* gain = nullptr;
          if (ph == PK_DOWN) {
#pragma unroll
            for (int m = 0; m < PK_MAX_B; ++m) in.p[m] = (const T*)a.h + (long long)m * a.F;
          } else {
            const bool from_emb = (l == 0 && ph == PK_QKV);
#pragma unroll
            for (int m = 0; m < PK_MAX_B; ++m) in.p[m] = from_emb ? emb.p[m] : (const T*)a.x + (long long)m * a.H;
            gain = ph == PK_HEAD ? (const T*)a.final_norm : (const T*)(ph == PK_QKV ? a.layers[l].in_norm : a.layers[l].post_norm);
          }
          pk_load_input(a, xs, scratch, in, K, gain);
        }
      }
      PK_PROF(1);

      // ---- this CTA's tiles of the phase ----
      for (int t = p.t_lo; t < p.t_hi && alive; ++t) {
        float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
        for (int ks = 0; ks < p.nseg; ++ks, ++n) {
          const int slot = n % nslots;
          if (!pk_wait(&full[slot], (uint32_t)((n / nslots) & 1), a)) { alive = false; break; }
          PK_PROF(2);
          const int seg = min(PK_KC, K - ks * PK_KC);
          const int nsteps = seg >> 4;
          const uint32_t abase = ring_u32 + (uint32_t)slot * PK_SLOT_BYTES + lm_off;
          const uint32_t bbase = xfrag_u32 + (uint32_t)ks * (PK_KC * 2);
#define PK_MMA_STEP(s_, c_)                                                                                             \
  do {                                                                                                                  \
    uint32_t a0, a1, a2, a3, b0 = 0u, b1 = 0u;                                                                          \
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"                                       \
                 : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3)                                                               \
                 : "r"(abase + (uint32_t)(s_) * 32u));                                                                  \
    if (g < B) asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(bbase + (uint32_t)(s_) * 32u)); \
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};" \
                 : "+f"(c_[0]), "+f"(c_[1]), "+f"(c_[2]), "+f"(c_[3])                                                   \
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));                                               \
  } while (0)
          // this warp's K-steps of the chunk, alternating between two accumulator sets (independent mma chains)
          int s = warp;
#pragma unroll 2
          for (; s + PK_COMPUTE_WARPS < nsteps; s += 2 * PK_COMPUTE_WARPS) {
            PK_MMA_STEP(s, c0);
            PK_MMA_STEP(s + PK_COMPUTE_WARPS, c1);
          }
          if (s < nsteps) PK_MMA_STEP(s, c0);
#undef PK_MMA_STEP
          __syncwarp();
          if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(pk_smem(&empty[slot])) : "memory");
          PK_PROF(3);
        }
        if (!alive) break;
        // ---- the eight warps' partial sums meet; rows x sequences: thread e = row * 8 + sequence ----
        float* redb = red + red_buf * (PK_COMPUTE_WARPS * PK_TILE_ROWS * PK_MAX_B);
        {
          float* w = redb + warp * (PK_TILE_ROWS * PK_MAX_B);
          const int col = 2 * tq;
          if (col < B) {
            w[g * PK_MAX_B + col] = c0[0] + c1[0];
            w[(g + 8) * PK_MAX_B + col] = c0[2] + c1[2];
          }
          if (col + 1 < B) {
            w[g * PK_MAX_B + col + 1] = c0[1] + c1[1];
            w[(g + 8) * PK_MAX_B + col + 1] = c0[3] + c1[3];
          }
        }
        pk_compute_sync();
        if (threadIdx.x < PK_TILE_ROWS * PK_MAX_B) {
          const int r = threadIdx.x >> 3, m = threadIdx.x & 7;
          if (m < B && (ph != PK_GU || r < 8)) {
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int w = 0; w < PK_COMPUTE_WARPS; ++w) s0 += redb[(w * PK_TILE_ROWS + r) * PK_MAX_B + m];
            if (ph == PK_GU) {
#pragma unroll
              for (int w = 0; w < PK_COMPUTE_WARPS; ++w) s1 += redb[(w * PK_TILE_ROWS + r + 8) * PK_MAX_B + m];
            }
            if (ph == PK_QKV) {
              ((T*)a.qkv)[(long long)m * NQKV + t * PK_TILE_ROWS + r] = Elem<T>::store(s0);
            } else if (ph == PK_O || ph == PK_DOWN) {
              // x = res + linear(.) (llama.rs:375,384): the linear output is a bf16 tensor, then one add in bf16
              const int nidx = t * PK_TILE_ROWS + r;
              const T* base = (const T*)a.x;
              long long off = (long long)m * a.H + nidx;
              if (l == 0 && ph == PK_O) {   // the residual of the first layer is the embedding row itself
                base = emb.p[m];
                off = nidx;
              }
              ((T*)a.x)[(long long)m * a.H + nidx] = Elem<T>::store(Elem<T>::load(__ldcg(base + off)) + pk_rt(s0));
            } else if (ph == PK_GU) {
              // silu(gate) * up (llama.rs:245; nn/mod.rs:124-148): silu in f32 as x * (1 / (1 + exp(-x))), cast back
              const float gt = pk_rt(s0), up = pk_rt(s1);
              const float sg = 1.f / (1.f + expf(-gt));
              const float si = pk_rt(gt * sg);
              ((T*)a.h)[(long long)m * a.F + t * (PK_TILE_ROWS / 2) + r] = Elem<T>::store(si * up);
            } else {
              const int nidx = t * PK_TILE_ROWS + r;
              const T lv = Elem<T>::store(s0);
              ((T*)a.logits)[(long long)m * a.V + nidx] = lv;
              const unsigned hiw = (unsigned)total_key(Elem<T>::load(lv)) ^ 0x80000000u;
              const unsigned long long key = ((unsigned long long)hiw << 32) | (unsigned)nidx;
              my_best = key > my_best ? key : my_best;
            }
          }
        }
        red_buf ^= 1;
        PK_PROF(4);
      }
    }
  }

  // ---- greedy pick (llama.rs:225): per-CTA keys, grid barrier, then every CTA reduces the keys to the next ids ----
  if (!alive) break;
  if (threadIdx.x < PK_TILE_ROWS * PK_MAX_B) best_s[threadIdx.x] = my_best;
  pk_compute_sync();
  if (threadIdx.x < B) {
    unsigned long long b = 0ull;
    for (int r = 0; r < PK_TILE_ROWS; ++r) {
      const unsigned long long k = best_s[r * PK_MAX_B + threadIdx.x];
      b = k > b ? k : b;
    }
    a.partials[(long long)cta * PK_MAX_B + threadIdx.x] = b;
  }
  alive = pk_grid_barrier(a, bar_target, ok_flag);
  if (!alive) break;
  if (warp < B) {
    unsigned long long b = 0ull;
    for (int c = lane; c < a.G; c += 32) {
      const unsigned long long k = __ldcg(a.partials + (long long)c * PK_MAX_B + warp);
      b = k > b ? k : b;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
      b = other > b ? other : b;
    }
    if (lane == 0) {
      const unsigned id = (unsigned)(b & 0xffffffffull);
      ids_s[warp] = id;
      if (cta == 0) {
        const int rec = *a.step_no + step;
        a.ids_cur[warp] = id;
        if (rec < a.out_cap_steps) a.out_ids[(long long)rec * B + warp] = id;
      }
    }
  }
  // the partial keys are rewritten only at the end of the next step, many barriers later
  pk_compute_sync();
  PK_PROF(0);
  if (cta == 0 && threadIdx.x == 0 && step + 1 == a.nsteps) {
    *a.ctx_len = pos + 1;
    *a.step_no = *a.step_no + a.nsteps;
  }
  }   // steps
  if (PROF && a.prof && threadIdx.x == 0) {
    unsigned long long* pr = a.prof + (long long)cta * PK_PROF_SLOTS;
    for (int i = 0; i < 6; ++i) pr[i] += (unsigned long long)pc[i];
    pr[6] += (unsigned long long)(clock64() - pt_start);
    pr[7] += (unsigned long long)a.nsteps;
  }
#undef PK_PROF
  asm volatile("bar.sync 2, %0;" ::"n"(PK_THREADS) : "memory");   // shared memory stays alive until the copy warp is done
}

}  // namespace cgk

// One decode step of the Llama term as ONE persistent kernel (batch <= 4).
//
// Why: a decode step of a 1B-parameter model is ~2.5 GB of weight traffic, 0.38 ms at HBM speed, spread over
// ~85 dependent sub-graphs (llama.rs:349-385 per layer: qkv, attention, o_proj, gate/up, down).  As separate
// launches each sub-graph pays launch latency, a cold pipeline and a drain, and the step takes ~3x the HBM time.
// Here one CTA per SM stays resident for the whole step:
//   * this CTA's share of every weight matrix, in the order the step consumes it, streams through a ring of
//     shared-memory slots with 1-D bulk async copies (cp.async.bulk, completion on mbarriers).  Weights do not
//     depend on activations, so the stream runs ahead of the dependent phases: the moment a slot has been
//     consumed, thread 0 refills it with the chunk `nslots` positions ahead, whatever phase or layer that chunk
//     belongs to; while the CTA sits in a grid barrier or in attention, its ring keeps filling from HBM;
//   * the eight warps multiply each slot (R weight rows x K) with the phase's input vector, reduce per row
//     in a fixed order, and apply the epilogue of the sub-graph (store / residual add / SiLU-mul / greedy pick);
//   * phases are separated by a grid-wide barrier (monotonic 64-bit counter in global memory).
// Rounding points are those of the separate kernels (llama_kernels.cuh).
//
// All waits are bounded (mbarrier waits, grid barrier): on a timeout the CTA records DEV_ERR_WAIT_TIMEOUT, raises a
// device-wide abort word that every other wait polls, drains its outstanding copies and returns.
// Must be launched cooperatively (all CTAs co-resident) with 256 threads.
//
// HBM-bound; algorithmic bytes per step = every weight once + KV cache read + new KV rows.
#pragma once
#include "llama_kernels.cuh"

namespace cgk {

constexpr int MEGA_THREADS = 256;
constexpr int MEGA_CONSUMERS = 256;
constexpr int MEGA_SLOT_BYTES = 32768;
constexpr int MEGA_RMAX = 16;  // most weight rows per slot
constexpr long long MEGA_WAIT_CYCLES = 4000000000ll;  // ~2 s

struct MegaLayer {
  const void *in_norm, *q, *k, *v, *o, *post_norm, *gate, *up, *down;
};

struct MegaArgs {
  int L, H, F, NQ, NKV, V, nh, nkv, P, B, G, nslots;
  float eps, scale;
  const void* embed;
  const void* final_norm;
  const void* head;
  const MegaLayer* layers;  // device array [L]
  void* x;       // [B, H] residual stream
  void* qkv;     // [B, NQ + 2 NKV]
  void* attn;    // [B, NQ]
  void* h;       // [B, F]
  void* logits;  // [B, V]
  void* kc;      // [L, Bmax, nkv, P, HD]
  void* vc;
  long long kv_layer_stride;
  const float* cos_t;
  const float* sin_t;
  unsigned* ids_cur;            // [B] in: this step's token ids; out: the next ones
  unsigned* out_ids;            // [steps, B] record
  int* ctx_len;
  int* step_no;
  int out_cap_steps;
  unsigned long long* partials;  // [G * B] scratch: per-CTA greedy-pick keys
  unsigned long long* bar_counter;
  unsigned long long bar_base;   // value of *bar_counter when this launch starts
  unsigned* err;
  unsigned* abort_word;
  unsigned long long* prof;      // optional [G][8] cycle counters (thread 0 of every CTA), or nullptr
};

__device__ __forceinline__ uint32_t mg_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mg_consumer_sync() { __syncthreads(); }

__device__ __forceinline__ bool mg_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred P1;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n"
      "selp.b32 %0, 1, 0, P1;\n}"
      : "=r"(ok)
      : "r"(mg_smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mg_aborted(const MegaArgs& a) { return *(volatile unsigned*)a.abort_word != 0u; }
__device__ __forceinline__ void mg_abort(const MegaArgs& a) {
  atomicOr(a.err, DEV_ERR_WAIT_TIMEOUT);
  atomicExch(a.abort_word, 1u);
}
// Bounded mbarrier wait; false = gave up (timeout here or abort raised elsewhere).
__device__ __forceinline__ bool mg_wait(uint64_t* bar, uint32_t parity, const MegaArgs& a) {
  if (mg_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  unsigned spins = 0;
  while (true) {
    if (mg_try_wait(bar, parity)) return true;
    if ((++spins & 255u) == 0u) {
      if (mg_aborted(a)) return false;
      if (clock64() - t0 > MEGA_WAIT_CYCLES) {
        mg_abort(a);
        return false;
      }
    }
  }
}

// ---- the sequence of weight chunks of one CTA ----------------------------------------------------
// Producer and consumers walk the same deterministic sequence.  Phases of a layer: 0 qkv (matrices q, k, v),
// 1 o_proj, 2 gate/up (chunks alternate: gate rows, then the same rows of up), 3 down; after the last layer:
// 4 lm_head.  A chunk is `rows` consecutive rows of one matrix, K elements each, contiguous in memory.
enum { PH_QKV = 0, PH_O = 1, PH_GU = 2, PH_DOWN = 3, PH_HEAD = 4 };

struct PhaseShape {
  int nmat;         // matrices in the phase
  int n0, n1, n2;   // rows of each (scalars, not an array: a runtime-indexed array would live in local memory)
  int o1, o2;       // offsets of matrices 1 and 2 in the phase's output vector (matrix 0 starts at 0)
  int K;
  bool interleave;  // gate/up: alternate chunks of the two matrices over the same rows
};
__device__ __forceinline__ PhaseShape mg_phase_shape(const MegaArgs& a, int ph) {
  PhaseShape p;
  p.nmat = 1;
  p.n0 = p.n1 = p.n2 = 0;
  p.o1 = p.o2 = 0;
  p.K = a.H;
  p.interleave = false;
  switch (ph) {
    case PH_QKV:
      p.nmat = 3;
      p.n0 = a.NQ; p.n1 = a.NKV; p.n2 = a.NKV;
      p.o1 = a.NQ; p.o2 = a.NQ + a.NKV;
      break;
    case PH_O: p.n0 = a.H; p.K = a.NQ; break;
    case PH_GU: p.nmat = 2; p.n0 = p.n1 = a.F; p.interleave = true; break;
    case PH_DOWN: p.n0 = a.H; p.K = a.F; break;
    default: p.n0 = a.V; break;
  }
  return p;
}
// rows [lo, hi) of an n-row matrix owned by CTA `cta` of G (n * G < 2^31 is checked on the host)
__device__ __forceinline__ void mg_share(int n, int cta, int G, int& lo, int& hi) {
  lo = (int)((unsigned)n * (unsigned)cta / (unsigned)G);
  hi = (int)((unsigned)n * (unsigned)(cta + 1) / (unsigned)G);
}
template <class T>
__device__ __forceinline__ int mg_rows_per_chunk(int K) {
  int r = MEGA_SLOT_BYTES / (K * (int)sizeof(T));
  return r > MEGA_RMAX ? MEGA_RMAX : (r < 1 ? 1 : r);
}
// Iterator over the chunks of one phase owned by one CTA, in ring order (plain state, no closures: everything
// stays in registers).
template <class T>
struct PhaseChunks {
  int mat = 0, row = 0, hi = 0, R = 1;
  bool up = false;
  __device__ __forceinline__ void begin(const PhaseShape& p, int cta, int G) {
    R = mg_rows_per_chunk<T>(p.K);
    mat = 0;
    up = false;
    mg_share(p.n0, cta, G, row, hi);
  }
  // Next chunk: matrix index, output offset of that matrix, first row, row count.
  __device__ __forceinline__ bool next(const PhaseShape& p, int cta, int G, int& cmat, int& out_off, int& row0, int& rows) {
    if (p.interleave) {
      if (row >= hi) return false;
      rows = hi - row < R ? hi - row : R;
      row0 = row;
      out_off = 0;
      cmat = up ? 1 : 0;
      if (up) row += rows;
      up = !up;
      return true;
    }
    while (mat < p.nmat) {
      if (row < hi) {
        rows = hi - row < R ? hi - row : R;
        row0 = row;
        cmat = mat;
        out_off = mat == 0 ? 0 : (mat == 1 ? p.o1 : p.o2);
        row += rows;
        return true;
      }
      ++mat;
      if (mat < p.nmat) mg_share(mat == 1 ? p.n1 : p.n2, cta, G, row, hi);
    }
    return false;
  }
};

// Cursor over the same chunk sequence, `nslots` chunks ahead of consumption, advanced by thread 0 only.
template <class T>
struct MegaFeed {
  int l = 0, pi = 0;       // layer (L = lm_head) and phase index within the layer
  int mat = 0, row = 0, hi = 0;
  bool started = false, up = false, done = false;
  PhaseShape p;
  const T *b0 = nullptr, *b1 = nullptr, *b2 = nullptr;

  __device__ __forceinline__ void enter_phase(const MegaArgs& a, int cta) {
    const int ph = l < a.L ? pi : PH_HEAD;
    p = mg_phase_shape(a, ph);
    if (ph == PH_HEAD) {
      b0 = (const T*)a.head;
    } else {
      const MegaLayer& w = a.layers[l];
      if (ph == PH_QKV) { b0 = (const T*)w.q; b1 = (const T*)w.k; b2 = (const T*)w.v; }
      else if (ph == PH_O) { b0 = (const T*)w.o; }
      else if (ph == PH_GU) { b0 = (const T*)w.gate; b1 = (const T*)w.up; }
      else { b0 = (const T*)w.down; }
    }
    mat = 0;
    up = false;
    mg_share(p.n0, cta, a.G, row, hi);
    started = true;
  }
  // Next chunk of this CTA: source address and size.  false when the step's weights are exhausted.
  __device__ __forceinline__ bool next(const MegaArgs& a, int cta, const T*& src, uint32_t& bytes) {
    while (!done) {
      if (!started) enter_phase(a, cta);
      const int R = mg_rows_per_chunk<T>(p.K);
      if (p.interleave) {
        if (row < hi) {
          const int rows = hi - row < R ? hi - row : R;
          src = (up ? b1 : b0) + (long long)row * p.K;
          bytes = (uint32_t)(rows * p.K * (int)sizeof(T));
          if (up) row += rows;
          up = !up;
          return true;
        }
      } else {
        while (mat < p.nmat) {
          if (row < hi) {
            const int rows = hi - row < R ? hi - row : R;
            src = (mat == 0 ? b0 : (mat == 1 ? b1 : b2)) + (long long)row * p.K;
            bytes = (uint32_t)(rows * p.K * (int)sizeof(T));
            row += rows;
            return true;
          }
          ++mat;
          if (mat < p.nmat) mg_share(mat == 1 ? p.n1 : p.n2, cta, a.G, row, hi);
        }
      }
      started = false;
      if (l >= a.L) {
        done = true;
      } else if (++pi == 4) {
        pi = 0;
        ++l;
      }
    }
    return false;
  }
};

// ---- deterministic reductions over the 256 consumer threads ---------------------------------------
__device__ __forceinline__ float mg_block_sum(float v, float* scratch) {
  v = warp_sum(v);
  mg_consumer_sync();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  mg_consumer_sync();
  float r = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) r += scratch[w];
  return r;
}
__device__ __forceinline__ float mg_block_max(float v, float* scratch) {
  v = warp_max(v);
  mg_consumer_sync();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  mg_consumer_sync();
  float r = -FLT_MAX;
#pragma unroll
  for (int w = 0; w < 8; ++w) r = fmaxf(r, scratch[w]);
  return r;
}

// Grid-wide barrier.  Thread 0 publishes the CTA's writes with a release add on the monotonic counter and
// acquires the others' by polling it; __syncthreads on both sides extends that to the whole CTA.
// Returns false if it gave up.
__device__ __forceinline__ bool mg_grid_barrier(const MegaArgs& a, unsigned long long& target, int* ok_flag) {
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long old;
    asm volatile("atom.add.release.gpu.global.u64 %0, [%1], %2;" : "=l"(old) : "l"(a.bar_counter), "l"(1ull) : "memory");
    target += (unsigned long long)a.G;
    int ok = 1;
    if (old + 1 < target) {
      const long long t0 = clock64();
      unsigned spins = 0;
      while (true) {
        unsigned long long v;
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(a.bar_counter) : "memory");
        if (v >= target) break;
        if ((++spins & 63u) == 0u) {
          if (mg_aborted(a)) { ok = 0; break; }
          if (clock64() - t0 > MEGA_WAIT_CYCLES) { mg_abort(a); ok = 0; break; }
        }
      }
    } else {
      asm volatile("fence.acq_rel.gpu;" ::: "memory");
    }
    *ok_flag = ok;
  }
  __syncthreads();
  return *(volatile int*)ok_flag != 0;
}

template <class T>
__device__ __forceinline__ VecT<T, 16 / sizeof(T)> mg_ldcg16(const T* p) {
  uint4 u = __ldcg(reinterpret_cast<const uint4*>(p));
  VecT<T, 16 / sizeof(T)> v;
  memcpy(&v, &u, 16);
  return v;
}

// Input vector of a phase into shared memory (as T), all consumer threads, one 16-byte L2 load per element
// group.  norm_gain != nullptr applies RMSNorm (helpers/tensors.rs:82-111) with the rounding points of the graph.
// Needs K / VEC <= 1024 (checked on the host).
template <class T, int MT>
struct RowPtrs {
  const T* p[MT];
};
template <class T, int MT>
__device__ __forceinline__ void mg_load_input(const MegaArgs& a, T* xs, float* scratch, RowPtrs<T, MT> rows, int K,
                                              const T* norm_gain) {
  constexpr int VEC = 16 / sizeof(T);
  const int nvec = K / VEC;
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    VecT<T, VEC> xv[4], gv[4];
    if (m < a.B) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int v = threadIdx.x + j * MEGA_CONSUMERS;
        if (v < nvec) {
          xv[j] = mg_ldcg16<T>(rows.p[m] + v * VEC);
          if (norm_gain) gv[j] = *reinterpret_cast<const VecT<T, VEC>*>(norm_gain + v * VEC);
        }
      }
    }
    if (m < a.B && norm_gain) {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int v = threadIdx.x + j * MEGA_CONSUMERS;
        if (v < nvec) {
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            float f = Elem<T>::load(xv[j].v[i]);
            ss += f * f;
          }
        }
      }
      ss = mg_block_sum(ss, scratch);
      const float rms = sqrtf(ss / (float)K + a.eps);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int v = threadIdx.x + j * MEGA_CONSUMERS;
        if (v < nvec) {
          VecT<T, VEC> o;
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            float nrm = rt<T>(Elem<T>::load(xv[j].v[i]) / rms);
            o.v[i] = Elem<T>::store(nrm * Elem<T>::load(gv[j].v[i]));
          }
          *reinterpret_cast<VecT<T, VEC>*>(xs + m * K + v * VEC) = o;
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int v = threadIdx.x + j * MEGA_CONSUMERS;
        if (v < nvec) {
          VecT<T, VEC> o;
          if (m < a.B) o = xv[j];
          else memset(&o, 0, sizeof(o));
          *reinterpret_cast<VecT<T, VEC>*>(xs + m * K + v * VEC) = o;
        }
      }
    }
  }
  mg_consumer_sync();
}

// Partial dot products of up to 8 weight rows (rows r0 .. r0+7 of the slot) with the MT input rows, one warp.
// Every lane accumulates its 16-byte columns of all 8 rows (independent loads in flight), then a transposing
// butterfly leaves the warp total of row j in the lanes whose bits 4..2 spell j: 9 shuffles instead of 40.
template <class T, int MT>
__device__ __forceinline__ void mg_multiply8(const T* wslot, const T* xs, int r0, int rows, int K, int nvec, int warp,
                                             int lane, float* redb) {
  constexpr int VEC = 16 / sizeof(T);
  float acc[8][MT];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[j][m] = 0.f;
  const int nr = rows - r0 < 8 ? rows - r0 : 8;
  for (int v = threadIdx.x; v < nvec; v += MEGA_CONSUMERS) {
    float xf[MT][VEC];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      VecT<T, VEC> xv = *reinterpret_cast<const VecT<T, VEC>*>(xs + m * K + v * VEC);
#pragma unroll
      for (int i = 0; i < VEC; ++i) xf[m][i] = Elem<T>::load(xv.v[i]);
    }
    VecT<T, VEC> wv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < nr) wv[j] = *reinterpret_cast<const VecT<T, VEC>*>(wslot + (long long)(r0 + j) * K + v * VEC);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < nr) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const float wf = Elem<T>::load(wv[j].v[i]);
#pragma unroll
          for (int m = 0; m < MT; ++m) acc[j][m] = fmaf(xf[m][i], wf, acc[j][m]);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    float b4[4], b2[2];
    const bool h16 = (lane & 16) != 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float send = h16 ? acc[j][m] : acc[j + 4][m];
      const float keep = h16 ? acc[j + 4][m] : acc[j][m];
      b4[j] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
    const bool h8 = (lane & 8) != 0;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const float send = h8 ? b4[j] : b4[j + 2];
      const float keep = h8 ? b4[j + 2] : b4[j];
      b2[j] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    const bool h4 = (lane & 4) != 0;
    float d = (h4 ? b2[1] : b2[0]) + __shfl_xor_sync(0xffffffffu, h4 ? b2[0] : b2[1], 4);
    d += __shfl_xor_sync(0xffffffffu, d, 2);
    d += __shfl_xor_sync(0xffffffffu, d, 1);
    const int j = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
    if ((lane & 3) == 0 && j < nr) redb[(warp * MEGA_RMAX + r0 + j) * MT + m] = d;
  }
}

// Attention for one (head, sequence), 256 consumer threads; same algorithm and rounding points as
// attn_decode_kernel (RoPE + KV append fused).  `sc` needs P + 1 + (256 / (HD/VEC)) * HD floats.
template <class T, int HD>
__device__ __forceinline__ void mg_attention(const MegaArgs& a, int layer, int h, int b, int pos, float* sc, float* scratch, float* q_s,
                             T* k_new, T* v_new) {
  constexpr int VEC = 16 / sizeof(T);
  constexpr int LPK = HD / VEC, KPW = 32 / LPK, half = HD / 2, UN = 4;
  const int rep = a.nh / a.nkv, kvh = h / rep;
  const int total = pos + 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LPK, kslot = lane / LPK;
  const long long NQKV = a.NQ + 2 * a.NKV;
  const T* qrow = (const T*)a.qkv + (long long)b * NQKV;
  T* kc = (T*)a.kc + (long long)layer * a.kv_layer_stride + ((long long)b * a.nkv + kvh) * a.P * HD;
  T* vc = (T*)a.vc + (long long)layer * a.kv_layer_stride + ((long long)b * a.nkv + kvh) * a.P * HD;
  if (threadIdx.x < HD) {
    const bool is_q = threadIdx.x < half;
    const int i = is_q ? threadIdx.x : threadIdx.x - half;
    const T* src = is_q ? qrow + h * HD : qrow + a.NQ + kvh * HD;
    float x1 = Elem<T>::load(__ldcg(src + i)), x2 = Elem<T>::load(__ldcg(src + i + half));
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
    v_new[i] = __ldcg(qrow + a.NQ + a.NKV + kvh * HD + i);
  }
  mg_consumer_sync();
  if (h % rep == 0 && threadIdx.x < HD) {
    kc[(long long)pos * HD + threadIdx.x] = k_new[threadIdx.x];
    vc[(long long)pos * HD + threadIdx.x] = v_new[threadIdx.x];
  }
  float qf[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) qf[i] = q_s[sub * VEC + i];
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
  if (warp == 0) {
    float d = 0.f;
    for (int i = lane; i < HD; i += 32) d = fmaf(q_s[i], Elem<T>::load(k_new[i]), d);
    d = warp_sum(d);
    if (lane == 0) sc[pos] = rt<T>(rt<T>(d) / a.scale);
  }
  mg_consumer_sync();
  float mx = -FLT_MAX;
  for (int t = threadIdx.x; t < total; t += MEGA_CONSUMERS) mx = fmaxf(mx, sc[t]);
  mx = mg_block_max(mx, scratch);
  float sum = 0.f;
  for (int t = threadIdx.x; t < total; t += MEGA_CONSUMERS) {
    float e = expf(sc[t] - mx);
    sc[t] = e;
    sum += e;
  }
  sum = mg_block_sum(sum, scratch);
  for (int t = threadIdx.x; t < total; t += MEGA_CONSUMERS) sc[t] = rt<T>(sc[t] / sum);
  mg_consumer_sync();
  constexpr int NCH = HD / VEC, TG = 256 / NCH;
  float* part = sc + a.P + 1;
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
  if (tg == (pos % TG)) {
    float p = sc[pos];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = fmaf(p, Elem<T>::load(v_new[ch * VEC + i]), acc[i]);
  }
#pragma unroll
  for (int i = 0; i < VEC; ++i) part[tg * HD + ch * VEC + i] = acc[i];
  mg_consumer_sync();
  if (threadIdx.x < HD) {
    float s = 0.f;
    for (int g = 0; g < TG; ++g) s += part[g * HD + threadIdx.x];
    ((T*)a.attn)[(long long)b * a.NQ + h * HD + threadIdx.x] = Elem<T>::store(s);
  }
  mg_consumer_sync();
}

// Shared memory: [nslots x 32 KiB ring][input vectors / attention scratch][small state]
template <class T, int MT, int HD, bool PROF>
__global__ void __launch_bounds__(MEGA_THREADS, 1) llama_decode_mega_kernel(MegaArgs a, int xs_bytes) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* ring = smem_raw;
  T* xs = reinterpret_cast<T*>(smem_raw + (size_t)a.nslots * MEGA_SLOT_BYTES);  // [MT][Kmax] or attention scratch
  unsigned char* tail = smem_raw + (size_t)a.nslots * MEGA_SLOT_BYTES + xs_bytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(tail);          // [nslots] (nslots <= 8)
  float* red = reinterpret_cast<float*>(full + 16);            // [2][8][RMAX][MT]
  float* scratch = red + 2 * 8 * MEGA_RMAX * MT;               // [8]
  float* q_s = scratch + 8;                                    // [HD]
  T* k_new = reinterpret_cast<T*>(q_s + HD);                   // [HD]
  T* v_new = k_new + HD;                                       // [HD]
  int* ok_flag = reinterpret_cast<int*>(v_new + HD);
  unsigned long long* best_s = reinterpret_cast<unsigned long long*>((reinterpret_cast<uintptr_t>(ok_flag + 2) + 7) & ~(uintptr_t)7);  // [RMAX*MT]

  constexpr int VEC = 16 / sizeof(T);
  const int cta = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nslots = a.nslots;

  // Weight feed (thread 0): one chunk into a slot whose previous contents have been consumed.
  MegaFeed<T> feed;
  int issued = 0;
#define MG_ISSUE(slot_)                                                                                              \
  do {                                                                                                               \
    const T* src_;                                                                                                   \
    uint32_t bytes_;                                                                                                 \
    if (feed.next(a, cta, src_, bytes_)) {                                                                           \
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mg_smem_u32(&full[slot_])),       \
                   "r"(bytes_)                                                                                       \
                   : "memory");                                                                                      \
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(  \
                       mg_smem_u32(ring + (size_t)(slot_) * MEGA_SLOT_BYTES)),                                       \
                   "l"(src_), "r"(bytes_), "r"(mg_smem_u32(&full[slot_]))                                            \
                   : "memory");                                                                                      \
      ++issued;                                                                                                      \
    }                                                                                                                \
  } while (0)

  constexpr int FEEDER = 7 * 32;  // the thread that owns the weight feed (not in the warp that leads the barriers)
  if (threadIdx.x == 0) {
    for (int s = 0; s < nslots; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mg_smem_u32(&full[s])), "r"(1));
    *ok_flag = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == FEEDER) {
    for (int s = 0; s < nslots; ++s) MG_ISSUE(s);  // fill the ring before anything else
  }

  const int B = a.B;
  const long long NQKV = a.NQ + 2 * a.NKV;
  unsigned long long bar_target = a.bar_base;
  const int pos = *a.ctx_len;  // position of the new token
  const bool dead = pos >= a.P;  // cache full: walk the ring to the end, write nothing
  if (dead && cta == 0 && threadIdx.x == 0) atomicOr(a.err, DEV_ERR_INDEX_OOB);

  // per-sequence embedding rows: the residual stream of layer 0 (helpers/tensors.rs:255-272)
  RowPtrs<T, MT> emb;
  bool bad_id = false;
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    unsigned id = m < B ? a.ids_cur[m] : 0u;
    if (id >= (unsigned)a.V) {
      bad_id = true;
      id = 0;
    }
    emb.p[m] = (const T*)a.embed + (long long)id * a.H;
  }
  if (bad_id && cta == 0 && threadIdx.x == 0) atomicOr(a.err, DEV_ERR_INDEX_OOB);

  // cycle counters (PROF builds only): barrier, prologue, wait for data, multiply, epilogue, attention
  long long pc0 = 0, pc1 = 0, pc2 = 0, pc3 = 0, pc4 = 0, pc5 = 0, pt = 0, pt_start = 0;
  if (PROF) pt = pt_start = clock64();
#define MG_PROF(slot) do { if (PROF) { long long now_ = clock64(); pc##slot += now_ - pt; pt = now_; } } while (0)
  int n = 0;
  int red_buf = 0;
  float gate_hold = 0.f;
  unsigned long long my_best = 0ull;  // greedy pick: thread (r, m) keeps the best key of its rows
  bool alive = true;

  // The barrier sequence is driven by the phase schedule, identical in every CTA, not by which CTA owns rows.
  for (int l = 0; l <= a.L && alive; ++l) {
    const int n_ph = l < a.L ? 4 : 1;
    for (int pi = 0; pi < n_ph && alive; ++pi) {
      const int ph = l < a.L ? pi : PH_HEAD;
      // ---- what must be complete before this phase: a grid barrier (except before the very first phase) ----
      if (!(l == 0 && ph == PH_QKV)) alive = mg_grid_barrier(a, bar_target, ok_flag);
      if (!alive) break;
      MG_PROF(0);
      if (ph == PH_O) {
        // attention for layer l sits between qkv and o_proj: work items (head, sequence) over the CTAs
        if (!dead) {
          for (int item = cta; item < a.nh * B; item += a.G)
            mg_attention<T, HD>(a, l, item % a.nh, item / a.nh, pos, reinterpret_cast<float*>(xs), scratch, q_s, k_new, v_new);
        }
        MG_PROF(5);
        alive = mg_grid_barrier(a, bar_target, ok_flag);
        if (!alive) break;
        MG_PROF(0);
      }
      // ---- input vector of the phase ----
      const PhaseShape p = mg_phase_shape(a, ph);
      const int K = p.K;
      RowPtrs<T, MT> in;
      const T* gain = nullptr;
      if (ph == PH_QKV || ph == PH_GU || ph == PH_HEAD) {
        const bool from_emb = (l == 0 && ph == PH_QKV);
#pragma unroll
        for (int m = 0; m < MT; ++m) in.p[m] = from_emb ? emb.p[m] : (const T*)a.x + (long long)m * a.H;
        gain = ph == PH_HEAD ? (const T*)a.final_norm
                             : (const T*)(ph == PH_QKV ? a.layers[l].in_norm : a.layers[l].post_norm);
      } else if (ph == PH_O) {
#pragma unroll
        for (int m = 0; m < MT; ++m) in.p[m] = (const T*)a.attn + (long long)m * a.NQ;
      } else {
#pragma unroll
        for (int m = 0; m < MT; ++m) in.p[m] = (const T*)a.h + (long long)m * a.F;
      }
      mg_load_input<T, MT>(a, xs, scratch, in, K, gain);
      const int nvec = K / VEC;
      MG_PROF(1);

      // ---- this CTA's chunks of the phase ----
      PhaseChunks<T> chunks;
      chunks.begin(p, cta, a.G);
      int mat, out_off, row0, rows;
      while (chunks.next(p, cta, a.G, mat, out_off, row0, rows)) {
        const int s = n % nslots;
        if (!mg_wait(&full[s], (uint32_t)((n / nslots) & 1), a)) {
          alive = false;
          break;
        }
        MG_PROF(2);
        const T* wslot = reinterpret_cast<const T*>(ring + (size_t)s * MEGA_SLOT_BYTES);
        float* redb = red + red_buf * 8 * MEGA_RMAX * MT;
        for (int r0 = 0; r0 < rows; r0 += 8) mg_multiply8<T, MT>(wslot, xs, r0, rows, K, nvec, warp, lane, redb);
        __syncthreads();
        MG_PROF(3);
        // every thread has read the slot: refill it with the chunk nslots positions ahead
        if (threadIdx.x == FEEDER) MG_ISSUE(s);
        MG_PROF(4);
        // epilogue item e = r * MT + m runs on lane e / 8 of warp e % 8: the row results are spread over the warps
        const int e_item = lane * 8 + warp;
        if (lane < 8 && e_item < rows * MT && !dead) {
          const int r = e_item / MT, m = e_item % MT;
          float sres = 0.f;
#pragma unroll
          for (int w = 0; w < 8; ++w) sres += redb[(w * MEGA_RMAX + r) * MT + m];
          const int nidx = out_off + row0 + r;
          if (m < B) {
            if (ph == PH_QKV) {
              ((T*)a.qkv)[(long long)m * NQKV + nidx] = Elem<T>::store(sres);
            } else if (ph == PH_O || ph == PH_DOWN) {
              T* xr = (T*)a.x + (long long)m * a.H;
              const T* base = (T*)a.x;
              long long off = (long long)m * a.H + nidx;
              if (l == 0 && ph == PH_O) {
                // the residual of the first layer is the embedding row itself
                base = (const T*)a.embed;
                unsigned id = a.ids_cur[m];
                off = (long long)(id < (unsigned)a.V ? id : 0u) * a.H + nidx;
              }
              xr[nidx] = Elem<T>::store(Elem<T>::load(__ldcg(base + off)) + rt<T>(sres));
            } else if (ph == PH_GU) {
              if (mat == 0) {
                gate_hold = sres;
              } else {
                float g = rt<T>(gate_hold), u = rt<T>(sres);
                float sg = 1.f / (1.f + expf(-g));
                float si = rt<T>(g * sg);
                ((T*)a.h)[(long long)m * a.F + nidx] = Elem<T>::store(si * u);
              }
            } else {
              T lv = Elem<T>::store(sres);
              ((T*)a.logits)[(long long)m * a.V + nidx] = lv;
              unsigned hiw = (unsigned)total_key(Elem<T>::load(lv)) ^ 0x80000000u;
              unsigned long long key = ((unsigned long long)hiw << 32) | (unsigned)nidx;
              my_best = key > my_best ? key : my_best;
            }
          }
        }
        red_buf ^= 1;
        ++n;
        MG_PROF(1);
      }
    }
  }

  // ---- greedy pick (llama.rs:225): per-CTA keys, grid barrier, CTA 0 finishes and advances the step ----
  if (alive) {
    if (lane < 8) best_s[lane * 8 + warp] = my_best;  // indexed by epilogue item e = r * MT + m
    __syncthreads();
    if (threadIdx.x < MT) {
      unsigned long long b = 0ull;
      for (int e = threadIdx.x; e < MEGA_RMAX * MT; e += MT) {
        unsigned long long k = best_s[e];
        b = k > b ? k : b;
      }
      if (threadIdx.x < B) a.partials[(long long)cta * MT + threadIdx.x] = b;
    }
    alive = mg_grid_barrier(a, bar_target, ok_flag);
  }
  if (!alive && threadIdx.x == FEEDER) {
    // bounded drain of copies still in flight, so none lands after the CTA has left
    for (int k = n; k < issued; ++k) {
      const long long t0 = clock64();
      while (!mg_try_wait(&full[k % nslots], (uint32_t)((k / nslots) & 1)) && clock64() - t0 < MEGA_WAIT_CYCLES) {
      }
    }
  }
  if (PROF && a.prof && threadIdx.x == 0) {
    MG_PROF(0);
    unsigned long long* pr = a.prof + (long long)cta * 8;
    pr[0] += (unsigned long long)pc0; pr[1] += (unsigned long long)pc1; pr[2] += (unsigned long long)pc2;
    pr[3] += (unsigned long long)pc3; pr[4] += (unsigned long long)pc4; pr[5] += (unsigned long long)pc5;
    pr[6] += (unsigned long long)(clock64() - pt_start);
    pr[7] += 1ull;
  }
#undef MG_PROF
#undef MG_ISSUE
  if (alive && cta == 0 && !dead) {
    const int step = *a.step_no;
    if (warp < B) {
      unsigned long long b = 0ull;
      for (int c = lane; c < a.G; c += 32) {
        unsigned long long k = __ldcg(a.partials + (long long)c * MT + warp);
        b = k > b ? k : b;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
        b = other > b ? other : b;
      }
      if (lane == 0) {
        unsigned id = (unsigned)(b & 0xffffffffull);
        a.ids_cur[warp] = id;
        if (step < a.out_cap_steps) a.out_ids[(long long)step * B + warp] = id;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      *a.ctx_len = pos + 1;
      *a.step_no = step + 1;
    }
  }
}

}  // namespace cgk

// The fused Llama runner behind cg_llama_* (include/catgrad_b200.h).
//
// It executes the Llama term (llama_term.cc, i.e. catgrad-llm-models/src/models/llama.rs:144-385) as a fixed
// plan instead of ~140 interpreter edges per layer:
//   * the plan is built once per model (the reference re-lowers and re-schedules the term on every token,
//     interpreter.rs:33-36 + ssa/mod.rs:24-76);
//   * every `linear` reads W[out,in] in place (no transpose/broadcast copy, nn/mod.rs:182-204);
//   * the KV cache lives on the device with spare capacity and is appended in place; the functional
//     slice/concat/re-stack of helpers/cache.rs:13-75 never runs; repeat_kv is an index computation;
//   * RoPE tables and all literals are computed once at creation (cache.rs:86-103 rebuilds them per step);
//   * the context length is a device-side scalar, so one captured CUDA graph replays for every decode step;
//   * greedy ids stay on the device between steps (the reference reads them back per token, main.rs:1031-1037).
// Observable behaviour kept: ids of the last position per sequence; K/V contents; rounding points (see
// llama_kernels.cuh).  The lm_head runs on the last position of each sequence only: the reference computes it
// for all S positions (llama.rs:217-225) and its runner reads only the last element.
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>

#include "../kernels/elementwise.h"
#include "../kernels/gemm_tcgen05.h"
#include "../kernels/llama_kernels.cuh"
#include "../kernels/attn_prefill_fused.cuh"
#include "../kernels/llama_persist.cuh"
#include "../kernels/matmul.h"
#include "c_api_internal.h"
#include "cuda_backend.h"
#include "tp_comm.h"

using namespace cg;

namespace {

struct LayerW {
  const void *in_norm, *q, *k, *v, *o, *post_norm, *gate, *up, *down;
  // stacked copies for the GEMM path (made on its first use): [q; k; v] and [gate; up], so that the three / two
  // projections of the same input are one product
  const void *qkv = nullptr, *gate_up = nullptr;
};

// Row interleave of the stacked [gate; up] weight: 32 gate rows, then the 32 up rows of the same features, so that a
// 64-column block of the product holds both halves of 32 outputs and SiLU(gate) * up can ride in the GEMM epilogue.
constexpr int64_t GU_BLOCK = 32;

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace

struct cg_llama {
  CudaBackend* be = nullptr;
  cg_ctx* ctx = nullptr;
  LlamaConfig cfg;            // heads and FFN width are this rank's share under tensor parallelism
  int64_t hd = 0;             // head dimension (of the unsharded model)
  // tensor parallelism: q/k/v/gate/up hold this rank's rows, o/down this rank's columns; the partial products
  // of o/down are summed over the ranks through `comm`, whose data area holds x and the partial buffer
  cg_comm* comm = nullptr;
  int64_t comm_tokens = 0;
  size_t comm_part_off = 0;
  Dtype dt = Dtype::BF16;
  size_t es = 2;
  int64_t max_batch = 0, P = 0;
  std::vector<Tensor> keep;  // parameter tensors kept alive
  std::vector<Tensor> stacked;  // [q; k; v] and [gate; up] per layer (GEMM path only)
  bool gu_interleaved = false;  // [gate; up] rows alternate in blocks of GU_BLOCK (FFN width a multiple of it)
  std::vector<LayerW> layers;
  const void *embed = nullptr, *final_norm = nullptr, *head = nullptr;

  // persistent device state
  Tensor kc, vc;              // [L, Bmax, nkv, P, hd]
  Tensor cos_t, sin_t;        // [P, hd/2] f32
  Tensor words;               // int32: [0] ctx_len, [1] step_no
  Tensor ids_in, ids_cur, ids_new, ids_out;  // u32: prompt ids [M], current [B], argmax result [B], record [steps*B]
  Tensor logits;              // [Bmax, V]
  Tensor partials;            // u64 [Bmax, ceil(V/4096)]: stage-1 keys of the greedy pick (scratch)
  int argmax_chunks = 0;
  // persistent one-kernel decode step (batch <= 4)
  Tensor mega_layers, mega_partials, mega_prof, mega_att;
  bool mega_enabled = false;
  bool mega_possible = false;   // cooperative launch available and no tensor parallelism
  bool mega_last_step = false;  // the most recent decode step ran as the persistent kernel
  unsigned long long bar_base = 0;
  int mega_grid = 0;
  bool use_pdl = true;        // programmatic dependent launch between the kernels of a step
  bool l2_prefetch = false;   // decode kernels pull the weights of later launches into L2 (opt-in)
  int64_t out_cap_steps = 0;
  // activation buffers sized for `cap_tokens` tokens
  int64_t cap_tokens = 0;
  Tensor x, xn, qkv, attn, h, g, u, tmp, scores, attn_bhsd;
  Tensor attn_scores, attn_partial, attn_counters;  // scratch of the key-split decode attention
  int64_t batch = 0;
  int64_t host_ctx_len = 0;   // mirror of words[0] (all steps are issued by this object)
  uint64_t launches = 0;

  cudaGraphExec_t graph = nullptr;
  int64_t graph_batch = -1;
  int graph_ctx_bucket = -1;   // 0: captured at a context <= 512, 1: above (the attention variant is chosen by that)
  uint64_t graph_nodes = 0;

  ~cg_llama() {
    if (graph) cudaGraphExecDestroy(graph);
  }
};

namespace {

template <class T>
struct Plan {
  cg_llama& m;
  cudaStream_t st;
  int sm;
  explicit Plan(cg_llama& mm) : m(mm), st(mm.be->stream()), sm(mm.be->sm_count()) {}

  void launched(const char* what) {
    ++m.launches;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) throw Error(ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
  }

  static int mt_for(int64_t M) { return M <= 1 ? 1 : M <= 2 ? 2 : M <= 4 ? 4 : M <= 8 ? 8 : 16; }
  static bool gemv_ok(int64_t M, int64_t K) {
    return M <= 16 && (size_t)mt_for(M) * K * sizeof(T) <= 160 * 1024 && K % (16 / sizeof(T)) == 0;
  }

  // Launch with the programmatic-stream-serialization attribute: the kernel may be scheduled while its
  // predecessor drains and blocks in griddepcontrol.wait until that one has completed.
  template <class... KArgs, class... Args>
  void launch(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = m.use_pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
    if (e != cudaSuccess) throw Error(ERR_CUDA, std::string("cudaLaunchKernelEx: ") + cudaGetErrorString(e));
  }

  // K split so that even the smallest projection puts >= 16 warps on every SM
  int ks_for(int n_pairs, int K) const {
    int nvec = K / (int)(16 / sizeof(T));
    int ks = 1;
    while (ks < 8 && (long long)n_pairs * ks < (long long)sm * 16 && nvec / (ks * 2) >= 64) ks *= 2;  // 16 warps per SM
    return ks;
  }

  template <int MT, int PRO, int EPI>
  void gemv_launch(cgk::GemvArgs a) {
    size_t smem = (size_t)MT * a.K * sizeof(T);
    auto kern = cgk::gemv_fused_kernel<T, MT, PRO, EPI>;
    static size_t smem_set_dev[64] = {0};  // per instantiation and device: raise the dynamic shared-memory limit once per size class
    size_t& smem_set = smem_set_dev[m.be->device() & 63];
    if (smem > 40 * 1024 && smem > smem_set) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      smem_set = smem;
    }
    int pairs = EPI == cgk::EPI_SILU_MUL ? a.N : (a.N + 1) / 2;
    a.ks = ks_for(pairs, a.K);
    int ppc = 8 / a.ks;
    int ctas_per_sm = smem > 100 * 1024 ? 1 : 2;  // 128 registers x 256 threads: two CTAs per SM
    int grid = std::min((pairs + ppc - 1) / ppc, sm * ctas_per_sm);
    launch(kern, dim3(grid), dim3(256), smem, a);
    launched("gemv");
  }
  template <int PRO, int EPI>
  void gemv_mt(const cgk::GemvArgs& a) {
    switch (mt_for(a.M)) {
      case 1: gemv_launch<1, PRO, EPI>(a); break;
      case 2: gemv_launch<2, PRO, EPI>(a); break;
      case 4: gemv_launch<4, PRO, EPI>(a); break;
      case 8: gemv_launch<8, PRO, EPI>(a); break;
      default: gemv_launch<16, PRO, EPI>(a); break;
    }
  }
  void gemv(int pro, int epi, const cgk::GemvArgs& a) {
    if (pro == cgk::PRO_NORM) {
      if (epi == cgk::EPI_STORE) gemv_mt<cgk::PRO_NORM, cgk::EPI_STORE>(a);
      else if (epi == cgk::EPI_SILU_MUL) gemv_mt<cgk::PRO_NORM, cgk::EPI_SILU_MUL>(a);
      else gemv_mt<cgk::PRO_NORM, cgk::EPI_RESIDUAL>(a);
    } else {
      if (epi == cgk::EPI_STORE) gemv_mt<cgk::PRO_NONE, cgk::EPI_STORE>(a);
      else if (epi == cgk::EPI_SILU_MUL) gemv_mt<cgk::PRO_NONE, cgk::EPI_SILU_MUL>(a);
      else gemv_mt<cgk::PRO_NONE, cgk::EPI_RESIDUAL>(a);
    }
  }

  // out[M,N] (row pitch ldo... contiguous) = xin[M,K] (row pitch ldx) @ W[N,K]^T
  // The early weight fetch under programmatic dependent launch is used from 256 rows up: measured +1..4 % there
  // (batch-256 decode, prefill) but -18 % on a batch-32 decode step, whose cluster launches it delays.
  // With `res`: res[M,N] += T(xin @ W^T) (the residual add of a block), through `scratch` when the add cannot ride
  // in the GEMM epilogue.
  // `silu_pairs`: W is the block-interleaved [gate; up] weight and out is [M, N / 2] (see launch_tcgen05_gemm);
  // returns false, with nothing launched, when the tensor-core kernel cannot take that product.
  bool gemm(const void* xin, int64_t ldx, const void* W, void* out, int64_t M, int64_t N, int64_t K, void* res = nullptr,
            bool silu_pairs = false) {
    cgk::View4 bt;
    std::memset(&bt, 0, sizeof(bt));
    bt.rank = 0;
    bt.total = 1;
    if (std::is_same<T, __nv_bfloat16>::value && cgk::tcgen05_gemm_applicable(bt, 1, xin, W, M, N, K, ldx, 1, 1, K) &&
        cgk::launch_tcgen05_gemm(bt, 1, xin, W, res ? res : out, M, N, K, ldx, K, m.be->dev_err(), sm, st, false, res,
                                 /*static_b=*/m.use_pdl && M >= 256, silu_pairs)) {
      launched("gemm(tcgen05)");
      return true;
    }
    if (silu_pairs) return false;
    cgk::launch_matmul((int)m.dt, bt, 1, xin, W, out, M, N, K, ldx, 1, 1, K, sm, st);
    launched("gemm");
    if (res) add_inplace(res, out, M * N);
    return true;
  }

  int grid_for(long long items) {
    long long blocks = (items + 255) / 256, cap = (long long)sm * 8;
    return (int)std::max<long long>(1, std::min(blocks, cap));
  }

  template <int NV>
  void rmsnorm_rows(const void* in, const void* gain, void* out, int64_t rows, int64_t row_mul, int64_t row_off) {
    launch(cgk::rmsnorm_rows_kernel<T, NV>, dim3((unsigned)((rows + 7) / 8)), dim3(256), 0, (const T*)in, (const T*)gain, (T*)out,
           (long long)rows, m.cfg.rms_norm_eps, (long long)row_mul, (long long)row_off);
  }
  void rmsnorm(const void* in, const void* gain, void* out, int64_t rows, int64_t H, int64_t row_mul, int64_t row_off) {
    // warp per row with the row in registers when the row is 1, 2, 4, 8 or 16 sixteen-byte vectors per lane and
    // everything is 16-byte aligned (activations and gains come from the allocator); one CTA per row otherwise
    const int64_t per_lane = 32 * (16 / (int64_t)sizeof(T));
    const bool aligned = (((uintptr_t)in | (uintptr_t)gain | (uintptr_t)out) & 15) == 0;
    const int64_t nv = H % per_lane == 0 ? H / per_lane : 0;
    // (a few hundred rows are too few warps for that shape: measured 7.7 us against 6.5 us at 256 rows of 2048)
    if (aligned && rows >= 1024 && (nv == 1 || nv == 2 || nv == 4 || nv == 8 || nv == 16)) {
      switch (nv) {
        case 1: rmsnorm_rows<1>(in, gain, out, rows, row_mul, row_off); break;
        case 2: rmsnorm_rows<2>(in, gain, out, rows, row_mul, row_off); break;
        case 4: rmsnorm_rows<4>(in, gain, out, rows, row_mul, row_off); break;
        case 8: rmsnorm_rows<8>(in, gain, out, rows, row_mul, row_off); break;
        default: rmsnorm_rows<16>(in, gain, out, rows, row_mul, row_off); break;
      }
    } else if (aligned && H % (16 / (int64_t)sizeof(T)) == 0 && H / (16 / (int64_t)sizeof(T)) <= 1024) {
      // one CTA per row, the row in registers, 16-byte accesses
      launch(cgk::rmsnorm_vec_kernel<T>, dim3((unsigned)rows), dim3(256), 0, (const T*)in, (const T*)gain, (T*)out, (int)H,
             m.cfg.rms_norm_eps, (long long)row_mul, (long long)row_off);
    } else {
      launch(cgk::rmsnorm_kernel<T>, dim3((unsigned)rows), dim3(256), 0, (const T*)in, (const T*)gain, (T*)out, (int)H,
             m.cfg.rms_norm_eps, (long long)row_mul, (long long)row_off);
    }
    launched("rmsnorm");
  }
  void add_inplace(void* xx, const void* y, int64_t n) {
    cgk::add_inplace_kernel<T><<<grid_for(n / (16 / sizeof(T))), 256, 0, st>>>((T*)xx, (const T*)y, n);
    launched("add");
  }

  // Decode attention with one warp per (kv head, sequence): taken when that alone gives every SM a warp or
  // more, for bf16, GQA groups of 1/2/4/8 and contexts up to 512 (a captured graph keeps the choice of its first step).
  // two warps per (kv head, sequence), two pairs per CTA
  template <int HD, int REP>
  void pair_attention_launch(const cgk::AttnArgs& a, int64_t B, int64_t nkv, unsigned* err) {
    const size_t per_pair = ((size_t)2 * HD * sizeof(T) + (size_t)(2 * REP * HD + 4 * REP + REP * (m.P + 1)) * 4 + 15) / 16 * 16;
    const size_t smem = 2 * per_pair;
    auto kern = cgk::attn_decode_pair_kernel<__nv_bfloat16, HD, REP>;
    static size_t smem_set_dev[64] = {0};
    size_t& smem_set = smem_set_dev[m.be->device() & 63];
    if (smem > 40 * 1024 && smem > smem_set) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      smem_set = smem;
    }
    launch(kern, dim3((unsigned)((nkv + 1) / 2), (unsigned)B), dim3(128), smem, a, err);
  }
  template <int HD, int REP>
  void group_attention_launch(const cgk::AttnArgs& a, int64_t B, int64_t nkv, unsigned* err) {
    // measured (8 kv heads): two warps per pair +8 % tokens/s at batch 32, -4 % at batch 256, where one warp per
    // pair already fills every SM
    if (B * nkv <= 8 * (int64_t)sm) {
      pair_attention_launch<HD, REP>(a, B, nkv, err);
      return;
    }
    size_t per_warp = (size_t)2 * HD * sizeof(T) + (size_t)REP * HD * 4 + (size_t)REP * (m.P + 1) * 4;
    per_warp = (per_warp + 15) / 16 * 16;
    size_t smem = 4 * per_warp;
    auto kern = cgk::attn_decode_group_kernel<__nv_bfloat16, HD, REP>;
    static size_t smem_set_dev[64] = {0};
            size_t& smem_set = smem_set_dev[m.be->device() & 63];
    if (smem > 40 * 1024 && smem > smem_set) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      smem_set = smem;
    }
    launch(kern, dim3((unsigned)((nkv + 3) / 4), (unsigned)B), dim3(128), smem, a, err);
  }
  bool launch_group_attention(const cgk::AttnArgs& a, int64_t B, int64_t nkv, int64_t rep, int64_t hd, unsigned* err) {
    if (!std::is_same<T, __nv_bfloat16>::value) return false;
    // measured at batch 32 and 64 (8 kv heads): 10 % and 21 % more tokens/s than one warp per query head
    if (B * nkv < (int64_t)sm || m.host_ctx_len > 512) return false;
    const size_t per_warp = (size_t)2 * hd * 2 + (size_t)rep * hd * 4 + (size_t)rep * (m.P + 1) * 4 + 16;
    if (4 * per_warp > 200 * 1024) return false;
    if (hd == 64) {
      switch (rep) {
        case 1: group_attention_launch<64, 1>(a, B, nkv, err); return true;
        case 2: group_attention_launch<64, 2>(a, B, nkv, err); return true;
        case 4: group_attention_launch<64, 4>(a, B, nkv, err); return true;
        case 8: group_attention_launch<64, 8>(a, B, nkv, err); return true;
        default: return false;
      }
    }
    if (hd == 128) {
      switch (rep) {
        case 1: group_attention_launch<128, 1>(a, B, nkv, err); return true;
        case 2: group_attention_launch<128, 2>(a, B, nkv, err); return true;
        case 4: group_attention_launch<128, 4>(a, B, nkv, err); return true;
        default: return false;
      }
    }
    return false;
  }

  // Decode attention with the keys split over CTAs (bf16, contexts above 512, GQA groups of 1/2/4/8).
  template <int HD, int REP>
  void split_attention_launch(const cgk::AttnSplitArgs& s, int64_t B, int64_t nkv, unsigned* err) {
    dim3 grid((unsigned)s.chunks_max, (unsigned)nkv, (unsigned)B);
    launch(cgk::attn_split_scores_kernel<__nv_bfloat16, HD, REP>, grid, dim3(128), 0, s, err);
    ++m.launches;
    launch(cgk::attn_split_pv_kernel<__nv_bfloat16, HD, REP>, grid, dim3(128), 0, s, err);
  }
  bool launch_split_attention(const cgk::AttnArgs& a, int64_t B, int64_t nkv, int64_t rep, int64_t hd, unsigned* err) {
    if (!std::is_same<T, __nv_bfloat16>::value) return false;
    // a single sequence is faster through the one-launch kernel (measured: 1.00 vs 1.12 ms per step at batch 1)
    if (m.host_ctx_len <= 512 || B > 65535 || B * nkv < 32) return false;
    const int64_t nh = nkv * rep;
    const int chunks_max = (int)((m.P + cgk::ATTN_CHUNK - 1) / cgk::ATTN_CHUNK);
    // the scratch is made by ensure_capacity: nothing may allocate here, this runs inside graph captures
    if (!m.attn_scores.defined() || !m.attn_partial.defined() || !m.attn_counters.defined()) return false;
    (void)nh;
    cgk::AttnSplitArgs s;
    s.a = a;
    s.scores = (float*)m.attn_scores.raw();
    s.partial = (float*)m.attn_partial.raw();
    s.counters = (unsigned*)m.attn_counters.raw();
    s.chunks_max = chunks_max;
    if (hd == 64) {
      switch (rep) {
        case 1: split_attention_launch<64, 1>(s, B, nkv, err); return true;
        case 2: split_attention_launch<64, 2>(s, B, nkv, err); return true;
        case 4: split_attention_launch<64, 4>(s, B, nkv, err); return true;
        case 8: split_attention_launch<64, 8>(s, B, nkv, err); return true;
        default: return false;
      }
    }
    if (hd == 128) {
      switch (rep) {
        case 1: split_attention_launch<128, 1>(s, B, nkv, err); return true;
        case 2: split_attention_launch<128, 2>(s, B, nkv, err); return true;
        case 4: split_attention_launch<128, 4>(s, B, nkv, err); return true;
        default: return false;
      }
    }
    return false;
  }

  // x += sum over the tensor-parallel ranks of the partial product in `tmp` (both live in the symmetric buffer)
  void reduce_partials(int64_t n) {
    m.comm->allreduce(m.dt, 0, m.comm_part_off, n, /*residual=*/true, sm, st, m.be->dev_err());
    ++m.launches;
  }

  // ---- the one-kernel decode step (llama_persist.cuh) ----
  struct MegaGeom { bool ok = false; int nslots = 0; int xs_bytes = 0; int xs_pitch = 0; size_t smem = 0; };
  MegaGeom mega_geom(int64_t B) const {
    MegaGeom g;
    const LlamaConfig& c = m.cfg;
    if (!m.mega_enabled || !std::is_same<T, __nv_bfloat16>::value || B > cgk::PK_MAX_B) return g;
    const int64_t hd = m.hd, H = c.hidden_size, F = c.intermediate_size, NQ = c.num_attention_heads * hd,
                  NKV = c.num_key_value_heads * hd, V = c.vocab_size, rep = c.num_attention_heads / c.num_key_value_heads;
    if (!(rep == 1 || rep == 2 || rep == 4)) return g;
    // whole 16-row tiles (8 + 8 for gate/up), whole 16-column K-steps, the norm loader holds 4 x 256 16-byte groups
    if (NQ % 16 || NKV % 16 || H % 16 || V % 16 || F % 16 || H / 4 > 8 * cgk::PK_COMPUTE_THREADS) return g;
    if (m.P > 16384) return g;   // attention chunk partials are combined by every CTA: keep that list short
    const int64_t kmax = std::max<int64_t>(std::max<int64_t>(H, F), NQ);
    const int64_t pitch = kmax * 2 + cgk::PK_XS_PAD;
    int64_t xs = std::max<int64_t>(B * pitch, cgk::pk_att_smem_bytes((int)hd, (int)rep));
    xs = (xs + 127) / 128 * 128;
    const int64_t budget = 227 * 1024;
    int64_t nslots = (budget - xs - cgk::pk_tail_bytes()) / cgk::PK_SLOT_BYTES;
    if (nslots > cgk::PK_MAX_SLOTS) nslots = cgk::PK_MAX_SLOTS;
    if (nslots < 3) return g;
    g.ok = true;
    g.nslots = (int)nslots;
    g.xs_bytes = (int)xs;
    g.xs_pitch = (int)pitch;
    g.smem = (size_t)(nslots * cgk::PK_SLOT_BYTES + xs + cgk::pk_tail_bytes());
    return g;
  }
  template <int HD, int REP>
  bool mega_launch_t(const cgk::PkArgs& a, const MegaGeom& g) {
    auto kern = m.mega_prof.defined() ? cgk::llama_decode_persistent_kernel<HD, REP, true> : cgk::llama_decode_persistent_kernel<HD, REP, false>;
    static size_t smem_set_dev[64][2] = {};
    size_t& smem_set_ref = smem_set_dev[m.be->device() & 63][m.mega_prof.defined() ? 1 : 0];
    if (g.smem > smem_set_ref) {
      cudaError_t e0 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem);
      int per_sm = 0;
      cudaError_t e1 = e0 == cudaSuccess ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, cgk::PK_THREADS, g.smem) : e0;
      if (e1 != cudaSuccess || per_sm < 1) {
        cudaGetLastError();
        std::fprintf(stderr, "[catgrad_b200] persistent decode kernel unavailable (shared memory %zu, occupancy %d: %s); using the kernel-per-sub-graph plan\n",
                     g.smem, per_sm, cudaGetErrorString(e1));
        m.mega_enabled = false;
        return false;
      }
      smem_set_ref = g.smem;
    }
    cgk::PkArgs args = a;
    int xs_bytes = g.xs_bytes;
    void* params[] = {(void*)&args, (void*)&xs_bytes};
    cudaError_t e = cudaLaunchCooperativeKernel((const void*)kern, dim3(a.G), dim3(cgk::PK_THREADS), params, g.smem, st);
    if (e != cudaSuccess) throw Error(ERR_CUDA, std::string("cooperative launch of the decode kernel: ") + cudaGetErrorString(e));
    return true;
  }
  // Runs `nsteps` (<= PK_MAX_STEPS) decode steps as one launch of the persistent kernel, starting from the ids in
  // ids_cur.  Returns false if this shape cannot use it.
  bool mega_steps(int64_t B, int nsteps) {
    MegaGeom g = mega_geom(B);
    if (!g.ok) return false;
    const LlamaConfig& c = m.cfg;
    const int64_t rep = c.num_attention_heads / c.num_key_value_heads;
    const int64_t NQ = c.num_attention_heads * m.hd, NKV = c.num_key_value_heads * m.hd;
    const int att_chunks = (int)((m.P + cgk::PK_ATT_CHUNK - 1) / cgk::PK_ATT_CHUNK);
    if (!m.mega_att.defined())
      m.mega_att = m.be->empty({std::min<int64_t>(m.max_batch, cgk::PK_MAX_B) * c.num_key_value_heads * att_chunks *
                                cgk::pk_att_item_floats((int)m.hd, (int)rep)},
                               Dtype::F32);
    cgk::PkArgs a{};
    a.L = (int)c.num_hidden_layers; a.H = (int)c.hidden_size; a.F = (int)c.intermediate_size;
    a.NQ = (int)NQ; a.NKV = (int)NKV;
    a.V = (int)c.vocab_size; a.nh = (int)c.num_attention_heads; a.nkv = (int)c.num_key_value_heads;
    a.P = (int)m.P; a.B = (int)B; a.G = m.mega_grid; a.nslots = g.nslots; a.xs_pitch = g.xs_pitch;
    a.nsteps = nsteps;
    a.eps = c.rms_norm_eps; a.scale = cgk_host_round((float)std::sqrt((float)m.hd));
    a.embed = m.embed; a.final_norm = m.final_norm; a.head = m.head;
    a.layers = (const cgk::PkLayer*)m.mega_layers.raw();
    a.x = m.x.raw(); a.qkv = m.qkv.raw(); a.h = m.h.raw(); a.logits = m.logits.raw();
    a.att = (float*)m.mega_att.raw(); a.att_chunks = att_chunks;
    a.kc = m.kc.raw(); a.vc = m.vc.raw();
    a.kv_layer_stride = m.max_batch * c.num_key_value_heads * m.P * m.hd;
    a.kv_seq_stride = m.P * m.hd;
    a.cos_t = (const float*)m.cos_t.raw(); a.sin_t = (const float*)m.sin_t.raw();
    a.ids_cur = (unsigned*)m.ids_cur.raw(); a.out_ids = (unsigned*)m.ids_out.raw();
    a.ctx_len = (int*)m.words.raw(); a.step_no = (int*)m.words.raw() + 1; a.out_cap_steps = (int)m.out_cap_steps;
    a.partials = (unsigned long long*)m.mega_partials.raw();
    a.bar_counter = (unsigned long long*)((unsigned*)m.words.raw() + 4);
    a.bar_base = m.bar_base;
    a.err = m.be->dev_err(); a.abort_word = (unsigned*)m.words.raw() + 2;
    a.prof = m.mega_prof.defined() ? (unsigned long long*)m.mega_prof.raw() : nullptr;
    bool ok = false;
    if (m.hd == 64) ok = rep == 1 ? mega_launch_t<64, 1>(a, g) : rep == 2 ? mega_launch_t<64, 2>(a, g) : mega_launch_t<64, 4>(a, g);
    else ok = rep == 1 ? mega_launch_t<128, 1>(a, g) : rep == 2 ? mega_launch_t<128, 2>(a, g) : mega_launch_t<128, 4>(a, g);
    if (!ok) return false;
    m.bar_base += (unsigned long long)nsteps * (unsigned long long)cgk::pk_barriers_per_step((int)c.num_hidden_layers) * (unsigned long long)a.G;
    ++m.launches;
    return true;
  }

  // One evaluation of the term on M = B*S tokens whose ids are in `ids` (device).
  void step(const unsigned* ids, int64_t B, int64_t S) {
    const LlamaConfig& c = m.cfg;
    const int64_t H = c.hidden_size, F = c.intermediate_size, nh = c.num_attention_heads, nkv = c.num_key_value_heads,
                  hd = m.hd, V = c.vocab_size, L = c.num_hidden_layers;
    const int64_t M = B * S, NQ = nh * hd, NKV = nkv * hd, NQKV = NQ + 2 * NKV;
    int* ctx_len = (int*)m.words.raw();
    unsigned* err = m.be->dev_err();
    T* x = (T*)m.x.raw();

    launch(cgk::embed_kernel<T>, dim3(grid_for(M * (H / (16 / sizeof(T))))), dim3(256), 0, ids, (const T*)m.embed, x,
           (int)M, (int)H, (int)V, err);
    launched("embed");

    const float scale = cgk_host_round((float)std::sqrt((float)hd));
    const bool pf_on = m.l2_prefetch && S == 1 && gemv_ok(M, H);
    const long long es = (long long)sizeof(T);
    auto region = [&](cgk::PrefetchArgs& pf, int i, const void* p, long long elems) {
      if (pf_on && p) { pf.ptr[i] = p; pf.bytes[i] = elems * es; }
    };
    for (int64_t l = 0; l < L; ++l) {
      const LayerW& w = m.layers[l];
      // ---- attention block ----
      T* qkv = (T*)m.qkv.raw();
      if (gemv_ok(M, H)) {
        cgk::GemvArgs a{};
        a.w[0] = w.q; a.w[1] = w.k; a.w[2] = w.v;
        a.n_end[0] = (int)NQ; a.n_end[1] = (int)(NQ + NKV); a.n_end[2] = (int)NQKV;
        a.x = x; a.x_row_stride = H; a.gain = w.in_norm; a.eps = c.rms_norm_eps;
        a.out = qkv; a.M = (int)M; a.N = (int)NQKV; a.K = (int)H;
        region(a.pf, 0, w.o, H * NQ); region(a.pf, 1, w.gate, F * H); region(a.pf, 2, w.up, F * H);
        gemv(cgk::PRO_NORM, cgk::EPI_STORE, a);
      } else {
        rmsnorm(x, w.in_norm, m.xn.raw(), M, H, 1, 0);
        gemm(m.xn.raw(), H, w.qkv, qkv, M, NQKV, H);   // one product over the stacked [q; k; v]
      }
      // rows hold q | k | v side by side (pitch NQKV) on both paths
      T* q = qkv;
      T* k = qkv + NQ;
      T* v = qkv + NQ + NKV;
      const int64_t qs = NQKV, ks = NQKV;
      T* kcl = (T*)m.kc.raw() + l * m.max_batch * nkv * m.P * hd;
      T* vcl = (T*)m.vc.raw() + l * m.max_batch * nkv * m.P * hd;
      T* attn = (T*)m.attn.raw();
      if (S == 1) {
        cgk::AttnArgs a{};
        a.q = q; a.q_row_stride = qs; a.k = k; a.k_row_stride = ks; a.v = v; a.v_row_stride = ks;
        a.kc = kcl; a.vc = vcl; a.out = attn; a.out_row_stride = NQ;
        a.cos_t = (const float*)m.cos_t.raw(); a.sin_t = (const float*)m.sin_t.raw();
        a.ctx_len = ctx_len; a.nh = (int)nh; a.nkv = (int)nkv; a.P = (int)m.P; a.scale = scale;
        constexpr int VEC = 16 / sizeof(T);
        const int64_t rep = nh / nkv;
        if (launch_group_attention(a, B, nkv, rep, hd, err)) {
          // one warp per (kv head, sequence)
        } else if (launch_split_attention(a, B, nkv, rep, hd, err)) {
          // long contexts: keys split over CTAs
        } else if (B * nh >= 4 * (int64_t)sm && rep <= 8 && m.host_ctx_len <= 512) {
          // many sequences with short contexts: one warp per query head, one CTA per (kv head, sequence); long
          // contexts keep a whole CTA per head (a captured graph keeps the choice made at its first step)
          size_t smem = (size_t)rep * (m.P + 1) * 4 + (size_t)rep * hd * 4 + 2 * hd * sizeof(T);
          dim3 grid((unsigned)nkv, (unsigned)B);
          if (hd == 64) {
            auto kern = cgk::attn_decode_warp_kernel<T, 64>;
            static size_t smem_set_dev[64] = {0};
            size_t& smem_set = smem_set_dev[m.be->device() & 63];
            if (smem > 40 * 1024 && smem > smem_set) {
              cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
              smem_set = smem;
            }
            launch(kern, grid, dim3((unsigned)(32 * rep)), smem, a, err);
          } else {
            auto kern = cgk::attn_decode_warp_kernel<T, 128>;
            static size_t smem_set_dev[64] = {0};
            size_t& smem_set = smem_set_dev[m.be->device() & 63];
            if (smem > 40 * 1024 && smem > smem_set) {
              cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
              smem_set = smem;
            }
            launch(kern, grid, dim3((unsigned)(32 * rep)), smem, a, err);
          }
        } else {
        size_t smem = (size_t)(m.P + 1) * 4 + (size_t)(256 / (hd / VEC)) * hd * 4;
        dim3 grid((unsigned)nh, (unsigned)B);
        if (hd == 64) {
          auto kern = cgk::attn_decode_kernel<T, 64>;
          static size_t smem_set_dev[64] = {0};
            size_t& smem_set = smem_set_dev[m.be->device() & 63];
          if (smem > 40 * 1024 && smem > smem_set) {
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            smem_set = smem;
          }
          launch(kern, grid, dim3(256), smem, a, err);
        } else {
          auto kern = cgk::attn_decode_kernel<T, 128>;
          static size_t smem_set_dev[64] = {0};
            size_t& smem_set = smem_set_dev[m.be->device() & 63];
          if (smem > 40 * 1024 && smem > smem_set) {
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            smem_set = smem;
          }
          launch(kern, grid, dim3(256), smem, a, err);
        }
        }
        launched("attn_decode");
      } else {
        cgk::RopeArgs r{};
        r.q = q; r.q_row_stride = qs; r.k = k; r.k_row_stride = ks; r.v = v; r.v_row_stride = ks;
        r.kc = kcl; r.vc = vcl; r.cos_t = (const float*)m.cos_t.raw(); r.sin_t = (const float*)m.sin_t.raw();
        r.ctx_len = ctx_len; r.B = (int)B; r.S = (int)S; r.nh = (int)nh; r.nkv = (int)nkv; r.HD = (int)hd; r.P = (int)m.P;
        cgk::rope_append_kernel<T><<<(int)M, 256, 0, st>>>(r, err);
        launched("rope_append");
        prefill_attention(q, qs, kcl, vcl, attn, B, S);
      }
      // ---- o_proj + residual ----
      if (gemv_ok(M, NQ)) {
        cgk::GemvArgs a{};
        a.w[0] = w.o; a.n_end[0] = a.n_end[1] = a.n_end[2] = (int)H;
        a.x = attn; a.x_row_stride = NQ; a.out = x; a.res = x; a.M = (int)M; a.N = (int)H; a.K = (int)NQ;
        region(a.pf, 0, w.down, H * F);
        if (m.comm) {
          a.out = m.tmp.raw(); a.res = nullptr;
          gemv(cgk::PRO_NONE, cgk::EPI_STORE, a);
        } else {
          gemv(cgk::PRO_NONE, cgk::EPI_RESIDUAL, a);
        }
      } else {
        gemm(attn, NQ, w.o, m.tmp.raw(), M, H, NQ, m.comm ? nullptr : x);
      }
      if (m.comm) reduce_partials(M * H);
      // ---- MLP ----
      T* hbuf = (T*)m.h.raw();
      if (gemv_ok(M, H)) {
        cgk::GemvArgs a{};
        a.w[0] = w.gate; a.w[1] = w.up; a.n_end[0] = a.n_end[1] = a.n_end[2] = (int)F;
        a.x = x; a.x_row_stride = H; a.gain = w.post_norm; a.eps = c.rms_norm_eps;
        a.out = hbuf; a.M = (int)M; a.N = (int)F; a.K = (int)H;
        if (l + 1 < L) {
          const LayerW& nx = m.layers[l + 1];
          region(a.pf, 0, nx.q, NQ * H); region(a.pf, 1, nx.k, NKV * H); region(a.pf, 2, nx.v, NKV * H);
        } else {
          region(a.pf, 0, m.head, std::min<long long>(V * H, 48ll << 20));  // the start of the lm_head
        }
        gemv(cgk::PRO_NORM, cgk::EPI_SILU_MUL, a);
      } else {
        rmsnorm(x, w.post_norm, m.xn.raw(), M, H, 1, 0);
        // one product over the interleaved [gate; up] with SiLU(gate) * up in its epilogue; where the tensor-core
        // kernel cannot take it (f32, odd sizes) the two halves are multiplied out and combined by a second kernel
        if (!(m.gu_interleaved && gemm(m.xn.raw(), H, w.gate_up, hbuf, M, 2 * F, H, nullptr, true))) {
          if (!m.g.defined() || m.g.size() < M * 2 * F) m.g = m.be->empty({M, 2 * F}, m.dt);
          gemm(m.xn.raw(), H, w.gate_up, m.g.raw(), M, 2 * F, H);
          launch(cgk::silu_mul_packed_kernel<T>, dim3((unsigned)grid_for(M * F / (16 / sizeof(T)))), dim3(256), 0,
                 (const T*)m.g.raw(), hbuf, (long long)M, (int)F, m.gu_interleaved ? (int)GU_BLOCK : 0);
          launched("silu_mul");
        }
      }
      if (gemv_ok(M, F)) {
        cgk::GemvArgs a{};
        a.w[0] = w.down; a.n_end[0] = a.n_end[1] = a.n_end[2] = (int)H;
        a.x = hbuf; a.x_row_stride = F; a.out = x; a.res = x; a.M = (int)M; a.N = (int)H; a.K = (int)F;
        if (m.comm) {
          a.out = m.tmp.raw(); a.res = nullptr;
          gemv(cgk::PRO_NONE, cgk::EPI_STORE, a);
        } else {
          gemv(cgk::PRO_NONE, cgk::EPI_RESIDUAL, a);
        }
      } else {
        gemm(hbuf, F, w.down, m.tmp.raw(), M, H, F, m.comm ? nullptr : x);
      }
      if (m.comm) reduce_partials(M * H);
    }
    // ---- final norm + lm_head on the last position of each sequence, argmax ----
    T* logits = (T*)m.logits.raw();
    if (gemv_ok(B, H)) {
      cgk::GemvArgs a{};
      a.w[0] = m.head; a.n_end[0] = a.n_end[1] = a.n_end[2] = (int)V;
      a.x = x + (S - 1) * H; a.x_row_stride = S * H; a.gain = m.final_norm; a.eps = c.rms_norm_eps;
      a.out = logits; a.M = (int)B; a.N = (int)V; a.K = (int)H;
      gemv(cgk::PRO_NORM, cgk::EPI_STORE, a);
    } else {
      rmsnorm(x, m.final_norm, m.xn.raw(), B, H, S, S - 1);
      gemm(m.xn.raw(), H, m.head, logits, B, V, H);
    }
    launch(cgk::argmax_partial_kernel<T>, dim3((unsigned)m.argmax_chunks, (unsigned)B), dim3(256), 0, (const T*)logits,
           (long long)V, (int)V, (unsigned long long*)m.partials.raw());
    launched("argmax_partial");
    launch(cgk::advance_kernel, dim3(1), dim3(cgk::ADVANCE_THREADS), 0, (const unsigned long long*)m.partials.raw(), m.argmax_chunks,
           (unsigned*)m.ids_cur.raw(), (unsigned*)m.ids_out.raw(), ctx_len, ctx_len + 1, (int)B, (int)S,
           (int)m.out_cap_steps);
    launched("advance");
  }

  // Greedy ids of ALL M = B*S positions from the residual stream the last step left in x (final norm, lm_head,
  // argmax per row: llama.rs:204-225 as the term types its output, [B,S,1]); rows are taken 2048 at a time so that the
  // logits buffer stays at 2048 x vocabulary.
  void all_position_ids(int64_t M, unsigned* out) {
    const LlamaConfig& c = m.cfg;
    const int64_t H = c.hidden_size, V = c.vocab_size, CH = std::min<int64_t>(M, 2048);
    Tensor xn = m.be->empty({CH, H}, m.dt), lg = m.be->empty({CH, V}, m.dt);
    Tensor part = m.be->empty({CH * m.argmax_chunks * 2}, Dtype::U32);
    const T* x = (const T*)m.x.raw();
    for (int64_t r0 = 0; r0 < M; r0 += CH) {
      const int64_t rows = std::min(CH, M - r0);
      rmsnorm(x + r0 * H, m.final_norm, xn.raw(), rows, H, 1, 0);
      gemm(xn.raw(), H, m.head, lg.raw(), rows, V, H);
      launch(cgk::argmax_partial_kernel<T>, dim3((unsigned)m.argmax_chunks, (unsigned)rows), dim3(256), 0, (const T*)lg.raw(), (long long)V,
             (int)V, (unsigned long long*)part.raw());
      launched("argmax_partial");
      cgk::ids_from_partials_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>((const unsigned long long*)part.raw(), m.argmax_chunks, (int)rows,
                                                                              out + r0);
      launched("ids_from_partials");
    }
  }

  // round sqrt(hd) through T like `cast(constant(sqrt(hd)), dtype(attn))` (llama.rs:331-332)
  static float cgk_host_round(float v) {
    if (std::is_same<T, float>::value) return v;
    uint32_t u;
    std::memcpy(&u, &v, 4);
    u += 0x7fffu + ((u >> 16) & 1u);
    u &= 0xffff0000u;
    float r;
    std::memcpy(&r, &u, 4);
    return r;
  }

  // Prefill attention through batched matmuls over views (no repeat_kv copy, no K transpose copy):
  // scores[b,kvh,r] = Q[b,:,kvh*rep+r,:] x K[b,kvh]^T ; softmax ; out = P x V[b,kvh].
  void prefill_attention(T* q, int64_t qs, T* kcl, T* vcl, T* attn_out, int64_t B, int64_t S) {
    const LlamaConfig& c = m.cfg;
    const int64_t nh = c.num_attention_heads, nkv = c.num_key_value_heads, hd = m.hd, rep = nh / nkv;
    const int64_t T0 = m.host_ctx_len, Tt = T0 + S;
    const float scale = cgk_host_round((float)std::sqrt((float)hd));
    unsigned* err = m.be->dev_err();
    if (fused_prefill_ok(m, Tt)) {
      // one kernel: scores, mask, softmax and P x V per 64-query tile, the score rows never leave shared memory
      cgk::PrefillAttnArgs a{};
      a.q = (const __nv_bfloat16*)q; a.q_row = qs; a.kc = (const __nv_bfloat16*)kcl; a.vc = (const __nv_bfloat16*)vcl;
      a.out = (__nv_bfloat16*)attn_out; a.S = (int)S; a.T0 = (int)T0; a.P = (int)m.P; a.nh = (int)nh; a.nkv = (int)nkv;
      a.scale = scale;
      a.pp = (int)((Tt + cgk::PA_KEYS - 1) / cgk::PA_KEYS * cgk::PA_KEYS + 8);
      const size_t smem = cgk::prefill_attn_smem((int)hd, (int)Tt);
      auto kern = hd == 64 ? cgk::attn_prefill_fused_kernel<64> : cgk::attn_prefill_fused_kernel<128>;
      static size_t smem_set_dev[64][2] = {};
      size_t& smem_set = smem_set_dev[m.be->device() & 63][hd == 64 ? 0 : 1];
      if (smem > smem_set) {
        CG_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        smem_set = smem;
      }
      kern<<<dim3((unsigned)((S + cgk::PA_ROWS - 1) / cgk::PA_ROWS), (unsigned)nh, (unsigned)B), 128, smem, st>>>(a);
      launched("attention(prefill, fused)");
      return;
    }
    const int64_t Tp = score_pitch(Tt);  // row pitch of the score matrix
    T* scores = (T*)m.scores.raw();
    bool tc = false;
    if (std::is_same<T, __nv_bfloat16>::value) {
      // tensor cores: scores[b, h] = Q[b, :, h, :] x K[b, h / rep]^T over 4-D tensor maps
      cgk::GroupedGemm g{};
      g.A = q; g.a_row = qs; g.a_head = hd; g.a_outer = S * qs;
      g.B = kcl; g.b_row = hd; g.b_head = m.P * hd; g.b_outer = nkv * m.P * hd; g.b_n_contiguous = false;
      g.C = scores; g.ldc = Tp; g.c_head = S * Tp; g.c_outer = nh * S * Tp;
      g.M = S; g.N = Tt; g.K = hd; g.heads = nh; g.outer = B; g.b_div = rep;
      tc = cgk::launch_tcgen05_gemm_grouped(g, err, st);
    }
    if (tc) {
      launched("scores(tcgen05)");
    } else {
      cgk::View4 bt;
      std::memset(&bt, 0, sizeof(bt));
      bt.rank = 3;
      bt.shape[0] = B; bt.shape[1] = nkv; bt.shape[2] = rep;
      bt.total = B * nh;
      bt.sa[0] = S * qs; bt.sa[1] = rep * hd; bt.sa[2] = hd;            // Q[b, s, h, :] with h = kvh*rep + r
      bt.sb[0] = nkv * m.P * hd; bt.sb[1] = m.P * hd; bt.sb[2] = 0;     // K[b, kvh, t, :]
      // scores: A = Q rows (pitch qs, K-contiguous), B = K^T: k-stride 1, n-stride hd; C rows Tt apart
      CG_CHECK(Tp == Tt, ERR_INVALID_ARG, "internal: padded score rows need the tensor-core path");
      cgk::launch_matmul((int)m.dt, bt, B * nh, q, kcl, scores, S, Tt, hd, qs, 1, 1, hd, sm, st);
      launched("scores");
    }
    if (std::is_same<T, __nv_bfloat16>::value && Tp <= 1024 && Tp % 8 == 0) {
      const long long rows = B * nh * S;
      int lpr = 1;   // lanes per row: the smallest power of two whose 16-byte vectors cover a row (at most a warp)
      while (lpr < 32 && lpr * 8 < Tp) lpr <<= 1;
      const long long rows_per_cta = 8 * (32 / lpr);
      cgk::softmax_mask_rows_kernel<T><<<(unsigned)((rows + rows_per_cta - 1) / rows_per_cta), 256, 0, st>>>(
          scores, rows, (int)S, (int)Tt, (int)Tp, (int)T0, scale, lpr);
    } else {
      if ((size_t)Tt * 4 > 40 * 1024)
        cudaFuncSetAttribute(cgk::softmax_mask_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(Tt * 4));
      cgk::softmax_mask_kernel<T><<<(unsigned)(B * nh * S), 256, (size_t)Tt * 4, st>>>(scores, (int)S, (int)Tt, (int)Tp, (int)T0, scale);
    }
    launched("softmax_mask");
    // out[b, s, h, :] = P[b, h, s, :] x V[b, h / rep]  (V rows are keys: K rows hd apart, N contiguous)
    tc = false;
    if (std::is_same<T, __nv_bfloat16>::value) {
      cgk::GroupedGemm g{};
      g.A = scores; g.a_row = Tp; g.a_head = S * Tp; g.a_outer = nh * S * Tp;
      g.B = vcl; g.b_row = hd; g.b_head = m.P * hd; g.b_outer = nkv * m.P * hd; g.b_n_contiguous = true;
      g.C = attn_out; g.ldc = nh * hd; g.c_head = hd; g.c_outer = S * nh * hd;   // straight into [B, S, nh*hd]
      g.M = S; g.N = hd; g.K = Tt; g.heads = nh; g.outer = B; g.b_div = rep;
      tc = cgk::launch_tcgen05_gemm_grouped(g, err, st);
    }
    if (tc) {
      launched("pv(tcgen05)");
      return;
    }
    cgk::View4 bp;
    std::memset(&bp, 0, sizeof(bp));
    bp.rank = 3;
    bp.shape[0] = B; bp.shape[1] = nkv; bp.shape[2] = rep;
    bp.total = B * nh;
    bp.sa[0] = nh * S * Tp; bp.sa[1] = rep * S * Tp; bp.sa[2] = S * Tp;
    bp.sb[0] = nkv * m.P * hd; bp.sb[1] = m.P * hd; bp.sb[2] = 0;
    T* obhsd = (T*)m.attn_bhsd.raw();
    cgk::launch_matmul((int)m.dt, bp, B * nh, scores, vcl, obhsd, S, hd, Tt, Tp, 1, hd, 1, sm, st);
    launched("pv");
    cgk::bhsd_to_bshd_kernel<T><<<grid_for(B * nh * S * (hd / (16 / sizeof(T)))), 256, 0, st>>>(obhsd, attn_out, (int)B,
                                                                                              (int)nh, (int)S, (int)hd);
    launched("bhsd_to_bshd");
  }

  // bf16, head dimension 64 or 128, at most 1024 keys (the score rows of a 64-query tile stay in shared memory)
  static bool fused_prefill_ok(const cg_llama& m, int64_t Tt) {
    return std::is_same<T, __nv_bfloat16>::value && (m.hd == 64 || m.hd == 128) && Tt <= cgk::PA_MAX_KEYS &&
           m.max_batch <= 65535 && m.cfg.num_attention_heads <= 65535;   // grid.y = heads, grid.z = sequences
  }

  // bf16 score rows are padded to a multiple of 16 bytes so that they can be tensor-map rows
  static int64_t score_pitch(int64_t Tt) {
    return std::is_same<T, __nv_bfloat16>::value && cgk::tcgen05_available() ? (Tt + 7) / 8 * 8 : Tt;
  }
};

const Tensor& find_param(const cg_params* p, const std::string& key, Dtype dt, const Shape& shape) {
  auto it = p->p.find(key);
  CG_CHECK(it != p->p.end(), ERR_INTERP, "Load: no parameter named " + key);
  const Tensor& t = it->second;
  CG_CHECK(t.dt == dt, ERR_DTYPE_MISMATCH, "parameter " + key + " has dtype " + dtype_name(t.dt));
  CG_CHECK(t.shape == shape, ERR_SHAPE_MISMATCH, "parameter " + key + " has shape " + shape_str(t.shape) + ", expected " + shape_str(shape));
  CG_CHECK(t.is_contiguous() && ((uintptr_t)t.raw() % 16 == 0), ERR_INVALID_ARG, "parameter " + key + " must be contiguous and 16-byte aligned");
  return t;
}

// The GEMM path multiplies the normed input by [q; k; v] and by [gate; up] in one product each; the stacked
// matrices are device-side copies made once (the originals, which the caller owns, keep serving the GEMV path).
void ensure_stacked_weights(cg_llama& m) {
  if (!m.stacked.empty()) return;
  const LlamaConfig& c = m.cfg;
  const int64_t H = c.hidden_size, F = c.intermediate_size, NQ = c.num_attention_heads * m.hd,
                NKV = c.num_key_value_heads * m.hd;
  cudaStream_t st = m.be->stream();
  for (auto& w : m.layers) {
    Tensor qkv = m.be->empty({NQ + 2 * NKV, H}, m.dt);
    Tensor gu = m.be->empty({2 * F, H}, m.dt);
    unsigned char* p = (unsigned char*)qkv.raw();
    CG_CUDA(cudaMemcpyAsync(p, w.q, (size_t)NQ * H * m.es, cudaMemcpyDeviceToDevice, st));
    CG_CUDA(cudaMemcpyAsync(p + (size_t)NQ * H * m.es, w.k, (size_t)NKV * H * m.es, cudaMemcpyDeviceToDevice, st));
    CG_CUDA(cudaMemcpyAsync(p + (size_t)(NQ + NKV) * H * m.es, w.v, (size_t)NKV * H * m.es, cudaMemcpyDeviceToDevice, st));
    unsigned char* g = (unsigned char*)gu.raw();
    m.gu_interleaved = F % GU_BLOCK == 0;
    if (m.gu_interleaved) {
      const size_t blk = (size_t)GU_BLOCK * H * m.es;   // one block of rows
      CG_CUDA(cudaMemcpy2DAsync(g, 2 * blk, w.gate, blk, blk, (size_t)(F / GU_BLOCK), cudaMemcpyDeviceToDevice, st));
      CG_CUDA(cudaMemcpy2DAsync(g + blk, 2 * blk, w.up, blk, blk, (size_t)(F / GU_BLOCK), cudaMemcpyDeviceToDevice, st));
    } else {
      CG_CUDA(cudaMemcpyAsync(g, w.gate, (size_t)F * H * m.es, cudaMemcpyDeviceToDevice, st));
      CG_CUDA(cudaMemcpyAsync(g + (size_t)F * H * m.es, w.up, (size_t)F * H * m.es, cudaMemcpyDeviceToDevice, st));
    }
    w.qkv = qkv.raw();
    w.gate_up = gu.raw();
    m.stacked.push_back(qkv);
    m.stacked.push_back(gu);
  }
  CG_CUDA(cudaStreamSynchronize(st));
}

void ensure_capacity(cg_llama& m, int64_t B, int64_t S) {
  const LlamaConfig& c = m.cfg;
  int64_t M = B * S;
  int64_t H = c.hidden_size, F = c.intermediate_size, nh = c.num_attention_heads, hd = m.hd,
          NQKV = (c.num_attention_heads + 2 * c.num_key_value_heads) * hd;
  if (M > m.cap_tokens) {
    if (m.graph) {
      cudaGraphExecDestroy(m.graph);
      m.graph = nullptr;
      m.graph_batch = -1;
    }
    m.be->synchronize();
    if (m.comm) {
      CG_CHECK(M <= m.comm_tokens, ERR_INVALID_ARG,
               "batch x sequence exceeds the max_tokens the tensor-parallel runner was created with");
      // x and the partial products live in the symmetric buffer (not owned: no deleter)
      auto wrap = [&](size_t off) {
        Tensor t;
        t.st = std::make_shared<Storage>(m.comm->data() + off, (size_t)(M * H) * m.es, nullptr);
        t.dt = m.dt;
        t.shape = {M, H};
        t.strides = contiguous_strides(t.shape);
        return t;
      };
      m.x = wrap(0);
    } else {
      m.x = m.be->empty({M, H}, m.dt);
    }
    m.xn = m.be->empty({M, H}, m.dt);
    m.qkv = m.be->empty({M, NQKV}, m.dt);
    m.attn = m.be->empty({M, nh * hd}, m.dt);
    m.h = m.be->empty({M, F}, m.dt);
    if (m.comm) {
      Tensor t;
      t.st = std::make_shared<Storage>(m.comm->data() + m.comm_part_off, (size_t)(M * H) * m.es, nullptr);
      t.dt = m.dt;
      t.shape = {M, H};
      t.strides = contiguous_strides(t.shape);
      m.tmp = t;
    } else {
      m.tmp = m.be->empty({M, H}, m.dt);
    }
    if (M > 16 || (size_t)16 * H * m.es > 160 * 1024) {  // GEMM path
      ensure_stacked_weights(m);
      // gate | up buffer: only where SiLU(gate) * up cannot ride in the tensor-core GEMM's epilogue
      // (the fused epilogue is taken only by products with several tiles per SM, where it runs under the next
      // tile's main loop; with one tile per SM - a decode step of a few hundred sequences - its exponentials would
      // be exposed and the separate, fully parallel SiLU kernel is faster)
      if (M <= 1024 || !(m.gu_interleaved && m.dt == Dtype::BF16 && cgk::tcgen05_available()))
        m.g = m.be->empty({M, 2 * F}, m.dt);
    }
    m.ids_in = m.be->empty({M}, Dtype::U32);
    m.cap_tokens = M;
  }
  if (m.dt == Dtype::BF16 && m.P > 512 && !m.attn_scores.defined()) {
    // scratch of the key-split decode attention (contexts above 512), sized for max_batch once
    const int64_t chunks_max = (m.P + cgk::ATTN_CHUNK - 1) / cgk::ATTN_CHUNK;
    m.attn_scores = m.be->empty({m.max_batch * nh * m.P}, Dtype::F32);
    m.attn_partial = m.be->empty({m.max_batch * nh * chunks_max * hd}, Dtype::F32);
    m.attn_counters = m.be->zeros({m.max_batch * c.num_key_value_heads}, Dtype::U32);
  }
  const bool fused_prefill = m.dt == Dtype::BF16 && Plan<__nv_bfloat16>::fused_prefill_ok(m, m.host_ctx_len + S);
  if (S > 1 && !fused_prefill) {   // score matrix and [B, nh, S, hd] staging of the unfused prefill attention
    int64_t Tt = m.host_ctx_len + S;
    int64_t need = B * nh * S * ((Tt + 7) / 8 * 8);
    if (!m.scores.defined() || m.scores.size() < need) m.scores = m.be->empty({need}, m.dt);
    int64_t need2 = B * nh * S * hd;
    if (!m.attn_bhsd.defined() || m.attn_bhsd.size() < need2) m.attn_bhsd = m.be->empty({need2}, m.dt);
  }
}

bool mega_available(cg_llama& m, int64_t B) { return m.dt == Dtype::BF16 && Plan<__nv_bfloat16>(m).mega_geom(B).ok; }

// allow_mega: decode steps that take their ids from the device id buffer may run as the single persistent
// kernel; a step being captured into a CUDA graph may not (cooperative launch, per-launch barrier base).
void run_step(cg_llama& m, const unsigned* ids, int64_t B, int64_t S, bool allow_mega = false) {
  if (allow_mega && S == 1 && ids == (const unsigned*)m.ids_cur.raw()) {
    bool done = m.dt == Dtype::BF16 && Plan<__nv_bfloat16>(m).mega_steps(B, 1);
    if (done) {
      m.host_ctx_len += 1;
      m.mega_last_step = true;
      return;
    }
  }
  if (S == 1) m.mega_last_step = false;
  if (m.dt == Dtype::BF16) Plan<__nv_bfloat16>(m).step(ids, B, S);
  else Plan<float>(m).step(ids, B, S);
  m.host_ctx_len += S;
}

cg_llama* L(cg_llama* m) {
  CG_CHECK(m != nullptr, ERR_BAD_HANDLE, "null runner");
  return m;
}
}  // namespace

extern "C" {

typedef struct {
  uint64_t hidden_size, intermediate_size, num_hidden_layers, num_attention_heads, num_key_value_heads, vocab_size;
  float rope_theta, rms_norm_eps;
  int tie_word_embeddings;
  int rope_scaling_type;
  float rope_factor, rope_low_freq_factor, rope_high_freq_factor;
  uint64_t rope_original_max_position;
} api_llama_config;

}  // extern "C"

namespace {
// comm == nullptr: the whole model on this GPU.  Otherwise `params` holds rank comm->rank's shard of a model whose
// unsharded shape is `cfg`: rows [r*n/size, (r+1)*n/size) of q/k/v/gate/up, the same range of columns of o/down;
// norms, embedding and lm_head whole.
int create_runner(cg_ctx* ctx, const api_llama_config* cfg, int dtype, const cg_params* params, uint64_t max_batch,
                  uint64_t max_positions, cg_comm* comm, uint64_t max_tokens, cg_llama** out) {
  CG_API_BEGIN
  CG_CHECK(ctx && ctx->be && cfg && params && out, ERR_BAD_HANDLE, "null argument");
  CG_CHECK(dtype == (int)Dtype::F32 || dtype == (int)Dtype::BF16, ERR_UNSUPPORTED_DTYPE,
           "the fused runner supports f32 and bf16");
  CG_CHECK(max_batch >= 1 && max_positions >= 1, ERR_INVALID_ARG, "max_batch and max_positions must be positive");
  std::unique_ptr<cg_llama> m(new cg_llama());
  m->ctx = ctx;
  m->be = static_cast<CudaBackend*>(ctx->be.get());
  m->be->guard();
  LlamaConfig& c = m->cfg;
  c.hidden_size = (int64_t)cfg->hidden_size;
  c.intermediate_size = (int64_t)cfg->intermediate_size;
  c.num_hidden_layers = (int64_t)cfg->num_hidden_layers;
  c.num_attention_heads = (int64_t)cfg->num_attention_heads;
  c.num_key_value_heads = (int64_t)cfg->num_key_value_heads;
  c.vocab_size = (int64_t)cfg->vocab_size;
  c.rope_theta = cfg->rope_theta;
  c.rms_norm_eps = cfg->rms_norm_eps;
  c.tie_word_embeddings = cfg->tie_word_embeddings;
  c.rope_scaling_type = cfg->rope_scaling_type;
  c.rope_factor = cfg->rope_factor;
  c.rope_low_freq_factor = cfg->rope_low_freq_factor;
  c.rope_high_freq_factor = cfg->rope_high_freq_factor;
  c.rope_original_max_position = (int64_t)cfg->rope_original_max_position;
  CG_CHECK(c.rope_scaling_type == 0 || (c.rope_scaling_type == 1 && c.rope_factor > 0.f && c.rope_original_max_position > 0 &&
                                        c.rope_high_freq_factor != c.rope_low_freq_factor && c.rope_low_freq_factor > 0.f &&
                                        c.rope_high_freq_factor > 0.f),
           ERR_INVALID_ARG, "rope_scaling: type must be 0 (none) or 1 (llama3) with positive factors");
  CG_CHECK(c.num_attention_heads > 0 && c.num_key_value_heads > 0 && c.hidden_size % c.num_attention_heads == 0 &&
               c.num_attention_heads % c.num_key_value_heads == 0 && c.num_hidden_layers > 0,
           ERR_INVALID_ARG, "inconsistent Llama config");
  const int64_t hd = c.head_dim();
  CG_CHECK(hd == 64 || hd == 128, ERR_INVALID_ARG, "the fused runner supports head_dim 64 and 128");
  m->hd = hd;
  m->dt = (Dtype)dtype;
  m->es = dtype_size(m->dt);
  if (comm) {
    const int64_t tp = comm->size;
    CG_CHECK(comm->ctx == ctx, ERR_INVALID_ARG, "communicator belongs to another context");
    CG_CHECK(comm->attached, ERR_INVALID_ARG, "communicator is not attached to its peers");
    CG_CHECK(c.num_key_value_heads % tp == 0 && c.intermediate_size % tp == 0, ERR_INVALID_ARG,
             "kv heads and intermediate size must divide by the number of tensor-parallel ranks");
    CG_CHECK(max_tokens >= max_batch, ERR_INVALID_ARG, "max_tokens must cover at least one token per sequence");
    // from here on the config describes this rank's share; the hidden size stays whole
    c.num_attention_heads /= tp;
    c.num_key_value_heads /= tp;
    c.intermediate_size /= tp;
    m->comm = comm;
    m->comm_tokens = (int64_t)max_tokens;
    m->comm_part_off = align_up((size_t)max_tokens * (size_t)c.hidden_size * m->es, 256);
    CG_CHECK(2 * m->comm_part_off <= comm->data_bytes, ERR_INVALID_ARG,
             "symmetric buffer too small: need 2 x align256(max_tokens x hidden x element size) bytes");
  }
  const int64_t vec = 16 / (int64_t)m->es;
  CG_CHECK(c.hidden_size % vec == 0 && c.intermediate_size % vec == 0, ERR_INVALID_ARG,
           "hidden and intermediate sizes must be multiples of 16 bytes");
  CG_CHECK((max_positions + 1) * 4 + 32 * 128 * 4 <= 200 * 1024, ERR_INVALID_ARG, "max_positions above 47000 is not supported");
  m->max_batch = (int64_t)max_batch;
  m->P = (int64_t)max_positions;

  const int64_t H = c.hidden_size, F = c.intermediate_size, NQ = c.num_attention_heads * hd,
                NKV = c.num_key_value_heads * hd, V = c.vocab_size;
  auto get = [&](const std::string& key, const Shape& shape) {
    const Tensor& t = find_param(params, key, m->dt, shape);
    m->keep.push_back(t);
    return (const void*)t.raw();
  };
  m->embed = get("model.embed_tokens.weight", {V, H});
  for (int64_t l = 0; l < c.num_hidden_layers; ++l) {
    std::string p = "model.layers." + std::to_string(l) + ".";
    LayerW w;
    w.in_norm = get(p + "input_layernorm.weight", {H});
    w.q = get(p + "self_attn.q_proj.weight", {NQ, H});
    w.k = get(p + "self_attn.k_proj.weight", {NKV, H});
    w.v = get(p + "self_attn.v_proj.weight", {NKV, H});
    w.o = get(p + "self_attn.o_proj.weight", {H, NQ});
    w.post_norm = get(p + "post_attention_layernorm.weight", {H});
    w.gate = get(p + "mlp.gate_proj.weight", {F, H});
    w.up = get(p + "mlp.up_proj.weight", {F, H});
    w.down = get(p + "mlp.down_proj.weight", {H, F});
    m->layers.push_back(w);
  }
  m->final_norm = get("model.norm.weight", {H});
  m->head = c.tie_word_embeddings ? m->embed : get("lm_head.weight", {V, H});

  CudaBackend& be = *m->be;
  m->kc = be.zeros({c.num_hidden_layers, m->max_batch, c.num_key_value_heads, m->P, hd}, m->dt);
  m->vc = be.zeros({c.num_hidden_layers, m->max_batch, c.num_key_value_heads, m->P, hd}, m->dt);
  m->cos_t = be.empty({m->P, hd / 2}, Dtype::F32);
  m->sin_t = be.empty({m->P, hd / 2}, Dtype::F32);
  cgk::rope_table_kernel<<<std::max<int>(1, (int)std::min<int64_t>((m->P * (hd / 2) + 255) / 256, 1024)), 256, 0,
                           be.stream()>>>((float*)m->cos_t.raw(), (float*)m->sin_t.raw(), (int)m->P, (int)(hd / 2),
                                          c.rope_theta, 2.0f / (float)hd,
                                          cgk::RopeScalingArgs{c.rope_scaling_type, c.rope_factor, c.rope_low_freq_factor,
                                                               c.rope_high_freq_factor, (float)c.rope_original_max_position});
  be.check_launch("rope_table");
  m->words = be.zeros({16}, Dtype::U32);
  m->ids_cur = be.zeros({m->max_batch}, Dtype::U32);
  m->ids_new = be.zeros({m->max_batch}, Dtype::U32);
  m->logits = be.zeros({m->max_batch, V}, m->dt);
  m->argmax_chunks = (int)((V + cgk::ARGMAX_CHUNK - 1) / cgk::ARGMAX_CHUNK);
  m->partials = be.zeros({m->max_batch * m->argmax_chunks * 2}, Dtype::U32);
  // programmatic dependent launch: the next kernel starts streaming its first weight rows while this one drains
  m->use_pdl = true;
  // cross-launch L2 prefetch of later weights: measured neutral-to-slower on B200 for this chain (the launches are
  // latency-bound, not HBM-bound), so it stays off
  m->l2_prefetch = false;
  m->out_cap_steps = 0;
  {
    // table of per-layer weight pointers for the persistent decode kernel
    std::vector<cgk::PkLayer> tab;
    for (auto& w : m->layers) tab.push_back(cgk::PkLayer{w.in_norm, w.q, w.k, w.v, w.o, w.post_norm, w.gate, w.up, w.down});
    m->mega_layers = be.empty({(int64_t)(tab.size() * sizeof(cgk::PkLayer) / 4)}, Dtype::U32);
    CG_CUDA(cudaMemcpyAsync(m->mega_layers.raw(), tab.data(), tab.size() * sizeof(cgk::PkLayer), cudaMemcpyHostToDevice,
                            be.stream()));
    CG_CUDA(cudaStreamSynchronize(be.stream()));
    m->mega_grid = be.sm_count();
    m->mega_partials = be.zeros({(int64_t)m->mega_grid * cgk::PK_MAX_B * 2}, Dtype::U32);
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, be.device());
    // on by default where the shape allows it (bf16, small batch); cg_llama_set_persistent turns it off
    m->mega_possible = coop != 0 && comm == nullptr && m->dt == Dtype::BF16;
    m->mega_enabled = m->mega_possible;
    // CATGRAD_B200_PERSIST_PROF: per-CTA cycle counters of the persistent kernel, printed by cg_llama_free
    if (std::getenv("CATGRAD_B200_PERSIST_PROF")) m->mega_prof = be.zeros({(int64_t)m->mega_grid * cgk::PK_PROF_SLOTS * 2}, Dtype::U32);
  }
  *out = m.release();
  CG_API_END(ctx)
}
}  // namespace

extern "C" {

int cg_llama_create(cg_ctx* ctx, const api_llama_config* cfg, int dtype, const cg_params* params, uint64_t max_batch,
                    uint64_t max_positions, cg_llama** out) {
  return create_runner(ctx, cfg, dtype, params, max_batch, max_positions, nullptr, 0, out);
}

int cg_llama_create_tp(cg_ctx* ctx, const api_llama_config* cfg, int dtype, const cg_params* params, uint64_t max_batch,
                       uint64_t max_positions, cg_comm* comm, uint64_t max_tokens, cg_llama** out) {
  if (!comm) return cg::record_error(ctx, (int)ERR_BAD_HANDLE, "null communicator");
  return create_runner(ctx, cfg, dtype, params, max_batch, max_positions, comm, max_tokens, out);
}

void cg_llama_free(cg_llama* m) {
  if (!m) return;
  if (m->be) {
    m->be->guard();
    cudaStreamSynchronize(m->be->stream());
    if (m->mega_prof.defined()) {
      const int NS = cgk::PK_PROF_SLOTS;
      std::vector<unsigned long long> h((size_t)m->mega_grid * NS);
      if (cudaMemcpy(h.data(), m->mega_prof.raw(), h.size() * 8, cudaMemcpyDeviceToHost) == cudaSuccess) {
        static const char* names[] = {"barrier", "input", "wait_chunk", "products", "epilogue", "attention", "total"};
        for (int c : {0, 1, 31, 32, 100, m->mega_grid - 1}) {
          if (c < 0 || c >= m->mega_grid || h[(size_t)c * NS + 7] == 0) continue;
          double steps = (double)h[(size_t)c * NS + 7];
          std::fprintf(stderr, "[persist prof] cta %3d steps %.0f cycles/step:", c, steps);
          for (int i = 0; i < 7; ++i) std::fprintf(stderr, " %s=%.0f", names[i], (double)h[(size_t)c * NS + i] / steps);
          std::fprintf(stderr, " copy_warp_waits_for_slot=%.0f\n", (double)h[(size_t)c * NS + 8] / steps);
        }
      }
    }
  }
  delete m;
}

int cg_llama_reset(cg_llama* mm, uint64_t batch) {
  cg_ctx* ctx = mm ? mm->ctx : nullptr;
  CG_API_BEGIN
  cg_llama& m = *L(mm);
  CG_CHECK(batch >= 1 && (int64_t)batch <= m.max_batch, ERR_INVALID_ARG, "batch exceeds max_batch");
  m.be->guard();
  CG_CUDA(cudaMemsetAsync(m.words.raw(), 0, 64, m.be->stream()));
  m.batch = (int64_t)batch;
  m.host_ctx_len = 0;
  m.bar_base = 0;  // the barrier counter lives in `words` and was just cleared
  CG_API_END(ctx)
}

int cg_llama_forward(cg_llama* mm, const uint32_t* ids, uint64_t batch, uint64_t seq, uint32_t* out_ids) {
  cg_ctx* ctx = mm ? mm->ctx : nullptr;
  CG_API_BEGIN
  cg_llama& m = *L(mm);
  CG_CHECK(ids != nullptr, ERR_INVALID_ARG, "ids is null");
  CG_CHECK((int64_t)batch == m.batch, ERR_INVALID_ARG, "batch differs from the one given to cg_llama_reset");
  CG_CHECK(seq >= 1 && m.host_ctx_len + (int64_t)seq <= m.P, ERR_INVALID_ARG, "sequence exceeds max_positions");
  m.be->guard();
  ensure_capacity(m, (int64_t)batch, (int64_t)seq);
  if (m.out_cap_steps < 1) {
    m.ids_out = m.be->zeros({m.max_batch}, Dtype::U32);
    m.out_cap_steps = 1;
  }
  cudaStream_t st = m.be->stream();
  // a single new token per sequence is a decode step: its ids go where the on-device loop keeps them
  void* ids_dst = seq == 1 ? m.ids_cur.raw() : m.ids_in.raw();
  CG_CUDA(cudaMemcpyAsync(ids_dst, ids, batch * seq * 4, cudaMemcpyHostToDevice, st));
  CG_CUDA(cudaMemsetAsync((int*)m.words.raw() + 1, 0, 4, st));  // step_no = 0
  run_step(m, (const unsigned*)ids_dst, (int64_t)batch, (int64_t)seq, /*allow_mega=*/true);
  if (out_ids) {
    CG_CUDA(cudaMemcpyAsync(out_ids, m.ids_cur.raw(), batch * 4, cudaMemcpyDeviceToHost, st));
    CG_CUDA(cudaStreamSynchronize(st));
    m.be->check_device_errors();
  }
  CG_API_END(ctx)
}

int cg_llama_decode(cg_llama* mm, uint64_t steps, uint32_t* out_ids) {
  cg_ctx* ctx = mm ? mm->ctx : nullptr;
  CG_API_BEGIN
  cg_llama& m = *L(mm);
  CG_CHECK(m.batch >= 1 && m.host_ctx_len >= 1, ERR_INVALID_ARG, "decode needs a prefilled context");
  CG_CHECK(m.host_ctx_len + (int64_t)steps <= m.P, ERR_INVALID_ARG, "decode would exceed max_positions");
  if (steps == 0) return 0;
  m.be->guard();
  const int64_t B = m.batch;
  ensure_capacity(m, B, 1);
  cudaStream_t st = m.be->stream();
  if (m.out_cap_steps < (int64_t)steps) {
    if (m.graph) {
      cudaGraphExecDestroy(m.graph);
      m.graph = nullptr;
      m.graph_batch = -1;
    }
    m.be->synchronize();
    m.ids_out = m.be->zeros({(int64_t)steps * m.max_batch}, Dtype::U32);
    m.out_cap_steps = (int64_t)steps;
  }
  CG_CUDA(cudaMemsetAsync((int*)m.words.raw() + 1, 0, 4, st));  // step_no = 0
  const bool mega = mega_available(m, B);
  const bool use_graph = !mega && std::getenv("CATGRAD_B200_NO_GRAPH") == nullptr;
  uint64_t first = 0;
  // The capture bakes in the attention variant picked from the context length at capture time (one launch up to 512
  // cached positions, keys split over CTAs above): a graph captured on the other side of 512 is captured again.  Within
  // one call the variant stays what it was at the call's first step (results are the same, only the speed differs).
  const int ctx_bucket = m.host_ctx_len + 1 > 512 ? 1 : 0;
  if (use_graph && (m.graph == nullptr || m.graph_batch != B || m.graph_ctx_bucket != ctx_bucket)) {
    // The first step of a new shape runs eagerly (it also loads the kernels and sets their attributes,
    // neither of which belongs inside a capture); the capture below records the same launches.
    run_step(m, (const unsigned*)m.ids_cur.raw(), B, 1);
    first = 1;
    if (m.graph) {
      cudaGraphExecDestroy(m.graph);
      m.graph = nullptr;
    }
    // One decode step captured once: the context length and step number are device scalars.
    uint64_t before = m.launches;
    int64_t ctx_before = m.host_ctx_len;
    cudaGraph_t g = nullptr;
    CG_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
    try {
      run_step(m, (const unsigned*)m.ids_cur.raw(), B, 1);
    } catch (...) {
      cudaStreamEndCapture(st, &g);
      if (g) cudaGraphDestroy(g);
      m.host_ctx_len = ctx_before;
      throw;
    }
    CG_CUDA(cudaStreamEndCapture(st, &g));
    m.host_ctx_len = ctx_before;  // capture only recorded the step
    m.graph_nodes = m.launches - before;
    m.launches = before;
    cudaError_t e = cudaGraphInstantiate(&m.graph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) throw Error(ERR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
    m.graph_batch = B;
    m.graph_ctx_bucket = ctx_bucket;
  }
  for (uint64_t i = first; i < steps;) {
    if (use_graph) {
      CG_CUDA(cudaGraphLaunch(m.graph, st));
      m.launches += m.graph_nodes;
      m.host_ctx_len += 1;
      ++i;
    } else if (mega && m.mega_enabled) {
      // the persistent kernel runs up to PK_MAX_STEPS steps per launch (ids fed back inside the kernel)
      const int n = (int)std::min<uint64_t>(steps - i, cgk::PK_MAX_STEPS);
      if (Plan<__nv_bfloat16>(m).mega_steps(B, n)) {
        m.host_ctx_len += n;
        m.mega_last_step = true;
        i += (uint64_t)n;
      }   // else: mega_enabled was switched off, the next turn takes the plain step
    } else {
      run_step(m, (const unsigned*)m.ids_cur.raw(), B, 1, /*allow_mega=*/false);
      ++i;
    }
  }
  if (out_ids) {
    std::vector<uint32_t> stage((size_t)steps * B);
    CG_CUDA(cudaMemcpyAsync(stage.data(), m.ids_out.raw(), stage.size() * 4, cudaMemcpyDeviceToHost, st));
    CG_CUDA(cudaStreamSynchronize(st));
    m.be->check_device_errors();
    for (uint64_t s = 0; s < steps; ++s)
      for (int64_t b = 0; b < B; ++b) out_ids[(size_t)b * steps + s] = stage[(size_t)s * B + b];
  }
  CG_API_END(ctx)
}

int cg_llama_last_logits(cg_llama* mm, float* dst, uint64_t cap_elems) {
  cg_ctx* ctx = mm ? mm->ctx : nullptr;
  CG_API_BEGIN
  cg_llama& m = *L(mm);
  int64_t n = m.batch * m.cfg.vocab_size;
  CG_CHECK((int64_t)cap_elems >= n, ERR_INVALID_ARG, "destination too small");
  m.be->guard();
  Tensor view = m.logits;
  view.shape = {m.batch, m.cfg.vocab_size};
  view.strides = contiguous_strides(view.shape);
  Tensor f = m.be->cast(view, Dtype::F32);
  m.be->to_vec(f, dst, (size_t)n * 4);
  CG_API_END(ctx)
}

int cg_llama_set_persistent(cg_llama* mm, int on) {
  cg_ctx* ctx = mm ? mm->ctx : nullptr;
  CG_API_BEGIN
  cg_llama& m = *L(mm);
  m.mega_enabled = on != 0 && m.mega_possible;
  CG_API_END(ctx)
}
int cg_llama_persistent_active(const cg_llama* m) { return m && m->mega_last_step ? 1 : 0; }

uint64_t cg_llama_context_len(const cg_llama* m) { return m ? (uint64_t)m->host_ctx_len : 0; }
uint64_t cg_llama_launch_count(const cg_llama* m) { return m ? m->launches : 0; }

// ---- timing and allocator introspection --------------------------------------------------------
int cg_event_record(cg_ctx* ctx, int slot) {
  CG_API_BEGIN
  CG_CHECK(ctx && ctx->be, ERR_BAD_HANDLE, "null context");
  CudaBackend* be = static_cast<CudaBackend*>(ctx->be.get());
  be->guard();
  CG_CUDA(cudaEventRecord(be->event(slot), be->stream()));
  CG_API_END(ctx)
}
int cg_event_elapsed_ms(cg_ctx* ctx, int a, int b, float* out_ms) {
  CG_API_BEGIN
  CG_CHECK(ctx && ctx->be && out_ms, ERR_BAD_HANDLE, "null argument");
  CudaBackend* be = static_cast<CudaBackend*>(ctx->be.get());
  be->guard();
  CG_CUDA(cudaEventSynchronize(be->event(b)));
  CG_CUDA(cudaEventElapsedTime(out_ms, be->event(a), be->event(b)));
  CG_API_END(ctx)
}
int cg_ctx_stats(cg_ctx* ctx, uint64_t stats[4]) {
  CG_API_BEGIN
  CG_CHECK(ctx && ctx->be, ERR_BAD_HANDLE, "null context");
  CudaBackend* be = static_cast<CudaBackend*>(ctx->be.get());
  stats[0] = be->allocator().live_bytes();
  stats[1] = be->allocator().cached_bytes();
  stats[2] = be->allocator().cuda_mallocs();
  stats[3] = be->launches;
  CG_API_END(ctx)
}
namespace {
__global__ void flush_kernel(uint4* p, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    p[i] = make_uint4((unsigned)i, 0, 0, 0);
}
}  // namespace
}  // extern "C"

namespace {
// Element i of a synthetic N(0, std) tensor: a hash of (seed, i) gives two uniforms, Box-Muller one normal.  The
// value depends only on the element's index in the WHOLE matrix, so any slice of it can be produced in place.
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
template <class T>
__global__ void random_normal_kernel(T* out, long long rows, long long cols, long long row0, long long col0,
                                     long long full_cols, unsigned long long seed, float std) {
  const long long n = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols, c = i - r * cols;
    const unsigned long long h = mix64(mix64(seed) ^ (unsigned long long)((row0 + r) * full_cols + col0 + c));
    const float u1 = ((float)(unsigned)(h >> 40) + 0.5f) * (1.0f / 16777216.0f);   // (0, 1)
    const float u2 = (float)(unsigned)((h >> 8) & 0xFFFFFFu) * (1.0f / 16777216.0f);
    const float z = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
    out[i] = cgk::Elem<T>::store(z * std);
  }
}
}  // namespace

extern "C" {

// Synthetic weights without a host copy (benchmarks of models too large to draw on the host): a new [rows, cols]
// tensor holding rows [row0, row0+rows) x columns [col0, col0+cols) of a virtual [*, full_cols] matrix of N(0, std)
// values determined by `seed`.  Not part of the trait.
int cg_random_normal(cg_ctx* ctx, uint64_t seed, float std, uint64_t rows, uint64_t cols, uint64_t row0, uint64_t col0,
                     uint64_t full_cols, int dtype, cg_tensor** out) {
  CG_API_BEGIN
  CG_CHECK(ctx && ctx->be && out, ERR_BAD_HANDLE, "null argument");
  CG_CHECK(dtype == (int)Dtype::F32 || dtype == (int)Dtype::BF16, ERR_UNSUPPORTED_DTYPE, "f32 or bf16");
  CG_CHECK(rows >= 1 && cols >= 1 && col0 + cols <= full_cols, ERR_INVALID_ARG, "slice outside the matrix");
  CudaBackend* be = static_cast<CudaBackend*>(ctx->be.get());
  Tensor t = be->empty({(int64_t)rows, (int64_t)cols}, (Dtype)dtype);
  const int grid = be->sm_count() * 8;
  if (dtype == (int)Dtype::F32)
    random_normal_kernel<float><<<grid, 256, 0, be->stream()>>>((float*)t.raw(), (long long)rows, (long long)cols, (long long)row0,
                                                               (long long)col0, (long long)full_cols, seed, std);
  else
    random_normal_kernel<__nv_bfloat16><<<grid, 256, 0, be->stream()>>>((__nv_bfloat16*)t.raw(), (long long)rows, (long long)cols,
                                                                       (long long)row0, (long long)col0, (long long)full_cols,
                                                                       seed, std);
  be->check_launch("random_normal");
  cg_tensor* h = new cg_tensor();
  h->t = t;
  *out = h;
  CG_API_END(ctx)
}

// Fused last-axis softmax (the graph of stdlib nn::softmax, nn/mod.rs:168-179, in one kernel).  Not part of the trait.
int cg_softmax(cg_ctx* ctx, const cg_tensor* x, cg_tensor** out) {
  CG_API_BEGIN
  CG_CHECK(ctx && ctx->be && x && out, ERR_BAD_HANDLE, "null argument");
  CudaBackend* be = static_cast<CudaBackend*>(ctx->be.get());
  be->guard();
  cg_tensor* h = new cg_tensor();
  h->t = be->softmax(x->t);
  *out = h;
  CG_API_END(ctx)
}

int cg_flush_l2(cg_ctx* ctx, uint64_t bytes) {
  CG_API_BEGIN
  CG_CHECK(ctx && ctx->be, ERR_BAD_HANDLE, "null context");
  CudaBackend* be = static_cast<CudaBackend*>(ctx->be.get());
  Tensor t = be->empty({(int64_t)(bytes / 4)}, Dtype::U32);
  flush_kernel<<<be->sm_count() * 8, 256, 0, be->stream()>>>((uint4*)t.raw(), (long long)(bytes / 16));
  be->check_launch("flush_l2");
  CG_API_END(ctx)
}

}  // extern "C"

// ---- term -> plan: the Llama term through cg_interp_run on the fused runner ---------------------------------------
// catgrad reaches a backend only through `interpreter.run(term, inputs)` per token (examples/llama/main.rs:955-1043;
// interpreter.rs:29-37), one Backend call per tensor edge.  On the first run of a term, this hook checks whether the
// term is, edge for edge, the term `LlamaModel` builds (llama_term.cc, i.e. llama.rs:144-401) for the configuration its
// parameters and constants imply.  If so, this and every later run of the term execute as the fused plan: the KV cache
// stays in the runner's device buffers and is appended in place; the `out_k`/`out_v` values handed back are strided
// views of those buffers ([L,B,Hkv,T+S,D] over the [L,B,Hkv,P,D] allocation), and when the caller threads them back
// in as `in_k`/`in_v` (helpers/cache.rs:13-75) they are recognised by their storage, so nothing is copied or
// re-stacked.  The ids output has the term's shape [B,S,1] (all positions).  Anything else - a term that differs in a
// single edge, logits tapped as a fourth output, a cache that is not the runner's own - runs op by op as before.
namespace {

struct LlamaPlan {
  bool tried = false, matched = false;
  LlamaConfig cfg;
  struct Slot {
    const cg_params* params = nullptr;
    uint64_t version = 0;
    cg_ctx* ctx = nullptr;
    int64_t batch = 0, positions = 0;
    cg_llama* model = nullptr;
  };
  std::vector<Slot> slots;
  ~LlamaPlan() {
    for (auto& s : slots) cg_llama_free(s.model);
  }
};

bool same_term(const Term& a, const Term& b) {
  if (a.nodes != b.nodes || a.sources != b.sources || a.targets != b.targets || a.edges.size() != b.edges.size()) return false;
  for (size_t i = 0; i < a.edges.size(); ++i) {
    const Edge &x = a.edges[i], &y = b.edges[i];
    if (x.sources != y.sources || x.targets != y.targets || x.op.kind != y.op.kind) return false;
    switch (x.op.kind) {
      case OpKind::Map: if (x.op.sop != y.op.sop) return false; break;
      case OpKind::NatConstant: if (x.op.nat != y.op.nat) return false; break;
      case OpKind::DtypeConstant: if (x.op.dtype != y.op.dtype) return false; break;
      case OpKind::ScalarF32: if (std::memcmp(&x.op.f32, &y.op.f32, 4) != 0) return false; break;
      case OpKind::ScalarU32: if (x.op.u32 != y.op.u32) return false; break;
      case OpKind::Load: case OpKind::Probe: if (x.op.str != y.op.str) return false; break;
      case OpKind::If: return false;
      default: break;
    }
  }
  return true;
}

// The configuration the parameters' shapes and the term's constants imply, verified by rebuilding the term from it.
bool match_llama(const Term& t, const Parameters& p, LlamaConfig& out) {
  if (t.sources.size() != 4 || t.targets.size() != 3) return false;
  auto find = [&](const std::string& k) -> const Tensor* {
    auto it = p.find(k);
    return it == p.end() ? nullptr : &it->second;
  };
  const Tensor* emb = find("model.embed_tokens.weight");
  const Tensor* q = find("model.layers.0.self_attn.q_proj.weight");
  const Tensor* k = find("model.layers.0.self_attn.k_proj.weight");
  const Tensor* gate = find("model.layers.0.mlp.gate_proj.weight");
  if (!emb || !q || !k || !gate || emb->rank() != 2 || q->rank() != 2 || k->rank() != 2 || gate->rank() != 2) return false;
  LlamaConfig c;
  c.vocab_size = emb->shape[0];
  c.hidden_size = emb->shape[1];
  c.intermediate_size = gate->shape[0];
  while (find("model.layers." + std::to_string(c.num_hidden_layers) + ".self_attn.q_proj.weight")) ++c.num_hidden_layers;
  c.tie_word_embeddings = find("lm_head.weight") ? 0 : 1;
  if (q->shape[0] != c.hidden_size) return false;   // head_dim = hidden / heads (llama.rs:54-56): q_proj is square
  // float constants of the term in edge order: eps is the small positive one, theta the large one; a 2 pi marks
  // llama3 RoPE scaling, whose six parameters are the constants just before it (rope.rs:252-268)
  std::vector<float> consts;
  for (auto& e : t.edges)
    if (e.op.kind == OpKind::ScalarF32) consts.push_back(e.op.f32);
  std::vector<float> eps_c, theta_c;
  for (float v : consts) {
    if (v > 0.f && v < 1e-3f && std::find(eps_c.begin(), eps_c.end(), v) == eps_c.end()) eps_c.push_back(v);
    if (v >= 100.f && std::isfinite(v) && std::find(theta_c.begin(), theta_c.end(), v) == theta_c.end()) theta_c.push_back(v);
  }
  const float two_pi = 2.0f * 3.14159265358979323846f;
  size_t pi_at = consts.size();
  for (size_t i = 0; i < consts.size(); ++i)
    if (consts[i] == two_pi) { pi_at = i; break; }
  for (int64_t hd : {64, 128}) {
    if (c.hidden_size % hd || k->shape[0] % hd) continue;
    c.num_attention_heads = c.hidden_size / hd;
    c.num_key_value_heads = k->shape[0] / hd;
    if (c.num_key_value_heads == 0 || c.num_attention_heads % c.num_key_value_heads) continue;
    for (float eps : eps_c) {
      for (float theta : theta_c) {
        c.rms_norm_eps = eps;
        c.rope_theta = theta;
        for (int scaling = 0; scaling < 2; ++scaling) {
          c.rope_scaling_type = scaling;
          if (scaling == 1) {
            if (pi_at < 6 || pi_at >= consts.size()) continue;
            c.rope_factor = consts[pi_at - 4];
            c.rope_low_freq_factor = consts[pi_at - 3];
            c.rope_high_freq_factor = consts[pi_at - 2];
            c.rope_original_max_position = (int64_t)consts[pi_at - 1];
            if (!(c.rope_factor > 0.f) || !(c.rope_low_freq_factor > 0.f) || c.rope_high_freq_factor == c.rope_low_freq_factor ||
                c.rope_original_max_position <= 0)
              continue;
          }
          if (same_term(t, build_llama_term(c, false))) {
            out = c;
            return true;
          }
        }
      }
    }
  }
  return false;
}

std::atomic<bool> g_planning{true};

bool llama_plan_hook(cg_ctx* ctx, const cg_term* term, const cg_params* params, std::vector<Value>& in, std::vector<Value>& out) {
  if (!g_planning.load() || !ctx || !ctx->be || std::string(ctx->be->name()) != "b200") return false;
  if (!term->plan) term->plan = std::make_shared<LlamaPlan>();
  LlamaPlan& plan = *static_cast<LlamaPlan*>(term->plan.get());
  if (!plan.tried) {
    plan.tried = true;
    plan.matched = match_llama(term->t, params->p, plan.cfg);
  }
  if (!plan.matched || in.size() != 4) return false;
  if (in[0].kind != Value::TensorV || in[1].kind != Value::TensorV || in[2].kind != Value::TensorV || in[3].kind != Value::Nat) return false;
  const Tensor &x = in[0].tensor, &ik = in[1].tensor, &iv = in[2].tensor;
  const LlamaConfig& c = plan.cfg;
  const int64_t hd = c.head_dim();
  if (x.dt != Dtype::U32 || x.rank() != 2 || !x.is_contiguous() || ik.rank() != 5 || iv.rank() != 5 || ik.shape != iv.shape) return false;
  const int64_t B = x.shape[0], S = x.shape[1], T = ik.shape[3], P = in[3].nat;
  if (B < 1 || S < 1 || ik.shape[0] != c.num_hidden_layers || ik.shape[1] != B || ik.shape[2] != c.num_key_value_heads ||
      ik.shape[4] != hd || T + S > P)
    return false;
  auto it0 = params->p.find("model.embed_tokens.weight");
  if (it0 == params->p.end()) return false;
  const Dtype dt = it0->second.dt;
  if ((dt != Dtype::F32 && dt != Dtype::BF16) || ik.dt != dt || iv.dt != dt) return false;
  // the runner for (parameters, batch, positions); rebuilt when the parameters were changed since
  LlamaPlan::Slot* slot = nullptr;
  for (auto& s : plan.slots)
    if (s.params == params && s.ctx == ctx && s.batch == B && s.positions == P) slot = &s;
  if (slot && slot->version != params->version) {
    cg_llama_free(slot->model);
    slot->model = nullptr;
  }
  if (!slot) {
    plan.slots.push_back(LlamaPlan::Slot{params, params->version, ctx, B, P, nullptr});
    slot = &plan.slots.back();
  }
  if (!slot->model) {
    api_llama_config ac{};
    ac.hidden_size = (uint64_t)c.hidden_size; ac.intermediate_size = (uint64_t)c.intermediate_size;
    ac.num_hidden_layers = (uint64_t)c.num_hidden_layers; ac.num_attention_heads = (uint64_t)c.num_attention_heads;
    ac.num_key_value_heads = (uint64_t)c.num_key_value_heads; ac.vocab_size = (uint64_t)c.vocab_size;
    ac.rope_theta = c.rope_theta; ac.rms_norm_eps = c.rms_norm_eps; ac.tie_word_embeddings = c.tie_word_embeddings;
    ac.rope_scaling_type = c.rope_scaling_type; ac.rope_factor = c.rope_factor; ac.rope_low_freq_factor = c.rope_low_freq_factor;
    ac.rope_high_freq_factor = c.rope_high_freq_factor; ac.rope_original_max_position = (uint64_t)c.rope_original_max_position;
    cg_llama* mm = nullptr;
    if (create_runner(ctx, &ac, (int)dt, params, (uint64_t)B, (uint64_t)P, nullptr, 0, &mm) != 0) {
      plan.matched = false;   // e.g. a parameter with an unexpected layout: leave this term to the evaluator for good
      return false;
    }
    slot->model = mm;
    slot->version = params->version;
  }
  cg_llama& m = *slot->model;
  // the incoming cache: empty (a new sequence), or the runner's own buffers at its current length
  if (T == 0) {
    if (cg_llama_reset(&m, (uint64_t)B) != 0) return false;
  } else {
    const bool own = ik.st == m.kc.st && iv.st == m.vc.st && ik.offset == m.kc.offset && iv.offset == m.vc.offset &&
                     ik.strides == m.kc.strides && iv.strides == m.vc.strides && T == m.host_ctx_len && m.batch == B;
    if (!own) return false;
  }
  m.be->guard();
  ensure_capacity(m, B, S);
  if (m.out_cap_steps < 1) {
    m.ids_out = m.be->zeros({m.max_batch}, Dtype::U32);
    m.out_cap_steps = 1;
  }
  cudaStream_t st = m.be->stream();
  void* ids_dst = S == 1 ? m.ids_cur.raw() : m.ids_in.raw();
  CG_CUDA(cudaMemcpyAsync(ids_dst, x.raw(), (size_t)(B * S) * 4, cudaMemcpyDeviceToDevice, st));
  CG_CUDA(cudaMemsetAsync((int*)m.words.raw() + 1, 0, 4, st));  // step_no = 0
  run_step(m, (const unsigned*)ids_dst, B, S, /*allow_mega=*/true);
  Tensor ids = m.be->empty({B, S, 1}, Dtype::U32);
  if (S == 1) {
    CG_CUDA(cudaMemcpyAsync(ids.raw(), m.ids_cur.raw(), (size_t)B * 4, cudaMemcpyDeviceToDevice, st));
  } else if (m.dt == Dtype::BF16) {
    Plan<__nv_bfloat16>(m).all_position_ids(B * S, (unsigned*)ids.raw());
  } else {
    Plan<float>(m).all_position_ids(B * S, (unsigned*)ids.raw());
  }
  auto cache_view = [&](const Tensor& full) {
    Tensor v = full;
    v.shape = {c.num_hidden_layers, B, c.num_key_value_heads, T + S, hd};
    return v;   // strides of the [L, Bmax, Hkv, P, D] allocation: a view, nothing moves
  };
  out.clear();
  out.push_back(Value::of_tensor(ids));
  out.push_back(Value::of_tensor(cache_view(m.kc)));
  out.push_back(Value::of_tensor(cache_view(m.vc)));
  return true;
}

struct PlanHookInstaller {
  PlanHookInstaller() { cg::g_plan_hook = &llama_plan_hook; }
} g_plan_hook_installer;

}  // namespace

extern "C" {
// 0: the term has not been run yet (or planning was off); 1: it was recognised and runs as the fused Llama plan;
// 2: it was not recognised and runs op by op.
int cg_term_plan_state(const cg_term* t) {
  if (!t || !t->plan) return 0;
  const LlamaPlan& p = *static_cast<const LlamaPlan*>(t->plan.get());
  return !p.tried ? 0 : (p.matched ? 1 : 2);
}
// Process-wide switch of the term -> plan step of cg_interp_run (on by default); off forces op-by-op evaluation.
void cg_interp_set_planning(int on) { g_planning.store(on != 0); }
}

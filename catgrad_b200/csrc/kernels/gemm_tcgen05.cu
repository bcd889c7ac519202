// bf16 GEMM on Blackwell tensor cores: C[M,N] = A[M,K] x B[N,K]^T, f32 accumulation in tensor memory.
//
// This is the tensor-core path of `matmul` (catgrad/src/interpreter/backend/mod.rs:61; ndarray.rs:732-816;
// bf16 semantics = candle.rs:601-610: bf16 operands, wide accumulate, bf16 result) for the layout every
// `linear` produces: activations [M,K] row-major times a weight kept as W[N,K] row-major
// (stdlib/nn/mod.rs:182-204: x @ broadcast(transpose(W)); both operands are K-contiguous, nothing is copied).
//
// Structure of one CTA (192 threads), one 128 x BN output tile:
//   warp 0, one lane : TMA producer.  cp.async.bulk.tensor loads 128x64 (A) and BNx64 (B) bf16 boxes with the
//                      128-byte swizzle into a ring of shared-memory stages; completion lands on an mbarrier.
//                      BN is 16..256: wide tiles for large products, narrow ones so that a product with a
//                      single row tile (a decode batch) still spreads the weight stream over all SMs.
//   warp 1, one lane : issues tcgen05.mma (kind::f16, M=128, N=BN, K=16) from shared-memory descriptors into a
//                      TMEM accumulator; tcgen05.commit releases each stage and finally signals the epilogue.
//                      Warp 1 also allocates/frees the TMEM columns.
//   warps 2..5       : epilogue.  tcgen05.ld pulls the f32 accumulator (each warp its 32 TMEM lanes = 32 rows),
//                      rounds once to bf16 and stores 64-byte row segments.
// Rows/columns beyond M, N, K are zero-filled by TMA on the way in and masked on the way out, so any M, N and any
// K that keeps rows 16-byte aligned work.  Every TMA load is a plain cp.async.bulk.tensor (no cluster multicast) over
// this GPU's own memory, so the kernel may run in multi-GPU jobs; the split-K variant launches thread-block clusters
// and uses them only for a cluster barrier and distributed-shared-memory reads of the partial tiles.
//
// Every wait on an mbarrier is bounded: after ~1 s a role records DEV_ERR_WAIT_TIMEOUT, raises a CTA-wide abort
// flag, all roles fall through, TMEM is freed and the kernel returns.
//
// Bound: bf16 tensor pipe for large M; for M <= 128 (decode of a batch) it streams W once and is HBM-bound.
// Algorithmic work: 2*M*N*K flop, (M*K + N*K + M*N) * 2 bytes.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "gemm_tcgen05.h"

namespace cgk {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr long long WAIT_CYCLES = 2000000000ll;  // ~1 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred P1;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n"
      "selp.b32 %0, 1, 0, P1;\n}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false if the barrier did not flip in time or another role aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > WAIT_CYCLES) {
      *abort_flag = 1;
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile written by TMA with the 128-byte swizzle:
// rows are 128 bytes, groups of 8 rows are 1024 bytes apart (stride byte offset), descriptor version 1,
// layout type 2 (SWIZZLE_128B).  The tile base is 1024-byte aligned.
__device__ __forceinline__ uint64_t make_smem_desc(const void* tile) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);  // start address, 16-byte units
  d |= (uint64_t)1 << 16;                            // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset
  d |= (uint64_t)1 << 46;                            // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                            // SWIZZLE_128B
  return d;
}

// Same for an MN-major operand tile (the row-major [K, N] right operand of the trait's matmul: N contiguous).
// TMA writes it as blocks of 64 columns x BK rows (rows of 128 bytes, swizzled); the next 64-column block starts
// BK * 128 bytes later (leading byte offset), groups of 8 K-rows are 1024 bytes apart (stride byte offset).
__device__ __forceinline__ uint64_t make_smem_desc_mn(const void* tile) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);
  d |= (uint64_t)((BK * 128) >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor for kind::f16: D = f32, A = B = bf16, both K-major, shape M x N.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool b_mn_major = false) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- thread-block cluster helpers (split-K: the CTAs of a cluster own consecutive K ranges of one tile) ----
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_cluster_f4(const void* local_smem, unsigned cta_rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_smem)), "r"(cta_rank));
  float4 v;
  // volatile keeps it behind the cluster barrier; no memory clobber, so several of these can be in flight
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote));
  return v;
}

template <int BN>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;  // BN >= 16: a multiple of 1024, so every tile base stays 1024-aligned
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
};

// Where a product of a batch sits: z = blockIdx.z.  BMODE 1: 3-D tensor maps {K, rows, z}.  BMODE 2: 4-D maps
// {K, rows, head, outer} with z = outer * heads + head; the right operand's head coordinate is head / b_div (grouped
// heads share it), and C may be strided: base + outer * c_outer + head * c_inner, rows ldc apart.
struct BatchGeom {
  int heads, b_div;
  long long c_outer, c_inner;
  int ldc;
  // optional residual with C's layout (may alias C): C = bf16(res + bf16(acc)), the `x + linear(...)` of a block
  const __nv_bfloat16* res;
  // BMODE 0 with a right operand that no earlier kernel of the stream writes (a weight): the kernel was launched
  // with programmatic stream serialization and may fetch its first B tiles before the preceding kernel has finished
  int early_b;
  // columns come in blocks of 64 = 32 `gate` columns followed by the 32 `up` columns of the same features (the
  // interleaved [gate; up] weight of an MLP): the epilogue writes bf16(bf16(g * sigmoid(g)) * u), 32 values per block,
  // to a C that is half as wide (ldc = N / 2).  bf16 output, no residual, N a multiple of 64; persistent kernel only.
  int silu = 0;
};

// One 64-column block of gate|up accumulators of one row -> 32 bf16 outputs (64 bytes).  The products are rounded
// to bf16 first, as a stand-alone GEMM would have stored them, then combined like `silu_mul_packed_kernel`.
__device__ __forceinline__ void store_silu_block(__nv_bfloat16* dst, const uint32_t (&rg)[32], const uint32_t (&ru)[32]) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float o[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float gf = __bfloat162float(__float2bfloat16_rn(__uint_as_float(rg[v * 8 + 2 * j + e])));
        const float uf = __bfloat162float(__float2bfloat16_rn(__uint_as_float(ru[v * 8 + 2 * j + e])));
        const float sg = 1.f / (1.f + expf(-gf));
        const float si = __bfloat162float(__float2bfloat16_rn(gf * sg));
        o[e] = si * uf;
      }
      __nv_bfloat162 h = __floats2bfloat162_rn(o[0], o[1]);
      w[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// bf16(r + bf16(a)) for two neighbouring elements
__device__ __forceinline__ uint32_t add_res2(float a0, float a1, uint32_t r) {
  const __nv_bfloat162 rv = *reinterpret_cast<const __nv_bfloat162*>(&r);
  const __nv_bfloat162 av = __floats2bfloat162_rn(a0, a1);
  const __nv_bfloat162 o = __floats2bfloat162_rn(__bfloat162float(rv.x) + __bfloat162float(av.x),
                                                 __bfloat162float(rv.y) + __bfloat162float(av.y));
  return *reinterpret_cast<const uint32_t*>(&o);
}

// Split-K reduction of one CTA's share of a tile: rows [z * rows_per, (z + 1) * rows_per) of the f32 partial tiles that
// the Z CTAs of the cluster parked in their shared memory (row r at r * (BN + 4) floats), summed in rank order, rounded
// once, residual added, stored.  128 threads (warps 2..5); U items (4 columns each) per thread are in flight at once.
struct ReduceArgs {
  __nv_bfloat16* C;
  const __nv_bfloat16* res;
  int ldc, M, N, m0, n0, z, rows_valid, rows_per;
};
template <int BN, int Z, int U>
__device__ __forceinline__ void splitk_reduce(const ReduceArgs& a, const float* park) {
  const int t = threadIdx.x - 64;  // 0..127
  const bool vec_ok = (a.ldc % 4 == 0) && (((uintptr_t)a.C & 7) == 0) && (((uintptr_t)a.res & 7) == 0);
  const int items = a.rows_per * (BN / 4);
  for (int base = t; base < items; base += 128 * U) {
    float4 part[U][Z];
    uint2 rv[U];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int item = base + u * 128;
      const int rr = a.z * a.rows_per + item / (BN / 4), c4 = (item % (BN / 4)) * 4;
      live[u] = item < items && rr < a.rows_valid;
      rv[u] = make_uint2(0u, 0u);
      if (live[u]) {
        const float* src = park + (size_t)rr * (BN + 4) + c4;
#pragma unroll
        for (int pz = 0; pz < Z; ++pz) part[u][pz] = ld_cluster_f4(src, (unsigned)pz);
        const int row = a.m0 + rr, col = a.n0 + c4;
        if (a.res && vec_ok && row < a.M && col + 4 <= a.N)
          rv[u] = *reinterpret_cast<const uint2*>(a.res + (long long)row * a.ldc + col);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!live[u]) continue;
      const int item = base + u * 128;
      const int rr = a.z * a.rows_per + item / (BN / 4), c4 = (item % (BN / 4)) * 4;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int pz = 0; pz < Z; ++pz) { acc.x += part[u][pz].x; acc.y += part[u][pz].y; acc.z += part[u][pz].z; acc.w += part[u][pz].w; }
      const int row = a.m0 + rr, col = a.n0 + c4;
      if (row < a.M && col < a.N) {
        __nv_bfloat16* dst = a.C + (long long)row * a.ldc + col;
        const __nv_bfloat16* rsrc = a.res ? a.res + (long long)row * a.ldc + col : nullptr;
        if (vec_ok && col + 4 <= a.N) {
          if (rsrc) {
            *reinterpret_cast<uint2*>(dst) = make_uint2(add_res2(acc.x, acc.y, rv[u].x), add_res2(acc.z, acc.w, rv[u].y));
          } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
            *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
          }
        } else {
          const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
          for (int j = 0; j < 4; ++j)
            if (col + j < a.N) {
              __nv_bfloat16 o = __float2bfloat16_rn(a4[j]);
              if (rsrc) o = __float2bfloat16_rn(__bfloat162float(rsrc[j]) + __bfloat162float(o));
              dst[j] = o;
            }
        }
      }
    }
  }
}

// grid: (ceil(N/BN), ceil(M/BM), batch).  BMODE: 0 = one product, 1/2 = see BatchGeom.  B_MN: the right
// operand is stored [K, N] with N contiguous (tensor map dims {N, K}); otherwise [N, K] with K contiguous.
// SPLITK (BMODE 0 only): launched as clusters of gridDim.z CTAs along z; CTA z of a cluster accumulates k-blocks
// [z*per, (z+1)*per) of the tile into its own TMEM, all CTAs park their f32 partial tile in shared memory, and after
// a cluster barrier CTA z sums rows [z*128/Z, (z+1)*128/Z) over the cluster in rank order (distributed shared
// memory reads), rounds once and stores.  A pass over a weight with few row tiles thus fills all SMs without
// re-reading the activations per narrow column tile, and the result does not depend on timing.
// OUT_F32: C is a float matrix and the accumulator is stored unrounded (the exact-f32 product built from bf16 pieces).
template <int BN, int STAGES, int BMODE, bool B_MN, bool SPLITK = false, bool OUT_F32 = false>
__global__ void __launch_bounds__(192) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                                                           const __grid_constant__ CUtensorMap tmB,
                                                           __nv_bfloat16* C, int M, int N, int K,
                                                           BatchGeom g, unsigned* err) {
  using L = SmemLayout<BN>;
  constexpr int TMEM_COLS = BN < 32 ? 32 : BN;  // allocations are powers of two >= 32 columns
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + STAGES * L::STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint32_t* tmem_slot = (uint32_t*)(tmem_full + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM, bz = blockIdx.z;
  const int zo = BMODE == 2 ? bz / g.heads : 0, zh = BMODE == 2 ? bz % g.heads : 0;
  const int num_k_total = (K + BK - 1) / BK;
  int k_first = 0, num_k = num_k_total;
  if (SPLITK) {
    const int per = (num_k_total + (int)gridDim.z - 1) / (int)gridDim.z;
    k_first = bz * per;
    num_k = num_k_total - k_first < per ? num_k_total - k_first : per;   // the host keeps every range non-empty
  }

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer ----
    int issued = 0;
    int k_start = 0;
    if (BMODE == 0 && !B_MN && g.early_b) {
      // the weight tiles of the first ring-full of stages do not depend on the preceding kernel: fetch them, then
      // wait for that kernel (its output is this kernel's A operand) and add the A tiles to the same stages
      const int pre = num_k < STAGES ? num_k : STAGES;
      for (int k = 0; k < pre; ++k) {
        mbar_expect_tx(&full[k], L::STAGE_BYTES);
        tma_load_2d(smem + k * L::STAGE_BYTES + L::A_BYTES, &tmB, &full[k], (k_first + k) * BK, n0);
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int k = 0; k < pre; ++k) tma_load_2d(smem + k * L::STAGE_BYTES, &tmA, &full[k], (k_first + k) * BK, m0);
      k_start = pre;
      issued = pre;
    } else {
      asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    for (int k = k_start; k < num_k; ++k) {
      const int s = k % STAGES;
      const uint32_t par = ((k / STAGES) & 1) ^ 1;
      if (!mbar_wait(&empty[s], par, abort_flag)) break;
      unsigned char* a_dst = smem + s * L::STAGE_BYTES;
      unsigned char* b_dst = a_dst + L::A_BYTES;
      mbar_expect_tx(&full[s], L::STAGE_BYTES);
      const int kx = (k_first + k) * BK;
      if (BMODE == 2) tma_load_4d(a_dst, &tmA, &full[s], kx, m0, zh, zo);
      else if (BMODE == 1) tma_load_3d(a_dst, &tmA, &full[s], kx, m0, bz);
      else tma_load_2d(a_dst, &tmA, &full[s], kx, m0);
      if (B_MN) {
        // one 64-column x BK-row box per 64 columns of the tile
#pragma unroll
        for (int nb = 0; nb < BN / 64; ++nb) {
          if (BMODE == 2) tma_load_4d(b_dst + nb * (BK * 128), &tmB, &full[s], n0 + nb * 64, kx, zh / g.b_div, zo);
          else if (BMODE == 1) tma_load_3d(b_dst + nb * (BK * 128), &tmB, &full[s], n0 + nb * 64, kx, bz);
          else tma_load_2d(b_dst + nb * (BK * 128), &tmB, &full[s], n0 + nb * 64, kx);
        }
      } else {
        if (BMODE == 2) tma_load_4d(b_dst, &tmB, &full[s], kx, n0, zh / g.b_div, zo);
        else if (BMODE == 1) tma_load_3d(b_dst, &tmB, &full[s], kx, n0, bz);
        else tma_load_2d(b_dst, &tmB, &full[s], kx, n0);
      }
      issued = k + 1;
    }
    if (*abort_flag) {
      // give copies already in flight a bounded time to land before the CTA's shared memory goes away
      for (int k = (issued > STAGES ? issued - STAGES : 0); k < issued; ++k) {
        const long long t0 = clock64();
        while (!mbar_try_wait(&full[k % STAGES], (k / STAGES) & 1) && clock64() - t0 < WAIT_CYCLES) {
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer ----
    constexpr uint32_t idesc = make_idesc(BM, BN, B_MN);
    bool ok = true;
    for (int k = 0; k < num_k && ok; ++k) {
      const int s = k % STAGES;
      ok = mbar_wait(&full[s], (k / STAGES) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const unsigned char* a_tile = smem + s * L::STAGE_BYTES;
      const uint64_t adesc = make_smem_desc(a_tile);
      const uint64_t bdesc = B_MN ? make_smem_desc_mn(a_tile + L::A_BYTES) : make_smem_desc(a_tile + L::A_BYTES);
#pragma unroll
      for (int kk = 0; kk < BK / UMMA_K; ++kk) {
        // K-major: 16 bf16 = 32 bytes along K inside the swizzle row: +2 in the 16-byte address field.
        // MN-major: 16 K-rows of 128 bytes: +128.
        const uint64_t bstep = B_MN ? (uint64_t)(kk * (UMMA_K * 128 / 16)) : (uint64_t)(kk * 2);
        umma_bf16(tmem_base, adesc + (uint64_t)(kk * 2), bdesc + bstep, idesc, (k | kk) != 0 ? 1u : 0u);
      }
      umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
    }
    if (ok) umma_commit(tmem_full);  // accumulator complete
  } else if (warp >= 2) {
    // ---- epilogue: warp w owns TMEM lanes 32*(w%4) .. +31 = rows m0 + 32*(w%4) + lane ----
    // the epilogue reads the residual and writes C: order it after the preceding kernel like the producer
    asm volatile("griddepcontrol.wait;" ::: "memory");
    bool ok = mbar_wait(tmem_full, 0, abort_flag);
    // all lanes of the warp must agree before the warp-collective tcgen05.ld
    ok = __all_sync(0xffffffffu, ok);
    if (ok && SPLITK) {
      // park the f32 partial tile in the (now idle) operand ring: row r at r * (BN + 4) floats; warps whose 32 rows
      // lie beyond M have nothing to park (a decode batch of 32 rows uses one warp of the four)
      tc_fence_after();
      const int q = warp & 3;
      float* prow = reinterpret_cast<float*>(smem) + (size_t)(q * 32 + lane) * (BN + 4);
#pragma unroll 1
      for (int c0 = 0; c0 < BN && m0 + q * 32 < M; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 8; ++v)
          *reinterpret_cast<float4*>(prow + c0 + v * 4) = make_float4(__uint_as_float(r[v * 4]), __uint_as_float(r[v * 4 + 1]),
                                                                     __uint_as_float(r[v * 4 + 2]), __uint_as_float(r[v * 4 + 3]));
      }
    } else if (ok) {
      tc_fence_after();
      const int q = warp & 3;
      const int row = m0 + q * 32 + lane;
      const long long c_off = BMODE == 2 ? (long long)zo * g.c_outer + (long long)zh * g.c_inner : (long long)bz * g.c_outer;
      __nv_bfloat16* crow = C + c_off + (long long)row * g.ldc;
      const __nv_bfloat16* rrow = g.res ? g.res + c_off + (long long)row * g.ldc : nullptr;
      // 16-byte stores need every row start and every 32-column group aligned
      const bool vec_ok = (g.ldc % 8 == 0) && (((uintptr_t)C & 15) == 0) && (((uintptr_t)g.res & 15) == 0) &&
                          (g.c_outer % 8 == 0) && (g.c_inner % 8 == 0);
#pragma unroll 1
      for (int c0 = 0; c0 < BN && m0 + q * 32 < M; c0 += 32) {   // a warp whose 32 rows lie beyond M stores nothing
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
        tmem_ld_wait();
        if (OUT_F32) {
          if (row < M) {
            float* frow = reinterpret_cast<float*>(C) + c_off + (long long)row * g.ldc;
            const int col = n0 + c0;
            const int width = BN - c0 < 32 ? BN - c0 : 32;
            if (width == 32 && (g.ldc % 4 == 0) && (((uintptr_t)C & 15) == 0) && (g.c_outer % 4 == 0) && col + 32 <= N) {
#pragma unroll
              for (int v = 0; v < 8; ++v)
                *reinterpret_cast<float4*>(frow + col + v * 4) =
                    make_float4(__uint_as_float(r[v * 4]), __uint_as_float(r[v * 4 + 1]), __uint_as_float(r[v * 4 + 2]),
                                __uint_as_float(r[v * 4 + 3]));
            } else {
              for (int j = 0; j < width; ++j)
                if (col + j < N) frow[col + j] = __uint_as_float(r[j]);
            }
          }
        } else if (row < M) {
          const int col = n0 + c0;
          const int width = BN - c0 < 32 ? BN - c0 : 32;  // columns of this tile in the 32 just loaded
          if (width == 32 && vec_ok && col + 32 <= N) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t w[4];
              if (rrow) {
                const uint4 rv = *reinterpret_cast<const uint4*>(rrow + col + v * 8);
                const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  w[j] = add_res2(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]), rw[j]);
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
                  w[j] = *reinterpret_cast<uint32_t*>(&h);
                }
              }
              *reinterpret_cast<uint4*>(crow + col + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          } else {
            for (int j = 0; j < width; ++j)
              if (col + j < N) {
                __nv_bfloat16 o = __float2bfloat16_rn(__uint_as_float(r[j]));
                if (rrow) o = __float2bfloat16_rn(__bfloat162float(rrow[col + j]) + __bfloat162float(o));
                crow[col + j] = o;
              }
          }
        }
      }
    }
  }
  if (*abort_flag && threadIdx.x == 0) atomicOr(err, DEV_ERR_WAIT_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (SPLITK) {
    // every thread of every CTA of the cluster passes both barriers, whatever happened before
    cluster_sync_all();
    const int Z = (int)gridDim.z;
    const int rows_valid = M - m0 < BM ? M - m0 : BM;   // rows of this tile that exist
    const int rows_per = (rows_valid + Z - 1) / Z;      // CTA z reduces rows [z * rows_per, (z + 1) * rows_per)
    if (warp >= 2 && !*abort_flag) {
      // each loop iteration costs a distributed-shared-memory round trip plus a global one (the residual): several
      // items are kept in flight per thread, as many as fit 16 float4 of partials
      const ReduceArgs ra{C, g.res, g.ldc, M, N, m0, n0, bz, rows_valid, rows_per};
      const float* park = reinterpret_cast<const float*>(smem);
      if (Z == 2) splitk_reduce<BN, 2, 8>(ra, park);
      else if (Z == 4) splitk_reduce<BN, 4, 4>(ra, park);
      else splitk_reduce<BN, 8, 2>(ra, park);
    }
    cluster_sync_all();  // peers may still be reading this CTA's partial tile
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
}


// ---- persistent variant ------------------------------------------------------------------------------------------
// Same roles as above, but a CTA (one per SM) walks a static list of output tiles: tile t of CTA b is number
// b + t * gridDim.x.  TMEM holds TWO accumulators, so the epilogue warps drain tile t (tcgen05.ld, round, store) while
// the MMA warp is already accumulating tile t + 1; TMEM allocation, barrier set-up and the pipeline fill are paid once
// per CTA instead of once per tile, and the operand ring keeps streaming across tile boundaries.  Tiles are numbered
// in bands of 8 row tiles (row tile fastest inside a band) so that the tiles in flight share a few column tiles of B
// and a band of A in L2.  BATCHED: 3-D tensor maps {K, rows, z}; tile numbers then run over the batch as well.
// Used when a product has more tiles than SMs (prefill, batched products).
constexpr int PERSIST_GROUP_M = 8;

struct TileCoord {
  int m0, n0, z;
};
template <int BN>
__device__ __forceinline__ TileCoord tile_coord(long long t, int tiles_m, int tiles_n) {
  const long long per_z = (long long)tiles_m * tiles_n;
  TileCoord c;
  c.z = (int)(t / per_z);
  const int r = (int)(t - (long long)c.z * per_z);
  const int band = r / (PERSIST_GROUP_M * tiles_n);
  const int first_m = band * PERSIST_GROUP_M;
  const int band_m = tiles_m - first_m < PERSIST_GROUP_M ? tiles_m - first_m : PERSIST_GROUP_M;
  const int q = r - band * (PERSIST_GROUP_M * tiles_n);
  c.n0 = (q / band_m) * BN;
  c.m0 = (first_m + q % band_m) * BM;
  return c;
}

template <int BN, int STAGES, bool BATCHED, bool B_MN>
__global__ void __launch_bounds__(192) gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap tmA,
                                                                      const __grid_constant__ CUtensorMap tmB,
                                                                      __nv_bfloat16* C, int M, int N, int K, int batch,
                                                                      BatchGeom g, unsigned* err) {
  using L = SmemLayout<BN>;
  constexpr int TMEM_COLS = 2 * BN;   // two accumulators; BN is 128 or 256, so this is a power of two <= 512
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(smem + STAGES * L::STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;    // [2]
  uint64_t* tmem_empty = tmem_full + 2;    // [2]
  uint32_t* tmem_slot = (uint32_t*)(tmem_empty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const long long total = (long long)tiles_m * tiles_n * batch;
  const int num_k = (K + BK - 1) / BK;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);   // one arrival per epilogue warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ---- TMA producer: one continuous sequence of k-blocks over all tiles of this CTA ----
    asm volatile("griddepcontrol.wait;" ::: "memory");
    long long it = 0;       // k-blocks issued so far
    bool ok = true;
    for (long long t = blockIdx.x; t < total && ok; t += gridDim.x) {
      const TileCoord tc = tile_coord<BN>(t, tiles_m, tiles_n);
      for (int k = 0; k < num_k; ++k, ++it) {
        const int s = (int)(it % STAGES);
        const uint32_t par = (uint32_t)((it / STAGES) & 1) ^ 1u;
        if (!mbar_wait(&empty[s], par, abort_flag)) { ok = false; break; }
        unsigned char* a_dst = smem + s * L::STAGE_BYTES;
        mbar_expect_tx(&full[s], L::STAGE_BYTES);
        unsigned char* b_dst = a_dst + L::A_BYTES;
        if (BATCHED) tma_load_3d(a_dst, &tmA, &full[s], k * BK, tc.m0, tc.z);
        else tma_load_2d(a_dst, &tmA, &full[s], k * BK, tc.m0);
        if (B_MN) {
          // row-major [K, N] right operand: one 64-column x BK-row box per 64 columns of the tile
#pragma unroll
          for (int nb = 0; nb < BN / 64; ++nb) {
            if (BATCHED) tma_load_3d(b_dst + nb * (BK * 128), &tmB, &full[s], tc.n0 + nb * 64, k * BK, tc.z);
            else tma_load_2d(b_dst + nb * (BK * 128), &tmB, &full[s], tc.n0 + nb * 64, k * BK);
          }
        } else {
          if (BATCHED) tma_load_3d(b_dst, &tmB, &full[s], k * BK, tc.n0, tc.z);
          else tma_load_2d(b_dst, &tmB, &full[s], k * BK, tc.n0);
        }
      }
    }
    if (*abort_flag) {
      // give copies already in flight a bounded time to land before the CTA's shared memory goes away
      for (long long k = (it > STAGES ? it - STAGES : 0); k < it; ++k) {
        const long long t0 = clock64();
        while (!mbar_try_wait(&full[k % STAGES], (uint32_t)((k / STAGES) & 1)) && clock64() - t0 < WAIT_CYCLES) {
        }
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---- MMA issuer ----
    constexpr uint32_t idesc = make_idesc(BM, BN, B_MN);
    long long it = 0;
    bool ok = true;
    int i = 0;   // this CTA's tile counter
    for (long long t = blockIdx.x; t < total && ok; t += gridDim.x, ++i) {
      const int acc = i & 1;
      // the epilogue must have drained this accumulator (its previous use was tile i - 2)
      ok = mbar_wait(&tmem_empty[acc], (uint32_t)((i >> 1) & 1) ^ 1u, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
      for (int k = 0; k < num_k && ok; ++k, ++it) {
        const int s = (int)(it % STAGES);
        ok = mbar_wait(&full[s], (uint32_t)((it / STAGES) & 1), abort_flag);
        if (!ok) break;
        tc_fence_after();
        const unsigned char* a_tile = smem + s * L::STAGE_BYTES;
        const uint64_t adesc = make_smem_desc(a_tile);
        const uint64_t bdesc = B_MN ? make_smem_desc_mn(a_tile + L::A_BYTES) : make_smem_desc(a_tile + L::A_BYTES);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
          const uint64_t bstep = B_MN ? (uint64_t)(kk * (UMMA_K * 128 / 16)) : (uint64_t)(kk * 2);
          umma_bf16(d_tmem, adesc + (uint64_t)(kk * 2), bdesc + bstep, idesc, (k | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
      }
      if (ok) umma_commit(&tmem_full[acc]);  // accumulator complete
    }
  } else if (warp >= 2) {
    // ---- epilogue: warp w owns TMEM lanes 32*(w%4) .. +31 = rows m0 + 32*(w%4) + lane ----
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int q = warp & 3;
    const bool vec_ok = (g.ldc % 8 == 0) && (((uintptr_t)C & 15) == 0) && (((uintptr_t)g.res & 15) == 0) && (g.c_outer % 8 == 0);
    int i = 0;
    for (long long t = blockIdx.x; t < total; t += gridDim.x, ++i) {
      const int acc = i & 1;
      bool ok = mbar_wait(&tmem_full[acc], (uint32_t)((i >> 1) & 1), abort_flag);
      ok = __all_sync(0xffffffffu, ok);   // all lanes must agree before the warp-collective tcgen05.ld
      if (!ok) break;
      tc_fence_after();
      const TileCoord tc = tile_coord<BN>(t, tiles_m, tiles_n);
      const int row = tc.m0 + q * 32 + lane;
      const long long c_off = (long long)tc.z * g.c_outer;
      __nv_bfloat16* crow = C + c_off + (long long)row * g.ldc;
      const __nv_bfloat16* rrow = g.res ? g.res + c_off + (long long)row * g.ldc : nullptr;
      if (g.silu) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN && tc.m0 + q * 32 < M; c0 += 64) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0), rg);
          tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0 + 32), ru);
          tmem_ld_wait();
          if (row < M && tc.n0 + c0 + 64 <= N) store_silu_block(crow + ((tc.n0 + c0) >> 1), rg, ru);
        }
      } else
#pragma unroll 1
      for (int c0 = 0; c0 < BN && tc.m0 + q * 32 < M; c0 += 32) {   // a warp whose 32 rows lie beyond M stores nothing
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c0), r);
        tmem_ld_wait();
        if (row < M) {
          const int col = tc.n0 + c0;
          if (vec_ok && col + 32 <= N) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t w[4];
              if (rrow) {
                const uint4 rv = *reinterpret_cast<const uint4*>(rrow + col + v * 8);
                const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  w[j] = add_res2(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]), rw[j]);
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[v * 8 + 2 * j]), __uint_as_float(r[v * 8 + 2 * j + 1]));
                  w[j] = *reinterpret_cast<uint32_t*>(&h);
                }
              }
              *reinterpret_cast<uint4*>(crow + col + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          } else {
            for (int j = 0; j < 32; ++j)
              if (col + j < N) {
                __nv_bfloat16 o = __float2bfloat16_rn(__uint_as_float(r[j]));
                if (rrow) o = __float2bfloat16_rn(__bfloat162float(rrow[col + j]) + __bfloat162float(o));
                crow[col + j] = o;
              }
          }
        }
      }
      // this warp has read its lanes of the accumulator: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&tmem_empty[acc])) : "memory");
    }
  }
  if (*abort_flag && threadIdx.x == 0) atomicOr(err, DEV_ERR_WAIT_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS));
  }
}

// ---- host side ----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is resolved through the runtime, so the library has no link-time dependency on libcuda.
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// rows x K bf16 matrix with K contiguous and a row pitch of ld elements; optional batch axis.
bool make_map(CUtensorMap* map, const void* base, long long K, long long rows, long long ld, long long batch,
              long long batch_stride, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)batch_stride * 2};
  cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  int rank = batch > 1 ? 3 : 2;
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// [K, N] matrix with N contiguous and a row pitch of ld elements: tensor map dims {N, K}, boxes of 64 x BK.
bool make_map_mn(CUtensorMap* map, const void* base, long long K, long long N, long long ld, long long batch,
                 long long batch_stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)K, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)batch_stride * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)BK, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  int rank = batch > 1 ? 3 : 2;
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// 4-D variants for grouped batches: element strides of the row, head and outer axes.
bool make_map4(CUtensorMap* map, const void* base, long long K, long long rows, long long heads, long long outer,
               long long s_row, long long s_head, long long s_outer, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)heads, (cuuint64_t)outer};
  cuuint64_t strides[3] = {(cuuint64_t)s_row * 2, (cuuint64_t)s_head * 2, (cuuint64_t)s_outer * 2};
  cuuint32_t box[4] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}
bool make_map4_mn(CUtensorMap* map, const void* base, long long K, long long N, long long heads, long long outer,
                  long long s_krow, long long s_head, long long s_outer) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)K, (cuuint64_t)heads, (cuuint64_t)outer};
  cuuint64_t strides[3] = {(cuuint64_t)s_krow * 2, (cuuint64_t)s_head * 2, (cuuint64_t)s_outer * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)BK, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

struct Problem {
  bool ok = false;
  bool b_mn = false;               // right operand stored [K, N], N contiguous
  long long M, batch, a_bs, b_bs;  // after folding a shared-B batch into M
};

Problem analyse(const View4& bt, long long batch, const void* A, const void* B, long long M, long long N, long long K,
                long long sam, long long sak, long long sbk, long long sbn) {
  Problem p;
  if (sak != 1) return p;
  if (sbk == 1) {
    if (sbn % 8 != 0 || sbn < K) return p;
  } else if (sbn == 1) {
    // MN-major right operand: 64-column boxes, so keep it to products with at least one full box
    if (sbk % 8 != 0 || sbk < N || N < 64 || N % 8 != 0) return p;
    p.b_mn = true;
  } else {
    return p;
  }
  if (K < 16 || K % 8 != 0 || sam % 8 != 0) return p;
  if (((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return p;
  if (sam < K) return p;
  if (N < 16) return p;
  p.M = M;
  p.batch = 1;
  p.a_bs = p.b_bs = 0;
  if (batch > 1) {
    if (bt.rank != 1) return p;
    long long as = bt.sa[0], bs = bt.sb[0];
    if (bs == 0 && as == M * sam) {
      p.M = M * batch;  // one weight shared by the whole batch: the batch is just more rows
    } else {
      if (as % 8 != 0 || bs % 8 != 0 || as <= 0 || bs <= 0 || batch > 65535) return p;
      p.batch = batch;
      p.a_bs = as;
      p.b_bs = bs;
    }
  }
  if (p.M * p.batch < 17) return p;  // tiny products stay on the streaming GEMV
  if (p.M > 0x7fffffffll || N > 0x7fffffffll || K > 0x7fffffffll) return p;
  p.ok = encode_fn() != nullptr;
  return p;
}

template <int BN, int STAGES, int BMODE, bool B_MN>
void launch_g(const CUtensorMap& ta, const CUtensorMap& tb, void* C, long long M, long long N, long long K,
              long long batch, const BatchGeom& g, unsigned* err, cudaStream_t st) {
  using L = SmemLayout<BN>;
  size_t smem = (size_t)STAGES * L::STAGE_BYTES + 1024 /* alignment slack */ + (2 * STAGES + 1) * 8 + 16;
  auto kern = gemm_tcgen05_kernel<BN, STAGES, BMODE, B_MN>;
  static bool attr_set_dev[64] = {false};   // function attributes are per device
  int dev = 0;
  cudaGetDevice(&dev);
  bool& attr_set = attr_set_dev[dev & 63];
  if (!attr_set) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_set = true;
  }
  dim3 grid((unsigned)((N + BN - 1) / BN), (unsigned)((M + BM - 1) / BM), (unsigned)batch);
  if (BMODE == 0 && !B_MN && g.early_b) {
    cudaLaunchConfig_t cfg;
    std::memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, ta, tb, (__nv_bfloat16*)C, (int)M, (int)N, (int)K, g, err) == cudaSuccess) return;
    cudaGetLastError();
  }
  BatchGeom plain = g;
  plain.early_b = 0;
  kern<<<grid, 192, smem, st>>>(ta, tb, (__nv_bfloat16*)C, (int)M, (int)N, (int)K, plain, err);
}

// How many clusters of `splits` CTAs of the split-K kernel the GPU can hold at once (0 if the query fails).  A grid
// with more clusters than that runs a second, nearly empty wave, which doubles the duration of these short kernels.
template <int BN, int STAGES>
int splitk_max_clusters(int splits) {
  static int cache[9] = {-1, -1, -1, -1, -1, -1, -1, -1, -1};
  if (splits < 1 || splits > 8) return 0;
  if (cache[splits] >= 0) return cache[splits];
  using L = SmemLayout<BN>;
  size_t smem = (size_t)STAGES * L::STAGE_BYTES + 1024 + (2 * STAGES + 1) * 8 + 16;
  auto kern = gemm_tcgen05_kernel<BN, STAGES, 0, false, true>;
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(1, 1, (unsigned)splits);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = (unsigned)splits;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  cache[splits] = n;
  return n;
}

// Split-K launch: grid (N tiles, M tiles, splits) in clusters of (1, 1, splits).
template <int BN, int STAGES>
bool launch_splitk(const CUtensorMap& ta, const CUtensorMap& tb, void* C, long long M, long long N, long long K, int splits,
                   const void* res, unsigned* err, cudaStream_t st, bool static_b) {
  using L = SmemLayout<BN>;
  static_assert((size_t)STAGES * L::STAGE_BYTES >= (size_t)BM * (BN + 4) * 4, "partial tile must fit in the operand ring");
  size_t smem = (size_t)STAGES * L::STAGE_BYTES + 1024 + (2 * STAGES + 1) * 8 + 16;
  auto kern = gemm_tcgen05_kernel<BN, STAGES, 0, false, true>;
  static bool attr_set_dev[64] = {false};   // function attributes are per device
  int dev = 0;
  cudaGetDevice(&dev);
  bool& attr_set = attr_set_dev[dev & 63];
  if (!attr_set) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_set = true;
  }
  BatchGeom g;
  g.heads = 1;
  g.b_div = 1;
  g.c_outer = 0;
  g.c_inner = 0;
  g.ldc = (int)N;
  g.res = (const __nv_bfloat16*)res;
  g.early_b = static_b ? 1 : 0;
  cudaLaunchConfig_t cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)((N + BN - 1) / BN), (unsigned)((M + BM - 1) / BM), (unsigned)splits);
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = (unsigned)splits;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = static_b ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, ta, tb, (__nv_bfloat16*)C, (int)M, (int)N, (int)K, g, err) == cudaSuccess;
}

// contiguous C[batch, M, N]
template <int BN, int STAGES, bool BATCHED, bool B_MN = false>
void launch_t(const CUtensorMap& ta, const CUtensorMap& tb, void* C, long long M, long long N, long long K,
              long long batch, unsigned* err, cudaStream_t st, const void* res = nullptr, bool static_b = false) {
  BatchGeom g;
  g.heads = 1;
  g.b_div = 1;
  g.c_outer = M * N;
  g.c_inner = 0;
  g.ldc = (int)N;
  g.res = (const __nv_bfloat16*)res;
  g.early_b = static_b ? 1 : 0;
  launch_g<BN, STAGES, BATCHED ? 1 : 0, B_MN>(ta, tb, C, M, N, K, batch, g, err, st);
}

// Persistent launch (one CTA per SM): bf16 output, optional residual.
template <int BN, int STAGES, bool BATCHED, bool B_MN = false>
void launch_persistent(const CUtensorMap& ta, const CUtensorMap& tb, void* C, long long M, long long N, long long K, long long batch,
                       unsigned* err, int sm_count, cudaStream_t st, const void* residual, bool silu = false) {
  using L = SmemLayout<BN>;
  size_t smem = (size_t)STAGES * L::STAGE_BYTES + 1024 /* alignment slack */ + (2 * STAGES + 4) * 8 + 16;
  auto kern = gemm_tcgen05_persistent_kernel<BN, STAGES, BATCHED, B_MN>;
  static bool attr_set_dev[64] = {false};   // function attributes are per device
  int dev = 0;
  cudaGetDevice(&dev);
  bool& attr_set = attr_set_dev[dev & 63];
  if (!attr_set) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_set = true;
  }
  BatchGeom g;
  g.heads = 1;
  g.b_div = 1;
  g.c_outer = silu ? M * N / 2 : M * N;
  g.c_inner = 0;
  g.ldc = (int)(silu ? N / 2 : N);
  g.res = (const __nv_bfloat16*)residual;
  g.early_b = 0;
  g.silu = silu ? 1 : 0;
  const long long total = ((M + BM - 1) / BM) * ((N + BN - 1) / BN) * batch;
  const unsigned grid = (unsigned)(total < sm_count ? total : sm_count);
  kern<<<grid, 192, smem, st>>>(ta, tb, (__nv_bfloat16*)C, (int)M, (int)N, (int)K, (int)batch, g, err);
}
}  // namespace

bool tcgen05_available();

bool tcgen05_gemm_applicable(const View4& bt, long long batch, const void* A, const void* B, long long M, long long N,
                             long long K, long long sam, long long sak, long long sbk, long long sbn) {
  static const bool disabled = std::getenv("CATGRAD_B200_NO_TCGEN05") != nullptr;
  if (disabled) return false;
  return analyse(bt, batch, A, B, M, N, K, sam, sak, sbk, sbn).ok;
}

bool launch_tcgen05_gemm(const View4& bt, long long batch, const void* A, const void* B, void* C, long long M,
                         long long N, long long K, long long lda, long long ldb, unsigned* err, int sm_count,
                         cudaStream_t st, bool b_n_contiguous, const void* residual, bool static_b, bool silu_pairs) {
  if (silu_pairs && (b_n_contiguous || residual || batch != 1 || N % 64 != 0)) return false;
  Problem p = b_n_contiguous ? analyse(bt, batch, A, B, M, N, K, lda, 1, ldb, 1) : analyse(bt, batch, A, B, M, N, K, lda, 1, 1, ldb);
  if (!p.ok) return false;
  CUtensorMap ta, tb;
  // Tile width: as wide as possible while the grid still covers every SM about twice; narrow tiles (down to 16
  // columns) keep all SMs streaming W when M fits one row tile (decode of a batch).
  const long long mtiles = ((p.M + BM - 1) / BM) * p.batch;
  const bool streaming = mtiles <= 2;                 // one or two row tiles: a pass over W, HBM-bound
  const int min_bn = streaming && !silu_pairs ? 16 : 64;   // compute-bound products keep the MMA reasonably wide
  // enough tiles to occupy ~60 % of the SMs, but do not cut tiles finer than that: a second wave of CTAs costs more
  // than narrower tiles gain
  const long long want = streaming ? (3ll * sm_count) / 5 : (3ll * sm_count) / 4;
  int bn = 256;
  while (bn > min_bn && mtiles * ((N + bn - 1) / bn) < want) bn >>= 1;
  if (p.b_mn) {
    if (residual) return false;
    if (bn < 64) bn = 64;
    if (!make_map(&ta, A, K, p.M, lda, p.batch, p.a_bs, BM) || !make_map_mn(&tb, B, K, N, ldb, p.batch, p.b_bs)) return false;
    const bool b3 = p.batch > 1;
    if ((bn == 256 || bn == 128) && mtiles * ((N + bn - 1) / bn) > sm_count) {
      if (bn == 256) b3 ? launch_persistent<256, 4, true, true>(ta, tb, C, p.M, N, K, p.batch, err, sm_count, st, nullptr)
                        : launch_persistent<256, 4, false, true>(ta, tb, C, p.M, N, K, 1, err, sm_count, st, nullptr);
      else b3 ? launch_persistent<128, 6, true, true>(ta, tb, C, p.M, N, K, p.batch, err, sm_count, st, nullptr)
              : launch_persistent<128, 6, false, true>(ta, tb, C, p.M, N, K, 1, err, sm_count, st, nullptr);
      return true;
    }
    switch (bn) {
      case 256: b3 ? launch_t<256, 4, true, true>(ta, tb, C, p.M, N, K, p.batch, err, st) : launch_t<256, 4, false, true>(ta, tb, C, p.M, N, K, 1, err, st); break;
      case 128: b3 ? launch_t<128, 6, true, true>(ta, tb, C, p.M, N, K, p.batch, err, st) : launch_t<128, 6, false, true>(ta, tb, C, p.M, N, K, 1, err, st); break;
      default: b3 ? launch_t<64, 8, true, true>(ta, tb, C, p.M, N, K, p.batch, err, st) : launch_t<64, 8, false, true>(ta, tb, C, p.M, N, K, 1, err, st); break;
    }
    return true;
  }
  // One or two row tiles and too few 128-wide column tiles to fill the GPU: split K over a cluster instead of
  // cutting the columns finer (narrow tiles re-read the activations once per tile).
  if (streaming && p.batch == 1 && N >= 64 && !silu_pairs) {
    const long long num_k = (K + BK - 1) / BK;
    // candidates: column tiles of 128 or 64, 2/4/8-way split; keep the one that occupies the most SMs in ONE wave
    // of clusters (ties: wider tiles, then fewer splits)
    int best_bn = 0, best_splits = 1;
    long long best_ctas = mtiles * ((N + 127) / 128);   // what plain 128-wide tiles without a split would occupy
    if (best_ctas > sm_count) best_ctas = sm_count;
    for (int sbn = 128; sbn >= 64; sbn >>= 1) {
      if (N < sbn) continue;
      const long long tiles = mtiles * ((N + sbn - 1) / sbn);
      for (int splits = 2; splits <= 8; splits <<= 1) {
        if (num_k / splits < 2) break;                                              // at least two k-blocks per CTA
        if ((long long)(splits - 1) * ((num_k + splits - 1) / splits) >= num_k) continue;  // no empty K range
        const int room = sbn == 128 ? splitk_max_clusters<128, 6>(splits) : splitk_max_clusters<64, 8>(splits);
        if (tiles > room) continue;
        const long long ctas = tiles * splits;
        if (ctas > best_ctas + best_ctas / 8) {   // a finer cut has to buy clearly more parallelism
          best_ctas = ctas;
          best_bn = sbn;
          best_splits = splits;
        }
      }
    }
    if (best_bn && make_map(&ta, A, K, p.M, lda, 1, 0, BM) && make_map(&tb, B, K, N, ldb, 1, 0, best_bn)) {
      const bool launched = best_bn == 128 ? launch_splitk<128, 6>(ta, tb, C, p.M, N, K, best_splits, residual, err, st, static_b)
                                           : launch_splitk<64, 8>(ta, tb, C, p.M, N, K, best_splits, residual, err, st, static_b);
      if (launched) return true;
      cudaGetLastError();  // cluster launch refused: fall through to the plain tiles
    }
  }
  if (bn > N) bn = N >= 256 ? 256 : (N >= 128 ? 128 : (N >= 64 ? 64 : (N >= 32 ? 32 : 16)));
  if (!make_map(&ta, A, K, p.M, lda, p.batch, p.a_bs, BM) || !make_map(&tb, B, K, N, ldb, p.batch, p.b_bs, bn)) return false;
  const bool bt3 = p.batch > 1;
  // more tiles than SMs: the persistent kernel (epilogue of one tile under the main loop of the next)
  const bool persistent = (bn == 256 || bn == 128) && mtiles * ((N + bn - 1) / bn) > sm_count;
  // SiLU(gate) * up costs the four epilogue warps a few microseconds per tile: worth fusing only where that runs under
  // the next tile's MMAs
  if (silu_pairs && !persistent) return false;
  if (persistent) {
    if (bn == 256) bt3 ? launch_persistent<256, 4, true>(ta, tb, C, p.M, N, K, p.batch, err, sm_count, st, residual)
                       : launch_persistent<256, 4, false>(ta, tb, C, p.M, N, K, 1, err, sm_count, st, residual, silu_pairs);
    else bt3 ? launch_persistent<128, 6, true>(ta, tb, C, p.M, N, K, p.batch, err, sm_count, st, residual)
             : launch_persistent<128, 6, false>(ta, tb, C, p.M, N, K, 1, err, sm_count, st, residual, silu_pairs);
    return true;
  }
  switch (bn) {
    case 256: bt3 ? launch_t<256, 4, true>(ta, tb, C, p.M, N, K, p.batch, err, st, residual, static_b) : launch_t<256, 4, false>(ta, tb, C, p.M, N, K, 1, err, st, residual, static_b); break;
    case 128: bt3 ? launch_t<128, 6, true>(ta, tb, C, p.M, N, K, p.batch, err, st, residual, static_b) : launch_t<128, 6, false>(ta, tb, C, p.M, N, K, 1, err, st, residual, static_b); break;
    case 64: bt3 ? launch_t<64, 8, true>(ta, tb, C, p.M, N, K, p.batch, err, st, residual, static_b) : launch_t<64, 8, false>(ta, tb, C, p.M, N, K, 1, err, st, residual, static_b); break;
    case 32: bt3 ? launch_t<32, 5, true>(ta, tb, C, p.M, N, K, p.batch, err, st, residual, static_b) : launch_t<32, 5, false>(ta, tb, C, p.M, N, K, 1, err, st, residual, static_b); break;
    default: bt3 ? launch_t<16, 5, true>(ta, tb, C, p.M, N, K, p.batch, err, st, residual, static_b) : launch_t<16, 5, false>(ta, tb, C, p.M, N, K, 1, err, st, residual, static_b); break;
  }
  return true;
}

// f32 result from bf16 operands (K-major both, optional batch): used by the split-operand exact-f32 product.
template <int BN, int STAGES, bool BATCHED>
void launch_f32out(const CUtensorMap& ta, const CUtensorMap& tb, float* C, long long M, long long N, long long K,
                   long long batch, unsigned* err, cudaStream_t st) {
  using L = SmemLayout<BN>;
  size_t smem = (size_t)STAGES * L::STAGE_BYTES + 1024 + (2 * STAGES + 1) * 8 + 16;
  auto kern = gemm_tcgen05_kernel<BN, STAGES, BATCHED ? 1 : 0, false, false, true>;
  static bool attr_set_dev[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set_dev[dev & 63]) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attr_set_dev[dev & 63] = true;
  }
  BatchGeom g;
  g.heads = 1;
  g.b_div = 1;
  g.c_outer = M * N;
  g.c_inner = 0;
  g.ldc = (int)N;
  g.res = nullptr;
  g.early_b = 0;
  dim3 grid((unsigned)((N + BN - 1) / BN), (unsigned)((M + BM - 1) / BM), (unsigned)batch);
  kern<<<grid, 192, smem, st>>>(ta, tb, reinterpret_cast<__nv_bfloat16*>(C), (int)M, (int)N, (int)K, g, err);
}

bool launch_tcgen05_gemm_f32out(const void* A, const void* B, float* C, long long M, long long N, long long K,
                                long long batch, long long a_bs, long long b_bs, unsigned* err, int sm_count,
                                cudaStream_t st) {
  if (!tcgen05_available()) return false;
  if (K % 8 != 0 || K < 16 || N < 16 || M < 1 || batch < 1 || batch > 65535) return false;
  if (((uintptr_t)A & 15) || ((uintptr_t)B & 15) || ((uintptr_t)C & 15)) return false;
  if (a_bs % 8 != 0 || b_bs % 8 != 0 || a_bs <= 0) return false;
  CUtensorMap ta, tb;
  const long long mtiles = ((M + BM - 1) / BM) * batch;
  int bn = 256;
  while (bn > 64 && mtiles * ((N + bn - 1) / bn) < (3ll * sm_count) / 4) bn >>= 1;
  if (bn > N) bn = N >= 256 ? 256 : (N >= 128 ? 128 : 64);
  if (N < 64) return false;
  // a right operand shared by the whole batch (b_bs == 0) is addressed through a 2-D map by every batch entry
  const bool b3 = batch > 1;
  if (!make_map(&ta, A, K, M, K, batch, a_bs, BM)) return false;
  if (b3 && b_bs == 0) return false;   // callers fold a shared right operand into M instead
  if (!make_map(&tb, B, K, N, K, batch, b_bs, bn)) return false;
  switch (bn) {
    case 256: b3 ? launch_f32out<256, 4, true>(ta, tb, C, M, N, K, batch, err, st) : launch_f32out<256, 4, false>(ta, tb, C, M, N, K, 1, err, st); break;
    case 128: b3 ? launch_f32out<128, 6, true>(ta, tb, C, M, N, K, batch, err, st) : launch_f32out<128, 6, false>(ta, tb, C, M, N, K, 1, err, st); break;
    default: b3 ? launch_f32out<64, 8, true>(ta, tb, C, M, N, K, batch, err, st) : launch_f32out<64, 8, false>(ta, tb, C, M, N, K, 1, err, st); break;
  }
  return true;
}

bool tcgen05_available() {
  static const bool disabled = std::getenv("CATGRAD_B200_NO_TCGEN05") != nullptr;
  return !disabled && encode_fn() != nullptr;
}

bool launch_tcgen05_gemm_grouped(const GroupedGemm& p, unsigned* err, cudaStream_t st) {
  if (!tcgen05_available()) return false;
  auto ok8 = [](long long v) { return v > 0 && v % 8 == 0; };
  if (p.M < 1 || p.N < 16 || p.K < 16 || p.heads < 1 || p.outer < 1 || p.b_div < 1 || p.heads % p.b_div != 0) return false;
  if ((long long)p.heads * p.outer > 65535) return false;
  if (!ok8(p.a_row) || !ok8(p.a_head) || !ok8(p.a_outer) || !ok8(p.b_row) || !ok8(p.b_head) || !ok8(p.b_outer)) return false;
  if (!ok8(p.ldc) || p.c_head % 8 != 0 || p.c_outer % 8 != 0) return false;
  if (((uintptr_t)p.A & 15) || ((uintptr_t)p.B & 15) || ((uintptr_t)p.C & 15)) return false;
  if (p.b_n_contiguous && (p.N < 64 || p.N % 8 != 0)) return false;
  BatchGeom g;
  g.heads = (int)p.heads;
  g.b_div = (int)p.b_div;
  g.c_outer = p.c_outer;
  g.c_inner = p.c_head;
  g.ldc = (int)p.ldc;
  g.res = nullptr;
  g.early_b = 0;
  const long long z = (long long)p.heads * p.outer;
  CUtensorMap ta, tb;
  if (!make_map4(&ta, p.A, p.K, p.M, p.heads, p.outer, p.a_row, p.a_head, p.a_outer, BM)) return false;
  const long long kv_heads = p.heads / p.b_div;
  if (p.b_n_contiguous) {
    if (!make_map4_mn(&tb, p.B, p.K, p.N, kv_heads, p.outer, p.b_row, p.b_head, p.b_outer)) return false;
    if (p.N >= 128) launch_g<128, 6, 2, true>(ta, tb, p.C, p.M, p.N, p.K, z, g, err, st);
    else launch_g<64, 8, 2, true>(ta, tb, p.C, p.M, p.N, p.K, z, g, err, st);
    return true;
  }
  const int bn = p.N >= 256 ? 256 : (p.N >= 128 ? 128 : (p.N >= 64 ? 64 : (p.N >= 32 ? 32 : 16)));
  if (!make_map4(&tb, p.B, p.K, p.N, kv_heads, p.outer, p.b_row, p.b_head, p.b_outer, bn)) return false;
  // short reductions (K = head dimension) need two stages only, which leaves room for several CTAs per SM
  const bool short_k = p.K <= 2 * BK;
  switch (bn) {
    case 256: short_k ? launch_g<256, 2, 2, false>(ta, tb, p.C, p.M, p.N, p.K, z, g, err, st) : launch_g<256, 4, 2, false>(ta, tb, p.C, p.M, p.N, p.K, z, g, err, st); break;
    case 128: short_k ? launch_g<128, 2, 2, false>(ta, tb, p.C, p.M, p.N, p.K, z, g, err, st) : launch_g<128, 6, 2, false>(ta, tb, p.C, p.M, p.N, p.K, z, g, err, st); break;
    case 64: short_k ? launch_g<64, 2, 2, false>(ta, tb, p.C, p.M, p.N, p.K, z, g, err, st) : launch_g<64, 8, 2, false>(ta, tb, p.C, p.M, p.N, p.K, z, g, err, st); break;
    case 32: launch_g<32, 2, 2, false>(ta, tb, p.C, p.M, p.N, p.K, z, g, err, st); break;
    default: launch_g<16, 2, 2, false>(ta, tb, p.C, p.M, p.N, p.K, z, g, err, st); break;
  }
  return true;
}

}  // namespace cgk

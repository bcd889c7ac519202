// cg_comm_*: symmetric buffers over CUDA IPC and the tensor-parallel all-reduce kernel (tp_comm.h).
//
// Protocol of one all-reduce (every rank launches the same kernel, sequence number `seq` from a device counter so
// that a captured CUDA graph replays it):
//   A. rank r stores seq into slot r of every peer's A-flags, then waits until its own A-flags are all >= seq:
//      every rank's partial product is complete and visible.
//   B. reduce.  Large messages ("two-shot"): rank r sums slice r of all ranks' partials in rank order (f32), rounds,
//      adds its residual slice and stores the result into x of EVERY rank.  Small messages ("one-shot"): every rank
//      sums everything itself and stores only locally.  Both give bit-identical x on all ranks.
//   C. the last CTA to finish stores seq into every peer's B-flags; all CTAs wait for all B-flags: nobody still
//      reads this rank's partial or writes its x when the kernel ends.
// Flags are pushed (remote store) and polled locally.  The grid never exceeds the SM count, so every CTA is
// resident while it waits.  Waits give up after the communicator's time limit (5 s unless changed): the communicator is then marked dead (later calls
// return at once) and DEV_ERR_WAIT_TIMEOUT is raised for the host.
#include "tp_comm.h"

#include <cuda_bf16.h>

#include <cstring>
#include <string>

#include "../kernels/common.cuh"
#include "c_api_internal.h"
#include "cuda_backend.h"

using namespace cg;

namespace {

constexpr size_t ONE_SHOT_BYTES = 1 << 20;

// header words (u32): [0..7] A-flags, [32..39] B-flags, [64] completed sequence number, [65] CTAs done, [66] dead
constexpr int HDR_A = 0, HDR_B = 32, HDR_SEQ = 64, HDR_DONE = 65, HDR_DEAD = 66;

struct CommDev {
  unsigned char* base[TP_MAX_RANKS];
  int rank, size;
  unsigned long long wait_ns;
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// true once all `size` flags have reached seq (wrap-safe), false after limit_ns
__device__ bool wait_flags(const unsigned* flags, unsigned seq, int size, unsigned long long limit_ns) {
  const unsigned long long t0 = now_ns();
  for (int p = 0; p < size; ++p) {
    while ((int)(ld_acquire_sys(flags + p) - seq) < 0) {
      if (now_ns() - t0 > limit_ns) return false;
      __nanosleep(40);
    }
  }
  return true;
}

template <class T>
__global__ void __launch_bounds__(512) tp_allreduce_kernel(CommDev c, size_t x_off, size_t part_off, long long nvec,
                                                           int two_shot, int residual, unsigned* err) {
  constexpr int VEC = 16 / sizeof(T);
  unsigned* hdr = reinterpret_cast<unsigned*>(c.base[c.rank]);
  __shared__ unsigned s_seq;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    const unsigned dead = ld_acquire_sys(hdr + HDR_DEAD);
    const unsigned seq = ld_acquire_sys(hdr + HDR_SEQ) + 1u;
    bool ok = dead == 0;
    if (ok) {
      if (blockIdx.x == 0) {
        __threadfence_system();
        for (int p = 0; p < c.size; ++p) st_release_sys(reinterpret_cast<unsigned*>(c.base[p]) + HDR_A + c.rank, seq);
      }
      ok = wait_flags(hdr + HDR_A, seq, c.size, c.wait_ns);
      if (!ok) {
        st_release_sys(hdr + HDR_DEAD, 1u);
        atomicOr(err, cgk::DEV_ERR_WAIT_TIMEOUT);
      }
    }
    s_seq = seq;
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const unsigned seq = s_seq;

  long long lo = 0, hi = nvec;
  if (two_shot) {
    const long long chunk = (nvec + c.size - 1) / c.size;
    lo = chunk * c.rank;
    hi = lo + chunk < nvec ? lo + chunk : nvec;
  }
  const size_t data = TP_HEADER_BYTES;
  unsigned char* x_local = c.base[c.rank] + data + x_off;
  for (long long v = lo + (long long)blockIdx.x * blockDim.x + threadIdx.x; v < hi; v += (long long)gridDim.x * blockDim.x) {
    uint4 in[TP_MAX_RANKS];
#pragma unroll
    for (int p = 0; p < TP_MAX_RANKS; ++p)
      if (p < c.size) in[p] = ld_peer16(c.base[p] + data + part_off + (size_t)v * 16);
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
#pragma unroll
    for (int p = 0; p < TP_MAX_RANKS; ++p) {
      if (p < c.size) {
        const T* e = reinterpret_cast<const T*>(&in[p]);
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] += cgk::Elem<T>::load(e[i]);
      }
    }
    uint4 outv;
    T* o = reinterpret_cast<T*>(&outv);
    if (residual) {
      const uint4 xv = *reinterpret_cast<const uint4*>(x_local + (size_t)v * 16);
      const T* xe = reinterpret_cast<const T*>(&xv);
#pragma unroll
      for (int i = 0; i < VEC; ++i)
        o[i] = cgk::Elem<T>::store(cgk::Elem<T>::load(xe[i]) + cgk::Elem<T>::load(cgk::Elem<T>::store(acc[i])));
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = cgk::Elem<T>::store(acc[i]);
    }
    if (two_shot) {
#pragma unroll
      for (int p = 0; p < TP_MAX_RANKS; ++p)
        if (p < c.size) *reinterpret_cast<uint4*>(c.base[p] + data + x_off + (size_t)v * 16) = outv;
    } else {
      *reinterpret_cast<uint4*>(x_local + (size_t)v * 16) = outv;
    }
  }
  // two-shot: the stores into the peers' x must be visible system-wide before the B flag; one-shot wrote only local
  // memory, and its reads of the peers' partials completed when their values were consumed
  if (two_shot) __threadfence_system();
  else __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned old = atomicAdd(hdr + HDR_DONE, 1u);
    if (old == gridDim.x - 1) {
      // every CTA of this launch has read the old sequence number and finished its stores
      atomicExch(hdr + HDR_DONE, 0u);
      st_release_sys(hdr + HDR_SEQ, seq);
      for (int p = 0; p < c.size; ++p) st_release_sys(reinterpret_cast<unsigned*>(c.base[p]) + HDR_B + c.rank, seq);
    }
    if (!wait_flags(hdr + HDR_B, seq, c.size, c.wait_ns)) {
      st_release_sys(hdr + HDR_DEAD, 1u);
      atomicOr(err, cgk::DEV_ERR_WAIT_TIMEOUT);
    }
  }
}

cg_comm* C(cg_comm* c) {
  CG_CHECK(c != nullptr, ERR_BAD_HANDLE, "null communicator");
  return c;
}

}  // namespace

void cg_comm::allreduce(Dtype dt, size_t x_off, size_t part_off, int64_t n, bool residual, int sm_count, cudaStream_t st,
                        unsigned* err) {
  CG_CHECK(attached, ERR_INVALID_ARG, "communicator is not attached to its peers");
  const size_t es = dtype_size(dt);
  const size_t bytes = (size_t)n * es;
  CG_CHECK(dt == Dtype::BF16 || dt == Dtype::F32, ERR_UNSUPPORTED_DTYPE, "all-reduce supports f32 and bf16");
  CG_CHECK(bytes % 16 == 0 && x_off % 16 == 0 && part_off % 16 == 0, ERR_INVALID_ARG, "all-reduce needs 16-byte granularity");
  CG_CHECK(x_off + bytes <= data_bytes && part_off + bytes <= data_bytes, ERR_INVALID_ARG, "all-reduce outside the symmetric buffer");
  CommDev c;
  for (int p = 0; p < TP_MAX_RANKS; ++p) c.base[p] = p < size ? peer[p] : nullptr;
  c.rank = rank;
  c.size = size;
  c.wait_ns = (unsigned long long)wait_ms * 1000000ull;
  const long long nvec = (long long)(bytes / 16);
  const int two_shot = (size > 1 && bytes > ONE_SHOT_BYTES) ? 1 : 0;
  const long long mine = two_shot ? (nvec + size - 1) / size : nvec;
  int grid = (int)std::min<long long>(sm_count, std::max<long long>(1, (mine + 511) / 512));
  if (dt == Dtype::BF16)
    tp_allreduce_kernel<__nv_bfloat16><<<grid, 512, 0, st>>>(c, x_off, part_off, nvec, two_shot, residual ? 1 : 0, err);
  else
    tp_allreduce_kernel<float><<<grid, 512, 0, st>>>(c, x_off, part_off, nvec, two_shot, residual ? 1 : 0, err);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw Error(ERR_CUDA, std::string("tp all-reduce launch: ") + cudaGetErrorString(e));
}

extern "C" {

// Allocates this rank's symmetric buffer (header + data_bytes, zeroed) on the context's device.
int cg_comm_create(cg_ctx* ctx, int rank, int size, uint64_t data_bytes, cg_comm** out) {
  CG_API_BEGIN
  CG_CHECK(ctx && ctx->be && out, ERR_BAD_HANDLE, "null argument");
  CG_CHECK(size >= 1 && size <= TP_MAX_RANKS && rank >= 0 && rank < size, ERR_INVALID_ARG, "need 0 <= rank < size <= 8");
  CG_CHECK(data_bytes >= 16 && data_bytes % 256 == 0, ERR_INVALID_ARG, "data_bytes must be a positive multiple of 256");
  CudaBackend* be = static_cast<CudaBackend*>(ctx->be.get());
  be->guard();
  std::unique_ptr<cg_comm> c(new cg_comm());
  c->ctx = ctx;
  c->rank = rank;
  c->size = size;
  c->device = be->device();
  c->data_bytes = (size_t)data_bytes;
  for (int p = 0; p < TP_MAX_RANKS; ++p) c->peer[p] = nullptr;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, TP_HEADER_BYTES + (size_t)data_bytes);
  if (e != cudaSuccess) throw Error(ERR_OOM, std::string("symmetric buffer: ") + cudaGetErrorString(e));
  c->local = (unsigned char*)p;
  c->peer[rank] = c->local;
  e = cudaMemset(p, 0, TP_HEADER_BYTES + (size_t)data_bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess && size > 1) e = cudaIpcGetMemHandle(&c->handle, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    throw Error(ERR_CUDA, std::string("symmetric buffer setup: ") + cudaGetErrorString(e));
  }
  c->attached = size == 1;
  *out = c.release();
  CG_API_END(ctx)
}

// Copies the 64-byte IPC handle of this rank's buffer; ranks exchange these out of band (any host channel).
int cg_comm_handle(cg_comm* cc, void* out64) {
  cg_ctx* ctx = cc ? cc->ctx : nullptr;
  CG_API_BEGIN
  cg_comm& c = *C(cc);
  CG_CHECK(out64 != nullptr, ERR_INVALID_ARG, "null destination");
  CG_CHECK(c.size > 1, ERR_INVALID_ARG, "a single-rank communicator has no handle to exchange");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  std::memcpy(out64, &c.handle, 64);
  CG_API_END(ctx)
}

// handles: size x 64 bytes in rank order (this rank's own entry is ignored).  Call once, after every rank has
// created its buffer; the exchange of handles is the barrier that orders the zeroing before any peer access.
int cg_comm_attach(cg_comm* cc, const void* handles) {
  cg_ctx* ctx = cc ? cc->ctx : nullptr;
  CG_API_BEGIN
  cg_comm& c = *C(cc);
  CG_CHECK(handles != nullptr, ERR_INVALID_ARG, "null handles");
  CG_CHECK(!c.attached, ERR_INVALID_ARG, "communicator already attached");
  static_cast<CudaBackend*>(c.ctx->be.get())->guard();
  for (int p = 0; p < c.size; ++p) {
    if (p == c.rank) continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, (const unsigned char*)handles + (size_t)p * 64, 64);
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      for (int q = 0; q < p; ++q)
        if (q != c.rank && c.peer[q]) {
          cudaIpcCloseMemHandle(c.peer[q]);
          c.peer[q] = nullptr;
        }
      throw Error(ERR_CUDA, "cudaIpcOpenMemHandle(rank " + std::to_string(p) + "): " + cudaGetErrorString(e));
    }
    c.peer[p] = (unsigned char*)ptr;
  }
  c.attached = true;
  CG_API_END(ctx)
}

// Same-process variant of cg_comm_attach for hosts that drive several GPUs from one process (IPC handles cannot be
// opened by the process that made them): `all` lists the communicators of all ranks in rank order.  Peer access
// between the devices is enabled when they differ.
int cg_comm_attach_local(cg_comm* cc, cg_comm* const* all) {
  cg_ctx* ctx = cc ? cc->ctx : nullptr;
  CG_API_BEGIN
  cg_comm& c = *C(cc);
  CG_CHECK(all != nullptr, ERR_INVALID_ARG, "null communicator list");
  CG_CHECK(!c.attached, ERR_INVALID_ARG, "communicator already attached");
  static_cast<CudaBackend*>(c.ctx->be.get())->guard();
  for (int p = 0; p < c.size; ++p) {
    CG_CHECK(all[p] != nullptr && all[p]->size == c.size && all[p]->rank == p && all[p]->data_bytes == c.data_bytes,
             ERR_INVALID_ARG, "communicator list does not match (rank order, size, data_bytes)");
    if (p == c.rank) continue;
    if (all[p]->device != c.device) {
      int can = 0;
      CG_CUDA(cudaDeviceCanAccessPeer(&can, c.device, all[p]->device));
      CG_CHECK(can != 0, ERR_CUDA, "no peer access between the devices of two ranks");
      cudaError_t e = cudaDeviceEnablePeerAccess(all[p]->device, 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
      else if (e != cudaSuccess) throw Error(ERR_CUDA, std::string("cudaDeviceEnablePeerAccess: ") + cudaGetErrorString(e));
    }
    c.peer[p] = all[p]->local;
  }
  c.local_peers = true;
  c.attached = true;
  CG_API_END(ctx)
}

// Time limit of the device-side waits of this communicator (default 5000 ms).
int cg_comm_set_timeout_ms(cg_comm* cc, uint64_t ms) {
  cg_ctx* ctx = cc ? cc->ctx : nullptr;
  CG_API_BEGIN
  cg_comm& c = *C(cc);
  CG_CHECK(ms >= 1 && ms <= 600000, ERR_INVALID_ARG, "timeout must be 1 ms .. 10 min");
  c.wait_ms = ms;
  CG_API_END(ctx)
}

// Device address of the data area (for callers that place their own operands in symmetric memory).
int cg_comm_data(cg_comm* cc, void** ptr, uint64_t* bytes) {
  cg_ctx* ctx = cc ? cc->ctx : nullptr;
  CG_API_BEGIN
  cg_comm& c = *C(cc);
  if (ptr) *ptr = c.data();
  if (bytes) *bytes = c.data_bytes;
  CG_API_END(ctx)
}

// Host <-> data area copies (stream-ordered on the context's stream; the read synchronises).
int cg_comm_write(cg_comm* cc, uint64_t off, const void* src, uint64_t bytes) {
  cg_ctx* ctx = cc ? cc->ctx : nullptr;
  CG_API_BEGIN
  cg_comm& c = *C(cc);
  CG_CHECK(src != nullptr && off + bytes <= c.data_bytes, ERR_INVALID_ARG, "write outside the symmetric buffer");
  CudaBackend* be = static_cast<CudaBackend*>(c.ctx->be.get());
  be->guard();
  CG_CUDA(cudaMemcpyAsync(c.data() + off, src, bytes, cudaMemcpyHostToDevice, be->stream()));
  CG_CUDA(cudaStreamSynchronize(be->stream()));
  CG_API_END(ctx)
}
int cg_comm_read(cg_comm* cc, uint64_t off, void* dst, uint64_t bytes) {
  cg_ctx* ctx = cc ? cc->ctx : nullptr;
  CG_API_BEGIN
  cg_comm& c = *C(cc);
  CG_CHECK(dst != nullptr && off + bytes <= c.data_bytes, ERR_INVALID_ARG, "read outside the symmetric buffer");
  CudaBackend* be = static_cast<CudaBackend*>(c.ctx->be.get());
  be->guard();
  CG_CUDA(cudaMemcpyAsync(dst, c.data() + off, bytes, cudaMemcpyDeviceToHost, be->stream()));
  CG_CUDA(cudaStreamSynchronize(be->stream()));
  be->check_device_errors();
  CG_API_END(ctx)
}

// x (+)= sum over ranks of part, element type dtype, n elements; offsets in bytes into the data area.
int cg_comm_allreduce(cg_comm* cc, int dtype, uint64_t x_off, uint64_t part_off, uint64_t n, int residual) {
  cg_ctx* ctx = cc ? cc->ctx : nullptr;
  CG_API_BEGIN
  cg_comm& c = *C(cc);
  CudaBackend* be = static_cast<CudaBackend*>(c.ctx->be.get());
  be->guard();
  c.allreduce((Dtype)dtype, (size_t)x_off, (size_t)part_off, (int64_t)n, residual != 0, be->sm_count(), be->stream(),
              be->dev_err());
  CG_API_END(ctx)
}

void cg_comm_free(cg_comm* c) {
  if (!c) return;
  if (c->ctx && c->ctx->be) static_cast<CudaBackend*>(c->ctx->be.get())->guard();
  cudaDeviceSynchronize();
  for (int p = 0; p < c->size; ++p)
    if (p != c->rank && c->peer[p] && !c->local_peers) cudaIpcCloseMemHandle(c->peer[p]);
  if (c->local) cudaFree(c->local);
  delete c;
}

}  // extern "C"

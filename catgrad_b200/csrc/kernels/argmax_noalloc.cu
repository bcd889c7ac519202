// cg_argmax_rows_noalloc: the two-stage greedy pick (last-axis argmax) for callers that must not allocate.
//
// Who needs it: code that runs where device allocation is off the table.  Examples are a serving loop whose
// memory was carved up front and is owned by another allocator (any cudaMalloc would fragment or fail it), a
// host callback or latency-critical section where cudaMalloc's implicit device synchronisation is unacceptable,
// and plug-ins that are handed raw device pointers and a stream but no allocator to ask.  The regular entry
// point cg_argmax returns a NEW tensor from the context's caching allocator, so it may call cudaMalloc.
//
// This variant takes caller-owned input and output buffers and keeps its only scratch (the stage-1 partial
// keys) in a fixed array that is part of the library image: every GPU that loads the library holds
// CG_NOALLOC_MAX_PARTIALS * 8 bytes (128 KiB) of it until the process exits.  It calls no cudaMalloc, cudaFree
// or any allocating routine.
//
// Sharing rules that follow from the fixed array:
//  * all calls on one GPU use the same scratch; two calls whose kernels overlap on the GPU (different streams,
//    different threads) race on it.  Serialise them.
//  * the array keeps whatever the last call left.  Nothing has to start at zero here: stage 1 writes every
//    entry [0, rows * chunks) that stage 2 of the same call reads.
//  * the first call on each device looks the array's device address up (cudaGetSymbolAddress).
//  * every call waits for its kernels (it synchronises `stream`), so no call may be made while `stream` is being
//    captured: such a call is refused with CG_ERR_INVALID_ARG and the capture is left intact.
//  * x and out must be device memory of the CURRENT device (checked with cudaPointerGetAttributes, which allocates
//    nothing): the kernels and the scratch follow the current device, and a foreign pointer would fault there.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "../host/c_api_internal.h"
#include "argmax_two_stage.cuh"
#include "elementwise.h"

#define CG_NOALLOC_MAX_PARTIALS 16384

namespace {

// Host code may only use this name to ask the runtime for its device address; kernels get the address as an
// ordinary pointer argument.
static __device__ __align__(256) unsigned long long g_noalloc_partials[CG_NOALLOC_MAX_PARTIALS];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
unsigned long long* g_scratch_ptr[kMaxDevices] = {nullptr};

using cgk::argmax_finish_kernel;
using cgk::argmax_stage1_kernel;
constexpr int kChunk = cgk::ARGMAX_STAGE_CHUNK;

// Device address of the scratch array on the current device, looked up once per device.
unsigned long long* scratch_for_current_device() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) throw cg::Error(cg::ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) throw cg::Error(cg::ERR_INVALID_ARG, "device index above 63");
  std::lock_guard<std::mutex> lk(g_setup_mu);
  if (!g_scratch_ptr[dev]) {
    unsigned long long* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_partials);
    if (e != cudaSuccess || p == nullptr)
      throw cg::Error(cg::ERR_CUDA, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
    g_scratch_ptr[dev] = p;
  }
  return g_scratch_ptr[dev];
}

}  // namespace

extern "C" int cg_argmax_rows_noalloc(const void* x, int dtype, uint64_t rows, uint64_t n, uint64_t row_stride,
                                      uint32_t* out, void* stream) {
  CG_API_BEGIN
  CG_CHECK(x != nullptr && out != nullptr, cg::ERR_INVALID_ARG, "cg_argmax_rows_noalloc: null buffer");
  CG_CHECK(dtype == cgk::DT_F32 || dtype == cgk::DT_BF16 || dtype == cgk::DT_F16, cg::ERR_UNSUPPORTED_DTYPE,
           "cg_argmax_rows_noalloc: dtype must be f32, bf16 or f16");
  CG_CHECK(rows >= 1 && n >= 1 && n <= 0x7fffffffull && row_stride >= n, cg::ERR_INVALID_ARG,
           "cg_argmax_rows_noalloc: need rows >= 1, 1 <= n < 2^31, row_stride >= n");
  const uint64_t chunks = (n + kChunk - 1) / kChunk;
  CG_CHECK(rows <= 65535 && rows * chunks <= CG_NOALLOC_MAX_PARTIALS, cg::ERR_INVALID_ARG,
           "cg_argmax_rows_noalloc: rows * ceil(n / 4096) = " + std::to_string(rows * chunks) +
               " exceeds the fixed scratch of " + std::to_string(CG_NOALLOC_MAX_PARTIALS) +
               " entries; use cg_argmax or split the rows");
  cudaStream_t st = (cudaStream_t)stream;
  {
    // refuse inside a stream capture: the synchronisation below would invalidate the caller's capture
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaError_t ce = cudaStreamIsCapturing(st, &cap);
    if (ce != cudaSuccess) {
      cudaGetLastError();
      throw cg::Error(cg::ERR_INVALID_ARG, std::string("cg_argmax_rows_noalloc: bad stream: ") + cudaGetErrorString(ce));
    }
    CG_CHECK(cap == cudaStreamCaptureStatusNone, cg::ERR_INVALID_ARG,
             "cg_argmax_rows_noalloc: the stream is being captured; this call synchronises and cannot be captured");
    // both buffers must be device memory of the current device
    int dev = -1;
    ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) throw cg::Error(cg::ERR_CUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(ce));
    const void* ptrs[2] = {x, (const void*)out};
    const char* names[2] = {"x", "out"};
    for (int i = 0; i < 2; ++i) {
      cudaPointerAttributes pa;
      ce = cudaPointerGetAttributes(&pa, ptrs[i]);
      if (ce != cudaSuccess) {
        cudaGetLastError();
        throw cg::Error(cg::ERR_INVALID_ARG, std::string("cg_argmax_rows_noalloc: ") + names[i] + " is not a CUDA pointer");
      }
      CG_CHECK((pa.type == cudaMemoryTypeDevice || pa.type == cudaMemoryTypeManaged) && pa.device == dev, cg::ERR_INVALID_ARG,
               std::string("cg_argmax_rows_noalloc: ") + names[i] + " must be device memory of the current device");
    }
  }
  unsigned long long* scratch = scratch_for_current_device();
  dim3 grid((unsigned)chunks, (unsigned)rows);
  switch (dtype) {
    case cgk::DT_F32:
      argmax_stage1_kernel<float><<<grid, 256, 0, st>>>((const float*)x, (long long)row_stride, (int)n, scratch);
      break;
    case cgk::DT_BF16:
      argmax_stage1_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (long long)row_stride,
                                                                     (int)n, scratch);
      break;
    default:
      argmax_stage1_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, (long long)row_stride, (int)n, scratch);
      break;
  }
  argmax_finish_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(scratch, (int)chunks, (int)rows, out);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw cg::Error(cg::ERR_CUDA, std::string("cg_argmax_rows_noalloc launch: ") + cudaGetErrorString(e));
  e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) throw cg::Error(cg::ERR_CUDA, std::string("cg_argmax_rows_noalloc: ") + cudaGetErrorString(e));
  CG_API_END(nullptr)
}

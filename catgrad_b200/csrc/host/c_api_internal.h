// Handle layouts behind the opaque C types (shared by c_api.cc and the CUDA-only entry points).
#pragma once
#include <atomic>
#include <memory>
#include <string>

#include "backend.h"
#include "ir.h"

struct cg_ctx {
  std::unique_ptr<cg::Backend> be;
  std::string last_error;
};
struct cg_tensor {
  std::atomic<int> rc{1};
  cg::Tensor t;
};
struct cg_term {
  cg::Term t;
};
struct cg_builder {
  cg::Builder b;
  std::vector<cg::Var> vars;
};
struct cg_params {
  cg::Parameters p;
};

namespace cg {
// Implemented once per library: the CUDA backend in the product, the CPU restatement in the oracle.
Backend* make_backend(int device);
// Records a failure on the context (or thread-locally when ctx is null) and returns its status.
int record_error(cg_ctx* ctx, int status, const std::string& msg);
}  // namespace cg

// Wraps a C entry point body: exceptions become status codes.
#define CG_API_BEGIN try {
#define CG_API_END(ctx)                                                   \
  return 0;                                                               \
  }                                                                       \
  catch (const cg::Error& e) {                                            \
    return cg::record_error((ctx), (int)e.status, e.what());              \
  }                                                                       \
  catch (const std::bad_alloc&) {                                         \
    return cg::record_error((ctx), (int)cg::ERR_OOM, "host out of memory"); \
  }                                                                       \
  catch (const std::exception& e) {                                       \
    return cg::record_error((ctx), (int)cg::ERR_INVALID_ARG, e.what());   \
  }

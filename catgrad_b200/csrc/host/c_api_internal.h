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
  // Slot for a compiled plan of this term (filled by the CUDA library on the term's first run, freed with the term).
  mutable std::shared_ptr<void> plan;
};
struct cg_builder {
  cg::Builder b;
  std::vector<cg::Var> vars;
};
struct cg_params {
  cg::Parameters p;
  uint64_t version = 0;   // bumped by every cg_params_set: plans built from older contents are rebuilt
};

namespace cg {
// Implemented once per library: the CUDA backend in the product, the CPU restatement in the oracle.
Backend* make_backend(int device);
// Records a failure on the context (or thread-locally when ctx is null) and returns its status.
int record_error(cg_ctx* ctx, int status, const std::string& msg);
// Term -> plan hook of cg_interp_run: when set (the CUDA library sets it) it is offered every run first; it returns
// true after filling `out` if it executed the term as a compiled plan, false to let the op-by-op evaluator run it.
using PlanHook = bool (*)(cg_ctx*, const cg_term*, const cg_params*, std::vector<Value>& in, std::vector<Value>& out);
extern PlanHook g_plan_hook;
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

// extern "C" entry points shared by every Backend implementation (see include/catgrad_b200.h for the
// contract of each).  The exported names are CG_PREFIX + name: `cg_` in the shipped library; the CPU
// oracle used by the tests compiles this same file with another prefix so both libraries can be loaded
// side by side.
#include <cstdio>
#include <cstring>
#include <sstream>

#include "c_api_internal.h"

#ifndef CG_PREFIX
#define CG_PREFIX cg_
#endif
#define CG_CAT2(a, b) a##b
#define CG_CAT(a, b) CG_CAT2(a, b)
#define API(name) CG_CAT(CG_PREFIX, name)

namespace cg {
static thread_local std::string g_last_error;
int record_error(cg_ctx* ctx, int status, const std::string& msg) {
  if (ctx)
    ctx->last_error = msg;
  else
    g_last_error = msg;
  return status;
}

// Default Backend::format_tensor: dtype, shape and the first elements (the reference prints ndarray's
// Debug form, mod.rs:117-125; the exact text is not part of any contract).
std::string Backend::format_tensor(const Tensor& x) {
  // plain snprintf: iostream number formatting goes through locale facets, which crashed when the process had
  // loaded another C++ runtime's copy of them first (numpy does)
  std::string s = std::string(dtype_name(x.dt)) + shape_str(x.shape) + " [";
  int64_t n = x.size();
  std::vector<char> buf((size_t)n * dtype_size(x.dt) + 1);
  to_vec(x, buf.data(), buf.size());
  int64_t shown = n < 16 ? n : 16;
  char num[64];
  for (int64_t i = 0; i < shown; ++i) {
    if (i) s += ", ";
    switch (x.dt) {
      case Dtype::F32: std::snprintf(num, sizeof(num), "%g", (double)((float*)buf.data())[i]); break;
      case Dtype::U32: std::snprintf(num, sizeof(num), "%u", ((uint32_t*)buf.data())[i]); break;
      case Dtype::BF16: {
        uint32_t u = (uint32_t)((uint16_t*)buf.data())[i] << 16;
        float f;
        std::memcpy(&f, &u, 4);
        std::snprintf(num, sizeof(num), "%g", (double)f);
        break;
      }
      case Dtype::F16: std::snprintf(num, sizeof(num), "0x%04x", (unsigned)((uint16_t*)buf.data())[i]); break;
      default: std::snprintf(num, sizeof(num), "0x%02x", (unsigned)((uint8_t*)buf.data())[i]); break;
    }
    s += num;
  }
  if (shown < n) s += ", ...";
  s += "]";
  return s;
}
}  // namespace cg

namespace cg {
PlanHook g_plan_hook = nullptr;
}

using namespace cg;

namespace {
Shape to_shape(const uint64_t* dims, int rank) {
  CG_CHECK(rank >= 0 && rank <= 8, ERR_INVALID_ARG, "rank must be in 0..8");
  Shape s;
  for (int i = 0; i < rank; ++i) s.push_back((int64_t)dims[i]);
  return s;
}
const Tensor& T(const cg_tensor* t) {
  CG_CHECK(t != nullptr && t->rc.load() > 0, ERR_BAD_HANDLE, "null or released tensor handle");
  return t->t;
}
cg_tensor* wrap(Tensor t) {
  cg_tensor* h = new cg_tensor();
  h->t = std::move(t);
  return h;
}
Backend& BE(cg_ctx* c) {
  CG_CHECK(c != nullptr && c->be, ERR_BAD_HANDLE, "null context");
  return *c->be;
}
}  // namespace

extern "C" {

int API(init)(int device, cg_ctx** out) {
  CG_API_BEGIN
  CG_CHECK(out != nullptr, ERR_INVALID_ARG, "out is null");
  std::unique_ptr<cg_ctx> c(new cg_ctx());
  c->be.reset(make_backend(device));
  *out = c.release();
  CG_API_END(nullptr)
}
void API(destroy)(cg_ctx* c) { delete c; }
const char* API(last_error)(cg_ctx* c) { return c ? c->last_error.c_str() : g_last_error.c_str(); }
int API(synchronize)(cg_ctx* c) {
  CG_API_BEGIN
  BE(c).synchronize();
  CG_API_END(c)
}
const char* API(backend_name)(cg_ctx* c) { return (c && c->be) ? c->be->name() : ""; }

void API(retain)(cg_tensor* t) {
  if (t) t->rc.fetch_add(1);
}
void API(release)(cg_tensor* t) {
  if (t && t->rc.fetch_sub(1) == 1) delete t;
}
int API(rank)(const cg_tensor* t) { return t ? t->t.rank() : -1; }
int API(shape)(const cg_tensor* t, uint64_t* dims, int* rank) {
  CG_API_BEGIN
  const Tensor& x = T(t);
  *rank = x.rank();
  for (int i = 0; i < x.rank(); ++i) dims[i] = (uint64_t)x.shape[i];
  CG_API_END(nullptr)
}
int API(dtype_of)(const cg_tensor* t) { return t ? (int)t->t.dt : -1; }
int API(is_contiguous)(const cg_tensor* t) { return t ? (int)t->t.is_contiguous() : 0; }
void* API(data_ptr)(const cg_tensor* t) { return (t && t->t.st) ? t->t.raw() : nullptr; }
int API(strides)(const cg_tensor* t, int64_t* strides, int* rank) {
  CG_API_BEGIN
  const Tensor& x = T(t);
  *rank = x.rank();
  for (int i = 0; i < x.rank(); ++i) strides[i] = x.strides[i];
  CG_API_END(nullptr)
}

int API(zeros)(cg_ctx* c, const uint64_t* dims, int rank, int dtype, cg_tensor** out) {
  CG_API_BEGIN
  CG_CHECK(dtype >= 0 && dtype <= 4, ERR_INVALID_ARG, "bad dtype");
  *out = wrap(BE(c).zeros(to_shape(dims, rank), (Dtype)dtype));
  CG_API_END(c)
}
#define FROM_VEC(name, ctype, DT)                                                                              \
  int API(name)(cg_ctx* c, const ctype* data, uint64_t n, const uint64_t* dims, int rank, cg_tensor** out) {   \
    CG_API_BEGIN                                                                                               \
    *out = wrap(BE(c).from_vec(data, (int64_t)n, to_shape(dims, rank), DT));                                   \
    CG_API_END(c)                                                                                              \
  }
FROM_VEC(from_vec_f32, float, Dtype::F32)
FROM_VEC(from_vec_f16, uint16_t, Dtype::F16)
FROM_VEC(from_vec_bf16, uint16_t, Dtype::BF16)
FROM_VEC(from_vec_fp8, uint8_t, Dtype::F8)
FROM_VEC(from_vec_u32, uint32_t, Dtype::U32)
#undef FROM_VEC

int API(arange)(cg_ctx* c, uint64_t end, cg_tensor** out) {
  CG_API_BEGIN
  *out = wrap(BE(c).arange((int64_t)end));
  CG_API_END(c)
}
int API(cast)(cg_ctx* c, const cg_tensor* x, int target, cg_tensor** out) {
  CG_API_BEGIN
  CG_CHECK(target >= 0 && target <= 4, ERR_INVALID_ARG, "bad dtype");
  *out = wrap(BE(c).cast(T(x), (Dtype)target));
  CG_API_END(c)
}
int API(matmul)(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor** out) {
  CG_API_BEGIN
  *out = wrap(BE(c).matmul(T(a), T(b)));
  CG_API_END(c)
}
#define BINARY(name, OP)                                                                  \
  int API(name)(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, cg_tensor** out) {     \
    CG_API_BEGIN                                                                          \
    *out = wrap(BE(c).binary(OP, T(a), T(b)));                                            \
    CG_API_END(c)                                                                         \
  }
BINARY(add, BinOp::Add)
BINARY(sub, BinOp::Sub)
BINARY(mul, BinOp::Mul)
BINARY(div, BinOp::Div)
BINARY(pow, BinOp::Pow)
BINARY(lt, BinOp::LT)
BINARY(gt, BinOp::GT)
BINARY(gte, BinOp::GTE)
BINARY(lte, BinOp::LTE)
BINARY(eq, BinOp::EQ)
#undef BINARY
int API(where_cond)(cg_ctx* c, const cg_tensor* m, const cg_tensor* x, const cg_tensor* y, cg_tensor** out) {
  CG_API_BEGIN
  *out = wrap(BE(c).where_cond(T(m), T(x), T(y)));
  CG_API_END(c)
}
#define UNARY(name, OP)                                               \
  int API(name)(cg_ctx* c, const cg_tensor* x, cg_tensor** out) {     \
    CG_API_BEGIN                                                      \
    *out = wrap(BE(c).unary(OP, T(x)));                               \
    CG_API_END(c)                                                     \
  }
UNARY(sin, UnOp::Sin)
UNARY(cos, UnOp::Cos)
UNARY(exp, UnOp::Exp)
UNARY(log, UnOp::Log)
UNARY(floor, UnOp::Floor)
UNARY(round, UnOp::Round)
UNARY(neg, UnOp::Neg)
#undef UNARY
int API(broadcast)(cg_ctx* c, const cg_tensor* x, const uint64_t* dims, int rank, cg_tensor** out) {
  CG_API_BEGIN
  *out = wrap(BE(c).broadcast(T(x), to_shape(dims, rank)));
  CG_API_END(c)
}
int API(reshape)(cg_ctx* c, const cg_tensor* x, const uint64_t* dims, int rank, cg_tensor** out) {
  CG_API_BEGIN
  *out = wrap(BE(c).reshape(T(x), to_shape(dims, rank)));
  CG_API_END(c)
}
int API(transpose)(cg_ctx* c, const cg_tensor* x, uint64_t d0, uint64_t d1, cg_tensor** out) {
  CG_API_BEGIN
  *out = wrap(BE(c).transpose(T(x), (int64_t)d0, (int64_t)d1));
  CG_API_END(c)
}
int API(max)(cg_ctx* c, const cg_tensor* x, cg_tensor** out) {
  CG_API_BEGIN
  *out = wrap(BE(c).max(T(x)));
  CG_API_END(c)
}
int API(sum)(cg_ctx* c, const cg_tensor* x, cg_tensor** out) {
  CG_API_BEGIN
  *out = wrap(BE(c).sum(T(x)));
  CG_API_END(c)
}
int API(argmax)(cg_ctx* c, const cg_tensor* x, cg_tensor** out) {
  CG_API_BEGIN
  *out = wrap(BE(c).argmax(T(x)));
  CG_API_END(c)
}
int API(topk)(cg_ctx* c, const cg_tensor* x, uint64_t k, cg_tensor** out_values, cg_tensor** out_indices) {
  CG_API_BEGIN
  auto pr = BE(c).topk(T(x), (int64_t)k);
  *out_values = wrap(pr.first);
  *out_indices = wrap(pr.second);
  CG_API_END(c)
}
int API(compare)(cg_ctx* c, const cg_tensor* a, const cg_tensor* b, int* out_equal) {
  CG_API_BEGIN
  *out_equal = BE(c).compare(T(a), T(b)) ? 1 : 0;
  CG_API_END(c)
}
int API(concat)(cg_ctx* c, const cg_tensor* x, const cg_tensor* y, uint64_t dim, cg_tensor** out) {
  CG_API_BEGIN
  *out = wrap(BE(c).concat(T(x), T(y), (int64_t)dim));
  CG_API_END(c)
}
int API(index)(cg_ctx* c, const cg_tensor* x, uint64_t dim, const cg_tensor* indices, cg_tensor** out) {
  CG_API_BEGIN
  *out = wrap(BE(c).index(T(x), (int64_t)dim, T(indices)));
  CG_API_END(c)
}
int API(slice)(cg_ctx* c, const cg_tensor* x, uint64_t dim, uint64_t start, uint64_t len, cg_tensor** out) {
  CG_API_BEGIN
  *out = wrap(BE(c).slice(T(x), (int64_t)dim, (int64_t)start, (int64_t)len));
  CG_API_END(c)
}
int API(to_bool)(cg_ctx* c, const cg_tensor* x, int* out) {
  CG_API_BEGIN
  *out = BE(c).to_bool(T(x)) ? 1 : 0;
  CG_API_END(c)
}
int API(to_vec)(cg_ctx* c, const cg_tensor* x, void* dst, uint64_t cap_bytes) {
  CG_API_BEGIN
  BE(c).to_vec(T(x), dst, (size_t)cap_bytes);
  CG_API_END(c)
}
int API(format)(cg_ctx* c, const cg_tensor* x, char* buf, uint64_t cap) {
  CG_API_BEGIN
  CG_CHECK(buf && cap > 0, ERR_INVALID_ARG, "empty buffer");
  std::string s = BE(c).format_tensor(T(x));
  std::snprintf(buf, (size_t)cap, "%s", s.c_str());
  CG_API_END(c)
}

// ---- terms ---------------------------------------------------------------------------------
int API(builder_new)(cg_builder** out) {
  CG_API_BEGIN
  *out = new cg_builder();
  CG_API_END(nullptr)
}
void API(builder_free)(cg_builder* b) { delete b; }
int API(builder_source)(cg_builder* b, int node_type, int* out_var) {
  CG_API_BEGIN
  CG_CHECK(b, ERR_BAD_HANDLE, "null builder");
  CG_CHECK(node_type >= 0 && node_type <= 4, ERR_INVALID_ARG, "bad node type");
  b->vars.push_back(b->b.source((NodeType)node_type));
  *out_var = (int)b->vars.size() - 1;
  CG_API_END(nullptr)
}
int API(builder_op)(cg_builder* b, int op_kind, int scalar_op, uint64_t nat, int dtype, float f32, uint32_t u32,
                    const char* str, const cg_term* then_term, const cg_term* else_term, const int* inputs,
                    int n_inputs, const int* output_types, int n_outputs, int* out_vars) {
  CG_API_BEGIN
  CG_CHECK(b, ERR_BAD_HANDLE, "null builder");
  CG_CHECK(op_kind >= 0 && op_kind <= (int)OpKind::Load, ERR_INVALID_ARG, "bad op kind");
  CG_CHECK(scalar_op >= 0 && scalar_op <= (int)ScalarOp::Where, ERR_INVALID_ARG, "bad scalar op");
  CG_CHECK(dtype >= 0 && dtype <= 4, ERR_INVALID_ARG, "bad dtype");
  Operation op;
  op.kind = (OpKind)op_kind;
  op.sop = (ScalarOp)scalar_op;
  op.nat = (int64_t)nat;
  op.dtype = (Dtype)dtype;
  op.f32 = f32;
  op.u32 = u32;
  if (str) op.str = str;
  if (op.kind == OpKind::If) {
    CG_CHECK(then_term && else_term, ERR_INVALID_ARG, "If needs both branch terms");
    op.then_term = std::make_shared<Term>(then_term->t);
    op.else_term = std::make_shared<Term>(else_term->t);
  }
  std::vector<Var> in;
  for (int i = 0; i < n_inputs; ++i) {
    CG_CHECK(inputs[i] >= 0 && inputs[i] < (int)b->vars.size(), ERR_INVALID_ARG, "unknown variable id");
    in.push_back(b->vars[inputs[i]]);
  }
  std::vector<NodeType> out;
  for (int i = 0; i < n_outputs; ++i) {
    CG_CHECK(output_types[i] >= 0 && output_types[i] <= 4, ERR_INVALID_ARG, "bad node type");
    out.push_back((NodeType)output_types[i]);
  }
  auto res = b->b.op(op, in, out);
  for (int i = 0; i < n_outputs; ++i) {
    b->vars.push_back(res[i]);
    out_vars[i] = (int)b->vars.size() - 1;
  }
  CG_API_END(nullptr)
}
int API(builder_finish)(cg_builder* b, const int* targets, int n_targets, cg_term** out) {
  CG_API_BEGIN
  CG_CHECK(b, ERR_BAD_HANDLE, "null builder");
  std::vector<Var> t;
  for (int i = 0; i < n_targets; ++i) {
    CG_CHECK(targets[i] >= 0 && targets[i] < (int)b->vars.size(), ERR_INVALID_ARG, "unknown variable id");
    t.push_back(b->vars[targets[i]]);
  }
  std::unique_ptr<cg_term> term(new cg_term());
  term->t = b->b.finish(t);
  schedule(term->t);
  *out = term.release();
  CG_API_END(nullptr)
}
void API(term_free)(cg_term* t) { delete t; }
int API(term_stats)(const cg_term* t, uint64_t counts[4]) {
  CG_API_BEGIN
  CG_CHECK(t, ERR_BAD_HANDLE, "null term");
  schedule(t->t);
  counts[0] = t->t.nodes.size();
  counts[1] = t->t.edges.size();
  uint64_t n = 0;
  for (auto& e : t->t.edges)
    if (e.op.kind >= OpKind::Map && e.op.kind <= OpKind::Index) n++;
  counts[2] = n;
  counts[3] = t->t.layers.size();
  CG_API_END(nullptr)
}

typedef struct {
  uint64_t hidden_size, intermediate_size, num_hidden_layers, num_attention_heads, num_key_value_heads, vocab_size;
  float rope_theta, rms_norm_eps;
  int tie_word_embeddings;
  int rope_scaling_type;
  float rope_factor, rope_low_freq_factor, rope_high_freq_factor;
  uint64_t rope_original_max_position;
} api_llama_config;

int API(llama_term)(const api_llama_config* cfg, int tap_logits, cg_term** out) {
  CG_API_BEGIN
  CG_CHECK(cfg && out, ERR_INVALID_ARG, "null argument");
  CG_CHECK(cfg->num_attention_heads > 0 && cfg->num_key_value_heads > 0 &&
               cfg->hidden_size % cfg->num_attention_heads == 0 &&
               cfg->num_attention_heads % cfg->num_key_value_heads == 0 && cfg->num_hidden_layers > 0,
           ERR_INVALID_ARG, "inconsistent Llama config");
  LlamaConfig c;
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
  std::unique_ptr<cg_term> term(new cg_term());
  term->t = build_llama_term(c, tap_logits != 0);
  schedule(term->t);
  *out = term.release();
  CG_API_END(nullptr)
}

int API(params_new)(cg_params** out) {
  CG_API_BEGIN
  *out = new cg_params();
  CG_API_END(nullptr)
}
void API(params_free)(cg_params* p) { delete p; }
int API(params_set)(cg_params* p, const char* path, const cg_tensor* t) {
  CG_API_BEGIN
  CG_CHECK(p && path, ERR_BAD_HANDLE, "null argument");
  p->p[path] = T(t);
  ++p->version;
  CG_API_END(nullptr)
}

typedef struct {
  int kind;
  uint64_t nat;
  int dtype;
  uint64_t dims[8];
  int rank;
  cg_tensor* tensor;
} api_value;

int API(interp_run)(cg_ctx* c, const cg_term* term, const cg_params* params, const api_value* inputs, int n_inputs,
                    api_value* outputs, int cap_outputs, int* n_outputs) {
  CG_API_BEGIN
  CG_CHECK(term, ERR_BAD_HANDLE, "null term");
  std::vector<Value> in;
  for (int i = 0; i < n_inputs; ++i) {
    const api_value& v = inputs[i];
    switch (v.kind) {
      case 1: in.push_back(Value::of_nat((int64_t)v.nat)); break;
      case 2: in.push_back(Value::of_dtype((Dtype)v.dtype)); break;
      case 3: in.push_back(Value::of_shape(to_shape(v.dims, v.rank))); break;
      case 4: in.push_back(Value::of_tensor(T(v.tensor))); break;
      default: throw Error(ERR_INVALID_ARG, "bad value kind");
    }
  }
  std::vector<Value> out;
  if (!(g_plan_hook && params && g_plan_hook(c, term, params, in, out))) {
    Interpreter interp(&BE(c), params ? &params->p : nullptr);
    out = interp.run(term->t, std::move(in));
  }
  CG_CHECK((int)out.size() <= cap_outputs, ERR_INVALID_ARG, "output array too small");
  *n_outputs = (int)out.size();
  for (size_t i = 0; i < out.size(); ++i) {
    api_value& v = outputs[i];
    std::memset(&v, 0, sizeof(v));
    v.kind = (int)out[i].kind;
    switch (out[i].kind) {
      case Value::Nat: v.nat = (uint64_t)out[i].nat; break;
      case Value::DtypeV: v.dtype = (int)out[i].dtype; break;
      case Value::ShapeV:
        v.rank = (int)out[i].shape.size();
        for (int d = 0; d < v.rank && d < 8; ++d) v.dims[d] = (uint64_t)out[i].shape[d];
        break;
      case Value::TensorV: v.tensor = wrap(out[i].tensor); break;
      default: break;
    }
  }
  CG_API_END(c)
}

// ---- per-operation counters of the evaluator (interp.cc) ----
void API(op_stats_set_mode)(int mode) { OpStats::set_mode(mode); }
void API(op_stats_reset)(void) { OpStats::reset(); }
int API(op_stats)(char* buf, uint64_t cap, uint64_t* needed) {
  try {
    const std::string js = OpStats::json();
    if (needed) *needed = js.size() + 1;
    if (buf == nullptr || cap < js.size() + 1) return (int)ERR_INVALID_ARG;
    std::memcpy(buf, js.c_str(), js.size() + 1);
    return 0;
  } catch (...) {
    return (int)ERR_INVALID_ARG;
  }
}

}  // extern "C"

// Builder, scheduler and evaluator for the restated core IR (see ir.h).
#include <algorithm>
#include <atomic>
#include <chrono>
#include <mutex>
#include <cstdio>
#include <cstdlib>

#include "ir.h"

namespace cg {

// ---------------------------------------------------------------------------------------------
// Builder
Var Builder::source(NodeType ty) {
  int id = (int)t_.nodes.size();
  t_.nodes.push_back(ty);
  t_.sources.push_back(id);
  return Var{this, id, ty};
}

std::vector<Var> Builder::op(const Operation& op, const std::vector<Var>& in, const std::vector<NodeType>& out) {
  Edge e;
  e.op = op;
  for (auto& v : in) e.sources.push_back(v.id);
  std::vector<Var> res;
  for (auto ty : out) {
    int id = (int)t_.nodes.size();
    t_.nodes.push_back(ty);
    e.targets.push_back(id);
    res.push_back(Var{this, id, ty});
  }
  t_.edges.push_back(std::move(e));
  return res;
}

// Makes the term strict: a node read k>1 times gets one Copy edge with k outputs (the role of
// `cartesian.copy` in the reference, pass/to_core.rs:96), a node never read is left dangling
// (the evaluator drops it at the end of the run).
Term Builder::finish(const std::vector<Var>& targets) {
  Term t = t_;
  for (auto& v : targets) t.targets.push_back(v.id);
  size_t n0 = t.nodes.size();
  std::vector<int> uses(n0, 0);
  for (auto& e : t.edges)
    for (int s : e.sources) uses[s]++;
  for (int s : t.targets) uses[s]++;
  std::vector<std::vector<int>> fresh(n0);
  size_t n_edges0 = t.edges.size();
  for (size_t n = 0; n < n0; ++n) {
    if (uses[n] <= 1) continue;
    Edge c;
    c.op.kind = OpKind::Copy;
    c.sources.push_back((int)n);
    for (int k = 0; k < uses[n]; ++k) {
      int id = (int)t.nodes.size();
      t.nodes.push_back(t.nodes[n]);
      c.targets.push_back(id);
      fresh[n].push_back(id);
    }
    t.edges.push_back(std::move(c));
  }
  std::vector<int> next(n0, 0);
  auto rewire = [&](int& s) {
    if (s < (int)n0 && !fresh[s].empty()) s = fresh[s][next[s]++];
  };
  for (size_t i = 0; i < n_edges0; ++i)
    for (int& s : t.edges[i].sources) rewire(s);
  for (int& s : t.targets) rewire(s);
  return t;
}

// ---------------------------------------------------------------------------------------------
// Layered topological order of edges (the reference gets it from open-hypergraphs'
// `layered_operations`, ssa/mod.rs:42): layer(e) = 1 + max layer over the edges producing e's sources.
void schedule(const Term& t) {
  if (t.scheduled) return;
  std::vector<int> producer(t.nodes.size(), -1);
  for (size_t i = 0; i < t.edges.size(); ++i)
    for (int n : t.edges[i].targets) {
      CG_CHECK(producer[n] == -1, ERR_INTERP, "term is not strict: node written twice");
      producer[n] = (int)i;
    }
  std::vector<int> layer(t.edges.size(), -1);
  // iterative DFS to get layers without assuming edge order
  std::vector<int> state(t.edges.size(), 0);
  for (size_t root = 0; root < t.edges.size(); ++root) {
    if (state[root] == 2) continue;
    std::vector<std::pair<int, size_t>> stack;
    stack.push_back({(int)root, 0});
    state[root] = 1;
    while (!stack.empty()) {
      auto& [e, k] = stack.back();
      if (k < t.edges[e].sources.size()) {
        int p = producer[t.edges[e].sources[k]];
        ++k;
        if (p >= 0 && state[p] != 2) {
          CG_CHECK(state[p] != 1, ERR_INTERP, "term has a cycle");
          state[p] = 1;
          stack.push_back({p, 0});
        }
      } else {
        int l = 0;
        for (int s : t.edges[e].sources) {
          int p = producer[s];
          if (p >= 0) l = std::max(l, layer[p] + 1);
        }
        layer[e] = l;
        state[e] = 2;
        stack.pop_back();
      }
    }
  }
  int nl = 0;
  for (int l : layer) nl = std::max(nl, l + 1);
  t.layers.assign(nl, {});
  for (size_t i = 0; i < t.edges.size(); ++i) t.layers[layer[i]].push_back((int)i);
  t.scheduled = true;
}

// ---------------------------------------------------------------------------------------------
// Evaluator
namespace {
std::string edge_msg(const char* what, int edge_id) { return std::string(what) + " at edge " + std::to_string(edge_id); }

const Tensor& as_tensor(const Value& v, int edge_id) {
  CG_CHECK(v.kind == Value::TensorV, ERR_INTERP, edge_msg("TypeError: expected a tensor", edge_id));
  return v.tensor;
}
int64_t as_nat(const Value& v, int edge_id) {
  CG_CHECK(v.kind == Value::Nat, ERR_INTERP, edge_msg("TypeError: expected a nat", edge_id));
  return v.nat;
}
const Shape& as_shape(const Value& v, int edge_id) {
  CG_CHECK(v.kind == Value::ShapeV, ERR_INTERP, edge_msg("TypeError: expected a shape", edge_id));
  return v.shape;
}
Dtype as_dtype(const Value& v, int edge_id) {
  CG_CHECK(v.kind == Value::DtypeV, ERR_INTERP, edge_msg("TypeError: expected a dtype", edge_id));
  return v.dtype;
}
void arity(const std::vector<Value>& a, size_t n, int edge_id) {
  CG_CHECK(a.size() == n, ERR_INTERP, edge_msg("ArityError", edge_id));
}
}  // namespace

// ---- per-operation counters ----------------------------------------------------------------------
namespace {
std::mutex g_stats_mu;
std::map<std::string, OpStats::Entry> g_stats;
std::atomic<int> g_stats_mode{[] {
  const char* e = std::getenv("CATGRAD_OP_STATS");   // "1" or "sync"
  return e == nullptr ? 0 : (std::string(e) == "sync" || std::string(e) == "2" ? 2 : 1);
}()};
}  // namespace
void OpStats::set_mode(int mode) { g_stats_mode.store(mode < 0 ? 0 : (mode > 2 ? 2 : mode)); }
int OpStats::mode() { return g_stats_mode.load(); }
void OpStats::reset() {
  std::lock_guard<std::mutex> lk(g_stats_mu);
  g_stats.clear();
}
void OpStats::add(const std::string& op, double seconds) {
  std::lock_guard<std::mutex> lk(g_stats_mu);
  Entry& e = g_stats[op];
  e.count += 1;
  e.seconds += seconds;
}
std::string OpStats::json() {
  std::lock_guard<std::mutex> lk(g_stats_mu);
  std::string out = "{";
  bool first = true;
  for (const auto& kv : g_stats) {
    char buf[96];
    std::snprintf(buf, sizeof(buf), "{\"count\": %llu, \"ms\": %.6f}", (unsigned long long)kv.second.count, kv.second.seconds * 1e3);
    out += (first ? "\"" : ", \"") + kv.first + "\": " + buf;
    first = false;
  }
  return out + "}";
}
std::string op_label(const Operation& op) {
  static const char* kinds[] = {"TypePack", "TypeUnpack", "TypeShape", "TypeDtype", "NatConstant", "NatMul", "NatAdd",
                                "DtypeConstant", "Map", "NatToU32", "Cast", "MatMul", "ScalarF32", "ScalarU32", "Sum", "Max",
                                "Argmax", "TopK", "Probe", "Broadcast", "Reshape", "Transpose", "Slice", "Concat", "Arange",
                                "Index", "If", "Copy", "Load"};
  static const char* sops[] = {"Add", "Sub", "Mul", "Div", "Neg", "Pow", "LT", "GT", "GTE", "LTE", "EQ", "Cos", "Sin", "Exp",
                               "Log", "Floor", "Round", "Where"};
  const int k = (int)op.kind;
  if (k < 0 || k >= (int)(sizeof(kinds) / sizeof(kinds[0]))) return "?";
  if (op.kind == OpKind::Map) {
    const int so = (int)op.sop;
    return std::string("Map.") + (so >= 0 && so < (int)(sizeof(sops) / sizeof(sops[0])) ? sops[so] : "?");
  }
  return kinds[k];
}

std::vector<Value> Interpreter::apply(const Edge& e, int id, std::vector<Value>& a) const {
  const Operation& op = e.op;
  auto T = [&](Tensor t) {
    std::vector<Value> r;
    r.push_back(Value::of_tensor(std::move(t)));
    return r;
  };
  // Operands of one Map/MatMul edge must share a dtype (interpreter/tensor_op.rs:254-256).
  auto same_dtype = [&](size_t n) {
    arity(a, n, id);
    Dtype d = as_tensor(a[0], id).dt;
    for (size_t i = 1; i < n; ++i)
      CG_CHECK(as_tensor(a[i], id).dt == d, ERR_DTYPE_MISMATCH, edge_msg("TypeError: operand dtypes differ", id));
  };
  switch (op.kind) {
    case OpKind::TypePack: {
      Shape s;
      for (auto& v : a) s.push_back(as_nat(v, id));
      return {Value::of_shape(std::move(s))};
    }
    case OpKind::TypeUnpack: {
      arity(a, 1, id);
      const Shape& s = as_shape(a[0], id);
      std::vector<Value> r;
      for (auto d : s) r.push_back(Value::of_nat(d));
      return r;
    }
    case OpKind::TypeShape:
      arity(a, 1, id);
      return {Value::of_shape(as_tensor(a[0], id).shape)};
    case OpKind::TypeDtype:
      arity(a, 1, id);
      return {Value::of_dtype(as_tensor(a[0], id).dt)};
    case OpKind::NatConstant:
      arity(a, 0, id);
      return {Value::of_nat(op.nat)};
    case OpKind::NatAdd:
      arity(a, 2, id);
      return {Value::of_nat(as_nat(a[0], id) + as_nat(a[1], id))};
    case OpKind::NatMul:
      arity(a, 2, id);
      return {Value::of_nat(as_nat(a[0], id) * as_nat(a[1], id))};
    case OpKind::DtypeConstant:
      return {Value::of_dtype(op.dtype)};
    case OpKind::Copy: {
      arity(a, 1, id);
      std::vector<Value> r(e.targets.size(), a[0]);
      return r;
    }
    case OpKind::Load: {
      auto it = params_ ? params_->find(op.str) : Parameters::const_iterator();
      CG_CHECK(params_ && it != params_->end(), ERR_INTERP, "Load: no parameter named " + op.str);
      return T(it->second);
    }
    case OpKind::If: {
      CG_CHECK(!a.empty(), ERR_INTERP, edge_msg("ArityError", id));
      bool c = be_->to_bool(as_tensor(a[0], id));
      std::vector<Value> rest(a.begin() + 1, a.end());
      return run(c ? *op.then_term : *op.else_term, std::move(rest));
    }
    default:
      break;
  }
  // tensor ops (interpreter/tensor_op.rs:9-51)
  ++tensor_ops;
  switch (op.kind) {
    case OpKind::Map:
      switch (op.sop) {
        case ScalarOp::Add: same_dtype(2); return T(be_->binary(BinOp::Add, a[0].tensor, a[1].tensor));
        case ScalarOp::Sub: same_dtype(2); return T(be_->binary(BinOp::Sub, a[0].tensor, a[1].tensor));
        case ScalarOp::Mul: same_dtype(2); return T(be_->binary(BinOp::Mul, a[0].tensor, a[1].tensor));
        case ScalarOp::Div: same_dtype(2); return T(be_->binary(BinOp::Div, a[0].tensor, a[1].tensor));
        case ScalarOp::Pow: same_dtype(2); return T(be_->binary(BinOp::Pow, a[0].tensor, a[1].tensor));
        case ScalarOp::LT: same_dtype(2); return T(be_->binary(BinOp::LT, a[0].tensor, a[1].tensor));
        case ScalarOp::GT: same_dtype(2); return T(be_->binary(BinOp::GT, a[0].tensor, a[1].tensor));
        case ScalarOp::GTE: same_dtype(2); return T(be_->binary(BinOp::GTE, a[0].tensor, a[1].tensor));
        case ScalarOp::LTE: same_dtype(2); return T(be_->binary(BinOp::LTE, a[0].tensor, a[1].tensor));
        case ScalarOp::EQ: same_dtype(2); return T(be_->binary(BinOp::EQ, a[0].tensor, a[1].tensor));
        case ScalarOp::Where: same_dtype(3); return T(be_->where_cond(a[0].tensor, a[1].tensor, a[2].tensor));
        case ScalarOp::Neg: arity(a, 1, id); return T(be_->unary(UnOp::Neg, as_tensor(a[0], id)));
        case ScalarOp::Sin: arity(a, 1, id); return T(be_->unary(UnOp::Sin, as_tensor(a[0], id)));
        case ScalarOp::Cos: arity(a, 1, id); return T(be_->unary(UnOp::Cos, as_tensor(a[0], id)));
        case ScalarOp::Exp: arity(a, 1, id); return T(be_->unary(UnOp::Exp, as_tensor(a[0], id)));
        case ScalarOp::Log: arity(a, 1, id); return T(be_->unary(UnOp::Log, as_tensor(a[0], id)));
        case ScalarOp::Floor: arity(a, 1, id); return T(be_->unary(UnOp::Floor, as_tensor(a[0], id)));
        case ScalarOp::Round: arity(a, 1, id); return T(be_->unary(UnOp::Round, as_tensor(a[0], id)));
      }
      break;
    case OpKind::NatToU32: {
      arity(a, 1, id);
      int64_t n = as_nat(a[0], id);
      CG_CHECK(n >= 0 && n <= 0xffffffffLL, ERR_INTERP, edge_msg("ApplyError: nat does not fit u32", id));
      uint32_t v = (uint32_t)n;
      return T(be_->from_vec(&v, 1, {}, Dtype::U32));
    }
    case OpKind::Cast:
      arity(a, 2, id);
      return T(be_->cast(as_tensor(a[0], id), as_dtype(a[1], id)));
    case OpKind::MatMul:
      same_dtype(2);
      return T(be_->matmul(a[0].tensor, a[1].tensor));
    case OpKind::ScalarF32:
      arity(a, 0, id);
      return T(be_->from_vec(&op.f32, 1, {}, Dtype::F32));
    case OpKind::ScalarU32:
      arity(a, 0, id);
      return T(be_->from_vec(&op.u32, 1, {}, Dtype::U32));
    case OpKind::Sum: arity(a, 1, id); return T(be_->sum(as_tensor(a[0], id)));
    case OpKind::Max: arity(a, 1, id); return T(be_->max(as_tensor(a[0], id)));
    case OpKind::Argmax: arity(a, 1, id); return T(be_->argmax(as_tensor(a[0], id)));
    case OpKind::TopK: {
      arity(a, 2, id);
      auto pr = be_->topk(as_tensor(a[0], id), as_nat(a[1], id));
      return {Value::of_tensor(pr.first), Value::of_tensor(pr.second)};
    }
    case OpKind::Probe: {
      // Debug print, only when CATGRAD_PROBE is set (tensor_op.rs:121-136).
      if (std::getenv("CATGRAD_PROBE")) {
        arity(a, 1, id);
        std::printf("[probe:%s] %s\n", op.str.c_str(), be_->format_tensor(as_tensor(a[0], id)).c_str());
        std::fflush(stdout);
      }
      return {};
    }
    case OpKind::Broadcast: arity(a, 2, id); return T(be_->broadcast(as_tensor(a[0], id), as_shape(a[1], id)));
    case OpKind::Reshape: arity(a, 2, id); return T(be_->reshape(as_tensor(a[1], id), as_shape(a[0], id)));
    case OpKind::Transpose:
      arity(a, 3, id);
      return T(be_->transpose(as_tensor(a[0], id), as_nat(a[1], id), as_nat(a[2], id)));
    case OpKind::Slice:
      arity(a, 4, id);
      return T(be_->slice(as_tensor(a[0], id), as_nat(a[1], id), as_nat(a[2], id), as_nat(a[3], id)));
    case OpKind::Concat:
      arity(a, 3, id);
      return T(be_->concat(as_tensor(a[0], id), as_tensor(a[1], id), as_nat(a[2], id)));
    case OpKind::Arange: arity(a, 1, id); return T(be_->arange(as_nat(a[0], id)));
    case OpKind::Index:
      arity(a, 3, id);
      return T(be_->index(as_tensor(a[0], id), as_nat(a[1], id), as_tensor(a[2], id)));
    default:
      break;
  }
  throw Error(ERR_INTERP, edge_msg("unknown operation", id));
}

std::vector<Value> Interpreter::run(const Term& term, std::vector<Value> inputs) const {
  CG_CHECK(inputs.size() == term.sources.size(), ERR_INTERP, "run: wrong number of input values");
  schedule(term);
  std::vector<Value> state(term.nodes.size());
  for (size_t i = 0; i < inputs.size(); ++i) state[term.sources[i]] = std::move(inputs[i]);
  std::vector<Value> args;
  for (auto& layer : term.layers) {
    for (int eid : layer) {
      const Edge& e = term.edges[eid];
      args.clear();
      for (int s : e.sources) {
        // each value is consumed exactly once (eval.rs:41-49)
        CG_CHECK(state[s].kind != Value::None, ERR_INTERP, "MultipleRead of node " + std::to_string(s));
        args.push_back(std::move(state[s]));
        state[s] = Value();
      }
      std::vector<Value> res;
      if (const int stats = OpStats::mode()) {
        const auto t0 = std::chrono::steady_clock::now();
        res = apply(e, eid, args);
        if (stats == 2 && e.op.kind != OpKind::If) be_->synchronize();   // an If is charged to the edges of its branch
        if (e.op.kind != OpKind::If)
          OpStats::add(op_label(e.op), std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
      } else {
        res = apply(e, eid, args);
      }
      CG_CHECK(res.size() == e.targets.size(), ERR_INTERP, edge_msg("ArityError: result count", eid));
      for (size_t i = 0; i < res.size(); ++i) {
        CG_CHECK(state[e.targets[i]].kind == Value::None, ERR_INTERP,
                 "MultipleWrite of node " + std::to_string(e.targets[i]));
        state[e.targets[i]] = std::move(res[i]);
      }
    }
  }
  std::vector<Value> out;
  for (int tnode : term.targets) {
    CG_CHECK(state[tnode].kind != Value::None, ERR_INTERP, "MultipleRead of node " + std::to_string(tnode));
    out.push_back(std::move(state[tnode]));
    state[tnode] = Value();
  }
  return out;
}

// ---------------------------------------------------------------------------------------------
// DSL
namespace dsl {
static Operation mk(OpKind k) {
  Operation o;
  o.kind = k;
  return o;
}
Var nat(Builder& b, int64_t n) {
  Operation o = mk(OpKind::NatConstant);
  o.nat = n;
  return b.op1(o, {}, NodeType::Nat);
}
Var dtype_constant(Builder& b, Dtype d) {
  Operation o = mk(OpKind::DtypeConstant);
  o.dtype = d;
  return b.op1(o, {}, NodeType::Dtype);
}
Var lit_f32(Builder& b, float x) {
  Operation o = mk(OpKind::ScalarF32);
  o.f32 = x;
  return b.op1(o, {}, NodeType::Tensor);
}
Var lit_u32(Builder& b, uint32_t x) {
  Operation o = mk(OpKind::ScalarU32);
  o.u32 = x;
  return b.op1(o, {}, NodeType::Tensor);
}
Var param(Builder& b, const std::string& path) {
  Operation o = mk(OpKind::Load);
  o.str = path;
  return b.op1(o, {}, NodeType::Tensor);
}
Var pack(Builder& b, const std::vector<Var>& extents) { return b.op1(mk(OpKind::TypePack), extents, NodeType::Shape); }
std::vector<Var> unpack(Builder& b, Var shape, int n) {
  return b.op(mk(OpKind::TypeUnpack), {shape}, std::vector<NodeType>(n, NodeType::Nat));
}
Var shape(Builder& b, Var x) { return b.op1(mk(OpKind::TypeShape), {x}, NodeType::Shape); }
Var dtype(Builder& b, Var x) { return b.op1(mk(OpKind::TypeDtype), {x}, NodeType::Dtype); }
Var map1(Builder& b, ScalarOp op, Var x) {
  Operation o = mk(OpKind::Map);
  o.sop = op;
  return b.op1(o, {x}, NodeType::Tensor);
}
Var map2(Builder& b, ScalarOp op, Var x, Var y) {
  Operation o = mk(OpKind::Map);
  o.sop = op;
  return b.op1(o, {x, y}, NodeType::Tensor);
}
Var where_cond(Builder& b, Var mask, Var x, Var y) {
  Operation o = mk(OpKind::Map);
  o.sop = ScalarOp::Where;
  return b.op1(o, {mask, x, y}, NodeType::Tensor);
}
Var broadcast(Builder& b, Var s, Var x) { return b.op1(mk(OpKind::Broadcast), {x, s}, NodeType::Tensor); }
Var reshape(Builder& b, Var s, Var x) { return b.op1(mk(OpKind::Reshape), {s, x}, NodeType::Tensor); }
Var transpose(Builder& b, Var d0, Var d1, Var x) { return b.op1(mk(OpKind::Transpose), {x, d0, d1}, NodeType::Tensor); }
Var index(Builder& b, Var dim, Var idx, Var x) { return b.op1(mk(OpKind::Index), {x, dim, idx}, NodeType::Tensor); }
Var slice(Builder& b, Var dim, Var start, Var len, Var x) {
  return b.op1(mk(OpKind::Slice), {x, dim, start, len}, NodeType::Tensor);
}
Var concat(Builder& b, Var dim, Var x, Var y) { return b.op1(mk(OpKind::Concat), {x, y, dim}, NodeType::Tensor); }
Var arange(Builder& b, Var end) { return b.op1(mk(OpKind::Arange), {end}, NodeType::Tensor); }
Var max(Builder& b, Var x) { return b.op1(mk(OpKind::Max), {x}, NodeType::Tensor); }
Var sum(Builder& b, Var x) { return b.op1(mk(OpKind::Sum), {x}, NodeType::Tensor); }
Var argmax(Builder& b, Var x) { return b.op1(mk(OpKind::Argmax), {x}, NodeType::Tensor); }
std::pair<Var, Var> topk(Builder& b, Var k, Var x) {
  auto r = b.op(mk(OpKind::TopK), {x, k}, {NodeType::Tensor, NodeType::Tensor});
  return {r[0], r[1]};
}
Var nat_to_u32(Builder& b, Var n) { return b.op1(mk(OpKind::NatToU32), {n}, NodeType::Tensor); }
Var matmul(Builder& b, Var f, Var g) { return b.op1(mk(OpKind::MatMul), {f, g}, NodeType::Tensor); }
Var cast(Builder& b, Var x, Var dt) { return b.op1(mk(OpKind::Cast), {x, dt}, NodeType::Tensor); }
Var nat_add(Builder& b, Var x, Var y) { return b.op1(mk(OpKind::NatAdd), {x, y}, NodeType::Nat); }
Var nat_mul(Builder& b, Var x, Var y) { return b.op1(mk(OpKind::NatMul), {x, y}, NodeType::Nat); }
void probe(Builder& b, const std::string& label, Var x) {
  Operation o = mk(OpKind::Probe);
  o.str = label;
  b.op(o, {x}, {});
}
std::vector<Var> cond(Builder& b, Var condition, std::shared_ptr<Term> then_t, std::shared_ptr<Term> else_t,
                      const std::vector<Var>& args, const std::vector<NodeType>& out) {
  Operation o = mk(OpKind::If);
  o.then_term = std::move(then_t);
  o.else_term = std::move(else_t);
  std::vector<Var> in{condition};
  in.insert(in.end(), args.begin(), args.end());
  return b.op(o, in, out);
}

// stdlib/ops.rs:21-30: a literal broadcast to a shape.
Var constant_f32(Builder& b, float x, Var s) { return broadcast(b, s, lit_f32(b, x)); }
Var constant_u32(Builder& b, uint32_t x, Var s) { return broadcast(b, s, lit_u32(b, x)); }
Var inverse(Builder& b, Var x) {
  Var one = constant_f32(b, 1.0f, shape(b, x));
  return map2(b, ScalarOp::Div, one, x);
}

// stdlib/nn/mod.rs:117-122: sqrt(x) = pow(x, 0.5) with the exponent cast to x's dtype.
Var nn_sqrt(Builder& b, Var x) {
  Var e = constant_f32(b, 0.5f, shape(b, x));
  e = cast(b, e, dtype(b, x));
  return map2(b, ScalarOp::Pow, x, e);
}
// nn/mod.rs:124-130: 1 / (1 + exp(-x))
Var nn_sigmoid(Builder& b, Var x) {
  Var one = constant_f32(b, 1.0f, shape(b, x));
  one = cast(b, one, dtype(b, x));
  Var den = map2(b, ScalarOp::Add, one, map1(b, ScalarOp::Exp, map1(b, ScalarOp::Neg, x)));
  return map2(b, ScalarOp::Div, one, den);
}
// nn/mod.rs:132-141: 2*sigmoid(2x) - 1
Var nn_tanh(Builder& b, Var x) {
  Var sh = shape(b, x);
  Var one = constant_f32(b, 1.0f, sh);
  Var two = constant_f32(b, 2.0f, sh);
  Var dt = dtype(b, x);
  one = cast(b, one, dt);
  two = cast(b, two, dt);
  Var s = nn_sigmoid(b, map2(b, ScalarOp::Mul, two, x));
  return map2(b, ScalarOp::Sub, map2(b, ScalarOp::Mul, two, s), one);
}
// nn/mod.rs:143-148: computed in f32, cast back
Var nn_silu(Builder& b, Var x) {
  Var dt = dtype(b, x);
  Var xf = cast(b, x, dtype_constant(b, Dtype::F32));
  Var y = map2(b, ScalarOp::Mul, xf, nn_sigmoid(b, xf));
  return cast(b, y, dt);
}
// nn/mod.rs:150-166: 0.5*x*(1+tanh(sqrt(2/pi)*(x+0.044715*x^3)))
Var nn_gelu(Builder& b, Var x) {
  Var sh = shape(b, x);
  Var dt = dtype(b, x);
  auto c = [&](float v) { return cast(b, constant_f32(b, v, sh), dt); };
  Var cc = c(0.7978845608028654f), one = c(1.0f), three = c(3.0f), half = c(0.5f), k = c(0.044715f);
  Var x3 = map2(b, ScalarOp::Pow, x, three);
  Var inner = map2(b, ScalarOp::Mul, cc, map2(b, ScalarOp::Add, x, map2(b, ScalarOp::Mul, k, x3)));
  Var t = nn_tanh(b, inner);
  return map2(b, ScalarOp::Mul, map2(b, ScalarOp::Mul, half, x), map2(b, ScalarOp::Add, one, t));
}
// nn/mod.rs:168-179
Var nn_softmax(Builder& b, Var x) {
  Var dt = dtype(b, x);
  Var xf = cast(b, x, dtype_constant(b, Dtype::F32));
  Var sh = shape(b, xf);
  Var m = max(b, xf);
  Var xs = map2(b, ScalarOp::Sub, xf, broadcast(b, sh, m));
  Var ex = map1(b, ScalarOp::Exp, xs);
  Var s = sum(b, ex);
  return cast(b, map2(b, ScalarOp::Div, ex, broadcast(b, sh, s)), dt);
}
// nn/mod.rs:182-204: x @ broadcast(transpose(W)) (+ broadcast bias)
Var linear_b_param(Builder& b, int64_t in_dim, int64_t out_dim, Var weight, const Var* bias, Var x) {
  Var wt = transpose(b, nat(b, 0), nat(b, 1), weight);
  auto dims = unpack(b, shape(b, x), 3);
  Var sh = pack(b, {dims[0], nat(b, in_dim), nat(b, out_dim)});
  wt = broadcast(b, sh, wt);
  Var m = matmul(b, x, wt);
  if (bias) {
    Var bb = broadcast(b, shape(b, m), *bias);
    return map2(b, ScalarOp::Add, m, bb);
  }
  return m;
}
Var linear_no_bias(Builder& b, int64_t in_dim, int64_t out_dim, const std::string& path, Var x) {
  Var w = param(b, path + ".weight");
  return linear_b_param(b, in_dim, out_dim, w, nullptr, x);
}
}  // namespace dsl

}  // namespace cg

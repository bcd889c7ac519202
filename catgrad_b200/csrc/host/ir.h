// Core IR restated for the C++ host: the operation set of
// catgrad/src/category/core.rs:104-290 (TensorOp, ScalarOp, NatOp, TypeOp,
// DtypeConstant, If, Copy, Load) over typed hypergraph nodes, plus a small
// builder that plays the role of the reference's `Builder`/`Var` DSL
// (catgrad/src/category/lang/ops.rs:74-428).
//
// A Term here is already "strict": every node is written by exactly one edge
// (or is a term source) and read exactly once, with explicit Copy edges for
// fan-out, which is the form the reference evaluator walks
// (catgrad/src/abstract_interpreter/eval.rs:18-77).
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "backend.h"
#include "tensor.h"

namespace cg {

enum class NodeType : int { Nat = 0, Dtype = 1, NdArrayType = 2, Shape = 3, Tensor = 4 };  // core.rs:84-90

enum class ScalarOp : int {  // core.rs:246-265, same order
  Add, Sub, Mul, Div, Neg, Pow, LT, GT, GTE, LTE, EQ, Cos, Sin, Exp, Log, Floor, Round, Where
};

enum class OpKind : int {
  // Operation::Type
  TypePack = 0, TypeUnpack, TypeShape, TypeDtype,
  // Operation::Nat
  NatConstant, NatMul, NatAdd,
  DtypeConstant,
  // Operation::Tensor
  Map, NatToU32, Cast, MatMul, ScalarF32, ScalarU32, Sum, Max, Argmax, TopK, Probe, Broadcast, Reshape,
  Transpose, Slice, Concat, Arange, Index,
  If, Copy, Load,
};

struct Term;

struct Operation {
  OpKind kind = OpKind::Copy;
  ScalarOp sop = ScalarOp::Add;  // Map
  int64_t nat = 0;               // NatConstant
  Dtype dtype = Dtype::F32;      // DtypeConstant
  float f32 = 0.f;               // ScalarF32
  uint32_t u32 = 0;              // ScalarU32
  std::string str;               // Probe label / Load path ("a.b.c")
  std::shared_ptr<Term> then_term, else_term;  // If
};

struct Edge {
  Operation op;
  std::vector<int> sources, targets;
};

struct Term {
  std::vector<NodeType> nodes;
  std::vector<Edge> edges;
  std::vector<int> sources, targets;
  // Layered topological order of edge ids (catgrad/src/ssa/mod.rs:24-76), computed once and kept:
  // the reference recomputes it on every run.
  mutable std::vector<std::vector<int>> layers;
  mutable bool scheduled = false;
};

// ---- runtime values (catgrad/src/interpreter/types.rs:10-16) --------------------------------
struct Value {
  enum Kind : int { None = 0, Nat = 1, DtypeV = 2, ShapeV = 3, TensorV = 4 } kind = None;
  int64_t nat = 0;
  Dtype dtype = Dtype::F32;
  Shape shape;
  Tensor tensor;
  static Value of_nat(int64_t n) { Value v; v.kind = Nat; v.nat = n; return v; }
  static Value of_dtype(Dtype d) { Value v; v.kind = DtypeV; v.dtype = d; return v; }
  static Value of_shape(Shape s) { Value v; v.kind = ShapeV; v.shape = std::move(s); return v; }
  static Value of_tensor(Tensor t) { Value v; v.kind = TensorV; v.tensor = std::move(t); return v; }
};

using Parameters = std::map<std::string, Tensor>;

// Evaluator (interp.cc).  `Interpreter::run` = catgrad/src/interpreter/interpreter.rs:29-37.
// Per-operation counters of the evaluator (tracing aid; off by default): how many edges of each kind were evaluated and
// the host time spent in them.  Mode 1 times the dispatch only (device work is asynchronous), mode 2 synchronises the
// backend after every edge so that the time is the operation's own.  Process-wide, guarded by a mutex.
struct OpStats {
  struct Entry { uint64_t count = 0; double seconds = 0.0; };
  static void set_mode(int mode);   // 0 off, 1 count + dispatch time, 2 count + synchronised time
  static int mode();
  static void reset();
  static void add(const std::string& op, double seconds);
  static std::string json();        // {"op name": {"count": n, "ms": t}, ...} sorted by name
};
std::string op_label(const Operation& op);   // "MatMul", "Map.Add", "Load", ...

class Interpreter {
 public:
  Interpreter(Backend* be, const Parameters* params) : be_(be), params_(params) {}
  std::vector<Value> run(const Term& term, std::vector<Value> inputs) const;
  // Number of backend tensor-op calls made by the last run (tracing aid).
  mutable int64_t tensor_ops = 0;

 private:
  std::vector<Value> apply(const Edge& e, int edge_id, std::vector<Value>& args) const;
  Backend* be_;
  const Parameters* params_;
};

void schedule(const Term& t);  // fills t.layers

// ---- builder -----------------------------------------------------------------------------------
class Builder;
struct Var {
  Builder* b = nullptr;
  int id = -1;
  NodeType ty = NodeType::Tensor;
};

// Records operations with free fan-out; finish() inserts the Copy edges.
class Builder {
 public:
  Var source(NodeType ty);
  std::vector<Var> op(const Operation& op, const std::vector<Var>& in, const std::vector<NodeType>& out);
  Var op1(const Operation& op, const std::vector<Var>& in, NodeType out) { return this->op(op, in, {out})[0]; }
  Term finish(const std::vector<Var>& targets);

 private:
  Term t_;
};

// DSL functions with the argument orders of lang/ops.rs (the edge's source order is what
// interpreter/tensor_op.rs unpacks: Broadcast[x,shape], Reshape[shape,x], Index[x,dim,idx], ...).
namespace dsl {
Var nat(Builder& b, int64_t n);
Var dtype_constant(Builder& b, Dtype d);
Var lit_f32(Builder& b, float x);
Var lit_u32(Builder& b, uint32_t x);
Var param(Builder& b, const std::string& path);
Var pack(Builder& b, const std::vector<Var>& extents);
std::vector<Var> unpack(Builder& b, Var shape, int n);
Var shape(Builder& b, Var x);
Var dtype(Builder& b, Var x);
Var map1(Builder& b, ScalarOp op, Var x);
Var map2(Builder& b, ScalarOp op, Var x, Var y);
Var where_cond(Builder& b, Var mask, Var x, Var y);
Var broadcast(Builder& b, Var s, Var x);
Var reshape(Builder& b, Var s, Var x);
Var transpose(Builder& b, Var d0, Var d1, Var x);
Var index(Builder& b, Var dim, Var idx, Var x);
Var slice(Builder& b, Var dim, Var start, Var len, Var x);
Var concat(Builder& b, Var dim, Var x, Var y);
Var arange(Builder& b, Var end);
Var max(Builder& b, Var x);
Var sum(Builder& b, Var x);
Var argmax(Builder& b, Var x);
std::pair<Var, Var> topk(Builder& b, Var k, Var x);
Var nat_to_u32(Builder& b, Var n);
Var matmul(Builder& b, Var f, Var g);
Var cast(Builder& b, Var x, Var dtype);
Var nat_add(Builder& b, Var x, Var y);
Var nat_mul(Builder& b, Var x, Var y);
void probe(Builder& b, const std::string& label, Var x);
std::vector<Var> cond(Builder& b, Var condition, std::shared_ptr<Term> then_t, std::shared_ptr<Term> else_t,
                      const std::vector<Var>& args, const std::vector<NodeType>& out);
// stdlib/ops.rs:21-30
Var constant_f32(Builder& b, float x, Var shape);
Var constant_u32(Builder& b, uint32_t x, Var shape);
Var inverse(Builder& b, Var x);
// stdlib/nn/mod.rs
Var nn_sqrt(Builder& b, Var x);
Var nn_sigmoid(Builder& b, Var x);
Var nn_tanh(Builder& b, Var x);
Var nn_silu(Builder& b, Var x);
Var nn_gelu(Builder& b, Var x);
Var nn_softmax(Builder& b, Var x);
Var linear_b_param(Builder& b, int64_t in_dim, int64_t out_dim, Var weight, const Var* bias, Var x);
Var linear_no_bias(Builder& b, int64_t in_dim, int64_t out_dim, const std::string& path, Var x);
}  // namespace dsl

// ---- Llama term (llama_term.cc) --------------------------------------------------------------
// Field names follow `LlamaConfig` (catgrad-llm-models/src/models/llama.rs:9-27).
struct LlamaConfig {
  int64_t hidden_size = 0, intermediate_size = 0, num_hidden_layers = 0, num_attention_heads = 0,
          num_key_value_heads = 0, vocab_size = 0;
  float rope_theta = 10000.f;
  float rms_norm_eps = 1e-5f;
  int tie_word_embeddings = 0;
  // rope_scaling (config.rs:10-18; helpers/rope.rs:14-60): 0 = absent (default tables), 1 = "llama3"
  int rope_scaling_type = 0;
  float rope_factor = 1.f, rope_low_freq_factor = 1.f, rope_high_freq_factor = 1.f;
  int64_t rope_original_max_position = 0;
  int64_t head_dim() const { return hidden_size / num_attention_heads; }  // llama.rs:54-56
};

// Sources: x [B,S] u32, in_k, in_v [L,B,Hkv,T,D], max_positions Nat.  Targets: ids [B,S,1] u32, out_k, out_v
// (llama.rs:393-401).  With tap_logits a 4th target carries the lm_head output the argmax consumed.
Term build_llama_term(const LlamaConfig& cfg, bool tap_logits);

}  // namespace cg

// The Llama term, restated op for op from the reference graph builders:
//   catgrad-llm-models/src/models/llama.rs:144-385   (forward, attention, mlp, layer)
//   catgrad-llm-models/src/helpers/tensors.rs        (embeddings, rmsnorm, causal_mask, repeat_kv, squeeze)
//   catgrad-llm-models/src/helpers/cache.rs:13-103   (functional KV cache, Cache::init)
//   catgrad-llm-models/src/helpers/rope.rs:14-60,65-104,232-314,423-451 (table choice, default and llama3 RoPE tables,
//                                                     rotate_half, apply)
// Every helper expands inline into primitive edges, as in the reference (no Definition edges).
// Parameter keys are the safetensors names (`model.layers.0.self_attn.q_proj.weight`, ...), i.e.
// what `to_load_ops` leaves after stripping the `llama.` prefix (stdlib_definitions.rs:43-54).
#include <cmath>
#include <limits>

#include "ir.h"

namespace cg {
namespace {
using namespace dsl;

struct G {
  Builder& b;
  const LlamaConfig& cfg;
  Var F32() { return dtype_constant(b, Dtype::F32); }
  Var N(int64_t n) { return nat(b, n); }
  Var add(Var x, Var y) { return map2(b, ScalarOp::Add, x, y); }
  Var mul(Var x, Var y) { return map2(b, ScalarOp::Mul, x, y); }
  Var div(Var x, Var y) { return map2(b, ScalarOp::Div, x, y); }
  Var sub(Var x, Var y) { return map2(b, ScalarOp::Sub, x, y); }
  Var neg(Var x) { return map1(b, ScalarOp::Neg, x); }

  // tensors.rs:27-45 (squeeze / unsqueeze via reshape)
  Var squeeze(int n, int dim, Var x) {
    auto s = unpack(b, shape(b, x), n);
    s.erase(s.begin() + dim);
    return reshape(b, pack(b, s), x);
  }
  Var unsqueeze(int n, int dim, Var x) {
    auto s = unpack(b, shape(b, x), n);
    s.insert(s.begin() + dim, N(1));
    return reshape(b, pack(b, s), x);
  }

  // tensors.rs:255-272
  Var embeddings(const std::string& p, Var x) {
    Var wte = param(b, p + ".weight");
    auto bs = unpack(b, shape(b, x), 2);
    Var flat = reshape(b, pack(b, {nat_mul(b, bs[0], bs[1])}), x);
    auto vh = unpack(b, shape(b, wte), 2);
    Var te = index(b, N(0), flat, wte);
    return reshape(b, pack(b, {bs[0], bs[1], vh[1]}), te);
  }

  // tensors.rs:207-224
  Var causal_mask(Var seq_len, Var pos) {
    Var size = nat_add(b, seq_len, pos);
    Var i = arange(b, size);
    Var sh = pack(b, {size, size});
    i = broadcast(b, sh, i);
    Var shr = pack(b, {size, N(1)});
    Var j = arange(b, size);
    j = reshape(b, shr, j);
    j = broadcast(b, sh, j);
    Var mask = map2(b, ScalarOp::LT, j, i);
    mask = cast(b, mask, F32());
    Var ninf = constant_f32(b, std::numeric_limits<float>::lowest(), sh);  // f32::MIN
    mask = mul(mask, ninf);
    return slice(b, N(0), pos, seq_len, mask);
  }

  // tensors.rs:82-111
  Var rmsnorm_raw(float eps, Var x) {
    Var x_dtype = dtype(b, x);
    Var x_shape = shape(b, x);
    auto u = unpack(b, x_shape, 3);
    Var n = u[2];
    Var xf = cast(b, x, F32());
    Var s = sum(b, mul(xf, xf));
    Var constn = nat_to_u32(b, n);
    constn = cast(b, constn, F32());
    constn = broadcast(b, shape(b, s), constn);
    Var mean = div(s, constn);
    Var epsilon = constant_f32(b, eps, shape(b, mean));
    epsilon = cast(b, epsilon, F32());
    Var rms = nn_sqrt(b, add(mean, epsilon));
    Var denom = broadcast(b, x_shape, rms);
    return cast(b, div(xf, denom), x_dtype);
  }
  Var rmsnorm(float eps, const std::string& p, Var x) {
    Var gamma = param(b, p + ".weight");
    Var lr = rmsnorm_raw(eps, x);
    gamma = broadcast(b, shape(b, lr), gamma);
    return mul(lr, gamma);
  }

  // tensors.rs:128-151
  Var repeat_kv(int64_t rep, Var x) {
    const int dim = 1;
    x = unsqueeze(4, dim + 1, x);
    auto sh = unpack(b, shape(b, x), 5);
    sh[dim + 1] = N(rep);
    Var orig = sh[dim];
    x = broadcast(b, pack(b, sh), x);
    sh.erase(sh.begin() + dim + 1);
    sh[dim] = nat_mul(b, orig, N(rep));
    return reshape(b, pack(b, sh), x);
  }

  // rope.rs:65-104
  std::pair<Var, Var> rope_tables_default(float theta, Var seq_len, int64_t head_dim, float factor) {
    int64_t half = head_dim / 2;
    Var f = arange(b, N(half));
    f = cast(b, f, F32());
    Var sh = shape(b, f);
    Var two = constant_f32(b, 2.0f / (float)head_dim, sh);
    f = mul(f, two);
    Var th = constant_f32(b, theta, sh);
    Var freq = map2(b, ScalarOp::Pow, th, f);
    Var inv_freq = inverse(b, freq);
    Var sh2 = pack(b, {seq_len, N(half)});
    inv_freq = broadcast(b, sh2, inv_freq);
    Var fac = constant_f32(b, factor, sh2);
    inv_freq = div(inv_freq, fac);
    Var pos = arange(b, seq_len);
    pos = cast(b, pos, F32());
    pos = reshape(b, pack(b, {seq_len, N(1)}), pos);
    pos = broadcast(b, shape(b, inv_freq), pos);
    pos = mul(pos, inv_freq);
    Var c = map1(b, ScalarOp::Cos, pos);
    Var s = map1(b, ScalarOp::Sin, pos);
    c = concat(b, N(1), c, c);
    s = concat(b, N(1), s, s);
    return {c, s};
  }

  // rope.rs:232-314: the "llama3" frequency rescaling (long wavelengths divided by `factor`, a smooth blend in between)
  std::pair<Var, Var> rope_tables_llama3(float theta, Var seq_len, int64_t head_dim) {
    int64_t half = head_dim / 2;
    Var f = arange(b, N(half));
    f = cast(b, f, F32());
    Var sh = shape(b, f);
    Var two = constant_f32(b, 2.0f / (float)head_dim, sh);
    f = mul(f, two);
    Var th = constant_f32(b, theta, sh);
    Var freq = map2(b, ScalarOp::Pow, th, f);
    Var inv_freq = inverse(b, freq);
    const float orig = (float)cfg.rope_original_max_position;
    sh = shape(b, inv_freq);
    Var low_wl = constant_f32(b, orig / cfg.rope_low_freq_factor, sh);
    Var high_wl = constant_f32(b, orig / cfg.rope_high_freq_factor, sh);
    Var factor = constant_f32(b, cfg.rope_factor, sh);
    Var low_ff = constant_f32(b, cfg.rope_low_freq_factor, sh);
    Var high_ff = constant_f32(b, cfg.rope_high_freq_factor, sh);
    Var old_len = constant_f32(b, orig, sh);
    Var pi_2 = constant_f32(b, 2.0f * 3.14159265358979323846f, sh);
    Var wavelen = div(pi_2, inv_freq);
    Var low_mask = cast(b, map2(b, ScalarOp::LT, low_wl, wavelen), F32());
    Var one = constant_f32(b, 1.0f, sh);
    Var scaled = div(inv_freq, factor);
    inv_freq = add(mul(low_mask, scaled), mul(sub(one, low_mask), inv_freq));
    Var high_mask = cast(b, map2(b, ScalarOp::LT, wavelen, high_wl), F32());
    Var not_high = sub(one, high_mask);
    Var not_low = sub(one, low_mask);
    Var mid_mask = mul(not_high, not_low);
    Var smooth = div(sub(div(old_len, wavelen), low_ff), sub(high_ff, low_ff));
    Var smoothed = add(mul(smooth, inv_freq), div(mul(sub(one, smooth), inv_freq), factor));
    inv_freq = add(mul(mid_mask, smoothed), mul(sub(one, mid_mask), inv_freq));
    Var sh2 = pack(b, {seq_len, N(half)});
    inv_freq = broadcast(b, sh2, inv_freq);
    Var pos = arange(b, seq_len);
    pos = cast(b, pos, F32());
    pos = reshape(b, pack(b, {seq_len, N(1)}), pos);
    pos = broadcast(b, shape(b, inv_freq), pos);
    pos = mul(pos, inv_freq);
    Var c = map1(b, ScalarOp::Cos, pos);
    Var s = map1(b, ScalarOp::Sin, pos);
    c = concat(b, N(1), c, c);
    s = concat(b, N(1), s, s);
    return {c, s};
  }

  // rope.rs:423-427 (chunk = two slices, tensors.rs:5-13)
  Var rotate_half(int64_t head_dim, Var x) {
    Var v0 = slice(b, N(3), N(0), N(head_dim / 2), x);
    Var v1 = slice(b, N(3), N(head_dim / 2), N(head_dim / 2), x);
    return concat(b, N(3), neg(v1), v0);
  }
  // rope.rs:430-451
  Var apply_rope_embedding(Var pos, int64_t head_dim, Var cos_t, Var sin_t, Var x) {
    Var sh = shape(b, x);
    auto d = unpack(b, sh, 4);
    Var seq_len = d[2];
    Var c = slice(b, N(0), pos, seq_len, cos_t);
    Var s = slice(b, N(0), pos, seq_len, sin_t);
    c = broadcast(b, sh, c);
    s = broadcast(b, sh, s);
    Var x_dtype = dtype(b, x);
    Var xf = cast(b, x, F32());
    Var rot = rotate_half(head_dim, xf);
    return cast(b, add(mul(c, xf), mul(s, rot)), x_dtype);
  }

  // cache.rs:13-75
  std::vector<std::pair<Var, Var>> kv;
  void kv_init(Var in_k, Var in_v) {
    for (int64_t l = 0; l < cfg.num_hidden_layers; ++l) {
      Var k = slice(b, N(0), N(l), N(1), in_k);
      Var v = slice(b, N(0), N(l), N(1), in_v);
      kv.push_back({squeeze(5, 0, k), squeeze(5, 0, v)});
    }
  }
  std::pair<Var, Var> kv_update(int64_t l, Var k, Var v) {
    Var nk = concat(b, N(2), kv[l].first, k);
    Var nv = concat(b, N(2), kv[l].second, v);
    kv[l] = {nk, nv};
    return kv[l];
  }
  std::pair<Var, Var> kv_output() {
    Var out_k = unsqueeze(4, 0, kv[0].first);
    Var out_v = unsqueeze(4, 0, kv[0].second);
    for (size_t l = 1; l < kv.size(); ++l) {
      Var k = unsqueeze(4, 0, kv[l].first);
      Var v = unsqueeze(4, 0, kv[l].second);
      out_k = concat(b, N(0), out_k, k);
      out_v = concat(b, N(0), out_v, v);
    }
    return {out_k, out_v};
  }

  // llama.rs:230-253
  Var mlp(const std::string& p, Var x) {
    Var gate = linear_no_bias(b, cfg.hidden_size, cfg.intermediate_size, p + ".gate_proj", x);
    Var up = linear_no_bias(b, cfg.hidden_size, cfg.intermediate_size, p + ".up_proj", x);
    Var h = mul(nn_silu(b, gate), up);
    return linear_no_bias(b, cfg.intermediate_size, cfg.hidden_size, p + ".down_proj", h);
  }

  // llama.rs:255-347
  Var attention(int64_t layer_id, Var attention_mask, Var cos_t, Var sin_t, Var pos, const std::string& p, Var x) {
    int64_t dim = cfg.hidden_size, nh = cfg.num_attention_heads, hd = cfg.head_dim(), nkv = cfg.num_key_value_heads;
    int64_t rep = nh / nkv;
    auto bs = unpack(b, shape(b, x), 3);
    Var B = bs[0], S = bs[1];
    Var q = linear_no_bias(b, dim, dim, p + ".q_proj", x);
    Var k = linear_no_bias(b, dim, dim / rep, p + ".k_proj", x);
    Var v = linear_no_bias(b, dim, dim / rep, p + ".v_proj", x);
    q = reshape(b, pack(b, {B, S, N(nh), N(hd)}), q);
    Var shkv = pack(b, {B, S, N(nkv), N(hd)});
    k = reshape(b, shkv, k);
    v = reshape(b, shkv, v);
    q = transpose(b, N(1), N(2), q);
    k = transpose(b, N(1), N(2), k);
    v = transpose(b, N(1), N(2), v);
    q = apply_rope_embedding(pos, hd, cos_t, sin_t, q);
    k = apply_rope_embedding(pos, hd, cos_t, sin_t, k);
    auto kvp = kv_update(layer_id, k, v);
    k = repeat_kv(rep, kvp.first);
    v = repeat_kv(rep, kvp.second);
    Var tk = transpose(b, N(2), N(3), k);
    Var attn = matmul(b, q, tk);
    Var sh = shape(b, attn);
    Var denom = constant_f32(b, std::sqrt((float)hd), sh);
    denom = cast(b, denom, dtype(b, attn));
    attn = div(attn, denom);
    Var m = cast(b, attention_mask, dtype(b, attn));
    m = broadcast(b, sh, m);
    attn = add(attn, m);
    attn = nn_softmax(b, attn);
    attn = matmul(b, attn, v);
    attn = transpose(b, N(1), N(2), attn);
    attn = reshape(b, pack(b, {B, S, N(dim)}), attn);
    return linear_no_bias(b, dim, dim, p + ".o_proj", attn);
  }

  // llama.rs:349-385
  Var layer(int64_t layer_id, Var mask, Var cos_t, Var sin_t, Var pos, const std::string& p, Var x) {
    Var res = x;
    Var h = rmsnorm(cfg.rms_norm_eps, p + ".input_layernorm", x);
    h = attention(layer_id, mask, cos_t, sin_t, pos, p + ".self_attn", h);
    h = add(res, h);
    res = h;
    Var y = rmsnorm(cfg.rms_norm_eps, p + ".post_attention_layernorm", h);
    y = mlp(p + ".mlp", y);
    return add(y, res);
  }
};
}  // namespace

Term build_llama_term(const LlamaConfig& cfg, bool tap_logits) {
  Builder b;
  Var x = b.source(NodeType::Tensor);
  Var in_k = b.source(NodeType::Tensor);
  Var in_v = b.source(NodeType::Tensor);
  Var max_positions = b.source(NodeType::Nat);
  G g{b, cfg};
  const std::string root = "model";
  // forward (llama.rs:144-164)
  Var h = g.embeddings(root + ".embed_tokens", x);
  auto bsd = unpack(b, shape(b, h), 3);
  auto kd = unpack(b, shape(b, in_k), 5);
  Var mask = g.causal_mask(bsd[1], kd[3]);
  // forward_embeddings (llama.rs:166-228): Cache::init = RoPE tables + per-layer KV slices
  // init_rope_tables (rope.rs:8-60): llama3 scaling when the config carries it, else the default tables
  auto tables = cfg.rope_scaling_type == 1 ? g.rope_tables_llama3(cfg.rope_theta, max_positions, cfg.head_dim())
                                           : g.rope_tables_default(cfg.rope_theta, max_positions, cfg.head_dim(), 1.0f);
  g.kv_init(in_k, in_v);
  auto kd2 = unpack(b, shape(b, in_k), 5);
  Var pos = kd2[3];
  for (int64_t i = 0; i < cfg.num_hidden_layers; ++i)
    h = g.layer(i, mask, tables.first, tables.second, pos, root + ".layers." + std::to_string(i), h);
  h = g.rmsnorm(cfg.rms_norm_eps, root + ".norm", h);
  std::string head = cfg.tie_word_embeddings ? root + ".embed_tokens" : std::string("lm_head");
  Var logits = linear_no_bias(b, cfg.hidden_size, cfg.vocab_size, head, h);
  Var ids = argmax(b, logits);
  auto out = g.kv_output();
  std::vector<Var> targets{ids, out.first, out.second};
  if (tap_logits) targets.push_back(logits);
  return b.finish(targets);
}

}  // namespace cg

// cg_runner_*: the batch-sharded multi-GPU runner behind the C ABI.
//
// The reference has no multi-device path (its runner is one device, batch 1: examples/llama/main.rs:947-951), but its
// Llama term is batch-polymorphic (llama.rs:159,271), so independent sequences can be split over GPUs without any
// exchange: one context, one weight replica and one fused Llama runner per device, each driven by its own host thread
// (a context is used by one thread at a time), and one gather of the generated ids on the host at the end.  This is
// the in-process alternative to one process per GPU (bench.py under torch.distributed.run does the same split with
// processes).
#include <algorithm>
#include <string>
#include <thread>
#include <vector>

#include "c_api_internal.h"

extern "C" {
typedef struct cg_llama cg_llama;
typedef struct {
  uint64_t hidden_size, intermediate_size, num_hidden_layers, num_attention_heads, num_key_value_heads, vocab_size;
  float rope_theta, rms_norm_eps;
  int tie_word_embeddings;
  int rope_scaling_type;
  float rope_factor, rope_low_freq_factor, rope_high_freq_factor;
  uint64_t rope_original_max_position;
} runner_llama_config;
int cg_init(int device, cg_ctx** out);
void cg_destroy(cg_ctx* c);
const char* cg_last_error(cg_ctx* c);
int cg_llama_create(cg_ctx* ctx, const runner_llama_config* cfg, int dtype, const cg_params* params, uint64_t max_batch,
                    uint64_t max_positions, cg_llama** out);
void cg_llama_free(cg_llama* m);
int cg_llama_reset(cg_llama* m, uint64_t batch);
int cg_llama_forward(cg_llama* m, const uint32_t* ids, uint64_t batch, uint64_t seq, uint32_t* out_ids);
int cg_llama_decode(cg_llama* m, uint64_t steps, uint32_t* out_ids);
}

struct cg_runner {
  struct Replica {
    cg_ctx* ctx = nullptr;
    cg_llama* model = nullptr;
  };
  std::vector<Replica> reps;
  runner_llama_config cfg;
  int dtype = 0;
  uint64_t max_batch = 0, max_positions = 0;
  std::string last_error;
  ~cg_runner() {
    for (auto& r : reps) {
      if (r.model) cg_llama_free(r.model);
      if (r.ctx) cg_destroy(r.ctx);
    }
  }
};

namespace {
// Contiguous share [lo, hi) of replica r; the first n % parts replicas hold one extra sequence.
void shard_range(uint64_t n, uint64_t parts, uint64_t r, uint64_t& lo, uint64_t& hi) {
  const uint64_t base = n / parts, extra = n % parts;
  lo = r * base + std::min(r, extra);
  hi = lo + base + (r < extra ? 1 : 0);
}
}  // namespace

extern "C" {

int cg_runner_create(const int* devices, int n_devices, const runner_llama_config* cfg, int dtype, uint64_t max_batch_per_device,
                     uint64_t max_positions, cg_runner** out) {
  CG_API_BEGIN
  CG_CHECK(devices && cfg && out && n_devices >= 1 && n_devices <= 64, cg::ERR_INVALID_ARG, "cg_runner_create: bad arguments");
  std::unique_ptr<cg_runner> r(new cg_runner());
  r->cfg = *cfg;
  r->dtype = dtype;
  r->max_batch = max_batch_per_device;
  r->max_positions = max_positions;
  for (int i = 0; i < n_devices; ++i) {
    cg_runner::Replica rep;
    int st = cg_init(devices[i], &rep.ctx);
    if (st != 0) throw cg::Error((cg::Status)st, std::string("cg_runner_create: device ") + std::to_string(devices[i]) + ": " + cg_last_error(nullptr));
    r->reps.push_back(rep);
  }
  *out = r.release();
  CG_API_END(nullptr)
}

int cg_runner_size(const cg_runner* r) { return r ? (int)r->reps.size() : 0; }
cg_ctx* cg_runner_ctx(cg_runner* r, int i) { return (r && i >= 0 && i < (int)r->reps.size()) ? r->reps[i].ctx : nullptr; }
const char* cg_runner_last_error(const cg_runner* r) { return r ? r->last_error.c_str() : ""; }

int cg_runner_set_params(cg_runner* r, int i, const cg_params* params) {
  CG_API_BEGIN
  CG_CHECK(r && params && i >= 0 && i < (int)r->reps.size(), cg::ERR_INVALID_ARG, "cg_runner_set_params: bad arguments");
  cg_runner::Replica& rep = r->reps[i];
  if (rep.model) {
    cg_llama_free(rep.model);
    rep.model = nullptr;
  }
  int st = cg_llama_create(rep.ctx, &r->cfg, r->dtype, params, r->max_batch, r->max_positions, &rep.model);
  if (st != 0) throw cg::Error((cg::Status)st, std::string("cg_runner_set_params: ") + cg_last_error(rep.ctx));
  CG_API_END(nullptr)
}

int cg_runner_generate(cg_runner* r, const uint32_t* prompts, uint64_t n_seq, uint64_t prompt_len, uint64_t steps, uint32_t* out_ids) {
  CG_API_BEGIN
  CG_CHECK(r && prompts && out_ids && n_seq >= 1 && prompt_len >= 1 && steps >= 1, cg::ERR_INVALID_ARG, "cg_runner_generate: bad arguments");
  const uint64_t parts = r->reps.size();
  for (auto& rep : r->reps) CG_CHECK(rep.model != nullptr, cg::ERR_INVALID_ARG, "cg_runner_generate: a replica has no parameters yet");
  CG_CHECK((n_seq + parts - 1) / parts <= r->max_batch, cg::ERR_INVALID_ARG, "cg_runner_generate: more sequences per device than max_batch_per_device");
  std::vector<int> status(parts, 0);
  std::vector<std::string> message(parts);
  std::vector<std::thread> threads;
  for (uint64_t p = 0; p < parts; ++p) {
    threads.emplace_back([&, p] {
      uint64_t lo, hi;
      shard_range(n_seq, parts, p, lo, hi);
      const uint64_t b = hi - lo;
      if (b == 0) return;
      cg_runner::Replica& rep = r->reps[p];
      std::vector<uint32_t> first(b), rest((size_t)b * (steps - 1));
      int st = cg_llama_reset(rep.model, b);
      if (st == 0) st = cg_llama_forward(rep.model, prompts + lo * prompt_len, b, prompt_len, first.data());
      if (st == 0 && steps > 1) st = cg_llama_decode(rep.model, steps - 1, rest.data());
      if (st != 0) {
        status[p] = st;
        message[p] = cg_last_error(rep.ctx);
        return;
      }
      // the one gather of this workload: this replica's rows of the [n_seq, steps] result
      for (uint64_t i = 0; i < b; ++i) {
        uint32_t* row = out_ids + (lo + i) * steps;
        row[0] = first[i];
        for (uint64_t s = 1; s < steps; ++s) row[s] = rest[(size_t)i * (steps - 1) + (s - 1)];
      }
    });
  }
  for (auto& t : threads) t.join();
  for (uint64_t p = 0; p < parts; ++p) {
    if (status[p] != 0) {
      r->last_error = "replica " + std::to_string(p) + ": " + message[p];
      throw cg::Error((cg::Status)status[p], r->last_error);
    }
  }
  CG_API_END(nullptr)
}

void cg_runner_free(cg_runner* r) { delete r; }

}  // extern "C"

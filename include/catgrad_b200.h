/* catgrad_b200 — C ABI of the B200 tensor backend for catgrad's interpreter.
 *
 * One entry point per method of `trait Backend`
 * (catgrad/src/interpreter/backend/mod.rs:24-122), with the trait's names, so that a Rust shim
 * `impl Backend for B200Backend` is a table of one-line FFI calls.  Conventions of the trait are kept
 * (mod.rs:18-23): the operands of one op share a dtype, nothing broadcasts implicitly, reductions keep
 * the rank.  Where the reference panics (ndarray.rs:27,34,365,444,485,530; candle.rs:1272-1274) or
 * returns BackendError::ShapeError (mod.rs:129-132), these functions return a status and leave a
 * message in cg_last_error(); nothing traps on the device.
 *
 * Plain pointers and sizes only.  Tensors are opaque reference-counted handles; every function that
 * returns a tensor returns a NEW handle the caller releases with cg_release().  Inputs are never
 * mutated and are not consumed (a Rust shim releases its `TaggedTensor` arguments when they drop).
 *
 * One cg_ctx = one device + one stream, used from one thread at a time.  Only cg_to_vec, cg_to_bool,
 * cg_compare, cg_format and cg_synchronize wait for the device.
 */
#ifndef CATGRAD_B200_H
#define CATGRAD_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cg_ctx cg_ctx;
typedef struct cg_tensor cg_tensor;
typedef struct cg_term cg_term;
typedef struct cg_builder cg_builder;
typedef struct cg_params cg_params;
typedef struct cg_llama cg_llama;

/* enum Dtype, catgrad/src/category/core.rs:23-29 (same order) */
typedef enum { CG_F32 = 0, CG_F16 = 1, CG_BF16 = 2, CG_F8E4M3 = 3, CG_U32 = 4 } cg_dtype;

typedef enum {
  CG_OK = 0,
  CG_ERR_SHAPE_MISMATCH = 1,    /* "Shape mismatch in operation" (candle.rs:1272-1274) */
  CG_ERR_DTYPE_MISMATCH = 2,    /* InterpreterError::TypeError (tensor_op.rs:254-256) */
  CG_ERR_UNSUPPORTED_DTYPE = 3, /* e.g. sin of a u32 tensor (ndarray.rs:361-367) */
  CG_ERR_OOM = 4,
  CG_ERR_CUDA = 5,
  CG_ERR_TIMEOUT = 6,
  CG_ERR_BAD_HANDLE = 7,
  CG_ERR_SHAPE = 8,             /* BackendError::ShapeError (mod.rs:129-132) */
  CG_ERR_INVALID_ARG = 9,
  CG_ERR_INTERP = 10            /* InterpreterError::{ArityError,MultipleRead,MultipleWrite,Load,...} */
} cg_status;

#define CG_MAX_RANK 8

/* ---- context ------------------------------------------------------------------------------ */
/* Creates a context on CUDA device `device` (replaces `CandleBackend::new_accel`/`NdArrayBackend`,
 * examples/llama/main.rs:199-210).  Fails with CG_ERR_CUDA when no device is usable: there is no
 * CPU fallback. */
cg_status cg_init(int device, cg_ctx** out);
void cg_destroy(cg_ctx* ctx);
/* Message of the last failing call on this context (or, with ctx == NULL, of the last failing call
 * that had no context).  Valid until the next call on the same context/thread. */
const char* cg_last_error(cg_ctx* ctx);
cg_status cg_synchronize(cg_ctx* ctx);
/* Name of the implementation behind the handle ("b200"). */
const char* cg_backend_name(cg_ctx* ctx);

/* ---- tensor handles (BackendTensorOps::shape, mod.rs:124-126; TaggedTensor::dtype, types.rs:18-60) */
void cg_retain(cg_tensor* t);
void cg_release(cg_tensor* t);
int cg_rank(const cg_tensor* t);
cg_status cg_shape(const cg_tensor* t, uint64_t* dims /* CG_MAX_RANK */, int* rank);
cg_dtype cg_dtype_of(const cg_tensor* t);
/* 1 if the handle is a contiguous row-major buffer (views made by transpose/slice/broadcast are not) */
int cg_is_contiguous(const cg_tensor* t);
/* Device address of element 0 and strides in elements (for zero-copy interop; not part of the trait). */
void* cg_data_ptr(const cg_tensor* t);
cg_status cg_strides(const cg_tensor* t, int64_t* strides /* CG_MAX_RANK */, int* rank);

/* ---- constructors (mod.rs:28-58) ---------------------------------------------------------- */
cg_status cg_zeros(cg_ctx*, const uint64_t* dims, int rank, cg_dtype dtype, cg_tensor** out);
/* `data` is host memory, n elements; n != product(dims) -> CG_ERR_SHAPE (BackendError::ShapeError) */
cg_status cg_from_vec_f32(cg_ctx*, const float* data, uint64_t n, const uint64_t* dims, int rank, cg_tensor** out);
cg_status cg_from_vec_f16(cg_ctx*, const uint16_t* data, uint64_t n, const uint64_t* dims, int rank, cg_tensor** out);
cg_status cg_from_vec_bf16(cg_ctx*, const uint16_t* data, uint64_t n, const uint64_t* dims, int rank, cg_tensor** out);
cg_status cg_from_vec_fp8(cg_ctx*, const uint8_t* data, uint64_t n, const uint64_t* dims, int rank, cg_tensor** out);
cg_status cg_from_vec_u32(cg_ctx*, const uint32_t* data, uint64_t n, const uint64_t* dims, int rank, cg_tensor** out);
cg_status cg_arange(cg_ctx*, uint64_t end, cg_tensor** out);                  /* mod.rs:111 */

/* ---- ops (mod.rs:60-110) ------------------------------------------------------------------- */
cg_status cg_cast(cg_ctx*, const cg_tensor* x, cg_dtype target, cg_tensor** out);
cg_status cg_matmul(cg_ctx*, const cg_tensor* lhs, const cg_tensor* rhs, cg_tensor** out);
cg_status cg_add(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
cg_status cg_sub(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
cg_status cg_mul(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
cg_status cg_div(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
cg_status cg_pow(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
cg_status cg_lt(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
cg_status cg_gt(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
cg_status cg_gte(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
cg_status cg_lte(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
cg_status cg_eq(cg_ctx*, const cg_tensor* a, const cg_tensor* b, cg_tensor** out);
cg_status cg_where_cond(cg_ctx*, const cg_tensor* mask, const cg_tensor* x, const cg_tensor* y, cg_tensor** out);
cg_status cg_sin(cg_ctx*, const cg_tensor* x, cg_tensor** out);
cg_status cg_cos(cg_ctx*, const cg_tensor* x, cg_tensor** out);
cg_status cg_exp(cg_ctx*, const cg_tensor* x, cg_tensor** out);
cg_status cg_log(cg_ctx*, const cg_tensor* x, cg_tensor** out);
cg_status cg_floor(cg_ctx*, const cg_tensor* x, cg_tensor** out);
cg_status cg_round(cg_ctx*, const cg_tensor* x, cg_tensor** out);
cg_status cg_neg(cg_ctx*, const cg_tensor* x, cg_tensor** out);
cg_status cg_broadcast(cg_ctx*, const cg_tensor* x, const uint64_t* dims, int rank, cg_tensor** out);
cg_status cg_reshape(cg_ctx*, const cg_tensor* x, const uint64_t* dims, int rank, cg_tensor** out);
cg_status cg_transpose(cg_ctx*, const cg_tensor* x, uint64_t dim0, uint64_t dim1, cg_tensor** out);
cg_status cg_max(cg_ctx*, const cg_tensor* x, cg_tensor** out);
cg_status cg_sum(cg_ctx*, const cg_tensor* x, cg_tensor** out);
cg_status cg_argmax(cg_ctx*, const cg_tensor* x, cg_tensor** out);
cg_status cg_topk(cg_ctx*, const cg_tensor* x, uint64_t k, cg_tensor** out_values, cg_tensor** out_indices);
cg_status cg_compare(cg_ctx*, const cg_tensor* a, const cg_tensor* b, int* out_equal);
cg_status cg_concat(cg_ctx*, const cg_tensor* x, const cg_tensor* y, uint64_t dim, cg_tensor** out);
cg_status cg_index(cg_ctx*, const cg_tensor* x, uint64_t dim, const cg_tensor* indices, cg_tensor** out);
cg_status cg_slice(cg_ctx*, const cg_tensor* x, uint64_t dim, uint64_t start, uint64_t len, cg_tensor** out);
cg_status cg_to_bool(cg_ctx*, const cg_tensor* x, int* out);                  /* mod.rs:113 */
/* Row-major contents to host memory, element type = the tensor's dtype (mod.rs:115, TaggedVec). */
cg_status cg_to_vec(cg_ctx*, const cg_tensor* x, void* dst, uint64_t cap_bytes);
/* Backend::format_tensor (mod.rs:117-125); writes a NUL-terminated string, truncated to cap. */
cg_status cg_format(cg_ctx*, const cg_tensor* x, char* buf, uint64_t cap);

/* ---- terms and the interpreter ------------------------------------------------------------
 * A restatement of catgrad's core IR (category/core.rs:104-290) and of the evaluator
 * (abstract_interpreter/eval.rs:18-187; interpreter/interpreter.rs:29-108; tensor_op.rs:9-275).
 * Node types and op kinds are the integer values of `cg::NodeType` / `cg::OpKind` / `cg::ScalarOp`
 * (catgrad_b200/csrc/host/ir.h), mirrored in catgrad_b200/ir.py. */
cg_status cg_builder_new(cg_builder** out);
void cg_builder_free(cg_builder* b);
/* Adds a term input of node type `node_type`; returns its variable id in *out_var. */
cg_status cg_builder_source(cg_builder* b, int node_type, int* out_var);
/* Adds one operation.  `str` is the Probe label or the Load path ("a.b.c"); then_term/else_term are
 * used by If (core.rs:112) and copied.  Variables may be used any number of times: the Copy edges the
 * evaluator needs are inserted by cg_builder_finish. */
cg_status cg_builder_op(cg_builder* b, int op_kind, int scalar_op, uint64_t nat, int dtype, float f32, uint32_t u32,
                        const char* str, const cg_term* then_term, const cg_term* else_term, const int* inputs,
                        int n_inputs, const int* output_types, int n_outputs, int* out_vars);
cg_status cg_builder_finish(cg_builder* b, const int* targets, int n_targets, cg_term** out);
void cg_term_free(cg_term* t);
/* counts[0..3] = nodes, edges, tensor-op edges, layers of the parallel SSA order (ssa/mod.rs:24-76) */
cg_status cg_term_stats(const cg_term* t, uint64_t counts[4]);

/* LlamaConfig (catgrad-llm-models/src/models/llama.rs:9-27), fields the Llama term reads; rope_scaling
 * (config.rs:10-18) selects the RoPE table builder as helpers/rope.rs:8-60 does: absent -> rope_tables_default,
 * "llama3" -> rope_tables_llama3 (rope.rs:232-310).  Yarn and longrope are not implemented: a config that
 * carries them must not be passed with rope_scaling_type 0. */
typedef struct {
  uint64_t hidden_size, intermediate_size, num_hidden_layers, num_attention_heads, num_key_value_heads, vocab_size;
  float rope_theta, rms_norm_eps;
  int tie_word_embeddings;
  int rope_scaling_type;                 /* 0: no rope_scaling block; 1: "llama3" */
  float rope_factor, rope_low_freq_factor, rope_high_freq_factor;
  uint64_t rope_original_max_position;   /* original_max_position_embeddings of the scaling block */
} cg_llama_config;
/* The term of LlamaModel::def (llama.rs:393-401): inputs x [B,S] u32, in_k, in_v [L,B,Hkv,T,D],
 * max_positions (nat); outputs ids [B,S,1] u32, out_k, out_v [L,B,Hkv,T+S,D].  tap_logits != 0 adds the
 * lm_head output as a 4th output. */
cg_status cg_llama_term(const cg_llama_config* cfg, int tap_logits, cg_term** out);

/* Parameters<B> (interpreter/parameters.rs): path -> tensor; Load(path) clones the handle. */
cg_status cg_params_new(cg_params** out);
void cg_params_free(cg_params* p);
cg_status cg_params_set(cg_params* p, const char* path, const cg_tensor* t);

/* Value<B> (interpreter/types.rs:10-16) crossing the ABI. */
typedef enum { CG_VALUE_NAT = 1, CG_VALUE_DTYPE = 2, CG_VALUE_SHAPE = 3, CG_VALUE_TENSOR = 4 } cg_value_kind;
typedef struct {
  int kind;              /* cg_value_kind */
  uint64_t nat;          /* CG_VALUE_NAT */
  int dtype;             /* CG_VALUE_DTYPE */
  uint64_t dims[CG_MAX_RANK];
  int rank;              /* CG_VALUE_SHAPE */
  cg_tensor* tensor;     /* CG_VALUE_TENSOR; outputs are new handles */
} cg_value;
/* Interpreter::run (interpreter.rs:33-36).  The schedule of a term is computed on its first run and
 * kept with the term. */
cg_status cg_interp_run(cg_ctx*, const cg_term* term, const cg_params* params, const cg_value* inputs, int n_inputs,
                        cg_value* outputs, int cap_outputs, int* n_outputs);

/* Term -> plan (B200 only).  cg_interp_run offers every term to a recogniser first: a term that is, edge for edge, the
 * Llama term of llama.rs:144-401 for the configuration its parameters and constants imply runs as the fused plan
 * below instead of one kernel per edge, with the KV cache kept in the runner's device buffers: the out_k / out_v values
 * are strided views of them, recognised by their storage when the caller threads them back in (helpers/cache.rs:13-75),
 * so nothing is copied or re-stacked; they stay valid until the term is run again with an empty cache.  Any other term
 * (one edge of difference is enough), or a cache that is not the runner's own, is evaluated op by op.
 * cg_term_plan_state: 0 not run yet, 1 runs as the fused plan, 2 runs op by op. */
int cg_term_plan_state(const cg_term* t);
/* Process-wide switch of the recogniser (on by default). */
void cg_interp_set_planning(int on);

/* ---- fused Llama runner (B200 only; not part of the trait) ---------------------------------
 * Executes the Llama term above as a fixed plan of fused kernels with a device-resident KV cache
 * instead of one kernel per IR edge.  It replaces the per-token `run_interpreter` loop of
 * examples/llama/main.rs:876-1043 (generate_stream): same inputs (token ids), same outputs (greedy ids),
 * with the rounding points of the term kept (bf16 at every op output the graph types as bf16). */
/* Parameters are looked up by their safetensors names (llama.rs Load paths).  dtype: CG_F32 or CG_BF16. */
cg_status cg_llama_create(cg_ctx*, const cg_llama_config* cfg, cg_dtype dtype, const cg_params* params,
                          uint64_t max_batch, uint64_t max_positions, cg_llama** out);
void cg_llama_free(cg_llama* m);

/* ---- tensor parallelism (B200 only; the reference has no multi-GPU path) ---------------------
 * One process per GPU.  Every rank creates a communicator (a symmetric device buffer), the ranks exchange the
 * 64-byte handles over any host channel and attach; after that the all-reduce is a single kernel per call that
 * sums over plain peer loads (NVLink), in rank order with f32 accumulation, so every rank holds bit-identical
 * results.  Device-side waits are bounded (5 s): a rank that never arrives turns into CG_ERR_TIMEOUT at the next
 * synchronising call, and the communicator stays unusable after that. */
typedef struct cg_comm cg_comm;
cg_status cg_comm_create(cg_ctx*, int rank, int size, uint64_t data_bytes, cg_comm** out);
cg_status cg_comm_handle(cg_comm*, void* out64);
cg_status cg_comm_attach(cg_comm*, const void* handles /* size x 64 bytes, rank order */);
/* Same-process alternative to cg_comm_attach (one process driving several GPUs, where IPC handles cannot be used):
 * `all` = the communicators of all ranks in rank order. */
cg_status cg_comm_attach_local(cg_comm*, cg_comm* const* all);
/* Limit of the device-side waits (default 5000 ms). */
cg_status cg_comm_set_timeout_ms(cg_comm*, uint64_t ms);
cg_status cg_comm_data(cg_comm*, void** device_ptr, uint64_t* bytes);
/* Host <-> data area copies at byte offset `off` (both synchronise the context's stream). */
cg_status cg_comm_write(cg_comm*, uint64_t off, const void* src, uint64_t bytes);
cg_status cg_comm_read(cg_comm*, uint64_t off, void* dst, uint64_t bytes);
/* x (+)= sum over ranks of part; x_off/part_off are byte offsets into the data area (same on every rank),
 * n elements of dtype CG_F32 or CG_BF16.  residual != 0: x = round(x + round(sum)); else x = round(sum). */
cg_status cg_comm_allreduce(cg_comm*, cg_dtype dtype, uint64_t x_off, uint64_t part_off, uint64_t n, int residual);
void cg_comm_free(cg_comm*);
/* Tensor-parallel fused runner: `cfg` is the unsharded model, `params` holds this rank's shard (rows
 * [r*n/size, (r+1)*n/size) of q/k/v/gate/up_proj, the same range of columns of o/down_proj, everything else
 * whole).  The partial products of o_proj and down_proj are all-reduced into the residual stream (llama.rs:303-385
 * with the projections split over heads / FFN columns).  The communicator's data area must hold
 * 2 x align256(max_tokens x hidden x element size) bytes; max_tokens bounds batch x seq of any forward call. */
cg_status cg_llama_create_tp(cg_ctx*, const cg_llama_config* cfg, cg_dtype dtype, const cg_params* params,
                             uint64_t max_batch, uint64_t max_positions, cg_comm* comm, uint64_t max_tokens,
                             cg_llama** out);
/* Clears the KV cache (context length 0) for a new batch of `batch` sequences. */
cg_status cg_llama_reset(cg_llama* m, uint64_t batch);
/* Runs one step of the term on `ids` (host memory, [batch, seq] u32, row-major) at the current context
 * length, appends K/V to the cache, and leaves the greedy id of the LAST position of every sequence on
 * the device (the element the reference runner reads, main.rs:1031-1037).  With out_ids != NULL they are
 * also copied to host ([batch] u32), which synchronises. */
cg_status cg_llama_forward(cg_llama* m, const uint32_t* ids, uint64_t batch, uint64_t seq, uint32_t* out_ids);
/* `steps` greedy decode steps, each consuming the ids the previous step left on the device (no host
 * round trip per token; EOS is ignored as in the reference's --bench loop, main.rs:919).  Writes
 * [batch, steps] u32 to out_ids (host) at the end. */
cg_status cg_llama_decode(cg_llama* m, uint64_t steps, uint32_t* out_ids);
/* Copies the logits of the last forward/decode step ([batch, vocab], last position only) to host as f32. */
cg_status cg_llama_last_logits(cg_llama* m, float* dst, uint64_t cap_elems);
/* Decode steps of small batches can run as ONE persistent kernel (weights streamed through shared memory by an
 * asynchronous-copy warp, grid barriers between the sub-graphs) instead of a captured graph of one kernel per
 * sub-graph.  on != 0 allows it where the shape permits (bf16, no tensor parallelism); on == 0 forces the
 * kernel-per-sub-graph plan.  Both keep the term's results within the bf16 tolerance of each other. */
cg_status cg_llama_set_persistent(cg_llama* m, int on);
/* 1 if the most recent decode step ran as the persistent kernel. */
int cg_llama_persistent_active(const cg_llama* m);
/* Current context length T. */
uint64_t cg_llama_context_len(const cg_llama* m);
/* Number of kernel launches issued by this runner since creation (graph replays count their nodes). */
uint64_t cg_llama_launch_count(const cg_llama* m);

/* ---- batch-sharded multi-GPU runner (B200 only; the reference runs one device, batch 1: main.rs:947-951) -----
 * One process drives several GPUs: a context, a weight replica and a fused Llama runner per device, each on its own
 * host thread; independent sequences are split into contiguous shares (the first n % devices shares hold one more),
 * there is no exchange while generating, and the ids are gathered on the host at the end.  Legal because the Llama
 * term is batch-polymorphic (llama.rs:159,271).  Usage: create, upload each replica's parameters through
 * cg_runner_ctx(r, i) (cg_from_vec_* / cg_params_set), cg_runner_set_params(r, i, params), then generate. */
typedef struct cg_runner cg_runner;
cg_status cg_runner_create(const int* devices, int n_devices, const cg_llama_config* cfg, cg_dtype dtype,
                           uint64_t max_batch_per_device, uint64_t max_positions, cg_runner** out);
int cg_runner_size(const cg_runner* r);
cg_ctx* cg_runner_ctx(cg_runner* r, int i);
cg_status cg_runner_set_params(cg_runner* r, int i, const cg_params* params);
/* prompts [n_seq, prompt_len] u32 (host) -> out_ids [n_seq, steps] u32 (host): the greedy ids generate_stream
 * (main.rs:876-1043) would produce for each sequence on its own, EOS ignored. */
cg_status cg_runner_generate(cg_runner* r, const uint32_t* prompts, uint64_t n_seq, uint64_t prompt_len, uint64_t steps,
                             uint32_t* out_ids);
const char* cg_runner_last_error(const cg_runner* r);
void cg_runner_free(cg_runner* r);

/* ---- per-operation counters of cg_interp_run (tracing aid, off by default; the reference has Probe and wall clocks only:
 * tensor_op.rs:121-136, main.rs:914-917) ------------------------------------------------------------------------------
 * mode 0 off, 1 count every evaluated edge by operation and time its dispatch on the host, 2 also synchronise after every
 * edge so that the time is the operation's own (slow).  The environment variable CATGRAD_OP_STATS=1|sync sets the
 * initial mode.  Process-wide.  cg_op_stats writes a JSON object {"MatMul": {"count": n, "ms": t}, "Map.Add": ...};
 * `needed` receives the size to pass when `cap` was too small (CG_ERR_INVALID_ARG).  A term that runs as the fused plan
 * evaluates no edges and leaves the counters untouched. */
void cg_op_stats_set_mode(int mode);
void cg_op_stats_reset(void);
cg_status cg_op_stats(char* buf, uint64_t cap, uint64_t* needed);

/* ---- timing and allocator introspection ---------------------------------------------------- */
/* CUDA events on the context's stream (the stream every kernel of this library is launched on). */
cg_status cg_event_record(cg_ctx*, int slot /* 0..63 */);
cg_status cg_event_elapsed_ms(cg_ctx*, int slot_start, int slot_end, float* out_ms);
/* bytes currently handed out / cached by the context's caching allocator, and launch counter */
cg_status cg_ctx_stats(cg_ctx*, uint64_t stats[4] /* live bytes, cached bytes, cudaMalloc calls, kernel launches */);
/* Synthetic weights without a host copy (for models too large to draw on the host): a new [rows, cols] tensor
 * holding rows [row0, row0+rows) x columns [col0, col0+cols) of a virtual [*, full_cols] matrix of N(0, std)
 * values determined by `seed` alone, so shards of one matrix can be made independently.  No reference counterpart. */
cg_status cg_random_normal(cg_ctx*, uint64_t seed, float std, uint64_t rows, uint64_t cols, uint64_t row0,
                           uint64_t col0, uint64_t full_cols, cg_dtype dtype, cg_tensor** out);

/* Fused softmax over the last axis: what the graph of stdlib nn::softmax (nn/mod.rs:168-179: cast f32, x - max,
 * exp, / sum, cast back) computes, in one kernel.  Not a trait method; a plan compiler would substitute it. */
cg_status cg_softmax(cg_ctx*, const cg_tensor* x, cg_tensor** out);

/* Writes `bytes` of device memory on the context's stream (used by benchmarks to evict L2). */
cg_status cg_flush_l2(cg_ctx*, uint64_t bytes);

/* ---- allocation-free entry point ------------------------------------------------------------
 * No counterpart in the reference (its backends allocate freely; argmax there is mod.rs:85).
 * Last-axis argmax of `rows` rows of `n` elements (row r starts at x + r * row_stride elements; dtype CG_F32,
 * CG_BF16 or CG_F16), same result as cg_argmax: the u32 index of the LAST maximum under f32::total_cmp.
 * For callers that cannot allocate device memory: x and out ([rows] u32) are caller-owned device buffers on the
 * CURRENT device, `stream` is a cudaStream_t (NULL = default stream), and the only scratch is a fixed 128 KiB
 * array inside the library.  Limits: rows <= 65535 and rows * ceil(n / 4096) <= 16384, otherwise
 * CG_ERR_INVALID_ARG.  The call returns after the kernels have finished (it synchronises `stream`) and calls no
 * cudaMalloc/cudaFree.  All calls on one GPU share the scratch: do not let two of them overlap on the device.
 * The first call on each device looks up the scratch address.  Because every call synchronises `stream`, a call on
 * a stream that is being captured is refused (CG_ERR_INVALID_ARG, the capture stays valid); so is a buffer that is
 * not device memory of the current device. */
cg_status cg_argmax_rows_noalloc(const void* x, cg_dtype dtype, uint64_t rows, uint64_t n, uint64_t row_stride,
                                 uint32_t* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif

"""Llama on the B200 backend: config, seeded synthetic weights, and the two ways to generate.

* `generate_with_interpreter` is the reference's loop (`generate_stream` + `run_interpreter`,
  catgrad-llm/examples/llama/main.rs:876-1043): the Llama term is evaluated edge by edge through the
  `Backend` entry points, the KV cache is a value threaded from step to step.
* `LlamaRunner` drives the fused plan (`cg_llama_*`): the same term executed as a fixed list of fused
  kernels with a device-resident KV cache and on-device greedy feedback.

Real checkpoints are not needed anywhere: weights are N(0, 0.02) from a seeded numpy PCG64 stream (norm
gains are 1.0), token ids are uniform.
"""
import ctypes as C
import dataclasses

import numpy as np

from . import _ffi
from .backend import Backend, BackendError, Dtype, Status, Tensor, f32_to_bf16_bits
from .ir import Interpreter, Parameters, Term


@dataclasses.dataclass
class LlamaConfig:
    """Fields of `LlamaConfig` the term reads (catgrad-llm-models/src/models/llama.rs:9-27)."""
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    vocab_size: int
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    tie_word_embeddings: bool = False
    # rope_scaling block of config.json (config.rs:10-18): None, or a dict with rope_type "llama3", factor,
    # low_freq_factor, high_freq_factor, original_max_position_embeddings (Llama-3.1 / 3.2 checkpoints carry it)
    rope_scaling: dict = None

    @property
    def head_dim(self):
        return self.hidden_size // self.num_attention_heads

    @classmethod
    def from_hf_config(cls, config):
        """From a checkpoint's config.json (a path or the parsed dict), the fields the reference deserialises for Llama
        (catgrad-llm-models/src/models/llama.rs:9-27, config.rs:10-49).  Features of that struct the Llama term here does
        not implement are refused rather than ignored: NoPE layer intervals, partial rotary factors other than 1,
        yarn / longrope scaling, quantised checkpoints."""
        import json
        if not isinstance(config, dict):
            with open(config) as f:
                config = json.load(f)
        if config.get("no_rope_layer_interval", 0):
            raise ValueError("no_rope_layer_interval is not implemented")
        if float(config.get("partial_rotary_factor", 1.0)) != 1.0:
            raise ValueError("partial_rotary_factor other than 1.0 is not implemented")
        if config.get("quantization_config"):
            raise ValueError("quantised checkpoints are not implemented")
        scaling = config.get("rope_scaling")
        if scaling is not None:
            kind = scaling.get("rope_type", scaling.get("type"))
            if kind != "llama3":
                raise ValueError(f"rope_scaling type {kind!r} is not implemented (only 'llama3')")
            scaling = {k: scaling[k] for k in ("factor", "low_freq_factor", "high_freq_factor",
                                               "original_max_position_embeddings")}
            scaling["rope_type"] = "llama3"
        heads = int(config["num_attention_heads"])
        cfg = cls(hidden_size=int(config["hidden_size"]), intermediate_size=int(config["intermediate_size"]),
                  num_hidden_layers=int(config["num_hidden_layers"]), num_attention_heads=heads,
                  num_key_value_heads=int(config.get("num_key_value_heads", heads)), vocab_size=int(config["vocab_size"]),
                  rope_theta=float(config.get("rope_theta", 10000.0)), rms_norm_eps=float(config["rms_norm_eps"]),
                  tie_word_embeddings=bool(config.get("tie_word_embeddings", False)), rope_scaling=scaling)
        if "head_dim" in config and int(config["head_dim"]) != cfg.head_dim:
            raise ValueError("head_dim other than hidden_size / num_attention_heads is not implemented")
        return cfg

    def to_struct(self):
        rs = self.rope_scaling
        if rs is None:
            scaling = (0, 1.0, 1.0, 1.0, 0)
        else:
            kind = rs.get("rope_type", rs.get("type"))
            if kind != "llama3":
                raise ValueError(f"rope_scaling type {kind!r} is not implemented (only 'llama3'; helpers/rope.rs:14-60 also "
                                 "knows yarn and longrope)")
            scaling = (1, float(rs["factor"]), float(rs["low_freq_factor"]), float(rs["high_freq_factor"]),
                       int(rs["original_max_position_embeddings"]))
        return _ffi.LlamaConfigStruct(self.hidden_size, self.intermediate_size, self.num_hidden_layers,
                                      self.num_attention_heads, self.num_key_value_heads, self.vocab_size,
                                      self.rope_theta, self.rms_norm_eps, int(self.tie_word_embeddings), *scaling)

    def param_shapes(self):
        """Parameter keys (HF layout [out, in]) in the order the weights are drawn."""
        h, f, v = self.hidden_size, self.intermediate_size, self.vocab_size
        kv = self.num_key_value_heads * self.head_dim
        out = [("model.embed_tokens.weight", (v, h))]
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            out += [(p + "input_layernorm.weight", (h,)),
                    (p + "self_attn.q_proj.weight", (h, h)),
                    (p + "self_attn.k_proj.weight", (kv, h)),
                    (p + "self_attn.v_proj.weight", (kv, h)),
                    (p + "self_attn.o_proj.weight", (h, h)),
                    (p + "post_attention_layernorm.weight", (h,)),
                    (p + "mlp.gate_proj.weight", (f, h)),
                    (p + "mlp.up_proj.weight", (f, h)),
                    (p + "mlp.down_proj.weight", (h, f))]
        out.append(("model.norm.weight", (h,)))
        if not self.tie_word_embeddings:
            out.append(("lm_head.weight", (v, h)))
        return out

    def num_params(self):
        return sum(int(np.prod(s)) for _, s in self.param_shapes())


# The model shapes of the benchmark configurations: the tiny f32 model, Llama-3.2-1B and Llama-3-8B.
TINY = LlamaConfig(256, 688, 2, 4, 4, 1024, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)
LLAMA_1B = LlamaConfig(2048, 8192, 16, 32, 8, 128256, rope_theta=500000.0, rms_norm_eps=1e-5,
                       tie_word_embeddings=True)
LLAMA_8B = LlamaConfig(4096, 14336, 32, 32, 8, 128256, rope_theta=500000.0, rms_norm_eps=1e-5,
                       tie_word_embeddings=False)


def random_weights(cfg, seed=0, std=0.02):
    """dict key -> float32 array.  Matrices N(0, std) drawn in `param_shapes` order; norm gains are 1."""
    rng = np.random.default_rng(seed)
    w = {}
    for key, shape in cfg.param_shapes():
        if len(shape) == 1:
            w[key] = np.ones(shape, dtype=np.float32)
        else:
            a = rng.standard_normal(shape, dtype=np.float32)
            a *= np.float32(std)
            w[key] = a
    return w


def upload_weights(backend, weights, dtype):
    """float32 host arrays -> Parameters on the backend in `dtype` (bf16 rounds to nearest even)."""
    params = Parameters(backend)
    for key, arr in weights.items():
        params[key] = backend.from_numpy(arr, dtype)
    return params


def llama_term(backend, cfg, tap_logits=False):
    """The term of `LlamaModel::def` (llama.rs:393-401), built by the library's restated graph builder."""
    h = C.c_void_p()
    st = cfg.to_struct()
    backend._check(backend._ns.llama_term(C.byref(st), int(tap_logits), C.byref(h)), ctx=False)
    return Term(backend, h)


def empty_state_cache(backend, cfg, batch, dtype):
    """zeros [L, B, Hkv, 0, D] twice (utils/mod.rs:570-583, with the batch the caller asks for)."""
    shape = (cfg.num_hidden_layers, batch, cfg.num_key_value_heads, 0, cfg.head_dim)
    return backend.zeros(shape, dtype), backend.zeros(shape, dtype)


def generate_with_interpreter(backend, term, params, cfg, prompt_ids, steps, dtype, max_positions, tap=False):
    """Greedy generation through the op-by-op interpreter.

    prompt_ids: [B, S] uint32.  Returns (ids [B, steps] uint32, list of per-call logits [B, S_call, V] f32 if
    the term was built with tap_logits and tap=True).  `steps` counts generated tokens: the prefill call yields
    the first, every later call one more (main.rs:908-925).
    """
    interp = Interpreter(backend, params)
    prompt_ids = np.ascontiguousarray(prompt_ids, dtype=np.uint32)
    batch = prompt_ids.shape[0]
    in_k, in_v = empty_state_cache(backend, cfg, batch, dtype)
    x = prompt_ids
    out_ids = np.zeros((batch, steps), dtype=np.uint32)
    logits = []
    for i in range(steps):
        xt = backend.ndarray_from_vec_u32(x, x.shape)
        res = interp.run(term, [xt, in_k, in_v, max_positions])
        ids, in_k, in_v = res[0], res[1], res[2]
        if tap and len(res) > 3:
            logits.append(backend.to_f32(res[3]))
        last = backend.to_numpy(ids)[:, -1, 0]          # the element the reference runner reads
        out_ids[:, i] = last
        x = last.reshape(batch, 1).astype(np.uint32)
    return out_ids, logits


def bench_table(model_name, size_gib, params_m, backend, pp, elapsed_pp_s, tg, elapsed_tg_s):
    """The prompt-processing / token-generation table of the reference's benchmark mode, column for column
    (catgrad-llm/src/utils/mod.rs:528-566): two rows, `pp<prompt tokens>` and `tg<generated tokens>`, tokens per second
    to two decimals.  Returns the four lines."""
    head = ("| model                                    | size       | params     | backend    |            test |"
            "                  t/s |")
    rule = ("| ---------------------------------------- | ---------- | ---------- | ---------- | --------------- |"
            " -------------------- |")
    rows = []
    for label, n, secs in ((f"pp{pp}", pp, elapsed_pp_s), (f"tg{tg}", tg, elapsed_tg_s)):
        rows.append(f"| {model_name:<40} | {size_gib:>6.2f} GiB | {params_m:>8.2f} M | {backend:<10} | {label:>15} | {n / secs:>20.2f} |")
    return [head, rule] + rows


class LlamaRunner:
    """Fused Llama plan with a device-resident KV cache (`cg_llama_*`)."""

    def __init__(self, backend, cfg, params, dtype, max_batch, max_positions, comm=None, max_tokens=None):
        """comm: a `catgrad_b200.tp.TpComm`; then `params` is this rank's shard (`tp.shard_weights`) of the model
        `cfg` describes, and max_tokens bounds batch x seq of any forward call."""
        if not hasattr(backend._ns, "llama_create"):
            raise BackendError(Status.CUDA, "the fused runner exists only in the CUDA library")
        self._be = backend
        self.cfg = cfg
        self.max_batch = max_batch
        self.max_positions = max_positions
        self._comm = comm
        h = C.c_void_p()
        st = cfg.to_struct()
        if comm is None:
            backend._check(backend._ns.llama_create(backend._ctx, C.byref(st), int(dtype), params.handle, max_batch,
                                                    max_positions, C.byref(h)))
        else:
            backend._check(backend._ns.llama_create_tp(backend._ctx, C.byref(st), int(dtype), params.handle, max_batch,
                                                       max_positions, comm.handle, int(max_tokens or max_batch),
                                                       C.byref(h)))
        self._h = h
        self._params = params
        self._batch = 0

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and self._be._ns is not None:
            self._be._ns.llama_free(h)

    def reset(self, batch):
        self._be._check(self._be._ns.llama_reset(self._h, batch))
        self._batch = batch

    def forward(self, ids, read=True):
        """ids [B, S] uint32 (host).  Returns the greedy id of the last position per sequence if read."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        b, s = ids.shape
        out = np.zeros(b, dtype=np.uint32) if read else None
        self._be._check(self._be._ns.llama_forward(self._h, ids.ctypes.data_as(C.c_void_p), b, s,
                                                   out.ctypes.data_as(C.c_void_p) if read else None))
        return out

    def decode(self, steps):
        """`steps` greedy steps fed on the device; returns [B, steps] uint32."""
        out = np.zeros((self._batch, steps), dtype=np.uint32)
        self._be._check(self._be._ns.llama_decode(self._h, steps, out.ctypes.data_as(C.c_void_p)))
        return out

    def last_logits(self):
        out = np.zeros((self._batch, self.cfg.vocab_size), dtype=np.float32)
        self._be._check(self._be._ns.llama_last_logits(self._h, out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def set_persistent(self, on):
        """Allow (or forbid) the one-kernel persistent decode step for small batches (`cg_llama_set_persistent`)."""
        self._be._check(self._be._ns.llama_set_persistent(self._h, int(bool(on))))

    @property
    def persistent_active(self):
        return bool(self._be._ns.llama_persistent_active(self._h))

    @property
    def context_len(self):
        return int(self._be._ns.llama_context_len(self._h))

    @property
    def launch_count(self):
        return int(self._be._ns.llama_launch_count(self._h))

    def generate(self, prompt_ids, steps):
        """Prefill + greedy decode: ids [B, steps] (first column comes from the prefill call)."""
        prompt_ids = np.ascontiguousarray(prompt_ids, dtype=np.uint32)
        self.reset(prompt_ids.shape[0])
        first = self.forward(prompt_ids, read=True)
        if steps <= 1:
            return first.reshape(-1, 1)[:, :steps]
        rest = self.decode(steps - 1)
        return np.concatenate([first.reshape(-1, 1), rest], axis=1)

"""Parity at the true dimensions of the benchmark configurations (not scaled-down stand-ins).

* Llama-3.2-1B shape, all 16 layers (hidden 2048, 32 query / 8 kv heads x 64, FFN 8192, vocabulary 128256, tied
  head): the CPU oracle (f32, weights rounded to bf16 first) runs a 16-token prompt and two decode steps; the fused
  f32 runner must give the same ids and logits within rel 1e-4, the fused bf16 runner (both decode plans) logits
  within the bf16 bar described below.
  This is the only place where the 128256-row head, the K = 8192 down projection and the stacked [q;k;v] /
  [gate;up] weights meet the oracle.
* The per-GPU batches of the batch-sharded workload (32 and 256 sequences: tensor-core GEMM path, split-K
  clusters, captured graph) against the f32 runner that the oracle has just pinned.
* Llama-3-8B dimensions (hidden 4096, 32 / 8 heads x 128, FFN 14336, untied head) at two layers against the oracle.
* The op-sweep shapes at full size where the oracle finishes in seconds (gather, argmax, pointwise in bf16).

Bars: ids exact (f32), f32 logits rel <= 1e-4, integer/index results and correctly rounded pointwise results
bit-exact.  bf16 logits: <= 2e-2 max-abs against f32 on the same weights wherever the reference's own bf16 semantics
meet that bar.  At the full 1B depth they do not: the CPU oracle in bf16 mode (every op output rounded to bf16,
candle.rs:1165-1192) is 0.09-0.10 max-abs and 0.016-0.017 mean-abs away from its own f32 run on these inputs
(tests/golden/llama1b_bf16_semantics.json, written by make_llama1b_bf16_semantics.py).  There the kernels are held
to "no worse than the reference semantics": max-abs and mean-abs error against the f32 oracle within 1.25x of the
bf16 oracle's, and the same greedy id wherever the f32 run's top-2 gap exceeds twice the error."""
import gc

import numpy as np
import pytest

import catgrad_b200 as cb
from catgrad_b200 import Dtype
import helpers
from test_gpu_ops import both, same_bits

pytestmark = pytest.mark.gpu

REL_F32 = 1e-4
ABS_BF16 = 2e-2
PROMPT = 16
DECODE = 2
SEM_1B = helpers.bf16_semantics("llama1b")
SEM_8B2L = helpers.bf16_semantics("llama8b2l")
assert SEM_1B["prompt_len"] == PROMPT and SEM_1B["decode_steps"] == DECODE


def bf16_bar_1b(step, got, want):
    helpers.check_bf16_against_f32(SEM_1B, step, got, want, small_bar=ABS_BF16)


def bf16_round(w):
    return {k: cb.bf16_bits_to_f32(cb.f32_to_bf16_bits(v)).reshape(v.shape) for k, v in w.items()}


def oracle_run(oracle, cfg, wb, ids, steps):
    """ids [1 + steps] and last-position logits [1 + steps, B, V] of the op-by-op oracle (f32)."""
    term = cb.llama_term(oracle, cfg, tap_logits=True)
    po = cb.upload_weights(oracle, wb, Dtype.F32)
    out, logits = cb.generate_with_interpreter(oracle, term, po, cfg, ids, 1 + steps, Dtype.F32,
                                               ids.shape[1] + steps + 1, tap=True)
    last = np.stack([l[:, -1] for l in logits])
    del po, term, logits
    gc.collect()
    return out, last


@pytest.fixture(scope="module")
def model_1b():
    cfg = cb.LLAMA_1B
    return cfg, bf16_round(cb.random_weights(cfg, seed=0))


@pytest.fixture(scope="module")
def oracle_1b(oracle, model_1b):
    cfg, wb = model_1b
    ids = np.random.default_rng(1).integers(0, cfg.vocab_size, size=(1, PROMPT), dtype=np.uint32)
    out, last = oracle_run(oracle, cfg, wb, ids, DECODE)
    return ids, out, last


@pytest.fixture(scope="module")
def gpu_params_1b(gpu, model_1b):
    cfg, wb = model_1b
    return {"f32": cb.upload_weights(gpu, wb, Dtype.F32), "bf16": cb.upload_weights(gpu, wb, Dtype.BF16)}


def test_1b_shape_f32_runner_equals_the_oracle(gpu, model_1b, oracle_1b, gpu_params_1b):
    cfg, _ = model_1b
    ids, ref_ids, ref_logits = oracle_1b
    r = cb.LlamaRunner(gpu, cfg, gpu_params_1b["f32"], Dtype.F32, max_batch=1, max_positions=PROMPT + DECODE + 1)
    r.reset(1)
    tok = r.forward(ids)
    assert tok[0] == ref_ids[0, 0]
    assert helpers.rel_err(r.last_logits()[0], ref_logits[0][0]) <= REL_F32
    for i in range(1, DECODE + 1):
        tok = r.forward(tok.reshape(1, 1))
        assert tok[0] == ref_ids[0, i]
        assert helpers.rel_err(r.last_logits()[0], ref_logits[i][0]) <= REL_F32
    # the on-device loop (captured graph) gives the same ids
    np.testing.assert_array_equal(r.generate(ids, DECODE + 1), ref_ids)


@pytest.mark.parametrize("persistent", [False, True], ids=["kernel-per-sub-graph", "persistent-kernel"])
def test_1b_shape_bf16_runner_against_the_f32_oracle(gpu, model_1b, oracle_1b, gpu_params_1b, persistent):
    """Teacher-forced with the oracle's ids so that a flipped near-tie cannot compound.  Both decode plans of a
    single sequence: the graph of per-sub-graph kernels and the one-kernel persistent step."""
    cfg, _ = model_1b
    ids, ref_ids, ref_logits = oracle_1b
    r = cb.LlamaRunner(gpu, cfg, gpu_params_1b["bf16"], Dtype.BF16, max_batch=1, max_positions=PROMPT + DECODE + 1)
    r.set_persistent(persistent)
    assert ref_ids[0].tolist() == SEM_1B["f32_ids"]          # the fixture was made from the same oracle run
    r.reset(1)
    r.forward(ids)
    bf16_bar_1b(0, r.last_logits()[0], ref_logits[0][0])
    for i in range(1, DECODE + 1):
        r.forward(ref_ids[:, i - 1].reshape(1, 1))
        bf16_bar_1b(i, r.last_logits()[0], ref_logits[i][0])
    if persistent:
        assert r.persistent_active, "the persistent decode kernel was not used for this shape"


@pytest.mark.parametrize("batch", [32, 256])
def test_1b_shape_batched_bf16_decode_against_the_pinned_f32_runner(gpu, model_1b, gpu_params_1b, batch):
    """The per-GPU batches of the batch-sharded workload on 8 GPUs and on 1: prefill, then decode through the
    captured graph (tensor-core GEMMs over the stacked weights, split-K clusters at 32 rows)."""
    cfg, _ = model_1b
    ids = np.random.default_rng(4).integers(0, cfg.vocab_size, size=(batch, PROMPT), dtype=np.uint32)
    P = PROMPT + DECODE + 2
    r16 = cb.LlamaRunner(gpu, cfg, gpu_params_1b["bf16"], Dtype.BF16, max_batch=batch, max_positions=P)
    r32 = cb.LlamaRunner(gpu, cfg, gpu_params_1b["f32"], Dtype.F32, max_batch=batch, max_positions=P)
    r16.reset(batch)
    r32.reset(batch)
    # see the module docstring; the maximum here is taken over up to 256 x 128256 logits instead of 128256, so the
    # max-abs bar gets twice the single-sequence figure while the mean-abs bar stays at 1.25x
    def close(a, b):
        helpers.check_bf16_against_f32(SEM_1B, None, a, b, small_bar=ABS_BF16, max_factor=2.0)

    first = r16.forward(ids)
    r32.forward(ids)
    close(r16.last_logits(), r32.last_logits())
    rest = r16.decode(DECODE)                       # the path the benchmark times
    tok = first
    for s in range(DECODE):                         # f32 runner fed the bf16 run's ids: same history on both sides
        r32.forward(tok.reshape(batch, 1))
        tok = rest[:, s]
    close(r16.last_logits(), r32.last_logits())
    # sequences are independent: row b of the batch equals running it alone (what batch sharding relies on)
    solo = cb.LlamaRunner(gpu, cfg, gpu_params_1b["bf16"], Dtype.BF16, max_batch=1, max_positions=P)
    solo.set_persistent(False)
    for b in (0, batch - 1):
        solo.reset(1)
        solo.forward(ids[b:b + 1])
        for s in range(DECODE):
            solo.forward(np.array([[first[b] if s == 0 else rest[b, s - 1]]], dtype=np.uint32))
        close(solo.last_logits()[0], r16.last_logits()[b])


def test_8b_dimensions_two_layers_against_the_oracle(oracle, gpu):
    """hidden 4096, 32 query / 8 kv heads x 128, FFN 14336, untied 128256-row head; two of the 32 layers.  The bf16 bar
    comes from tests/golden/llama8b2l_bf16_semantics.json (same model, prompt and steps)."""
    cfg = cb.LlamaConfig(4096, 14336, 2, 32, 8, 128256, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)
    wb = bf16_round(cb.random_weights(cfg, seed=3))
    ids = np.random.default_rng(5).integers(0, cfg.vocab_size, size=(1, 8), dtype=np.uint32)
    ref_ids, ref_logits = oracle_run(oracle, cfg, wb, ids, 1)
    assert ref_ids[0].tolist() == SEM_8B2L["f32_ids"]
    p32 = cb.upload_weights(gpu, wb, Dtype.F32)
    r32 = cb.LlamaRunner(gpu, cfg, p32, Dtype.F32, max_batch=1, max_positions=12)
    np.testing.assert_array_equal(r32.generate(ids, 2), ref_ids)
    assert helpers.rel_err(r32.last_logits()[0], ref_logits[1][0]) <= REL_F32
    p16 = cb.upload_weights(gpu, wb, Dtype.BF16)
    del wb
    gc.collect()
    # one sequence (weight-streaming path) and 32 copies of it (the benchmark's batch: tensor-core path)
    for batch in (1, 32):
        r16 = cb.LlamaRunner(gpu, cfg, p16, Dtype.BF16, max_batch=batch, max_positions=12)
        r16.reset(batch)
        r16.forward(np.repeat(ids, batch, 0))
        for b in range(batch):
            helpers.check_bf16_against_f32(SEM_8B2L, 0, r16.last_logits()[b], ref_logits[0][0], small_bar=ABS_BF16)
        r16.forward(np.repeat(ref_ids[:, :1], batch, 0))
        for b in range(batch):
            helpers.check_bf16_against_f32(SEM_8B2L, 1, r16.last_logits()[b], ref_logits[1][0], small_bar=ABS_BF16)
        del r16


def test_op_sweep_shapes_at_full_size(oracle, gpu):
    """Gather of 4096 rows from [32000, 2048], argmax over [64, 32000], pointwise ops on [4096, 8192] with an
    explicitly broadcast row vector: bit-exact in f32 and bf16."""
    rng = np.random.default_rng(2)
    table = rng.standard_normal((32000, 2048)).astype(np.float32)
    idx = rng.integers(0, 32000, 4096, dtype=np.uint32)
    am = rng.standard_normal((64, 32000)).astype(np.float32)
    x = rng.uniform(-4, 4, (4096, 8192)).astype(np.float32)
    v = rng.uniform(-4, 4, (8192,)).astype(np.float32)
    for dtype in (Dtype.F32, Dtype.BF16):
        to, tg = both(oracle, gpu, table, dtype)
        io, ig = both(oracle, gpu, idx)
        same_bits(oracle, gpu, oracle.index(to, 0, io), gpu.index(tg, 0, ig), "gather")
        del to, tg
        ao, ag = both(oracle, gpu, am, dtype)
        same_bits(oracle, gpu, oracle.argmax(ao), gpu.argmax(ag), "argmax")
        same_bits(oracle, gpu, oracle.max(ao), gpu.max(ag), "max")
    xo, xg = both(oracle, gpu, x, Dtype.BF16)
    vo, vg = both(oracle, gpu, v, Dtype.BF16)
    bo, bg = oracle.broadcast(vo, x.shape), gpu.broadcast(vg, x.shape)
    for op in ("add", "mul", "div"):
        same_bits(oracle, gpu, getattr(oracle, op)(xo, bo), getattr(gpu, op)(xg, bg), op)

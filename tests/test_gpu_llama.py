"""Llama through the C ABI on the GPU against the CPU oracle (the tiny f32 configuration and reduced bf16 shapes).

Bars: greedy ids exact and f32 logits within rel 1e-4 on the tiny model; bf16 logits within 2e-2 max-abs of the
f32 oracle run on the same (bf16-rounded) weights."""
import numpy as np
import pytest

import catgrad_b200 as cb
from catgrad_b200 import Dtype
import helpers

pytestmark = pytest.mark.gpu

REL_F32 = 1e-4
ABS_BF16 = 2e-2


def tiny_inputs():
    cfg = cb.TINY
    w = cb.random_weights(cfg, seed=0)
    ids = np.random.default_rng(1).integers(0, cfg.vocab_size, size=(1, 64), dtype=np.uint32)
    return cfg, w, ids


@pytest.fixture(scope="module")
def oracle_tiny(oracle):
    cfg, w, ids = tiny_inputs()
    term = cb.llama_term(oracle, cfg, tap_logits=True)
    params = cb.upload_weights(oracle, w, Dtype.F32)
    out, logits = cb.generate_with_interpreter(oracle, term, params, cfg, ids, 33, Dtype.F32, 97, tap=True)
    return out, logits


def test_config1_interpreter_path(gpu, oracle_tiny):
    """64-token prompt + 32 greedy steps through the op-by-op interpreter: ids exact, logits rel <= 1e-4."""
    cfg, w, ids = tiny_inputs()
    ref_ids, ref_logits = oracle_tiny
    term = cb.llama_term(gpu, cfg, tap_logits=True)
    params = cb.upload_weights(gpu, w, Dtype.F32)
    out, logits = cb.generate_with_interpreter(gpu, term, params, cfg, ids, 33, Dtype.F32, 97, tap=True)
    np.testing.assert_array_equal(out, ref_ids)
    for a, b in zip(logits, ref_logits):
        assert helpers.rel_err(a, b) <= REL_F32


def test_config1_fused_runner(gpu, oracle_tiny):
    cfg, w, ids = tiny_inputs()
    ref_ids, ref_logits = oracle_tiny
    params = cb.upload_weights(gpu, w, Dtype.F32)
    runner = cb.LlamaRunner(gpu, cfg, params, Dtype.F32, max_batch=1, max_positions=97)
    out = runner.generate(ids, 33)
    np.testing.assert_array_equal(out, ref_ids)
    # logits after the prefill and after every decode step, stepping by hand
    runner.reset(1)
    first = runner.forward(ids)
    assert helpers.rel_err(runner.last_logits()[0], ref_logits[0][0, -1]) <= REL_F32
    tok = first
    for i in range(1, 6):
        tok = runner.forward(tok.reshape(1, 1))
        assert helpers.rel_err(runner.last_logits()[0], ref_logits[i][0, -1]) <= REL_F32
        assert tok[0] == ref_ids[0, i]
    assert runner.context_len == 64 + 5
    assert runner.launch_count > 0


def test_fused_runner_batch_and_graph_replay_match_stepwise(gpu):
    """Batch of 3 sequences: decode through the captured graph equals stepping one call at a time, and every
    sequence equals running it alone (batch independence, which batch-sharding across GPUs relies on)."""
    cfg, w, _ = tiny_inputs()
    ids = np.random.default_rng(11).integers(0, cfg.vocab_size, size=(3, 16), dtype=np.uint32)
    params = cb.upload_weights(gpu, w, Dtype.F32)
    runner = cb.LlamaRunner(gpu, cfg, params, Dtype.F32, max_batch=3, max_positions=64)
    out = runner.generate(ids, 12)
    runner.reset(3)
    tok = runner.forward(ids)
    cols = [tok]
    for _ in range(11):
        tok = runner.forward(tok.reshape(3, 1))
        cols.append(tok)
    np.testing.assert_array_equal(out, np.stack(cols, 1))
    solo = cb.LlamaRunner(gpu, cfg, params, Dtype.F32, max_batch=1, max_positions=64)
    for b in range(3):
        np.testing.assert_array_equal(solo.generate(ids[b:b + 1], 12)[0], out[b])


def test_many_sequences_use_the_warp_per_head_attention_and_match_solo_runs(gpu):
    """With batch x heads above four CTAs per SM the decode step switches to the warp-per-head attention kernel
    (one CTA per kv head and sequence).  Every sequence must still equal running it alone, which goes through the
    CTA-per-head kernel: same ids, logits to f32 round-off."""
    cfg, w, _ = tiny_inputs()
    B = 160
    ids = np.random.default_rng(5).integers(0, cfg.vocab_size, size=(B, 12), dtype=np.uint32)
    params = cb.upload_weights(gpu, w, Dtype.F32)
    runner = cb.LlamaRunner(gpu, cfg, params, Dtype.F32, max_batch=B, max_positions=48)
    out = runner.generate(ids, 9)
    logits = runner.last_logits()
    solo = cb.LlamaRunner(gpu, cfg, params, Dtype.F32, max_batch=1, max_positions=48)
    for b in (0, 1, 77, 159):
        np.testing.assert_array_equal(solo.generate(ids[b:b + 1], 9)[0], out[b])
        assert helpers.rel_err(solo.last_logits()[0], logits[b]) <= REL_F32


@pytest.mark.parametrize("B,kv_heads", [(96, 2), (600, 2), (80, 1)])
def test_many_sequences_bf16_gqa(gpu, B, kv_heads):
    """Same check in bf16 with grouped heads.  With 2 kv heads there are at least as many (kv head, sequence) pairs as
    SMs: 96 sequences take two warps per pair, 600 sequences (more than 8 pairs per SM) one warp per pair, each
    computing the 4 query heads of the group.  80 sequences x 1 kv head is below that but has 640 (head, sequence)
    pairs: one warp per query head, the 8 heads of the kv head sharing a CTA."""
    cfg, wb, _ = small_bf16_model()
    if kv_heads != cfg.num_key_value_heads:
        cfg = cb.LlamaConfig(512, 1536, 2, 8, kv_heads, 4096, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=True)
        w = cb.random_weights(cfg, seed=0)
        wb = {k: cb.bf16_bits_to_f32(cb.f32_to_bf16_bits(v)).reshape(v.shape) for k, v in w.items()}
    ids = np.random.default_rng(6).integers(0, cfg.vocab_size, size=(B, 20), dtype=np.uint32)
    pg = cb.upload_weights(gpu, wb, Dtype.BF16)
    runner = cb.LlamaRunner(gpu, cfg, pg, Dtype.BF16, max_batch=B, max_positions=40)
    runner.reset(B)
    tok = runner.forward(ids)
    picks = (0, 50, B - 1)
    solos = {}
    for b in picks:
        solos[b] = cb.LlamaRunner(gpu, cfg, pg, Dtype.BF16, max_batch=1, max_positions=40)
        solos[b].reset(1)
        solos[b].forward(ids[b:b + 1])
    for _ in range(5):
        nxt = runner.forward(tok.reshape(B, 1))
        lg = runner.last_logits()
        for b in picks:
            # the solo run is fed the batch's ids, so both see the same history
            solos[b].forward(np.array([[tok[b]]], dtype=np.uint32))
            assert np.abs(solos[b].last_logits()[0] - lg[b]).max() <= ABS_BF16
        tok = nxt


@pytest.mark.parametrize("heads,kv_heads", [(8, 2), (4, 2)])
def test_long_context_uses_key_split_attention(gpu, heads, kv_heads):
    """Beyond 512 cached positions the bf16 decode step splits the keys of every (sequence, kv head) over CTAs (two
    launches, partial sums combined in chunk order).  Held to the f32 model on the same weights, step by step with
    the same history, like every bf16 path; head_dim 64 (8 heads) and 128 (4 heads)."""
    cfg = cb.LlamaConfig(512, 1536, 2, heads, kv_heads, 4096, rope_theta=500000.0, rms_norm_eps=1e-5,
                         tie_word_embeddings=True)
    w = cb.random_weights(cfg, seed=0)
    wb = {k: cb.bf16_bits_to_f32(cb.f32_to_bf16_bits(v)).reshape(v.shape) for k, v in w.items()}
    B, S = 16, 600     # 16 sequences x 2 kv heads: the smallest batch that takes the key-split path
    ids = np.random.default_rng(9).integers(0, cfg.vocab_size, size=(B, S), dtype=np.uint32)
    run16 = cb.LlamaRunner(gpu, cfg, cb.upload_weights(gpu, wb, Dtype.BF16), Dtype.BF16, max_batch=B, max_positions=S + 140)
    run32 = cb.LlamaRunner(gpu, cfg, cb.upload_weights(gpu, wb, Dtype.F32), Dtype.F32, max_batch=B, max_positions=S + 140)
    run16.reset(B)
    run32.reset(B)
    tok = run16.forward(ids)
    run32.forward(ids)
    assert np.abs(run16.last_logits() - run32.last_logits()).max() <= ABS_BF16
    for _ in range(3):
        nxt = run16.forward(tok.reshape(B, 1))
        run32.forward(tok.reshape(B, 1))
        assert np.abs(run16.last_logits() - run32.last_logits()).max() <= ABS_BF16
        tok = nxt
    # the captured graph replays the same two launches while the context crosses a chunk boundary (640 = 5 x 128)
    more = run16.decode(45)
    assert run16.context_len == S + 3 + 45
    again = cb.LlamaRunner(gpu, cfg, run16._params, Dtype.BF16, max_batch=B, max_positions=S + 140)
    again.reset(B)
    t2 = again.forward(ids)
    for _ in range(3):
        t2 = again.forward(t2.reshape(B, 1))
    cols = []
    for _ in range(45):
        t2 = again.forward(t2.reshape(B, 1))
        cols.append(t2)
    np.testing.assert_array_equal(more, np.stack(cols, 1))


def test_graph_capture_right_at_the_attention_switch_point(gpu):
    """A 512-token prompt: the first decode step (context 512) still takes the single-launch attention, the captured
    step (context 513) the key-split one.  Nothing may allocate inside the capture, and the ids must equal stepping."""
    cfg, wb, _ = small_bf16_model()
    B = 16
    ids = np.random.default_rng(3).integers(0, cfg.vocab_size, size=(B, 512), dtype=np.uint32)
    pg = cb.upload_weights(gpu, wb, Dtype.BF16)
    runner = cb.LlamaRunner(gpu, cfg, pg, Dtype.BF16, max_batch=B, max_positions=560)
    out = runner.generate(ids, 10)
    step = cb.LlamaRunner(gpu, cfg, pg, Dtype.BF16, max_batch=B, max_positions=560)
    step.reset(B)
    tok = step.forward(ids)
    cols = [tok]
    for _ in range(9):
        tok = step.forward(tok.reshape(B, 1))
        cols.append(tok)
    np.testing.assert_array_equal(out, np.stack(cols, 1))


def small_bf16_model():
    # Llama-3.2-1B proportions (GQA 4:1, head_dim 64, tied head, theta 5e5) at 2 layers / hidden 512
    cfg = cb.LlamaConfig(512, 1536, 2, 8, 2, 4096, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=True)
    w = cb.random_weights(cfg, seed=0)
    wb = {k: cb.bf16_bits_to_f32(cb.f32_to_bf16_bits(v)).reshape(v.shape) for k, v in w.items()}
    ids = np.random.default_rng(1).integers(0, cfg.vocab_size, size=(2, 40), dtype=np.uint32)
    return cfg, wb, ids


def test_bf16_logits_against_f32_oracle(oracle, gpu):
    cfg, wb, ids = small_bf16_model()
    term_o = cb.llama_term(oracle, cfg, tap_logits=True)
    po = cb.upload_weights(oracle, wb, Dtype.F32)
    ref_ids, ref_logits = cb.generate_with_interpreter(oracle, term_o, po, cfg, ids, 4, Dtype.F32, 64, tap=True)

    # op-by-op interpreter on the GPU in bf16
    term_g = cb.llama_term(gpu, cfg, tap_logits=True)
    pg = cb.upload_weights(gpu, wb, Dtype.BF16)
    out_i, logits_i = cb.generate_with_interpreter(gpu, term_g, pg, cfg, ids, 4, Dtype.BF16, 64, tap=True)
    for a, b in zip(logits_i, ref_logits):
        assert np.abs(a[:, -1] - b[:, -1]).max() <= ABS_BF16

    # fused runner in bf16: same bar against the oracle, and near-identical to the unfused GPU path
    runner = cb.LlamaRunner(gpu, cfg, pg, Dtype.BF16, max_batch=2, max_positions=64)
    runner.reset(2)
    tok = runner.forward(ids)
    lg = runner.last_logits()
    assert np.abs(lg - ref_logits[0][:, -1]).max() <= ABS_BF16
    assert np.abs(lg - logits_i[0][:, -1]).max() <= ABS_BF16
    for i in range(1, 4):
        tok = runner.forward(ref_ids[:, i - 1].reshape(2, 1))   # teacher-forced with the oracle's ids
        lg = runner.last_logits()
        assert np.abs(lg - ref_logits[i][:, -1]).max() <= ABS_BF16


def test_oracle_bf16_interpreter_matches_gpu_bf16_interpreter(oracle, gpu):
    """Same bf16 op stream on both sides (the oracle rounds at every op output like the GPU kernels): logits agree
    to bf16 resolution."""
    cfg, wb, ids = small_bf16_model()
    res = []
    for be in (oracle, gpu):
        term = cb.llama_term(be, cfg, tap_logits=True)
        p = cb.upload_weights(be, wb, Dtype.BF16)
        _, logits = cb.generate_with_interpreter(be, term, p, cfg, ids[:, :12], 1, Dtype.BF16, 32, tap=True)
        res.append(logits[0])
    assert np.abs(res[0] - res[1]).max() <= ABS_BF16


def test_kv_cache_roundtrip_property(gpu):
    """Prefill(prompt) then one decode step equals prefill(prompt + token): the appended cache row and the
    single-row attention path reproduce what the full causal pass computes."""
    cfg, w, _ = tiny_inputs()
    params = cb.upload_weights(gpu, w, Dtype.F32)
    ids = np.random.default_rng(5).integers(0, cfg.vocab_size, size=(2, 24), dtype=np.uint32)
    r = cb.LlamaRunner(gpu, cfg, params, Dtype.F32, max_batch=2, max_positions=64)
    r.reset(2)
    r.forward(ids[:, :23])
    r.forward(ids[:, 23:24])
    a = r.last_logits()
    r.reset(2)
    r.forward(ids)
    b = r.last_logits()
    assert helpers.rel_err(a, b) <= REL_F32


def test_runner_refuses_bad_use(gpu):
    cfg, w, ids = tiny_inputs()
    params = cb.upload_weights(gpu, w, Dtype.F32)
    r = cb.LlamaRunner(gpu, cfg, params, Dtype.F32, max_batch=1, max_positions=32)
    r.reset(1)
    with pytest.raises(cb.BackendError):
        r.forward(ids)                       # 64 tokens > max_positions
    with pytest.raises(cb.BackendError):
        cb.LlamaRunner(gpu, cfg, cb.Parameters(gpu), Dtype.F32, 1, 32)   # missing parameters
    bad = np.full((1, 4), cfg.vocab_size + 5, np.uint32)
    r.reset(1)
    with pytest.raises(cb.BackendError):
        r.forward(bad)                       # token id outside the vocabulary: reported, not trapped
    r.reset(1)
    assert r.forward(ids[:, :8]).shape == (1,)


def test_persistent_decode_kernel_matches_the_multi_kernel_plan(gpu):
    """Decode steps of a few bf16 sequences run as one persistent kernel unless cg_llama_set_persistent(0) asks for
    the graph of per-sub-graph kernels.  Same rounding points except inside attention (chunked softmax, see
    llama_persist.cuh), different summation order: logits agree to bf16 resolution (teacher-forced so that one
    flipped argmax cannot compound), and the KV caches they build are interchangeable."""
    cfg, wb, ids = small_bf16_model()
    pg = cb.upload_weights(gpu, wb, Dtype.BF16)
    mega = cb.LlamaRunner(gpu, cfg, pg, Dtype.BF16, max_batch=2, max_positions=64)
    plain = cb.LlamaRunner(gpu, cfg, pg, Dtype.BF16, max_batch=2, max_positions=64)
    plain.set_persistent(False)
    mega.reset(2)
    plain.reset(2)
    ta = mega.forward(ids)
    tb = plain.forward(ids)
    np.testing.assert_array_equal(ta, tb)           # the prefill is the same code in both
    tok = ta
    for _ in range(8):
        ta = mega.forward(tok.reshape(2, 1))
        tb = plain.forward(tok.reshape(2, 1))
        assert mega.persistent_active and not plain.persistent_active
        la, lb = mega.last_logits(), plain.last_logits()
        assert np.abs(la - lb).max() <= ABS_BF16
        tok = tb
    # on-device loop of the persistent kernel == stepping it from the host
    mega.reset(2)
    first = mega.forward(ids)
    out = mega.decode(6)
    mega.reset(2)
    t = mega.forward(ids)
    cols = []
    for _ in range(6):
        t = mega.forward(t.reshape(2, 1))
        cols.append(t)
    np.testing.assert_array_equal(out, np.stack(cols, 1))
    assert mega.launch_count < plain.launch_count   # one launch per decode step
    # a cache built by one plan serves the other: switch plans in the middle of a sequence
    mega.set_persistent(False)
    plain.set_persistent(True)
    ta = mega.forward(t.reshape(2, 1))
    plain.reset(2)
    plain.forward(ids)
    for c in [first] + cols:                       # the same history: prompt, its greedy token, the six decoded ones
        plain.forward(c.reshape(2, 1))
    assert np.abs(mega.last_logits() - plain.last_logits()).max() <= ABS_BF16


@pytest.mark.parametrize("heads,kv_heads,batch,ctx", [(8, 2, 1, 300), (4, 2, 3, 140), (8, 8, 4, 20)])
def test_persistent_decode_kernel_long_contexts_and_head_shapes(gpu, heads, kv_heads, batch, ctx):
    """The persistent kernel's attention splits the keys into 128-key chunks over the CTAs and combines the chunk
    partials when it loads the o_proj input: contexts spanning several chunks, head_dim 64 and 128, GQA groups of
    4, 2 and 1, against the f32 runner on the same weights (same history on both sides)."""
    cfg = cb.LlamaConfig(512, 1536, 2, heads, kv_heads, 4096, rope_theta=500000.0, rms_norm_eps=1e-5,
                         tie_word_embeddings=True)
    w = cb.random_weights(cfg, seed=0)
    wb = {k: cb.bf16_bits_to_f32(cb.f32_to_bf16_bits(v)).reshape(v.shape) for k, v in w.items()}
    ids = np.random.default_rng(12).integers(0, cfg.vocab_size, size=(batch, ctx), dtype=np.uint32)
    r16 = cb.LlamaRunner(gpu, cfg, cb.upload_weights(gpu, wb, Dtype.BF16), Dtype.BF16, max_batch=batch, max_positions=ctx + 140)
    r32 = cb.LlamaRunner(gpu, cfg, cb.upload_weights(gpu, wb, Dtype.F32), Dtype.F32, max_batch=batch, max_positions=ctx + 140)
    r16.reset(batch)
    r32.reset(batch)
    tok = r16.forward(ids)
    r32.forward(ids)
    for _ in range(4):
        nxt = r16.forward(tok.reshape(batch, 1))
        assert r16.persistent_active
        r32.forward(tok.reshape(batch, 1))
        assert np.abs(r16.last_logits() - r32.last_logits()).max() <= ABS_BF16
        tok = nxt
    # the on-device loop crosses a chunk boundary (a multiple of 128) and must equal stepping from the host
    more = r16.decode(130)
    again = cb.LlamaRunner(gpu, cfg, r16._params, Dtype.BF16, max_batch=batch, max_positions=ctx + 140)
    again.reset(batch)
    t2 = again.forward(ids)
    for _ in range(4):
        t2 = again.forward(t2.reshape(batch, 1))
    cols = []
    for _ in range(130):
        t2 = again.forward(t2.reshape(batch, 1))
        cols.append(t2)
    np.testing.assert_array_equal(more, np.stack(cols, 1))


def test_device_runner_shards_sequences_over_replicas(gpu):
    """cg_runner_*: sequences split over replicas (two contexts here; on a box with several GPUs one per GPU), ids
    gathered on the host: every row must equal what a single runner produces for it, in the right place."""
    import torch
    from catgrad_b200.runner import DeviceRunner, shard_range
    cfg, w, _ = tiny_inputs()
    n_dev = torch.cuda.device_count()
    devices = [0, 1 % n_dev, 0]                      # three replicas; 7 sequences split 3 + 2 + 2
    ids = np.random.default_rng(17).integers(0, cfg.vocab_size, size=(7, 10), dtype=np.uint32)
    params = cb.upload_weights(gpu, w, Dtype.F32)
    want = cb.LlamaRunner(gpu, cfg, params, Dtype.F32, max_batch=7, max_positions=32).generate(ids, 6)
    r = DeviceRunner(devices, cfg, Dtype.F32, max_batch_per_device=3, max_positions=32)
    assert r.size == 3 and shard_range(7, 3, 0) == (0, 3) and shard_range(7, 3, 2) == (5, 7)
    with pytest.raises(cb.BackendError):
        r.generate(ids, 6)                           # no parameters yet
    for i in range(r.size):
        r.set_params(i, cb.upload_weights(r.backend(i), w, Dtype.F32))
    np.testing.assert_array_equal(r.generate(ids, 6), want)
    np.testing.assert_array_equal(r.generate(ids[:2], 6), want[:2])          # fewer sequences than replicas: one idles
    with pytest.raises(cb.BackendError):
        r.generate(np.zeros((10, 10), np.uint32), 2)     # 4 sequences on a replica sized for 3
    r.close()


def test_llama3_rope_scaling_on_the_gpu(oracle, gpu):
    """rope_scaling "llama3": the fused runner's tables (rope_table_kernel) and the op-by-op term on the GPU against the
    oracle's term, f32, positions up to 300 where scaled and unscaled tables differ widely."""
    scaling = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 8192}
    cfg = cb.LlamaConfig(256, 512, 2, 4, 2, 1024, rope_theta=500000.0, tie_word_embeddings=True, rope_scaling=scaling)
    w = cb.random_weights(cfg, 5)
    ids = np.random.default_rng(6).integers(0, cfg.vocab_size, size=(1, 300), dtype=np.uint32)
    term_o = cb.llama_term(oracle, cfg, tap_logits=True)
    ref_ids, ref_logits = cb.generate_with_interpreter(oracle, term_o, cb.upload_weights(oracle, w, Dtype.F32), cfg, ids, 3,
                                                       Dtype.F32, 310, tap=True)
    params = cb.upload_weights(gpu, w, Dtype.F32)
    runner = cb.LlamaRunner(gpu, cfg, params, Dtype.F32, max_batch=1, max_positions=310)
    np.testing.assert_array_equal(runner.generate(ids, 3), ref_ids)
    assert helpers.rel_err(runner.last_logits()[0], ref_logits[2][0, -1]) <= REL_F32
    term_g = cb.llama_term(gpu, cfg, tap_logits=True)
    out, logits = cb.generate_with_interpreter(gpu, term_g, params, cfg, ids, 2, Dtype.F32, 310, tap=True)
    np.testing.assert_array_equal(out, ref_ids[:, :2])
    assert helpers.rel_err(logits[1][0, -1], ref_logits[1][0, -1]) <= REL_F32


# ---- term -> plan: the Llama term through cg_interp_run on the fused runner -------------------------------------
def test_llama_term_through_the_interpreter_entry_point_runs_as_the_fused_plan(gpu, oracle_tiny):
    """The route catgrad itself takes (interpreter.run(term) per token, the cache threaded as a value): the term is
    recognised on its first run, ids are those of the oracle and of cg_llama_forward, the cache values handed back are
    views of the runner's buffers (nothing is re-stacked), and far fewer kernels launch than one per edge."""
    cfg, w, ids = tiny_inputs()
    ref_ids, _ = oracle_tiny
    params = cb.upload_weights(gpu, w, Dtype.F32)
    term = cb.llama_term(gpu, cfg)
    assert term.plan_state == 0
    before = gpu.stats()[3]
    out, _ = cb.generate_with_interpreter(gpu, term, params, cfg, ids, 33, Dtype.F32, 97)
    assert term.plan_state == 1
    np.testing.assert_array_equal(out, ref_ids)
    runner = cb.LlamaRunner(gpu, cfg, params, Dtype.F32, max_batch=1, max_positions=97)
    np.testing.assert_array_equal(out, runner.generate(ids, 33))
    # op by op the same loop is ~300 backend calls per token; planned it is a few dozen launches of fused kernels,
    # none of them through the per-edge entry points counted here
    assert gpu.stats()[3] - before < 33 * 40
    # one call by hand: ids of ALL positions come back ([B, S, 1], as the term types them), and the cache is a view
    interp = cb.Interpreter(gpu, params)
    k0, v0 = cb.empty_state_cache(gpu, cfg, 1, Dtype.F32)
    res = interp.run(term, [gpu.ndarray_from_vec_u32(ids, ids.shape), k0, v0, 97])
    all_ids, k1, v1 = res[0], res[1], res[2]
    assert all_ids.shape == (1, 64, 1) and k1.shape == (cfg.num_hidden_layers, 1, cfg.num_key_value_heads, 64, cfg.head_dim)
    assert not k1.is_contiguous and k1.strides[2] == 97 * cfg.head_dim        # [L, B, Hkv, P, D] allocation underneath
    gpu._ns.interp_set_planning(0)
    try:
        slow = cb.Interpreter(gpu, params).run(cb.llama_term(gpu, cfg), [gpu.ndarray_from_vec_u32(ids, ids.shape), k0, v0, 97])
    finally:
        gpu._ns.interp_set_planning(1)
    np.testing.assert_array_equal(gpu.to_numpy(all_ids), gpu.to_numpy(slow[0]))          # every position's id
    assert helpers.rel_err(gpu.to_numpy(k1), gpu.to_numpy(slow[1])) <= REL_F32
    assert helpers.rel_err(gpu.to_numpy(v1), gpu.to_numpy(slow[2])) <= REL_F32
    # threading the views back in continues the same sequence in place
    nxt = gpu.to_numpy(all_ids)[:, -1, 0].reshape(1, 1).astype(np.uint32)
    res2 = interp.run(term, [gpu.ndarray_from_vec_u32(nxt, nxt.shape), k1, v1, 97])
    assert res2[1].shape[3] == 65 and gpu.to_numpy(res2[0])[0, 0, 0] == ref_ids[0, 1]


def test_terms_that_are_not_the_llama_term_fall_back_to_op_by_op(gpu, oracle):
    """One edge of difference is enough: the term with its logits tapped as a fourth output, and a model whose head
    dimension the fused runner does not support, run op by op and still agree with the oracle.  A cache that is not the
    runner's own (here: one produced op by op) is also left to the evaluator."""
    cfg, w, ids = tiny_inputs()
    params = cb.upload_weights(gpu, w, Dtype.F32)
    tapped = cb.llama_term(gpu, cfg, tap_logits=True)
    out, logits = cb.generate_with_interpreter(gpu, tapped, params, cfg, ids[:, :20], 3, Dtype.F32, 32, tap=True)
    assert tapped.plan_state == 2 and len(logits) == 3
    term_o = cb.llama_term(oracle, cfg)
    want, _ = cb.generate_with_interpreter(oracle, term_o, cb.upload_weights(oracle, w, Dtype.F32), cfg, ids[:, :20], 3, Dtype.F32, 32)
    np.testing.assert_array_equal(out, want)
    odd = cb.LlamaConfig(128, 256, 1, 4, 2, 512, rope_theta=10000.0)           # head_dim 32
    w2 = cb.random_weights(odd, 2)
    ids2 = np.random.default_rng(3).integers(0, 512, size=(1, 9), dtype=np.uint32)
    t2 = cb.llama_term(gpu, odd)
    got, _ = cb.generate_with_interpreter(gpu, t2, cb.upload_weights(gpu, w2, Dtype.F32), odd, ids2, 3, Dtype.F32, 16)
    assert t2.plan_state == 2
    want2, _ = cb.generate_with_interpreter(oracle, cb.llama_term(oracle, odd), cb.upload_weights(oracle, w2, Dtype.F32), odd, ids2, 3,
                                            Dtype.F32, 16)
    np.testing.assert_array_equal(got, want2)
    # a foreign cache: prefill op by op (planning off), then continue with the recognised term
    term = cb.llama_term(gpu, cfg)
    k0, v0 = cb.empty_state_cache(gpu, cfg, 1, Dtype.F32)
    gpu._ns.interp_set_planning(0)
    try:
        r1 = cb.Interpreter(gpu, params).run(term, [gpu.ndarray_from_vec_u32(ids[:, :20], (1, 20)), k0, v0, 32])
    finally:
        gpu._ns.interp_set_planning(1)
    tok = gpu.to_numpy(r1[0])[:, -1, 0].reshape(1, 1).astype(np.uint32)
    r2 = cb.Interpreter(gpu, params).run(term, [gpu.ndarray_from_vec_u32(tok, (1, 1)), r1[1], r1[2], 32])
    assert gpu.to_numpy(r2[0])[0, 0, 0] == want[0, 1] and r2[1].shape[3] == 21


def test_planned_bf16_decode_takes_the_persistent_kernel_and_handles_batches(gpu):
    cfg, wb, ids = small_bf16_model()
    pg = cb.upload_weights(gpu, wb, Dtype.BF16)
    term = cb.llama_term(gpu, cfg)
    out, _ = cb.generate_with_interpreter(gpu, term, pg, cfg, ids, 6, Dtype.BF16, 64)
    assert term.plan_state == 1
    runner = cb.LlamaRunner(gpu, cfg, pg, Dtype.BF16, max_batch=2, max_positions=64)
    np.testing.assert_array_equal(out, runner.generate(ids, 6))


def test_safetensors_checkpoint_loads_onto_the_gpu(tmp_path, oracle, gpu):
    """The loader (utils/mod.rs:321-449, dense-model part) feeding the CUDA backend: a sharded bf16 checkpoint is read
    into device tensors (values exact), and the loaded model generates, through the fused runner and through the Llama
    term in the interpreter, the ids the CPU oracle generates from the in-memory weights."""
    from catgrad_b200 import safetensors as st
    cfg = cb.TINY
    w = cb.random_weights(cfg, seed=0)
    keys = sorted(w)
    half = len(keys) // 2
    st.save_file(tmp_path / "model-00001-of-00002.safetensors", {k: w[k] for k in keys[:half]}, bf16=True)
    st.save_file(tmp_path / "model-00002-of-00002.safetensors", {k: w[k] for k in keys[half:]}, bf16=True)
    files = [str(tmp_path / f"model-0000{i}-of-00002.safetensors") for i in (1, 2)]
    loaded, n = st.load_parameters(gpu, files, Dtype.F32)            # BF16 file -> f32 model: exact widening
    assert n == cfg.num_params() and sorted(loaded.keys()) == keys
    wb = {k: cb.bf16_bits_to_f32(cb.f32_to_bf16_bits(v)).reshape(v.shape) for k, v in w.items()}
    for k in keys:
        np.testing.assert_array_equal(gpu.to_numpy(loaded[k]), wb[k])
    ids = np.random.default_rng(1).integers(0, cfg.vocab_size, size=(2, 8), dtype=np.uint32)
    want = cb.generate_with_interpreter(oracle, cb.llama_term(oracle, cfg), cb.upload_weights(oracle, wb, Dtype.F32), cfg,
                                        ids, 4, Dtype.F32, 16)[0]
    runner = cb.LlamaRunner(gpu, cfg, loaded, Dtype.F32, max_batch=2, max_positions=16)
    np.testing.assert_array_equal(runner.generate(ids, 4), want)
    got = cb.generate_with_interpreter(gpu, cb.llama_term(gpu, cfg), loaded, cfg, ids, 4, Dtype.F32, 16)[0]
    np.testing.assert_array_equal(got, want)
    l16, _ = st.load_parameters(gpu, files, Dtype.BF16)              # kept as bf16 on the device
    assert all(l16[k].dtype == Dtype.BF16 for k in keys)
    np.testing.assert_array_equal(gpu.to_f32(l16[keys[0]]), wb[keys[0]])


@pytest.mark.parametrize("heads,kv_heads", [(8, 2), (4, 4)], ids=["hd64", "hd128"])
def test_fused_prefill_attention_with_a_cached_prefix(gpu, heads, kv_heads):
    """A prompt fed in two calls (100 tokens, then 90 more on top of the cache): the fused prefill attention then runs
    with a non-empty prefix (keys 0..99 from the cache, causal mask offset by 100, ragged last query and key tiles).
    bf16 against the f32 runner driven the same way, and against the bf16 one-call prefill of all 190 tokens."""
    cfg = cb.LlamaConfig(512, 1536, 2, heads, kv_heads, 4096, rope_theta=500000.0, rms_norm_eps=1e-5,
                         tie_word_embeddings=True)
    w = cb.random_weights(cfg, seed=4)
    wb = {k: cb.bf16_bits_to_f32(cb.f32_to_bf16_bits(v)).reshape(v.shape) for k, v in w.items()}
    B = 3
    ids = np.random.default_rng(31).integers(0, cfg.vocab_size, size=(B, 190), dtype=np.uint32)
    p16 = cb.upload_weights(gpu, wb, Dtype.BF16)
    r16 = cb.LlamaRunner(gpu, cfg, p16, Dtype.BF16, max_batch=B, max_positions=256)
    r32 = cb.LlamaRunner(gpu, cfg, cb.upload_weights(gpu, wb, Dtype.F32), Dtype.F32, max_batch=B, max_positions=256)
    for r in (r16, r32):
        r.reset(B)
        r.forward(ids[:, :100])
        r.forward(ids[:, 100:])
    two_calls = r16.last_logits().copy()
    assert np.abs(two_calls - r32.last_logits()).max() <= ABS_BF16
    tok = r16.forward(ids[:, :1] * 0 + 7)          # one decode step on top: the cache rows of both calls are in place
    r32.forward(ids[:, :1] * 0 + 7)
    assert np.abs(r16.last_logits() - r32.last_logits()).max() <= ABS_BF16
    one = cb.LlamaRunner(gpu, cfg, p16, Dtype.BF16, max_batch=B, max_positions=256)
    one.reset(B)
    one.forward(ids)
    assert np.abs(one.last_logits() - two_calls).max() <= ABS_BF16


def test_prefill_with_ragged_row_tiles_on_the_persistent_gemm(gpu):
    """5 x 333 = 1665 prompt tokens: 13 full row tiles and one of a single row, more output tiles than SMs in the
    [gate;up] product (persistent kernel, SiLU(gate)*up in the epilogue) and in the other projections (residual in the
    epilogue); bf16 against the f32 runner on the same weights, then two decode steps."""
    cfg = cb.LlamaConfig(512, 4096, 2, 8, 2, 4096, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=True)
    w = cb.random_weights(cfg, seed=6)
    wb = {k: cb.bf16_bits_to_f32(cb.f32_to_bf16_bits(v)).reshape(v.shape) for k, v in w.items()}
    B, S = 5, 333
    ids = np.random.default_rng(41).integers(0, cfg.vocab_size, size=(B, S), dtype=np.uint32)
    r16 = cb.LlamaRunner(gpu, cfg, cb.upload_weights(gpu, wb, Dtype.BF16), Dtype.BF16, max_batch=B, max_positions=S + 8)
    r32 = cb.LlamaRunner(gpu, cfg, cb.upload_weights(gpu, wb, Dtype.F32), Dtype.F32, max_batch=B, max_positions=S + 8)
    r16.reset(B)
    r32.reset(B)
    tok = r16.forward(ids)
    r32.forward(ids)
    assert np.abs(r16.last_logits() - r32.last_logits()).max() <= ABS_BF16
    for _ in range(2):
        nxt = r16.forward(tok.reshape(B, 1))
        r32.forward(tok.reshape(B, 1))
        assert np.abs(r16.last_logits() - r32.last_logits()).max() <= ABS_BF16
        tok = nxt


def test_operation_counters_see_the_op_by_op_route_only(gpu):
    """cg_op_stats on the CUDA backend: a Llama term that runs as the fused plan evaluates no edge and records nothing; the
    same term op by op records every edge (synchronised timing mode)."""
    cfg, w, _ = tiny_inputs()
    params = cb.upload_weights(gpu, w, Dtype.F32)
    ids = np.random.default_rng(2).integers(0, cfg.vocab_size, size=(1, 6), dtype=np.uint32)
    try:
        gpu.op_stats(mode=2, reset=True)
        term = cb.llama_term(gpu, cfg)
        planned = cb.generate_with_interpreter(gpu, term, params, cfg, ids, 2, Dtype.F32, 12)[0]
        assert term.plan_state == 1 and gpu.op_stats() == {}
        gpu._ns.interp_set_planning(0)
        term2 = cb.llama_term(gpu, cfg)
        stepwise = cb.generate_with_interpreter(gpu, term2, params, cfg, ids, 2, Dtype.F32, 12)[0]
        st = gpu.op_stats()
    finally:
        gpu._ns.interp_set_planning(1)
        gpu.op_stats(mode=0, reset=True)
    np.testing.assert_array_equal(planned, stepwise)
    assert st["MatMul"]["count"] == 2 * (9 * cfg.num_hidden_layers + 1) and st["Argmax"]["count"] == 2
    assert sum(v["ms"] for v in st.values()) > 0.0

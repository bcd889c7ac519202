"""Host-side checks that need no GPU: the C-ABI library loads and exports what include/*.h declares, the term
builder/evaluator behave like the reference's, and the Llama term is a Llama."""
import ctypes
import os
import re

import numpy as np
import pytest

import catgrad_b200 as cb
from catgrad_b200 import Dtype, NodeType, OpKind
from catgrad_b200 import _ffi
import helpers
import llama_numpy

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "catgrad_b200.h")).read()
    names = sorted(set(re.findall(r"\b(cg_[a-z0-9_]+)\s*\(", hdr)))
    assert len(names) > 70
    path = _ffi.library_path()
    assert os.path.exists(path), "build the library first: python -m catgrad_b200._build"
    lib = ctypes.CDLL(path)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    _ffi.bind(lib, "cg_")          # every symbol the host wrapper binds exists too


def _param_count(arglist):
    arglist = re.sub(r"/\*.*?\*/", "", arglist, flags=re.S).strip()
    return 0 if arglist in ("", "void") else arglist.count(",") + 1


def test_rust_shim_binds_existing_entry_points_with_matching_arity():
    """shim/b200.rs cannot be compiled here (no Rust toolchain); at least every `cg_*` function it declares must be
    exported by the library and take as many arguments as the header says."""
    hdr = open(os.path.join(ROOT, "include", "catgrad_b200.h")).read()
    rs = open(os.path.join(ROOT, "shim", "b200.rs")).read()
    header_args = {m.group(1): _param_count(m.group(2))
                   for m in re.finditer(r"\b(cg_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", hdr, flags=re.S)}
    decls = re.findall(r"\bfn (cg_[a-z0-9_]+)\s*\(([^)]*)\)", rs)
    assert len(decls) >= 45
    lib = ctypes.CDLL(_ffi.library_path())
    for name, args in decls:
        assert hasattr(lib, name), name
        assert name in header_args, name
        assert _param_count(args) == header_args[name], (name, args, header_args[name])
    # all 41 trait methods are implemented
    trait_methods = ["zeros", "ndarray_from_vec_f32", "ndarray_from_vec_f16", "ndarray_from_vec_bf16",
                     "ndarray_from_vec_fp8", "ndarray_from_vec_u32", "cast", "matmul", "add", "sub", "mul", "div", "pow",
                     "lt", "gt", "gte", "lte", "eq", "where_cond", "sin", "cos", "exp", "log", "floor", "round", "neg",
                     "broadcast", "reshape", "transpose", "max", "sum", "argmax", "topk", "compare", "concat", "index",
                     "slice", "arange", "to_bool", "to_vec", "format_tensor"]
    body = rs[rs.index("impl Backend for B200Backend"):]
    for mth in trait_methods:
        assert re.search(r"\bfn %s\s*\(" % mth, body), mth


def test_no_cpu_fallback():
    """Without a GPU the product refuses to start; nothing silently computes on the host."""
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        pytest.skip("a GPU is present")
    with pytest.raises(cb.BackendError) as e:
        cb.Backend(0)
    assert e.value.status == cb.Status.CUDA


def test_product_sources_do_not_reach_into_the_oracle():
    for base in ("catgrad_b200", "include"):
        for root, _, files in os.walk(os.path.join(ROOT, base)):
            for f in files:
                if f.endswith((".py", ".cc", ".cu", ".cuh", ".h")):
                    text = open(os.path.join(root, f)).read()
                    assert "oracle/" not in text and "ndarray_ref" not in text, os.path.join(root, f)


def test_builder_inserts_copies_and_evaluator_consumes_once(oracle):
    tb = cb.TermBuilder(oracle)
    x = tb.source()
    y = x * x + x                       # x used three times -> one Copy edge with three outputs
    term = tb.finish([y, x])            # and once more as an output
    st = term.stats()
    assert st["tensor_ops"] == 2 and st["edges"] == 3
    a = oracle.from_numpy(np.array([1.0, 2.0, 3.0], np.float32))
    r = cb.Interpreter(oracle).run(term, [a])
    assert oracle.to_numpy(r[0]).tolist() == [2.0, 6.0, 12.0]
    assert oracle.to_numpy(r[1]).tolist() == [1.0, 2.0, 3.0]


def test_interpreter_errors(oracle):
    tb = cb.TermBuilder(oracle)
    x, y = tb.source(), tb.source()
    term = tb.finish([x + y])
    interp = cb.Interpreter(oracle)
    f = oracle.from_numpy(np.zeros(3, np.float32))
    u = oracle.from_numpy(np.zeros(3, np.uint32))
    with pytest.raises(cb.BackendError) as e:
        interp.run(term, [f, u])                       # TypeError: dtypes of one op differ
    assert e.value.status == cb.Status.DTYPE_MISMATCH
    with pytest.raises(cb.BackendError) as e:
        interp.run(term, [f])                          # wrong number of inputs
    assert e.value.status == cb.Status.INTERP
    tb = cb.TermBuilder(oracle)
    term = tb.finish([tb.param("no.such.weight")])
    with pytest.raises(cb.BackendError) as e:
        cb.Interpreter(oracle, cb.Parameters(oracle)).run(term, [])
    assert "no.such.weight" in str(e.value)


def test_nat_shape_and_dtype_values(oracle):
    tb = cb.TermBuilder(oracle)
    x = tb.source()
    d = tb.unpack(tb.shape(x), 3)
    n = tb.nat_add(tb.nat_mul(d[0], d[1]), d[2])
    term = tb.finish([n, tb.shape(x), tb.dtype(x), tb.nat_to_u32(d[2])])
    r = cb.Interpreter(oracle).run(term, [oracle.zeros((2, 3, 5), Dtype.U32)])
    assert r[0] == 11 and r[1] == (2, 3, 5) and r[2] == Dtype.U32
    assert oracle.to_numpy(r[3]).tolist() == 5


def test_llama_term_shape(oracle):
    """~137 tensor ops per layer plus prologue/epilogue; prefill and decode run the same term."""
    t2 = cb.llama_term(oracle, cb.TINY).stats()
    cfg4 = cb.LlamaConfig(256, 688, 4, 4, 4, 1024)
    t4 = cb.llama_term(oracle, cfg4).stats()
    per_layer = (t4["tensor_ops"] - t2["tensor_ops"]) / 2
    assert 120 <= per_layer <= 150
    assert t2["layers"] < t2["edges"]


def test_tiny_llama_oracle_equals_textbook_llama(oracle):
    cfg = cb.TINY
    w = cb.random_weights(cfg, 0)
    ids = np.random.default_rng(1).integers(0, cfg.vocab_size, size=(1, 64), dtype=np.uint32)
    term = cb.llama_term(oracle, cfg, tap_logits=True)
    params = cb.upload_weights(oracle, w, Dtype.F32)
    out, logits = cb.generate_with_interpreter(oracle, term, params, cfg, ids, 3, Dtype.F32, 96, tap=True)
    lg, cache = llama_numpy.forward(cfg, w, ids.astype(np.int64))
    assert helpers.rel_err(logits[0], lg) < 1e-5
    assert int(lg[0, -1].argmax()) == int(out[0, 0])
    lg2, cache = llama_numpy.forward(cfg, w, out[:, :1].astype(np.int64), cache)
    assert helpers.rel_err(logits[1], lg2) < 1e-5
    # GQA + tied head + batch 2 take the other branches of the term
    cfg2 = cb.LlamaConfig(128, 256, 2, 8, 2, 512, rope_theta=500000.0, tie_word_embeddings=True)
    w2 = cb.random_weights(cfg2, 3)
    ids2 = np.random.default_rng(4).integers(0, 512, size=(2, 9), dtype=np.uint32)
    term2 = cb.llama_term(oracle, cfg2, tap_logits=True)
    out2, logits2 = cb.generate_with_interpreter(oracle, term2, cb.upload_weights(oracle, w2, Dtype.F32), cfg2, ids2, 1,
                                                 Dtype.F32, 16, tap=True)
    lgb, _ = llama_numpy.forward(cfg2, w2, ids2.astype(np.int64))
    assert helpers.rel_err(logits2[0], lgb) < 1e-5


def test_config1_golden_ids(oracle):
    """Config 1 of the baseline (tiny f32 model, seed-0 weights, seed-1 prompt, 32 greedy steps after the prefill
    token) against the committed fixture written by tests/golden/make_tiny_llama_fixture.py."""
    import json
    fx = json.load(open(os.path.join(helpers.GOLDEN, "tiny_llama_c1.json")))
    cfg = cb.TINY
    w = cb.random_weights(cfg, fx["weight_seed"])
    ids = np.random.default_rng(fx["prompt_seed"]).integers(0, cfg.vocab_size, size=(1, 64), dtype=np.uint32)
    assert ids[0, :8].tolist() == fx["prompt_head"]
    term = cb.llama_term(oracle, cfg, tap_logits=True)
    params = cb.upload_weights(oracle, w, Dtype.F32)
    out, logits = cb.generate_with_interpreter(oracle, term, params, cfg, ids, 33, Dtype.F32, 97, tap=True)
    assert out[0].tolist() == fx["ids"]
    np.testing.assert_allclose(logits[0][0, -1, :16], np.array(fx["prefill_logits_head"], np.float32), rtol=1e-5, atol=1e-6)


def test_reduced_precision_conversions(oracle):
    """The oracle's bf16/f16 rounding against numpy's (f16) and the bit formula (bf16), incl. ties, subnormals, NaN."""
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(5000) * 10.0 ** rng.integers(-8, 6, 5000),
                        [0.0, -0.0, np.inf, -np.inf, np.nan, 65504.0, 65519.9, 65520.0, 6e-8, 2.98e-8, 2.99e-8, 1.00390625]]).astype(np.float32)
    t = oracle.from_numpy(x)
    h = oracle.to_numpy(oracle.cast(t, Dtype.F16))
    with np.errstate(over="ignore"):
        want = x.astype(np.float16)
    np.testing.assert_array_equal(h.view(np.uint16)[~np.isnan(x)], want.view(np.uint16)[~np.isnan(x)])
    assert np.isnan(h[np.isnan(x)]).all()
    b = oracle.to_numpy(oracle.cast(t, Dtype.BF16))
    wantb = cb.f32_to_bf16_bits(x)
    np.testing.assert_array_equal(b[~np.isnan(x)], wantb[~np.isnan(x)])
    back = oracle.to_numpy(oracle.cast(oracle.cast(t, Dtype.F16), Dtype.F32))
    np.testing.assert_array_equal(back[~np.isnan(x)], want.astype(np.float32)[~np.isnan(x)])


def _probe_term(be):
    tb = cb.TermBuilder(be)
    x = tb.source(cb.NodeType.Tensor)
    y = x + x
    tb.probe("doubled", y)
    return tb.finish([y])


def test_probe_prints_only_when_asked_and_format_names_dtype_shape_values(oracle, capfd, monkeypatch):
    """Probe (tensor_op.rs:121-136): a debug print of format_tensor, only with CATGRAD_PROBE set, no outputs."""
    x = np.array([[1.5, -2.0, 3.25]], np.float32)
    term = _probe_term(oracle)
    monkeypatch.delenv("CATGRAD_PROBE", raising=False)
    out = cb.Interpreter(oracle).run(term, [oracle.from_numpy(x)])
    assert len(out) == 1 and "[probe:" not in capfd.readouterr().out
    monkeypatch.setenv("CATGRAD_PROBE", "1")
    out = cb.Interpreter(oracle).run(term, [oracle.from_numpy(x)])
    np.testing.assert_array_equal(oracle.to_numpy(out[0]), 2 * x)
    text = capfd.readouterr().out
    assert "[probe:doubled]" in text and "f32" in text and "[1,3]" in text and "-4" in text and "6.5" in text
    # format_tensor on its own: dtype, shape, leading values; u32 and bf16 too
    assert "u32" in oracle.format_tensor(oracle.from_numpy(np.arange(5, dtype=np.uint32)))
    s = oracle.format_tensor(oracle.from_numpy(np.array([0.5, 2.0], np.float32), cb.Dtype.BF16))
    assert "bf16" in s and "0.5" in s and "2" in s


LLAMA3_SCALING = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                  "original_max_position_embeddings": 8192}


def test_llama3_rope_scaling_term_equals_textbook_llama(oracle):
    """rope_scaling "llama3" (helpers/rope.rs:232-310; what Llama-3.1/3.2 checkpoints configure): the term's tables against
    the published formula in float64.  Head dim 64 with theta 5e5 has frequencies in all three bands (kept, blended,
    divided by 32), and positions in the hundreds make the difference to unscaled tables large."""
    cfg = cb.LlamaConfig(128, 256, 2, 2, 1, 512, rope_theta=500000.0, tie_word_embeddings=True, rope_scaling=LLAMA3_SCALING)
    inv = 1.0 / 500000.0 ** (np.arange(32) * 2.0 / 64)
    scaled = llama_numpy.llama3_inv_freq(inv, LLAMA3_SCALING)
    ratio = scaled / inv
    assert (ratio == 1.0).any() and np.isclose(ratio, 1 / 32).any() and ((ratio > 1 / 32 + 1e-3) & (ratio < 1 - 1e-3)).any()
    w = cb.random_weights(cfg, 5)
    ids = np.random.default_rng(6).integers(0, 512, size=(2, 300), dtype=np.uint32)
    term = cb.llama_term(oracle, cfg, tap_logits=True)
    params = cb.upload_weights(oracle, w, Dtype.F32)
    out, logits = cb.generate_with_interpreter(oracle, term, params, cfg, ids, 2, Dtype.F32, 320, tap=True)
    lg, cache = llama_numpy.forward(cfg, w, ids.astype(np.int64))
    assert helpers.rel_err(logits[0][:, -1], lg[:, -1]) < 2e-5
    lg2, _ = llama_numpy.forward(cfg, w, out[:, :1].astype(np.int64), cache)
    assert helpers.rel_err(logits[1][:, -1], lg2[:, -1]) < 2e-5
    # and the scaling matters at these positions: the unscaled model is far away
    plain = cb.LlamaConfig(128, 256, 2, 2, 1, 512, rope_theta=500000.0, tie_word_embeddings=True)
    lg0, _ = llama_numpy.forward(plain, w, ids.astype(np.int64))
    assert helpers.rel_err(lg0[:, -1], lg[:, -1]) > 1e-4       # ten times the agreement asked for above
    with pytest.raises(ValueError):
        cb.LlamaConfig(128, 256, 2, 2, 1, 512, rope_scaling={"rope_type": "yarn", "factor": 4.0}).to_struct()


def test_bench_table_has_the_reference_layout():
    """print_bench_table (catgrad-llm/src/utils/mod.rs:528-566): header, rule, a pp row and a tg row; widths and
    precision as the reference formats them."""
    lines = cb.bench_table("llama-3.2-1b", 2.30, 1235.81, "b200", 512, 0.004, 128, 0.1)
    assert len(lines) == 4 and len({len(x) for x in lines}) == 1
    assert lines[0].startswith("| model ") and lines[0].endswith("t/s |") and set(lines[1]) <= set("| -")
    cells = [c.strip() for c in lines[2].split("|")[1:-1]]
    assert cells == ["llama-3.2-1b", "2.30 GiB", "1235.81 M", "b200", "pp512", "128000.00"]
    assert [c.strip() for c in lines[3].split("|")[1:-1]][-2:] == ["tg128", "1280.00"]


def test_per_operation_counters_of_the_evaluator(oracle):
    """cg_op_stats*: off by default; when on, every evaluated edge of a term is counted under its operation's name (the
    Llama term: 7 linear layers per layer + the head as MatMul, one Argmax, one Load per parameter) and timed; a reset
    clears them; the mode is process-wide, so it is switched off again here."""
    cfg = cb.TINY
    w = cb.random_weights(cfg, seed=0)
    params = cb.upload_weights(oracle, w, cb.Dtype.F32)
    term = cb.llama_term(oracle, cfg)
    ids = np.random.default_rng(0).integers(0, cfg.vocab_size, size=(1, 5), dtype=np.uint32)
    assert oracle.op_stats(mode=0, reset=True) == {}
    cb.generate_with_interpreter(oracle, term, params, cfg, ids, 1, cb.Dtype.F32, 8)
    assert oracle.op_stats() == {}                      # off: nothing recorded
    try:
        oracle.op_stats(mode=2)
        cb.generate_with_interpreter(oracle, term, params, cfg, ids, 1, cb.Dtype.F32, 8)
        st = oracle.op_stats()
    finally:
        oracle.op_stats(mode=0)
    L = cfg.num_hidden_layers
    # q, k, v, o, gate, up, down per layer, the head, and the two attention products per layer
    assert st["MatMul"]["count"] == 9 * L + 1
    assert st["Argmax"]["count"] == 1
    assert st["Load"]["count"] == len(cfg.param_shapes())
    assert all(v["count"] > 0 and v["ms"] >= 0.0 for v in st.values())
    assert any(k.startswith("Map.") for k in st) and "Concat" in st and "Broadcast" in st
    assert oracle.op_stats(reset=True) == {}

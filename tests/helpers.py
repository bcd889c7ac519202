"""Shared test helpers: running golden cases on a backend, the reference's helper graphs, comparisons."""
import json
import os

import numpy as np

import catgrad_b200 as cb
from catgrad_b200 import Dtype, NodeType, ScalarOp

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DT = {"f32": Dtype.F32, "u32": Dtype.U32, "bf16": Dtype.BF16, "f16": Dtype.F16}
NP = {"f32": np.float32, "u32": np.uint32}


def golden_cases(kind=None):
    with open(os.path.join(GOLDEN, "reference_vectors.json")) as f:
        cases = json.load(f)["cases"]
    return [c for c in cases if kind is None or c["kind"] == kind]


def make_input(be, t, dtype):
    arr = np.array(t["data"], dtype=NP[dtype]).reshape(t["shape"])
    return be.from_numpy(arr)


def call_op(be, case):
    """Runs one golden 'op' or 'error' case through the Backend methods; returns a list of result tensors."""
    xs = [make_input(be, t, case["dtype"]) for t in case["inputs"]]
    op, args = case["op"], case.get("args", [])
    if op in ("add", "sub", "mul", "div", "pow", "matmul", "lt", "gt", "gte", "lte", "eq"):
        return [getattr(be, op)(xs[0], xs[1])]
    if op in ("sum", "max", "argmax", "log", "exp", "floor", "neg", "round", "sin", "cos"):
        return [getattr(be, op)(xs[0])]
    if op == "reshape":
        return [be.reshape(xs[0], args[0])]
    if op == "broadcast":
        return [be.broadcast(xs[0], args[0])]
    if op == "cast":
        return [be.cast(xs[0], DT[args[0]])]
    if op == "topk":
        return list(be.topk(xs[0], args[0]))
    raise KeyError(op)


def call_op_via_interpreter(be, case):
    """Same, but as a one-op term through the interpreter (the reference's tests/test_interpreter.rs)."""
    tb = cb.TermBuilder(be)
    srcs = [tb.source(NodeType.Tensor) for _ in case["inputs"]]
    op = case["op"]
    if op == "add":
        outs = [srcs[0] + srcs[1]]
    elif op == "matmul":
        outs = [tb.matmul(srcs[0], srcs[1])]
    elif op == "exp":
        outs = [tb.exp(srcs[0])]
    elif op == "topk":
        outs = list(tb.topk(case["args"][0], srcs[0]))
    else:
        raise KeyError(op)
    term = tb.finish(outs)
    xs = [make_input(be, t, case["dtype"]) for t in case["inputs"]]
    return cb.Interpreter(be).run(term, xs)


def check_expect(be, results, case):
    assert len(results) == len(case["expect"])
    for r, e in zip(results, case["expect"]):
        assert r.dtype == DT[e["dtype"]], (case["name"], r.dtype)
        assert list(r.shape) == e["shape"], (case["name"], r.shape)
        got = be.to_numpy(r).reshape(-1)
        want = np.array(e["data"], dtype=NP[e["dtype"]])
        if "atol" in case or "rtol" in case:
            np.testing.assert_allclose(got, want, rtol=case.get("rtol", 0), atol=case.get("atol", 0), err_msg=case["name"])
        else:
            np.testing.assert_array_equal(got, want, err_msg=case["name"])


# ---- the reference's helper definitions, restated with the term builder --------------------------------
# catgrad-llm-models/src/helpers/tensors.rs (chunk/split :5-25, squeeze/unsqueeze :27-45, repeat_interleave :128-151,
# avgpool2d :153-185, clamp :187-205, where_broadcast :274-282, masked_fill :284-288, tril_mask/cumsum :306-350)
def squeeze(tb, n, dim, x):
    s = tb.unpack(tb.shape(x), n)
    s.pop(dim)
    return tb.reshape(tb.pack(s), x)


def unsqueeze(tb, n, dim, x):
    s = tb.unpack(tb.shape(x), n)
    s.insert(dim, tb.nat(1))
    return tb.reshape(tb.pack(s), x)


def repeat_interleave(tb, dim, rep, x):
    x = unsqueeze(tb, 4, dim + 1, x)
    sh = tb.unpack(tb.shape(x), 5)
    sh[dim + 1] = tb.nat(rep)
    orig = sh[dim]
    x = tb.broadcast(tb.pack(sh), x)
    sh.pop(dim + 1)
    sh[dim] = tb.nat_mul(orig, rep)
    return tb.reshape(tb.pack(sh), x)


def clamp(tb, x, lo, hi):
    sh = tb.shape(x)
    dt = tb.dtype(x)
    mn = tb.cast(tb.constant(float(lo), sh), dt)
    mx = tb.cast(tb.constant(float(hi), sh), dt)
    below = tb.cast(tb.lt(x, mn), dt)
    x = tb.where_cond(below, mn, x)
    above = tb.cast(tb.lt(mx, x), dt)
    return tb.where_cond(above, mx, x)


def tril_mask(tb, size):
    sh = tb.pack([size, size])
    diag = tb.constant(0, sh)
    idx = tb.arange(size)
    row = tb.reshape(tb.pack([size, 1]), idx)
    col = tb.reshape(tb.pack([1, size]), idx)
    row = tb.broadcast(sh, row)
    col = tb.broadcast(sh, col)
    row = row + diag
    return tb.cast(tb.lte(col, row), Dtype.F32)


def build_graph(tb, name):
    """Returns (sources, targets) of the named helper graph."""
    T = NodeType.Tensor
    if name == "if_double":
        x, c = tb.source(T), tb.source(T)
        t_then = cb.TermBuilder(tb._be)
        a = t_then.source(T)
        then_term = t_then.finish([a + a])
        t_else = cb.TermBuilder(tb._be)
        b = t_else.source(T)
        else_term = t_else.finish([b])
        tb._keep = (then_term, else_term)
        return [x, c], tb.cond(c, then_term, else_term, [x], [T])
    if name == "split_2_2":
        x = tb.source(T)
        return [x], [tb.slice(1, 0, 2, x), tb.slice(1, 2, 2, x)]
    if name == "squeeze_3_1":
        x = tb.source(T)
        return [x], [squeeze(tb, 3, 1, x)]
    if name == "unsqueeze_2_1":
        x = tb.source(T)
        return [x], [unsqueeze(tb, 2, 1, x)]
    if name == "repeat_kv_3":
        x = tb.source(T)
        return [x], [repeat_interleave(tb, 1, 3, x)]
    if name == "repeat_interleave_2_2":
        x = tb.source(T)
        return [x], [repeat_interleave(tb, 2, 2, x)]
    if name == "clamp_m1_1p5":
        x = tb.source(T)
        return [x], [clamp(tb, x, -1.0, 1.5)]
    if name == "avgpool2d_1_2_2":
        x = tb.source(T)
        dim, h, w, k = 1, 2, 2, 2
        y = tb.reshape(tb.pack([1, dim, h // k, k, w // k, k]), x)
        y = tb.transpose(3, 4, y)
        y = tb.reshape(tb.pack([1, dim, (h // k) * (w // k), k * k]), y)
        y = tb.sum(y)
        return [x], [y * tb.constant(1.0 / (k * k), tb.shape(y))]
    if name == "where_broadcast":
        m, x, y = tb.source(T), tb.source(T), tb.source(T)
        mm = tb.cast(tb.broadcast(tb.shape(x), m), tb.dtype(x))
        return [m, x, y], [tb.where_cond(mm, x, y)]
    if name == "masked_fill_9":
        m, x = tb.source(T), tb.source(T)
        fill = tb.constant(9.0, tb.shape(x))
        return [m, x], [tb.where_cond(m, fill, x)]
    if name == "cumsum_4":
        x = tb.source(T)
        sh = tb.unpack(tb.shape(x), 4)
        ldim = sh[3]
        new_sh = tb.pack([sh[0], sh[1], ldim, ldim])
        lower = tb.transpose(0, 1, tril_mask(tb, ldim))
        lower = tb.broadcast(new_sh, lower)
        return [x], [tb.matmul(x, lower)]
    raise KeyError(name)


def run_graph_case(be, case):
    tb = cb.TermBuilder(be)
    srcs, outs = build_graph(tb, case["graph"])
    term = tb.finish(outs)
    xs = [make_input(be, t, case["dtype"]) for t in case["inputs"]]
    return cb.Interpreter(be).run(term, xs)


def rel_err(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


# ---- the bf16 bar at full model dimensions ---------------------------------------------------------------
def bf16_semantics(name):
    """tests/golden/<name>_bf16_semantics.json: how far the reference's own bf16 semantics (the CPU oracle rounding every
    op output to bf16) land from its f32 run on a fixed model and prompt; written by make_llama1b_bf16_semantics.py."""
    with open(os.path.join(GOLDEN, name + "_bf16_semantics.json")) as f:
        return json.load(f)


def check_bf16_against_f32(sem, step, got, want, small_bar=2e-2, max_factor=1.25, mean_factor=1.25):
    """bf16 logits `got` of call `step` (0 = prefill; None = the worst call of the fixture) against f32 logits `want`: no
    worse than the reference semantics themselves by more than the given factors, never tighter than the small-model
    bar; and the same greedy id wherever the f32 top-2 gap clearly exceeds the error."""
    pick = (lambda v: max(v)) if step is None else (lambda v: v[step])
    d = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))
    max_bar = max(small_bar, max_factor * pick(sem["bf16_vs_f32_max_abs"]))
    mean_bar = mean_factor * pick(sem["bf16_vs_f32_mean_abs"])
    assert d.max() <= max_bar, ("max-abs", step, float(d.max()), max_bar)
    assert d.mean() <= mean_bar, ("mean-abs", step, float(d.mean()), mean_bar)
    if step is not None and got.ndim == 1 and sem["top2_gap_f32"][step] > 2 * d.max():
        assert int(np.argmax(got)) == int(np.argmax(want))

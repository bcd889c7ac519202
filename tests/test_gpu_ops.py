"""Parity of the CUDA backend with the CPU oracle, op by op, through the C ABI.

Bit-exact for integer/index/shape ops and for the correctly-rounded float ops (add/sub/mul/div/neg/floor/round/
compare/where/cast/max); libm-vs-CUDA ulp tolerance for exp/log/sin/cos/pow; accumulation-order tolerance for
sum/matmul (tolerances stated per test)."""
import numpy as np
import pytest

import catgrad_b200 as cb
from catgrad_b200 import Dtype
import helpers

pytestmark = pytest.mark.gpu

FLOAT_DTYPES = [Dtype.F32, Dtype.BF16, Dtype.F16]


def both(oracle, gpu, arr, dtype=None):
    return oracle.from_numpy(arr, dtype), gpu.from_numpy(arr, dtype)


def same_bits(oracle, gpu, ro, rg, what=""):
    assert ro.dtype == rg.dtype and ro.shape == rg.shape
    a, b = oracle.to_numpy(ro), gpu.to_numpy(rg)
    # bit patterns must agree, except that a NaN may carry any payload (x86 and the GPU pick different ones)
    if ro.dtype == Dtype.BF16:
        nan = (a & 0x7FFF) > 0x7F80
        assert ((b & 0x7FFF) > 0x7F80)[nan].all()
        a, b = np.where(nan, 0, a), np.where(nan, 0, b)
    elif a.dtype in (np.float32, np.float16):
        nan = np.isnan(a)
        assert np.isnan(b[nan]).all()
        bits = np.uint32 if a.dtype == np.float32 else np.uint16
        a, b = np.where(nan, 0, a.view(bits)), np.where(nan, 0, b.view(bits))
    np.testing.assert_array_equal(a, b, err_msg=what)


@pytest.mark.parametrize("case", helpers.golden_cases("op"), ids=lambda c: c["name"])
def test_reference_vectors(gpu, case):
    run = helpers.call_op_via_interpreter if case.get("via_interpreter") else helpers.call_op
    helpers.check_expect(gpu, run(gpu, case), case)


@pytest.mark.parametrize("case", helpers.golden_cases("error"), ids=lambda c: c["name"])
def test_shape_mismatch_is_refused(gpu, case):
    with pytest.raises(cb.BackendError) as e:
        helpers.call_op(gpu, case)
    assert e.value.status.name == case["error"]
    assert "Shape mismatch in operation" in str(e.value)


@pytest.mark.parametrize("case", helpers.golden_cases("graph"), ids=lambda c: c["name"])
def test_helper_graphs(gpu, case):
    helpers.check_expect(gpu, helpers.run_graph_case(gpu, case), case)


@pytest.mark.parametrize("dtype", FLOAT_DTYPES, ids=lambda d: d.name)
@pytest.mark.parametrize("shape", [(4096, 1024), (37, 129), (1,), (3, 5, 7, 2), (0, 4)], ids=str)
def test_exact_float_binary_ops(oracle, gpu, dtype, shape):
    rng = np.random.default_rng(2)
    a = rng.uniform(-4, 4, shape).astype(np.float32)
    b = rng.uniform(-4, 4, shape).astype(np.float32)
    if a.size > 4:
        b.reshape(-1)[:3] = [0.0, -0.0, np.inf]
        a.reshape(-1)[:3] = [1.0, -1.0, np.nan]
    ao, ag = both(oracle, gpu, a, dtype)
    bo, bg = both(oracle, gpu, b, dtype)
    for op in ("add", "sub", "mul", "div", "lt", "gt", "gte", "lte", "eq"):
        same_bits(oracle, gpu, getattr(oracle, op)(ao, bo), getattr(gpu, op)(ag, bg))
    same_bits(oracle, gpu, oracle.where_cond(ao, ao, bo), gpu.where_cond(ag, ag, bg))
    for op in ("neg", "floor", "round"):
        same_bits(oracle, gpu, getattr(oracle, op)(ao), getattr(gpu, op)(ag))


def test_broadcast_row_vector_sweep_shape(oracle, gpu):
    """The op-sweep layout: [4096, 8192] against an explicitly broadcast [8192] row vector (scaled down in rows
    so the CPU oracle finishes in seconds; the row length is the full 8192)."""
    rng = np.random.default_rng(2)
    x = rng.uniform(-4, 4, (256, 8192)).astype(np.float32)
    v = rng.uniform(-4, 4, (8192,)).astype(np.float32)
    for dtype in (Dtype.F32, Dtype.BF16):
        xo, xg = both(oracle, gpu, x, dtype)
        vo, vg = both(oracle, gpu, v, dtype)
        bo, bg = oracle.broadcast(vo, x.shape), gpu.broadcast(vg, x.shape)
        assert bg.strides == (0, 1)          # a view, not a copy
        for op in ("add", "mul", "div"):
            same_bits(oracle, gpu, getattr(oracle, op)(xo, bo), getattr(gpu, op)(xg, bg))
        eo, eg = oracle.exp(xo), gpu.exp(xg)
        tol = 2e-6 if dtype == Dtype.F32 else 1e-2
        np.testing.assert_allclose(gpu.to_f32(eg), oracle.to_f32(eo), rtol=tol)


def test_strided_and_column_broadcast_operands(oracle, gpu):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((6, 10, 12)).astype(np.float32)
    y = rng.standard_normal((6, 12, 10)).astype(np.float32)
    c = rng.standard_normal((6, 10, 1)).astype(np.float32)
    for dtype in (Dtype.F32, Dtype.BF16):
        xo, xg = both(oracle, gpu, x, dtype)
        yo, yg = both(oracle, gpu, y, dtype)
        co, cg = both(oracle, gpu, c, dtype)
        same_bits(oracle, gpu, oracle.add(xo, oracle.transpose(yo, 1, 2)), gpu.add(xg, gpu.transpose(yg, 1, 2)))
        same_bits(oracle, gpu, oracle.sub(xo, oracle.broadcast(co, x.shape)), gpu.sub(xg, gpu.broadcast(cg, x.shape)))
        so, sg = oracle.slice(xo, 2, 3, 5), gpu.slice(xg, 2, 3, 5)
        same_bits(oracle, gpu, oracle.mul(so, so), gpu.mul(sg, sg))
        same_bits(oracle, gpu, oracle.reshape(oracle.transpose(xo, 0, 2), (12, 60)), gpu.reshape(gpu.transpose(xg, 0, 2), (12, 60)))


def test_u32_ops(oracle, gpu):
    rng = np.random.default_rng(4)
    a = rng.integers(0, 2**32, (33, 17), dtype=np.uint32)
    b = rng.integers(1, 2**32, (33, 17), dtype=np.uint32)
    ao, ag = both(oracle, gpu, a)
    bo, bg = both(oracle, gpu, b)
    for op in ("add", "sub", "mul", "div", "lt", "gt", "gte", "lte", "eq"):
        same_bits(oracle, gpu, getattr(oracle, op)(ao, bo), getattr(gpu, op)(ag, bg))
    e = rng.integers(0, 6, (33, 17), dtype=np.uint32)
    eo, eg = both(oracle, gpu, e)
    same_bits(oracle, gpu, oracle.pow(ao, eo), gpu.pow(ag, eg))
    same_bits(oracle, gpu, oracle.neg(ao), gpu.neg(ag))
    same_bits(oracle, gpu, oracle.where_cond(eo, ao, bo), gpu.where_cond(eg, ag, bg))
    same_bits(oracle, gpu, oracle.sum(ao), gpu.sum(ag))
    same_bits(oracle, gpu, oracle.max(ao), gpu.max(ag))
    same_bits(oracle, gpu, oracle.argmax(ao), gpu.argmax(ag))
    small = rng.integers(0, 50, (4, 6, 5), dtype=np.uint32)
    so, sg = both(oracle, gpu, small)
    same_bits(oracle, gpu, oracle.matmul(so, oracle.transpose(so, 1, 2)), gpu.matmul(sg, gpu.transpose(sg, 1, 2)))
    with pytest.raises(cb.BackendError):
        gpu.sin(ag)


@pytest.mark.parametrize("dtype", FLOAT_DTYPES, ids=lambda d: d.name)
def test_transcendentals(oracle, gpu, dtype):
    """libm (the reference's f32::exp etc.) vs CUDA's full-precision functions: a few ulp in f32."""
    rng = np.random.default_rng(5)
    x = rng.uniform(-4, 4, (513, 77)).astype(np.float32)
    xo, xg = both(oracle, gpu, x, dtype)
    rtol, atol = (4e-6, 1e-6) if dtype == Dtype.F32 else (1e-2, 1e-2)
    for op in ("exp", "sin", "cos"):
        np.testing.assert_allclose(gpu.to_f32(getattr(gpu, op)(xg)), oracle.to_f32(getattr(oracle, op)(xo)), rtol=rtol, atol=atol)
    p = np.abs(x) + 0.5
    po, pg = both(oracle, gpu, p, dtype)
    np.testing.assert_allclose(gpu.to_f32(gpu.log(pg)), oracle.to_f32(oracle.log(po)), rtol=rtol, atol=atol)
    np.testing.assert_allclose(gpu.to_f32(gpu.pow(pg, xg)), oracle.to_f32(oracle.pow(po, xo)), rtol=2e-5 if dtype == Dtype.F32 else 2e-2)


def test_casts(oracle, gpu):
    rng = np.random.default_rng(6)
    x = np.concatenate([rng.uniform(-10, 300, 1000), [np.nan, np.inf, -np.inf, 5e9, -0.0, 0.49999997, 2.5, 16777217.0]]).astype(np.float32)
    xo, xg = both(oracle, gpu, x)
    for target in (Dtype.U32, Dtype.BF16, Dtype.F16, Dtype.F32):
        same_bits(oracle, gpu, oracle.cast(xo, target), gpu.cast(xg, target))
    u = rng.integers(0, 2**32, 1000, dtype=np.uint32)
    uo, ug = both(oracle, gpu, u)
    for target in (Dtype.F32, Dtype.BF16, Dtype.F16):
        same_bits(oracle, gpu, oracle.cast(uo, target), gpu.cast(ug, target))
    bo, bg = both(oracle, gpu, x, Dtype.BF16)
    for target in (Dtype.F32, Dtype.U32, Dtype.F16):
        same_bits(oracle, gpu, oracle.cast(bo, target), gpu.cast(bg, target))
    # strided source
    m = rng.standard_normal((9, 16)).astype(np.float32)
    mo, mg = both(oracle, gpu, m)
    same_bits(oracle, gpu, oracle.cast(oracle.transpose(mo, 0, 1), Dtype.BF16), gpu.cast(gpu.transpose(mg, 0, 1), Dtype.BF16))


@pytest.mark.parametrize("shape", [(512, 4096), (7, 3, 1000), (5, 1), (3, 33)], ids=str)
def test_reductions(oracle, gpu, shape):
    rng = np.random.default_rng(7)
    x = rng.standard_normal(shape).astype(np.float32)
    for dtype in (Dtype.F32, Dtype.BF16):
        xo, xg = both(oracle, gpu, x, dtype)
        same_bits(oracle, gpu, oracle.max(xo), gpu.max(xg))
        same_bits(oracle, gpu, oracle.argmax(xo), gpu.argmax(xg))
        tol = 1e-5 if dtype == Dtype.F32 else 1e-2
        np.testing.assert_allclose(gpu.to_f32(gpu.sum(xg)), oracle.to_f32(oracle.sum(xo)), rtol=tol, atol=tol * shape[-1] ** 0.5)
        # strided rows (reduce over a transposed view)
        if len(shape) == 2:
            to, tg = oracle.transpose(xo, 0, 1), gpu.transpose(xg, 0, 1)
            same_bits(oracle, gpu, oracle.max(to), gpu.max(tg))
            same_bits(oracle, gpu, oracle.argmax(to), gpu.argmax(tg))


def test_softmax_graph_sweep_shape(oracle, gpu):
    """nn::softmax (stdlib/nn/mod.rs:168-179) as the 9-op graph, rows of 4096 (fewer rows than the sweep's 8192)."""
    rng = np.random.default_rng(2)
    x = rng.uniform(-4, 4, (128, 4096)).astype(np.float32)
    outs = []
    for be in (oracle, gpu):
        tb = cb.TermBuilder(be)
        s = tb.source()
        xf = tb.cast(s, Dtype.F32)
        sh = tb.shape(xf)
        e = tb.exp(xf - tb.broadcast(sh, tb.max(xf)))
        y = tb.cast(e / tb.broadcast(sh, tb.sum(e)), tb.dtype(s))
        term = tb.finish([y])
        outs.append(be.to_f32(cb.Interpreter(be).run(term, [be.from_numpy(x)])[0]))
    np.testing.assert_allclose(outs[1], outs[0], rtol=1e-5, atol=1e-9)
    np.testing.assert_allclose(outs[1].sum(-1), 1.0, rtol=1e-5)


def test_argmax_ties_nan_and_signed_zero(oracle, gpu):
    rows = np.array([[1, 7, 7, 2, 7, 0], [-0.0, 0.0, -0.0, 0.0, -0.0, -0.0], [np.nan, 1, 2, 3, 4, 5],
                     [-np.inf] * 6, [3, 3, 3, 3, 3, 3]], np.float32)
    for dtype in (Dtype.F32, Dtype.BF16):
        xo, xg = both(oracle, gpu, rows, dtype)
        same_bits(oracle, gpu, oracle.argmax(xo), gpu.argmax(xg), what=f"argmax {dtype.name}")
        # max of a row holding both zeros: the sign of the result depends on the fold order in the reference too
        # (f32::max does not order -0.0 and +0.0), so compare by value
        np.testing.assert_array_equal(oracle.to_f32(oracle.max(xo)), gpu.to_f32(gpu.max(xg)))
    assert gpu.to_numpy(gpu.argmax(gpu.from_numpy(rows))).reshape(-1).tolist() == [4, 3, 0, 5, 5]
    # wide vocabulary row with many ties, as bf16 logits have
    rng = np.random.default_rng(8)
    wide = np.round(rng.standard_normal((64, 32000)) * 4) / 4
    xo, xg = both(oracle, gpu, wide.astype(np.float32), Dtype.BF16)
    same_bits(oracle, gpu, oracle.argmax(xo), gpu.argmax(xg))


def test_topk_tie_order(oracle, gpu):
    rng = np.random.default_rng(9)
    x = np.round(rng.standard_normal((5, 300)) * 3).astype(np.float32)
    xo, xg = both(oracle, gpu, x)
    for k in (1, 4, 17):
        vo, io = oracle.topk(xo, k)
        vg, ig = gpu.topk(xg, k)
        same_bits(oracle, gpu, vo, vg)
        same_bits(oracle, gpu, io, ig)


def test_gather_concat_slice_arange(oracle, gpu):
    rng = np.random.default_rng(2)
    table = rng.standard_normal((32000, 256)).astype(np.float32)
    idx = rng.integers(0, 32000, 4096, dtype=np.uint32)
    for dtype in (Dtype.F32, Dtype.BF16):
        to, tg = both(oracle, gpu, table, dtype)
        io, ig = both(oracle, gpu, idx)
        same_bits(oracle, gpu, oracle.index(to, 0, io), gpu.index(tg, 0, ig))
    small = rng.standard_normal((3, 7, 5)).astype(np.float32)
    so, sg = both(oracle, gpu, small)
    j = np.array([6, 0, 0, 3], np.uint32)
    jo, jg = both(oracle, gpu, j)
    same_bits(oracle, gpu, oracle.index(so, 1, jo), gpu.index(sg, 1, jg))
    same_bits(oracle, gpu, oracle.index(so, 2, oracle.slice(jo, 0, 1, 3)), gpu.index(sg, 2, gpu.slice(jg, 0, 1, 3)))
    for dim in (0, 1, 2):
        same_bits(oracle, gpu, oracle.concat(so, so, dim), gpu.concat(sg, sg, dim))
    same_bits(oracle, gpu, oracle.concat(oracle.transpose(so, 0, 2), oracle.transpose(so, 0, 2), 1),
              gpu.concat(gpu.transpose(sg, 0, 2), gpu.transpose(sg, 0, 2), 1))
    eo, eg = oracle.zeros((3, 0, 5), Dtype.F32), gpu.zeros((3, 0, 5), Dtype.F32)
    same_bits(oracle, gpu, oracle.concat(eo, so, 1), gpu.concat(eg, sg, 1))
    same_bits(oracle, gpu, oracle.arange(1000), gpu.arange(1000))
    assert gpu.arange(0).shape == (0,)
    assert gpu.compare(sg, sg) and not gpu.compare(sg, gpu.neg(sg))
    assert gpu.to_bool(gpu.from_numpy(np.array([0.0, -1.0, 2.0], np.float32)))
    assert not gpu.to_bool(gpu.from_numpy(np.array([0.0, -1.0, np.nan], np.float32)))
    assert not gpu.compare(gpu.from_numpy(np.array([np.nan], np.float32)), gpu.from_numpy(np.array([np.nan], np.float32)))


@pytest.mark.parametrize("dtype", [Dtype.F32, Dtype.BF16], ids=lambda d: d.name)
def test_matmul(oracle, gpu, dtype):
    rng = np.random.default_rng(2)
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == Dtype.F32 else dict(rtol=2e-2, atol=2e-2)
    cases = [((4, 96, 80), (4, 80, 72)), ((2, 3, 5, 7), (2, 3, 7, 1)), ((33, 65), (65, 17)), ((1, 1, 256), (1, 256, 384)),
             ((2, 130, 64), (2, 64, 130))]
    for sa, sb in cases:
        a = rng.standard_normal(sa).astype(np.float32)
        b = rng.standard_normal(sb).astype(np.float32)
        ao, ag = both(oracle, gpu, a, dtype)
        bo, bg = both(oracle, gpu, b, dtype)
        np.testing.assert_allclose(gpu.to_f32(gpu.matmul(ag, bg)), oracle.to_f32(oracle.matmul(ao, bo)), **tol)
    # the `linear` pattern: x @ broadcast(transpose(W)) with W [out, in]; nothing is copied on the GPU
    x = rng.standard_normal((2, 5, 256)).astype(np.float32)
    w = (rng.standard_normal((384, 256)) * 0.05).astype(np.float32)
    res = []
    for be in (oracle, gpu):
        xt, wt = be.from_numpy(x, dtype), be.from_numpy(w, dtype)
        wv = be.broadcast(be.transpose(wt, 0, 1), (2, 256, 384))
        res.append(be.to_f32(be.matmul(xt, wv)))
    np.testing.assert_allclose(res[1], res[0], **tol)
    # single-row products take the weight-streaming kernel
    x1 = rng.standard_normal((1, 1, 256)).astype(np.float32)
    res = []
    for be in (oracle, gpu):
        xt, wt = be.from_numpy(x1, dtype), be.from_numpy(w, dtype)
        res.append(be.to_f32(be.matmul(xt, be.broadcast(be.transpose(wt, 0, 1), (1, 256, 384)))))
    np.testing.assert_allclose(res[1], res[0], **tol)
    with pytest.raises(cb.BackendError):
        gpu.matmul(gpu.from_numpy(x), gpu.from_numpy(w))


@pytest.mark.parametrize("case", [((3, 256, 512), (3, 512, 320), "row-major right operand"),
                                  ((1024, 256), (256, 640), "rank 2"),
                                  ((4, 128, 264), (264, 200), "weight shared by the batch, stored [N, K]")], ids=lambda c: c[2])
def test_f32_matmul_on_tensor_cores_from_split_operands(gpu, case):
    """Large f32 products run on the bf16 tensor cores from three-way split operands (six partial products, f32
    accumulate).  Against float64 numpy the error must stay near f32 level (the tensor core's truncating accumulation
    costs a few 1e-6 of the largest entry), far below what a single bf16 or TF32 rounding of the operands would
    give (~4e-3)."""
    import os
    sa, sb, kind = case
    rng = np.random.default_rng(17)
    a = rng.standard_normal(sa).astype(np.float32)
    if kind.startswith("weight"):
        w = rng.standard_normal((sb[1], sb[0])).astype(np.float32)           # [N, K]
        bg = gpu.broadcast(gpu.transpose(gpu.from_numpy(w), 0, 1), (sa[0],) + sb)
        ref = a.astype(np.float64) @ w.T.astype(np.float64)
    else:
        b = rng.standard_normal(sb).astype(np.float32)
        bg = gpu.from_numpy(b)
        ref = a.astype(np.float64) @ b.astype(np.float64)
    got = gpu.to_numpy(gpu.matmul(gpu.from_numpy(a), bg))
    scale = np.abs(ref).max()
    assert np.abs(got - ref).max() / scale < 1e-5
    # scaled inputs with a wide dynamic range: the split must not lose small operands next to large ones
    a2 = (a * np.exp(rng.uniform(-8, 8, size=a.shape))).astype(np.float32)
    got2 = gpu.to_numpy(gpu.matmul(gpu.from_numpy(a2), bg))
    ref2 = a2.astype(np.float64) @ (w.T if kind.startswith("weight") else b).astype(np.float64)
    assert np.abs(got2 - ref2).max() / np.abs(ref2).max() < 1e-5


@pytest.mark.parametrize("dtype", [Dtype.F32, Dtype.BF16], ids=lambda d: d.name)
@pytest.mark.parametrize("shape", [(7, 33), (64, 1024), (5, 3, 4096), (3, 10000), (4, 40000)], ids=str)
def test_fused_softmax_equals_the_nn_softmax_graph(oracle, gpu, dtype, shape):
    """cg_softmax against the nine-op graph of stdlib nn::softmax run on the oracle (cast f32, x - max, exp, / sum,
    cast back): f32 to 1e-6, bf16 to one bf16 ulp of the largest probability; rows sum to 1."""
    rng = np.random.default_rng(sum(shape))
    x = rng.uniform(-6, 6, shape).astype(np.float32)
    x[0, ..., 0] = 30.0     # a dominant entry: the others underflow towards 0 without overflow anywhere
    xo, xg = both(oracle, gpu, x, dtype)

    def graph(be, t):
        xf = be.cast(t, Dtype.F32)
        e = be.exp(be.sub(xf, be.broadcast(be.max(xf), xf.shape)))
        return be.cast(be.div(e, be.broadcast(be.sum(e), xf.shape)), dtype)
    want = oracle.to_f32(graph(oracle, xo))
    got = gpu.to_f32(gpu.softmax(xg))
    tol = 1e-6 if dtype == Dtype.F32 else 2 ** -8
    assert np.abs(got - want).max() <= tol
    assert np.abs(got.sum(-1) - 1.0).max() <= (1e-5 if dtype == Dtype.F32 else 2e-2)
    # a strided view goes through a contiguous copy
    if len(shape) == 2:
        xt = gpu.transpose(gpu.from_numpy(np.ascontiguousarray(x.T), dtype), 0, 1)
        np.testing.assert_array_equal(gpu.to_f32(gpu.softmax(xt)), got)


def test_matmul_sweep_shape_linearity(gpu):
    """Full op-sweep size [16,1024,1024]^2 (too slow for the scalar oracle): checked through linearity,
    (A1+A2) B = A1 B + A2 B, and against a float64 numpy product on a sampled block."""
    rng = np.random.default_rng(2)
    a1 = rng.standard_normal((16, 1024, 1024)).astype(np.float32)
    a2 = rng.standard_normal((16, 1024, 1024)).astype(np.float32)
    b = rng.standard_normal((16, 1024, 1024)).astype(np.float32)
    A1, A2, B = gpu.from_numpy(a1), gpu.from_numpy(a2), gpu.from_numpy(b)
    lhs = gpu.to_numpy(gpu.matmul(gpu.add(A1, A2), B))
    rhs = gpu.to_numpy(gpu.add(gpu.matmul(A1, B), gpu.matmul(A2, B)))
    assert helpers.rel_err(lhs, rhs) < 1e-5
    ref = (a1[3, :64].astype(np.float64) + a2[3, :64]) @ b[3].astype(np.float64)
    assert helpers.rel_err(lhs[3, :64], ref) < 1e-5


def test_fp8_moves_and_casts(oracle, gpu):
    bits = np.arange(256, dtype=np.uint8)
    fo, fg = oracle.ndarray_from_vec_fp8(bits, (256,)), gpu.ndarray_from_vec_fp8(bits, (256,))
    a, b = oracle.to_f32(oracle.cast(fo, Dtype.F32)), gpu.to_f32(gpu.cast(fg, Dtype.F32))
    np.testing.assert_array_equal(np.nan_to_num(a, nan=12345.0), np.nan_to_num(b, nan=12345.0))
    x = np.linspace(-500, 500, 4001).astype(np.float32)
    np.testing.assert_array_equal(oracle.to_numpy(oracle.cast(oracle.from_numpy(x), Dtype.F8)),
                                  gpu.to_numpy(gpu.cast(gpu.from_numpy(x), Dtype.F8)))
    with pytest.raises(cb.BackendError):
        gpu.add(fg, fg)


def _bf16_round(a):
    return cb.bf16_bits_to_f32(cb.f32_to_bf16_bits(a)).reshape(a.shape)


@pytest.mark.parametrize("mnk", [(128, 128, 64), (300, 200, 264), (17, 2048, 512), (512, 384, 2048), (1000, 136, 72),
                                 (129, 257, 1032), (64, 16, 16), (128, 4096, 256), (100, 8200, 128), (32, 40, 64),
                                 (2048, 2048, 512), (2048, 4096, 512), (1000, 8200, 264), (2500, 1160, 136),
                                 (4100, 4104, 72)], ids=str)
def test_tensor_core_gemm_against_f32_path(gpu, mnk):
    """bf16 `x @ W^T` products (both operands K-contiguous) run on the tcgen05 kernel; the same bf16-rounded
    operands multiplied by the exact-f32 SIMT kernel give the reference.  Only the accumulation order differs, so
    after one rounding to bf16 the results agree to 1 bf16 ulp of the row scale."""
    m, n, k = mnk
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    x = _bf16_round(rng.standard_normal((m, k)).astype(np.float32))
    w = _bf16_round((rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32))
    got = gpu.to_f32(gpu.matmul(gpu.from_numpy(x, Dtype.BF16), gpu.transpose(gpu.from_numpy(w, Dtype.BF16), 0, 1)))
    ref = gpu.to_numpy(gpu.matmul(gpu.from_numpy(x), gpu.transpose(gpu.from_numpy(w), 0, 1)))
    np.testing.assert_allclose(got, ref, rtol=1e-2, atol=1e-2)
    assert helpers.rel_err(got, ref) < 6e-3
    # float64 check of a corner block, independent of any GPU kernel
    ref64 = x[:8].astype(np.float64) @ w[-8:].astype(np.float64).T
    np.testing.assert_allclose(got[:8, -8:], ref64, rtol=1e-2, atol=1e-2)


def test_tensor_core_gemm_batched_and_shared_weight(oracle, gpu):
    rng = np.random.default_rng(12)
    # a weight shared by the batch (the `linear` pattern): the batch folds into rows
    x = _bf16_round(rng.standard_normal((4, 40, 256)).astype(np.float32))
    w = _bf16_round((rng.standard_normal((192, 256)) / 16).astype(np.float32))
    res = []
    for be in (oracle, gpu):
        xt, wt = be.from_numpy(x, Dtype.BF16), be.from_numpy(w, Dtype.BF16)
        res.append(be.to_f32(be.matmul(xt, be.broadcast(be.transpose(wt, 0, 1), (4, 256, 192)))))
    np.testing.assert_allclose(res[1], res[0], rtol=2e-2, atol=2e-2)
    # a true batch: q @ k^T per head, k stored [heads, T, D]
    q = _bf16_round(rng.standard_normal((3, 150, 64)).astype(np.float32))
    kk = _bf16_round(rng.standard_normal((3, 96, 64)).astype(np.float32))
    res = []
    for be in (oracle, gpu):
        res.append(be.to_f32(be.matmul(be.from_numpy(q, Dtype.BF16), be.transpose(be.from_numpy(kk, Dtype.BF16), 1, 2))))
    np.testing.assert_allclose(res[1], res[0], rtol=2e-2, atol=6e-2)
    ref64 = np.einsum("bmk,bnk->bmn", q.astype(np.float64), kk.astype(np.float64))
    np.testing.assert_allclose(res[1], ref64, rtol=2e-2, atol=8e-2)


@pytest.mark.parametrize("mnk", [(128, 128, 64), (300, 200, 264), (512, 384, 2048), (129, 264, 1032), (1024, 64, 128),
                                 (40, 4096, 256)], ids=str)
def test_tensor_core_gemm_row_major_right_operand(gpu, mnk):
    """The trait's own layout: lhs [M,K] @ rhs [K,N], both row-major (rhs is N-contiguous, an MN-major tensor-core
    operand).  Reference: the exact-f32 kernel on the same bf16-rounded values."""
    m, n, k = mnk
    rng = np.random.default_rng(m + 5 * n + 11 * k)
    x = _bf16_round(rng.standard_normal((m, k)).astype(np.float32))
    w = _bf16_round((rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32))
    got = gpu.to_f32(gpu.matmul(gpu.from_numpy(x, Dtype.BF16), gpu.from_numpy(w, Dtype.BF16)))
    ref = gpu.to_numpy(gpu.matmul(gpu.from_numpy(x), gpu.from_numpy(w)))
    np.testing.assert_allclose(got, ref, rtol=1e-2, atol=1e-2)
    assert helpers.rel_err(got, ref) < 6e-3
    ref64 = x[-8:].astype(np.float64) @ w[:, :8].astype(np.float64)
    np.testing.assert_allclose(got[-8:, :8], ref64, rtol=1e-2, atol=1e-2)


def test_tensor_core_gemm_more_tiles_than_sms(gpu):
    """Products with more output tiles than SMs run on the persistent kernel (a CTA walks several tiles, two
    accumulators in tensor memory).  Every output element is checked against a float64 product, for a batched K-major
    product with ragged row tiles and for a product with a fused residual in the Llama runner's shapes."""
    rng = np.random.default_rng(77)
    q = _bf16_round(rng.standard_normal((8, 900, 64)).astype(np.float32))
    kk = _bf16_round(rng.standard_normal((8, 1024, 64)).astype(np.float32))
    got = gpu.to_f32(gpu.matmul(gpu.from_numpy(q, Dtype.BF16), gpu.transpose(gpu.from_numpy(kk, Dtype.BF16), 1, 2)))
    ref64 = np.einsum("bmk,bnk->bmn", q.astype(np.float64), kk.astype(np.float64))
    np.testing.assert_allclose(got, ref64, rtol=2e-2, atol=8e-2)
    # every tile must land where it belongs: compare the position of the largest element of each row
    assert (got.argmax(-1) == _bf16_round(ref64.astype(np.float32)).argmax(-1)).mean() > 0.98
    # many launches in a row on the same buffers: barrier phases and accumulator hand-over start afresh each time
    x = _bf16_round(rng.standard_normal((1536, 320)).astype(np.float32))
    w = _bf16_round((rng.standard_normal((6400, 320)) / 18).astype(np.float32))
    X, Wt = gpu.from_numpy(x, Dtype.BF16), gpu.transpose(gpu.from_numpy(w, Dtype.BF16), 0, 1)
    ref64 = x.astype(np.float64) @ w.astype(np.float64).T
    for _ in range(3):
        np.testing.assert_allclose(gpu.to_f32(gpu.matmul(X, Wt)), ref64, rtol=2e-2, atol=2e-2)


def test_tensor_core_gemm_row_major_batched(gpu):
    rng = np.random.default_rng(33)
    a = _bf16_round(rng.standard_normal((5, 160, 96)).astype(np.float32))
    b = _bf16_round((rng.standard_normal((5, 96, 192)) / 10).astype(np.float32))
    got = gpu.to_f32(gpu.matmul(gpu.from_numpy(a, Dtype.BF16), gpu.from_numpy(b, Dtype.BF16)))
    ref64 = np.einsum("bmk,bkn->bmn", a.astype(np.float64), b.astype(np.float64))
    np.testing.assert_allclose(got, ref64, rtol=2e-2, atol=3e-2)


def test_probe_and_format_on_the_gpu(gpu, capfd, monkeypatch):
    """Probe through cg_interp_run on the CUDA backend (a synchronising read-back) and cg_format."""
    tb = cb.TermBuilder(gpu)
    x = tb.source(cb.NodeType.Tensor)
    y = x * x
    tb.probe("squared", y)
    term = tb.finish([y])
    a = np.array([[3.0, -1.5], [0.25, 8.0]], np.float32)
    monkeypatch.setenv("CATGRAD_PROBE", "1")
    out = cb.Interpreter(gpu).run(term, [gpu.from_numpy(a)])
    np.testing.assert_array_equal(gpu.to_numpy(out[0]), a * a)
    text = capfd.readouterr().out
    assert "[probe:squared]" in text and "f32" in text and "[2,2]" in text and "2.25" in text and "64" in text
    monkeypatch.delenv("CATGRAD_PROBE")
    cb.Interpreter(gpu).run(term, [gpu.from_numpy(a)])
    assert "[probe:" not in capfd.readouterr().out
    s = gpu.format_tensor(gpu.transpose(gpu.from_numpy(a, Dtype.BF16), 0, 1))      # a strided view prints in logical order
    assert "bf16" in s and s.index("0.25") < s.index("-1.5")

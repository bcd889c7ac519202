"""Writes tests/golden/reference_vectors.json: the known-answer vectors of the reference's own tests for the
backend/interpreter path, transcribed with their source locations (paths inside hellas-ai/catgrad).

When a checkout of the reference is given (first argument, or the environment variable CATGRAD_REFERENCE) every case is checked
against the cited lines: each number of the case must appear as a literal in that line range.  The JSON is what
the test-suite reads; this script is only needed to regenerate or re-verify it.

Case kinds:
  op      : one Backend call.            {"op", "dtype", "inputs": [{"shape","data"}], "args", "expect": [{"dtype","shape","data"}]}
  error   : a call that must be refused. {"op", ..., "error": "SHAPE_MISMATCH"}
  graph   : a small term built from the reference's helper definitions (tests/test_helpers_graphs.py builds them).
"""
import json
import os
import re
import sys

ND = "catgrad/src/interpreter/backend/ndarray.rs"
CT = "catgrad/tests/test_interpreter_candle.rs"
IT = "catgrad/tests/test_interpreter.rs"
CA = "catgrad/src/interpreter/backend/candle.rs"
HT = "catgrad-llm/src/helpers_tests.rs"
IF = "catgrad/tests/test_if.rs"


def T(shape, data):
    return {"shape": list(shape), "data": list(data)}


def E(dtype, shape, data):
    return {"dtype": dtype, "shape": list(shape), "data": list(data)}


CASES = [
    # ---- ndarray.rs unit tests ----
    dict(kind="op", name="nd_batched_matmul", src=f"{ND}:832-875", op="matmul", dtype="f32",
         inputs=[T([2, 3, 2, 2], [float(i) for i in range(1, 25)]), T([2, 3, 2, 1], [float(i) for i in range(1, 13)])],
         expect=[E("f32", [2, 3, 2, 1], [5.0, 11.0, 39.0, 53.0, 105.0, 127.0, 203.0, 233.0, 333.0, 371.0, 495.0, 541.0])]),
    dict(kind="op", name="nd_add", src=f"{ND}:877-896", op="add", dtype="f32",
         inputs=[T([2, 2], [1.0, 2.0, 3.0, 4.0]), T([2, 2], [5.0, 6.0, 7.0, 8.0])],
         expect=[E("f32", [2, 2], [6.0, 8.0, 10.0, 12.0])]),
    dict(kind="op", name="nd_sub", src=f"{ND}:898-917", op="sub", dtype="f32",
         inputs=[T([2, 2], [10.0, 8.0, 6.0, 4.0]), T([2, 2], [1.0, 2.0, 3.0, 4.0])],
         expect=[E("f32", [2, 2], [9.0, 6.0, 3.0, 0.0])]),
    dict(kind="op", name="nd_sum_u32", src=f"{ND}:919-938", op="sum", dtype="u32",
         inputs=[T([2, 3], [1, 2, 3, 4, 5, 6])], expect=[E("u32", [2, 1], [6, 15])]),
    dict(kind="op", name="nd_sum_3d", src=f"{ND}:940-961", op="sum", dtype="f32",
         inputs=[T([2, 2, 3], [float(i) for i in range(1, 13)])], expect=[E("f32", [2, 2, 1], [6.0, 15.0, 24.0, 33.0])]),
    dict(kind="op", name="nd_max", src=f"{ND}:962-982", op="max", dtype="f32",
         inputs=[T([2, 3], [1.0, 5.0, 3.0, 2.0, 8.0, 4.0])], expect=[E("f32", [2, 1], [5.0, 8.0])]),
    dict(kind="op", name="nd_max_u32", src=f"{ND}:984-1000", op="max", dtype="u32",
         inputs=[T([2, 2], [1, 5, 3, 2])], expect=[E("u32", [2, 1], [5, 3])]),
    dict(kind="op", name="nd_max_3d", src=f"{ND}:1002-1022", op="max", dtype="f32",
         inputs=[T([2, 2, 3], [float(i) for i in range(1, 13)])], expect=[E("f32", [2, 2, 1], [3.0, 6.0, 9.0, 12.0])]),
    # ---- backend-trait tests (candle CPU, same trait) ----
    dict(kind="op", name="ct_add", src=f"{CT}:38-72", op="add", dtype="f32",
         inputs=[T([2, 2], [1.0, 2.0, 3.0, 4.0]), T([2, 2], [2.0, 3.0, 4.0, 5.0])],
         expect=[E("f32", [2, 2], [3.0, 5.0, 7.0, 9.0])]),
    dict(kind="op", name="ct_mul", src=f"{CT}:74-105", op="mul", dtype="f32",
         inputs=[T([2, 2], [1.0, 2.0, 3.0, 4.0]), T([2, 2], [2.0, 3.0, 4.0, 5.0])],
         expect=[E("f32", [2, 2], [2.0, 6.0, 12.0, 20.0])]),
    dict(kind="op", name="ct_sub_u32", src=f"{CT}:144-176", op="sub", dtype="u32",
         inputs=[T([2, 2], [10, 8, 6, 4]), T([2, 2], [1, 2, 3, 4])], expect=[E("u32", [2, 2], [9, 6, 3, 0])]),
    dict(kind="op", name="ct_argmax", src=f"{CT}:233-258", op="argmax", dtype="f32",
         inputs=[T([2, 3], [1.0, 5.0, 3.0, 2.0, 8.0, 4.0])], expect=[E("u32", [2, 1], [1, 1])]),
    dict(kind="op", name="ct_argmax_u32", src=f"{CT}:260-284", op="argmax", dtype="u32",
         inputs=[T([2, 2], [1, 5, 3, 2])], expect=[E("u32", [2, 1], [1, 0])]),
    dict(kind="op", name="ct_sum", src=f"{CT}:288-312", op="sum", dtype="f32",
         inputs=[T([2, 3], [1.0, 2.0, 3.0, 4.0, 5.0, 6.0])], expect=[E("f32", [2, 1], [6.0, 15.0])]),
    dict(kind="op", name="ct_matmul", src=f"{CT}:341-376", op="matmul", dtype="f32",
         inputs=[T([2, 3], [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]), T([3, 2], [1.0, 2.0, 3.0, 4.0, 5.0, 6.0])],
         expect=[E("f32", [2, 2], [22.0, 28.0, 49.0, 64.0])]),
    dict(kind="op", name="ct_reshape", src=f"{CT}:379-398", op="reshape", dtype="f32",
         inputs=[T([2, 3], [1.0, 2.0, 3.0, 4.0, 5.0, 6.0])], args=[[3, 2]],
         expect=[E("f32", [3, 2], [1.0, 2.0, 3.0, 4.0, 5.0, 6.0])]),
    dict(kind="op", name="ct_cast_u32", src=f"{CT}:401-430", op="cast", dtype="f32",
         inputs=[T([2, 2], [1.0, 2.0, 3.0, 4.0])], args=["u32"], expect=[E("u32", [2, 2], [1, 2, 3, 4])]),
    dict(kind="op", name="ct_div", src=f"{CT}:433-466", op="div", dtype="f32",
         inputs=[T([2, 2], [6.0, 8.0, 10.0, 12.0]), T([2, 2], [2.0, 4.0, 5.0, 3.0])],
         expect=[E("f32", [2, 2], [3.0, 2.0, 2.0, 4.0])]),
    dict(kind="op", name="ct_div_u32", src=f"{CT}:468-500", op="div", dtype="u32",
         inputs=[T([2, 2], [6, 8, 10, 12]), T([2, 2], [2, 4, 5, 3])], expect=[E("u32", [2, 2], [3, 2, 2, 4])]),
    dict(kind="op", name="ct_pow", src=f"{CT}:504-538", op="pow", dtype="f32",
         inputs=[T([2, 2], [2.0, 3.0, 4.0, 5.0]), T([2, 2], [2.0, 2.0, 2.0, 2.0])],
         expect=[E("f32", [2, 2], [4.0, 9.0, 16.0, 25.0])]),
    dict(kind="op", name="ct_log", src=f"{CT}:542-574", op="log", dtype="f32", atol=1e-6,
         inputs=[T([2, 2], [1.0, 2.0, 3.0, 4.0])],
         expect=[E("f32", [2, 2], [0.0, 0.6931471805599453, 1.0986122886681098, 1.3862943611198906])], derived="ln(x)"),
    dict(kind="op", name="ct_floor", src=f"{CT}:577-603", op="floor", dtype="f32",
         inputs=[T([2, 2], [1.1, 2.9, -3.5, 4.0])], expect=[E("f32", [2, 2], [1.0, 2.0, -4.0, 4.0])]),
    dict(kind="op", name="ct_neg", src=f"{CT}:607-632", op="neg", dtype="f32",
         inputs=[T([2, 2], [1.0, -2.0, 3.0, -4.0])], expect=[E("f32", [2, 2], [-1.0, 2.0, -3.0, 4.0])]),
    dict(kind="op", name="ct_broadcast_1", src=f"{CT}:636-656", op="broadcast", dtype="f32",
         inputs=[T([2, 2], [1.0, 2.0, 3.0, 4.0])], args=[[1, 2, 2]],
         expect=[E("f32", [1, 2, 2], [1.0, 2.0, 3.0, 4.0])]),
    dict(kind="op", name="ct_broadcast_5", src=f"{CT}:636-672", op="broadcast", dtype="f32",
         inputs=[T([1, 2, 2], [1.0, 2.0, 3.0, 4.0])], args=[[5, 2, 2]],
         expect=[E("f32", [5, 2, 2], [1.0, 2.0, 3.0, 4.0] * 5)], derived="repeat"),
    dict(kind="op", name="ct_broadcast_u32", src=f"{CT}:674-693", op="broadcast", dtype="u32",
         inputs=[T([2, 2], [1, 2, 3, 4])], args=[[2, 1, 2, 2]], expect=[E("u32", [2, 1, 2, 2], [1, 2, 3, 4] * 2)],
         derived="repeat"),
    dict(kind="op", name="ct_broadcast_front", src=f"{CT}:697-724", op="broadcast", dtype="f32",
         inputs=[T([2, 2], [1.0, 2.0, 3.0, 4.0])], args=[[2, 2, 2]],
         expect=[E("f32", [2, 2, 2], [1.0, 2.0, 3.0, 4.0] * 2)], derived="repeat",
         note="the reference test is should_panic: the broadcast succeeds with shape [2,2,2] and its assert on [1,2,2] fails"),
    dict(kind="error", name="ct_add_mismatch", src=f"{CT}:726-750", op="add", dtype="f32",
         inputs=[T([2, 2], [1.0, 2.0, 3.0, 4.0]), T([3], [1.0, 2.0, 3.0])], error="SHAPE_MISMATCH"),
    dict(kind="error", name="ct_mul_mismatch", src=f"{CT}:752-778", op="mul", dtype="f32",
         inputs=[T([2, 3], [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]), T([2, 2], [1.0, 2.0, 3.0, 4.0])], error="SHAPE_MISMATCH"),
    dict(kind="error", name="ct_div_mismatch", src=f"{CT}:780-804", op="div", dtype="f32",
         inputs=[T([2, 2], [1.0, 2.0, 3.0, 4.0]), T([2], [1.0, 2.0])], error="SHAPE_MISMATCH"),
    dict(kind="error", name="ct_pow_mismatch", src=f"{CT}:806-832", op="pow", dtype="f32",
         inputs=[T([2, 2], [1.0, 2.0, 3.0, 4.0]), T([2, 3], [1.0, 2.0, 3.0, 4.0, 5.0, 6.0])], error="SHAPE_MISMATCH"),
    dict(kind="error", name="ct_sub_mismatch", src=f"{CT}:834-862", op="sub", dtype="f32",
         inputs=[T([2, 2], [1.0, 2.0, 3.0, 4.0]), T([2], [1.0, 2.0])], error="SHAPE_MISMATCH"),
    dict(kind="op", name="ca_round_ties_even", src=f"{CA}:1607-1635", op="round", dtype="f32",
         inputs=[T([8], [1.2, 1.8, 2.5, 3.5, -1.2, -1.8, -2.5, -3.5])],
         expect=[E("f32", [8], [1.0, 2.0, 2.0, 4.0, -1.0, -2.0, -2.0, -4.0])]),
    # ---- interpreter integration tests (ndarray) ----
    dict(kind="op", name="it_add_u32", src=f"{IT}:50-75", op="add", dtype="u32", via_interpreter=True,
         inputs=[T([2, 1, 3], [1, 2, 3, 4, 5, 6]), T([2, 1, 3], [1, 2, 3, 4, 5, 6])],
         expect=[E("u32", [2, 1, 3], [2, 4, 6, 8, 10, 12])], derived="x*2"),
    dict(kind="op", name="it_batch_matmul", src=f"{IT}:77-114", op="matmul", dtype="f32", via_interpreter=True,
         inputs=[T([2, 2, 2], [1.0, 2.0, 3.0, 4.0, 5.0, 6.0, 7.0, 8.0]), T([2, 2, 1], [1.0, 2.0, 3.0, 4.0])],
         expect=[E("f32", [2, 2, 1], [5.0, 11.0, 39.0, 53.0])]),
    dict(kind="op", name="it_exp", src=f"{IT}:126-152", op="exp", dtype="f32", via_interpreter=True, rtol=1e-5, atol=1e-8,
         inputs=[T([2, 2], [0.0, 1.0, 2.0, -1.0])],
         expect=[E("f32", [2, 2], [1.0, 2.718281828459045, 7.38905609893065, 0.36787944117144233])], derived="exp(x)"),
    dict(kind="op", name="it_topk", src=f"{IT}:154-191", op="topk", dtype="f32", via_interpreter=True,
         inputs=[T([2, 5], [0.1, 5.0, 3.0, 10.0, 5.0, 8.0, 9.0, 7.0, 6.0, 8.0])], args=[2],
         expect=[E("f32", [2, 2], [10.0, 5.0, 9.0, 8.0]), E("u32", [2, 2], [3, 1, 1, 0])]),
    # ---- control flow ----
    dict(kind="graph", name="if_true", src=f"{IF}:9-60", graph="if_double", dtype="f32",
         inputs=[T([], [5.0]), T([], [1.0])], expect=[E("f32", [], [10.0])]),
    dict(kind="graph", name="if_false", src=f"{IF}:62-110", graph="if_double", dtype="f32",
         inputs=[T([], [5.0]), T([], [0.0])], expect=[E("f32", [], [5.0])]),
    # ---- helper graphs ----
    dict(kind="graph", name="split", src=f"{HT}:116-135", graph="split_2_2", dtype="f32",
         inputs=[T([1, 4], [1.0, 2.0, 3.0, 4.0])], expect=[E("f32", [1, 2], [1.0, 2.0]), E("f32", [1, 2], [3.0, 4.0])]),
    dict(kind="graph", name="squeeze", src=f"{HT}:158-172", graph="squeeze_3_1", dtype="f32",
         inputs=[T([2, 1, 3], [1.0, 2.0, 3.0, 4.0, 5.0, 6.0])], expect=[E("f32", [2, 3], [1.0, 2.0, 3.0, 4.0, 5.0, 6.0])]),
    dict(kind="graph", name="unsqueeze", src=f"{HT}:174-188", graph="unsqueeze_2_1", dtype="f32",
         inputs=[T([2, 3], [1.0, 2.0, 3.0, 4.0, 5.0, 6.0])], expect=[E("f32", [2, 1, 3], [1.0, 2.0, 3.0, 4.0, 5.0, 6.0])]),
    dict(kind="graph", name="repeat_kv", src=f"{HT}:190-209", graph="repeat_kv_3", dtype="f32",
         inputs=[T([1, 2, 1, 2], [1.0, 2.0, 3.0, 4.0])],
         expect=[E("f32", [1, 6, 1, 2], [1.0, 2.0, 1.0, 2.0, 1.0, 2.0, 3.0, 4.0, 3.0, 4.0, 3.0, 4.0])]),
    dict(kind="graph", name="repeat_interleave", src=f"{HT}:212-229", graph="repeat_interleave_2_2", dtype="f32",
         inputs=[T([1, 1, 2, 2], [1.0, 2.0, 3.0, 4.0])],
         expect=[E("f32", [1, 1, 4, 2], [1.0, 2.0, 1.0, 2.0, 3.0, 4.0, 3.0, 4.0])]),
    dict(kind="graph", name="clamp", src=f"{HT}:231-242", graph="clamp_m1_1p5", dtype="f32",
         inputs=[T([4], [-2.0, -1.0, 0.5, 2.0])], expect=[E("f32", [4], [-1.0, -1.0, 0.5, 1.5])]),
    dict(kind="graph", name="avgpool2d", src=f"{HT}:244-259", graph="avgpool2d_1_2_2", dtype="f32",
         inputs=[T([1, 1, 2, 2], [1.0, 3.0, 5.0, 7.0])], expect=[E("f32", [1, 1, 1, 1], [4.0])]),
    dict(kind="graph", name="where_broadcast", src=f"{HT}:261-278", graph="where_broadcast", dtype="f32",
         inputs=[T([1, 1], [0.0]), T([1, 2], [1.0, 2.0]), T([1, 2], [5.0, 6.0])], expect=[E("f32", [1, 2], [5.0, 6.0])]),
    dict(kind="graph", name="masked_fill", src=f"{HT}:280-296", graph="masked_fill_9", dtype="f32",
         inputs=[T([2], [1.0, 0.0]), T([2], [1.0, 2.0])], expect=[E("f32", [2], [9.0, 2.0])]),
    dict(kind="graph", name="cumsum", src=f"{HT}:298-312", graph="cumsum_4", dtype="f32",
         inputs=[T([1, 1, 1, 3], [1.0, 2.0, 3.0])], expect=[E("f32", [1, 1, 1, 3], [1.0, 3.0, 6.0])]),
]


def _numbers(case):
    """Literals that must be findable in the cited lines (inputs and, unless derived, expectations)."""
    vals = []
    for t in case.get("inputs", []):
        vals += t["data"]
    if "derived" not in case:
        for t in case.get("expect", []):
            vals += t["data"]
    return vals


def verify(ref_root):
    bad = []
    for c in CASES:
        path, rng = c["src"].rsplit(":", 1)
        lo, hi = [int(x) for x in rng.split("-")]
        with open(os.path.join(ref_root, path)) as f:
            lines = f.read().split("\n")
        text = "\n".join(lines[lo - 1:hi])
        found = set(float(x) for x in re.findall(r"-?\d+\.?\d*", re.sub(r"//[^\n]*", "", text)))
        for v in _numbers(c):
            if float(v) not in found:
                bad.append((c["name"], v, c["src"]))
    return bad


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("CATGRAD_REFERENCE", "")
    if ref_root and os.path.isdir(ref_root):
        bad = verify(ref_root)
        if bad:
            for b in bad:
                print("literal not found in cited lines:", b)
            sys.exit(1)
        print(f"verified {len(CASES)} cases against {ref_root}")
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.json")
    with open(out, "w") as f:
        json.dump({"source": "hellas-ai/catgrad v0.2.1 test-suite literals", "cases": CASES}, f, indent=1)
    print("wrote", out)


if __name__ == "__main__":
    main()

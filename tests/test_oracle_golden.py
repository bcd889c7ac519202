"""The CPU oracle against every known-answer vector the reference's own tests hold for the backend path
(tests/golden/reference_vectors.json; sources cited per case)."""
import numpy as np
import pytest

import catgrad_b200 as cb
import helpers


@pytest.mark.parametrize("case", helpers.golden_cases("op"), ids=lambda c: c["name"])
def test_op_vectors(oracle, case):
    run = helpers.call_op_via_interpreter if case.get("via_interpreter") else helpers.call_op
    helpers.check_expect(oracle, run(oracle, case), case)


@pytest.mark.parametrize("case", helpers.golden_cases("error"), ids=lambda c: c["name"])
def test_shape_mismatch_is_refused(oracle, case):
    with pytest.raises(cb.BackendError) as e:
        helpers.call_op(oracle, case)
    assert e.value.status.name == case["error"]
    assert "Shape mismatch in operation" in str(e.value)   # message pinned by the reference's should_panic tests


@pytest.mark.parametrize("case", helpers.golden_cases("graph"), ids=lambda c: c["name"])
def test_helper_graphs(oracle, case):
    helpers.check_expect(oracle, helpers.run_graph_case(oracle, case), case)


def test_constructor_shape_error(oracle):
    with pytest.raises(cb.BackendError) as e:
        oracle.ndarray_from_vec_f32(np.zeros(5, np.float32), (2, 3))
    assert e.value.status == cb.Status.SHAPE


def test_unpinned_semantics_follow_the_source(oracle):
    """Behaviour no reference test pins, stated by the source (ndarray.rs): argmax takes the LAST maximum under
    total_cmp, max folds from f32::MIN and ignores NaN, casts saturate, where treats NaN masks as false."""
    be = oracle
    x = be.from_numpy(np.array([[1.0, 3.0, 3.0, -0.0, 0.0], [np.nan, 1.0, np.inf, np.inf, -np.inf]], np.float32))
    assert be.to_numpy(be.argmax(x)).reshape(-1).tolist() == [2, 0]        # ties -> last; +NaN is the greatest
    z = be.from_numpy(np.array([[-0.0, 0.0, -0.0]], np.float32))
    assert be.to_numpy(be.argmax(z)).reshape(-1).tolist() == [1]           # -0.0 < +0.0
    m = be.from_numpy(np.array([[-np.inf, -np.inf], [np.nan, 2.0]], np.float32))
    got = be.to_numpy(be.max(m)).reshape(-1)
    assert got[0] == np.finfo(np.float32).min and got[1] == 2.0
    c = be.from_numpy(np.array([-1.5, 3.99, 5e9, np.nan], np.float32))
    assert be.to_numpy(be.cast(c, cb.Dtype.U32)).tolist() == [0, 3, 0xFFFFFFFF, 0]
    u = be.from_numpy(np.array([0, 5], np.uint32))
    assert be.to_numpy(be.neg(u)).tolist() == [0, 0xFFFFFFFB]
    mask = be.from_numpy(np.array([np.nan, 1.0, 0.0, -1.0], np.float32))
    a = be.from_numpy(np.array([1, 2, 3, 4], np.float32))
    b = be.from_numpy(np.array([5, 6, 7, 8], np.float32))
    assert be.to_numpy(be.where_cond(mask, a, b)).tolist() == [5, 2, 7, 8]
    assert be.to_numpy(be.arange(5)).tolist() == [0, 1, 2, 3, 4]
    e1 = be.zeros((2, 0, 3), cb.Dtype.F32)
    e2 = be.from_numpy(np.ones((2, 1, 3), np.float32))
    assert be.concat(e1, e2, 1).shape == (2, 1, 3)                         # empty left operand (empty KV cache)
    with pytest.raises(cb.BackendError):
        be.sin(u)

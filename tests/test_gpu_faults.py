"""Error paths on the GPU that never fault it: host-side checks, the sticky device error word, a capped allocator."""
import numpy as np
import pytest

import catgrad_b200 as cb
from catgrad_b200 import Dtype

pytestmark = pytest.mark.gpu


def test_u32_division_by_zero_is_reported_not_trapped(gpu):
    a = gpu.from_numpy(np.array([6, 8], np.uint32))
    b = gpu.from_numpy(np.array([2, 0], np.uint32))
    r = gpu.div(a, b)
    with pytest.raises(cb.BackendError) as e:
        gpu.to_numpy(r)
    assert "divide by zero" in str(e.value)
    assert gpu.to_numpy(gpu.div(a, gpu.from_numpy(np.array([2, 4], np.uint32)))).tolist() == [3, 2]   # context still usable


def test_index_out_of_bounds_is_reported_not_trapped(gpu):
    x = gpu.from_numpy(np.arange(12, dtype=np.float32).reshape(3, 4))
    r = gpu.index(x, 0, gpu.from_numpy(np.array([1, 7], np.uint32)))
    with pytest.raises(cb.BackendError) as e:
        gpu.to_numpy(r)
    assert "out of bounds" in str(e.value)
    assert gpu.to_numpy(gpu.index(x, 0, gpu.from_numpy(np.array([2], np.uint32)))).tolist() == [[8, 9, 10, 11]]


def test_host_side_refusals(gpu):
    x = gpu.from_numpy(np.zeros((2, 3), np.float32))
    u = gpu.from_numpy(np.zeros((2, 3), np.uint32))
    with pytest.raises(cb.BackendError) as e:
        gpu.add(x, u)
    assert e.value.status == cb.Status.DTYPE_MISMATCH
    with pytest.raises(cb.BackendError) as e:
        gpu.ndarray_from_vec_u32(np.zeros(5, np.uint32), (2, 3))
    assert e.value.status == cb.Status.SHAPE
    with pytest.raises(cb.BackendError):
        gpu.slice(x, 1, 2, 5)
    with pytest.raises(cb.BackendError):
        gpu.reshape(x, (4, 2))
    with pytest.raises(cb.BackendError):
        gpu.broadcast(x, (3, 3))
    with pytest.raises(cb.BackendError):
        gpu.concat(x, gpu.from_numpy(np.zeros((3, 3), np.float32)), 1)


def test_allocator_reuses_blocks_and_reports_oom(gpu):
    import ctypes as C
    stats = (C.c_uint64 * 4)()
    a = gpu.zeros((1 << 20,), Dtype.F32)
    del a
    gpu._check(gpu._ns.ctx_stats(gpu._ctx, stats))
    mallocs = stats[2]
    for _ in range(8):
        t = gpu.zeros((1 << 20,), Dtype.F32)
        del t
    gpu._check(gpu._ns.ctx_stats(gpu._ctx, stats))
    assert stats[2] == mallocs                      # served from the cache
    # out-of-memory is injected on the host: a second context whose allocator is capped at 1 MiB
    import os
    os.environ["CATGRAD_B200_MEM_CAP"] = str(1 << 20)
    try:
        capped = cb.Backend(0)
    finally:
        del os.environ["CATGRAD_B200_MEM_CAP"]
    small = capped.zeros((1024,), Dtype.F32)
    with pytest.raises(cb.BackendError) as e:
        capped.zeros((1 << 20,), Dtype.F32)
    assert e.value.status == cb.Status.OOM
    assert capped.to_numpy(small).sum() == 0        # the context survives the refusal
    capped.close()


def test_matmul_refuses_dimensions_the_kernels_cannot_index(gpu):
    """A 2^31-row operand (a broadcast view: no memory behind it) is refused on the host before anything is allocated or
    launched; a tall product just below the old 65535-row-tile limit of grid.y still computes."""
    one = gpu.from_numpy(np.ones((1, 8), np.float32))
    huge = gpu.broadcast(one, (1 << 31, 8))
    w = gpu.from_numpy(np.ones((8, 4), np.float32))
    with pytest.raises(cb.BackendError) as ei:
        gpu.matmul(huge, w)
    assert ei.value.status == cb.Status.INVALID_ARG
    tall = gpu.broadcast(one, (70000 * 64, 8))          # 70000 row tiles: beyond what grid.y could hold
    y = gpu.matmul(gpu.cast(tall, cb.Dtype.F16), gpu.cast(w, cb.Dtype.F16))      # f16 takes the SIMT kernel
    assert y.shape == (70000 * 64, 4)
    v = gpu.to_numpy(gpu.slice(y, 0, 70000 * 64 - 3, 3)).astype(np.float32)
    np.testing.assert_array_equal(v, np.full((3, 4), 8.0, np.float32))


def test_allocator_size_classes_absorb_slowly_growing_tensors(gpu):
    """A tensor that grows by a row per step (the KV cache an op-by-op evaluation re-concatenates per token) must not
    reach cudaMalloc at every step: sizes fall into four classes per power of two, and a freed block of the class is
    reused."""
    import ctypes as C
    stats = (C.c_uint64 * 4)()
    rows = lambda n: gpu.zeros((n, 512), Dtype.F32)          # 2 KiB per row
    t = rows(100)
    del t
    gpu._check(gpu._ns.ctx_stats(gpu._ctx, stats))
    before = stats[2]
    for n in range(100, 228):                                # 200 KiB .. 456 KiB in steps of 2 KiB: 128 distinct sizes
        t = rows(n)
        del t
    gpu._check(gpu._ns.ctx_stats(gpu._ctx, stats))
    assert stats[2] - before <= 6                            # classes of 32 / 64 KiB: a handful of new blocks, not 128

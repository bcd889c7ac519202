"""cg_argmax_rows_noalloc, the entry point for callers that cannot allocate device memory (a serving loop with
pre-carved memory, a latency-critical section that must not hit cudaMalloc's implicit synchronisation, a plug-in
that only gets raw pointers): checked against the regular cg_argmax on the same device buffers, twice in a row
because every call reuses the library's fixed scratch array.  Integer results: the comparison is exact."""
import ctypes as C

import numpy as np
import pytest

import catgrad_b200 as cb
from catgrad_b200 import Dtype

pytestmark = pytest.mark.gpu


def noalloc_argmax(gpu, x, rows, n):
    out = gpu.zeros((rows,), Dtype.U32)            # caller-owned output buffer
    gpu.synchronize()                              # inputs were produced on the context's stream
    st = gpu._ns.argmax_rows_noalloc(C.c_void_p(x.data_ptr), int(x.dtype), rows, n, n, C.c_void_p(out.data_ptr), None)
    if st != 0:
        raise cb.BackendError(st, gpu._ns.last_error(None).decode())
    return gpu.to_numpy(out)


def test_matches_cg_argmax_on_two_calls_in_a_row(gpu, oracle):
    rng = np.random.default_rng(21)
    # call 1: bf16 logits of a 128256-wide vocabulary with many ties (quantised values)
    a = (np.round(rng.standard_normal((4, 128256)) * 8) / 8).astype(np.float32)
    xa = gpu.from_numpy(a, Dtype.BF16)
    want_a = gpu.to_numpy(gpu.argmax(xa)).reshape(-1)
    # both must equal the CPU oracle's argmax (last index among equal maxima, ndarray.rs:670-694)
    np.testing.assert_array_equal(want_a, oracle.to_numpy(oracle.argmax(oracle.from_numpy(a, Dtype.BF16))).reshape(-1))
    got_a = noalloc_argmax(gpu, xa, 4, 128256)
    np.testing.assert_array_equal(got_a, want_a)
    # call 2, right after: other shape and dtype, fewer chunks than call 1 left behind in the scratch
    b = rng.standard_normal((7, 5000)).astype(np.float32)
    b[3, :] = 1.0                                   # a full tie: the last index wins
    b[5, 17] = np.nan                               # positive NaN is the greatest under total_cmp
    xb = gpu.from_numpy(b)
    want_b = gpu.to_numpy(gpu.argmax(xb)).reshape(-1)
    np.testing.assert_array_equal(want_b, oracle.to_numpy(oracle.argmax(oracle.from_numpy(b))).reshape(-1))
    got_b = noalloc_argmax(gpu, xb, 7, 5000)
    np.testing.assert_array_equal(got_b, want_b)
    assert got_b[3] == 4999 and got_b[5] == 17
    # and the first input again: same answer as before
    np.testing.assert_array_equal(noalloc_argmax(gpu, xa, 4, 128256), want_a)


def test_rejects_sizes_beyond_the_fixed_scratch(gpu):
    x = gpu.zeros((8, 16), Dtype.F32)
    out = gpu.zeros((8,), Dtype.U32)
    gpu.synchronize()
    # 8192 rows x 3 chunks = 24576 partial keys > 16384
    st = gpu._ns.argmax_rows_noalloc(C.c_void_p(x.data_ptr), int(Dtype.F32), 8192, 3 * 4096, 3 * 4096,
                                     C.c_void_p(out.data_ptr), None)
    assert st == int(cb.Status.INVALID_ARG)
    assert b"exceeds the fixed scratch" in gpu._ns.last_error(None)
    st = gpu._ns.argmax_rows_noalloc(C.c_void_p(x.data_ptr), int(Dtype.U32), 8, 16, 16, C.c_void_p(out.data_ptr), None)
    assert st == int(cb.Status.UNSUPPORTED_DTYPE)


def test_refuses_foreign_pointers_and_streams_under_capture(gpu):
    """Host-side refusals only: nothing here launches a kernel on a bad pointer."""
    import torch
    x = gpu.zeros((4, 64), Dtype.F32)
    out = gpu.zeros((4,), Dtype.U32)
    gpu.synchronize()
    host = np.zeros(256, np.float32)
    # a host pointer as input, then as output
    st = gpu._ns.argmax_rows_noalloc(C.c_void_p(host.ctypes.data), int(Dtype.F32), 4, 64, 64, C.c_void_p(out.data_ptr), None)
    assert st == int(cb.Status.INVALID_ARG)
    st = gpu._ns.argmax_rows_noalloc(C.c_void_p(x.data_ptr), int(Dtype.F32), 4, 64, 64, C.c_void_p(host.ctypes.data), None)
    assert st == int(cb.Status.INVALID_ARG)
    # a stream that is being captured: refused, and the capture stays usable
    s = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    t = torch.zeros(8, device="cuda")
    with torch.cuda.stream(s):
        g.capture_begin()
        try:
            st = gpu._ns.argmax_rows_noalloc(C.c_void_p(x.data_ptr), int(Dtype.F32), 4, 64, 64, C.c_void_p(out.data_ptr),
                                             C.c_void_p(s.cuda_stream))
            t += 1
        finally:
            g.capture_end()
    assert st == int(cb.Status.INVALID_ARG)
    assert b"captured" in gpu._ns.last_error(None)
    g.replay()
    torch.cuda.synchronize()
    assert float(t[0]) == 1.0
    # and the entry point still works afterwards
    np.testing.assert_array_equal(noalloc_argmax(gpu, x, 4, 64), np.full(4, 63, np.uint32))

"""Host-side mirror of catgrad's `Backend` trait over the C ABI.

`Backend` has one method per trait method (catgrad/src/interpreter/backend/mod.rs:24-122) with the same
names and argument meaning; tensors are `Tensor` objects wrapping an opaque reference-counted handle.
Errors the reference raises as panics or `BackendError::ShapeError` surface as `BackendError` with the
C status code and message.

There is no CPU fallback: constructing a `Backend` without the CUDA library or without a GPU raises.
"""
import ctypes as C
import enum

import numpy as np

from . import _ffi


class Dtype(enum.IntEnum):
    """`enum Dtype` (catgrad/src/category/core.rs:23-29)."""
    F32 = 0
    F16 = 1
    BF16 = 2
    F8 = 3
    U32 = 4


class Status(enum.IntEnum):
    OK = 0
    SHAPE_MISMATCH = 1
    DTYPE_MISMATCH = 2
    UNSUPPORTED_DTYPE = 3
    OOM = 4
    CUDA = 5
    TIMEOUT = 6
    BAD_HANDLE = 7
    SHAPE = 8
    INVALID_ARG = 9
    INTERP = 10


class BackendError(RuntimeError):
    def __init__(self, status, message):
        self.status = Status(status)
        super().__init__(f"{self.status.name}: {message}")


_NP_STORAGE = {Dtype.F32: np.float32, Dtype.U32: np.uint32, Dtype.F16: np.float16, Dtype.BF16: np.uint16,
               Dtype.F8: np.uint8}


def f32_to_bf16_bits(a):
    """float32 array -> bf16 bit patterns (uint16), round to nearest even, NaN kept."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32)
    rounded = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    return np.where(nan, ((u >> 16) | 0x40).astype(np.uint16), rounded)


def bf16_bits_to_f32(b):
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32)


class Tensor:
    """Owning wrapper of a `cg_tensor*`."""

    def __init__(self, backend, handle):
        self._be = backend
        self._h = handle

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and self._be is not None and self._be._ns is not None:
            self._be._ns.release(h)

    @property
    def handle(self):
        return self._h

    @property
    def shape(self):
        """BackendTensorOps::shape (mod.rs:124-126)."""
        dims = (C.c_uint64 * _ffi.MAX_RANK)()
        rank = C.c_int()
        self._be._check(self._be._ns.shape(self._h, dims, C.byref(rank)))
        return tuple(int(dims[i]) for i in range(rank.value))

    @property
    def strides(self):
        st = (C.c_int64 * _ffi.MAX_RANK)()
        rank = C.c_int()
        self._be._check(self._be._ns.strides(self._h, st, C.byref(rank)))
        return tuple(int(st[i]) for i in range(rank.value))

    @property
    def dtype(self):
        return Dtype(self._be._ns.dtype_of(self._h))

    @property
    def is_contiguous(self):
        return bool(self._be._ns.is_contiguous(self._h))

    @property
    def data_ptr(self):
        return self._be._ns.data_ptr(self._h)

    def numpy(self):
        return self._be.to_numpy(self)

    def __repr__(self):
        return f"Tensor({self.dtype.name}, {list(self.shape)})"


def _dims(shape):
    shape = tuple(int(s) for s in shape)
    return (C.c_uint64 * max(len(shape), 1))(*shape), len(shape)


class Backend:
    """The B200 backend.  `Backend()` opens CUDA device 0 through the in-tree library."""

    def __init__(self, device=0, *, _cdll=None, _prefix="cg_", _borrowed_ctx=None):
        self._ns = None
        self._ctx = None
        if _borrowed_ctx is not None:
            # a view of a context that something else owns (a replica of catgrad_b200.runner.DeviceRunner)
            self._ns = _ffi.bind(C.CDLL(_ffi.library_path()), _prefix)
            self._ctx = _borrowed_ctx
            return
        if _cdll is None:
            path = _ffi.library_path()
            try:
                _cdll = C.CDLL(path)
            except OSError as e:
                raise BackendError(Status.CUDA, f"CUDA library not built or not loadable ({path}): {e}; "
                                                "run __graft_entry__.build()") from e
        self._ns = _ffi.bind(_cdll, _prefix, require_cuda_entry_points=(_prefix == "cg_"))
        ctx = C.c_void_p()
        st = self._ns.init(int(device), C.byref(ctx))
        if st != 0:
            msg = self._ns.last_error(None).decode()
            self._ns = None
            raise BackendError(st, msg)
        self._ctx = ctx

    def close(self):
        if self._ctx is not None and self._ns is not None:
            self._ns.destroy(self._ctx)
        self._ctx = None

    def __del__(self):
        # Tensors may outlive the backend object in interpreter shutdown order; leak the context then.
        pass

    @property
    def name(self):
        return self._ns.backend_name(self._ctx).decode()

    # -- plumbing -------------------------------------------------------------------------------
    def _check(self, status, ctx=True):
        if status != 0:
            msg = self._ns.last_error(self._ctx if ctx else None).decode()
            if not msg:
                msg = self._ns.last_error(None).decode()
            raise BackendError(status, msg)

    def _out(self, fn, *args):
        out = C.c_void_p()
        self._check(fn(self._ctx, *args, C.byref(out)))
        return Tensor(self, out)

    def op_stats(self, mode=None, reset=False):
        """Per-operation counters of the evaluator behind `cg_interp_run` (`cg_op_stats*`): with `mode` (0 off, 1 count and
        dispatch time, 2 synchronised time) sets the mode, with `reset` clears them; returns {op: {"count", "ms"}}."""
        import json
        if mode is not None:
            self._ns.op_stats_set_mode(int(mode))
        if reset:
            self._ns.op_stats_reset()
        need = C.c_uint64(0)
        self._ns.op_stats(None, 0, C.byref(need))
        buf = C.create_string_buffer(int(need.value) + 16)
        if self._ns.op_stats(buf, len(buf), C.byref(need)) != 0:
            raise BackendError(Status.INVALID_ARG, "cg_op_stats failed")
        return json.loads(buf.value.decode())

    def stats(self):
        """(live bytes, cached bytes, cudaMalloc calls, kernel launches) of the context (`cg_ctx_stats`)."""
        out = (C.c_uint64 * 4)()
        self._check(self._ns.ctx_stats(self._ctx, out))
        return tuple(int(v) for v in out)

    def synchronize(self):
        self._check(self._ns.synchronize(self._ctx))

    # -- constructors (mod.rs:28-58) --------------------------------------------------------------
    def zeros(self, shape, target_dtype):
        d, r = _dims(shape)
        return self._out(self._ns.zeros, d, r, int(target_dtype))

    def _from_vec(self, fn, data, np_dtype, shape):
        arr = np.ascontiguousarray(data, dtype=np_dtype).reshape(-1)
        d, r = _dims(shape)
        return self._out(fn, arr.ctypes.data_as(C.c_void_p), arr.size, d, r)

    def ndarray_from_vec_f32(self, data, shape):
        return self._from_vec(self._ns.from_vec_f32, data, np.float32, shape)

    def ndarray_from_vec_f16(self, data, shape):
        return self._from_vec(self._ns.from_vec_f16, data, np.float16, shape)

    def ndarray_from_vec_bf16(self, data, shape):
        """`data`: bf16 bit patterns as uint16."""
        return self._from_vec(self._ns.from_vec_bf16, data, np.uint16, shape)

    def ndarray_from_vec_fp8(self, data, shape):
        """`data`: e4m3 bit patterns as uint8."""
        return self._from_vec(self._ns.from_vec_fp8, data, np.uint8, shape)

    def ndarray_from_vec_u32(self, data, shape):
        return self._from_vec(self._ns.from_vec_u32, data, np.uint32, shape)

    def arange(self, end):
        return self._out(self._ns.arange, int(end))

    # -- ops ----------------------------------------------------------------------------------------
    def cast(self, x, target_dtype):
        return self._out(self._ns.cast, x.handle, int(target_dtype))

    def softmax(self, x):
        """Fused last-axis softmax (stdlib nn::softmax in one kernel; CUDA library only, not a trait method)."""
        if not hasattr(self._ns, "softmax"):
            raise BackendError(Status.CUDA, "the fused softmax exists only in the CUDA library")
        return self._out(self._ns.softmax, x.handle)

    def matmul(self, lhs, rhs):
        return self._out(self._ns.matmul, lhs.handle, rhs.handle)

    def add(self, a, b):
        return self._out(self._ns.add, a.handle, b.handle)

    def sub(self, a, b):
        return self._out(self._ns.sub, a.handle, b.handle)

    def mul(self, a, b):
        return self._out(self._ns.mul, a.handle, b.handle)

    def div(self, a, b):
        return self._out(self._ns.div, a.handle, b.handle)

    def pow(self, a, b):
        return self._out(self._ns.pow, a.handle, b.handle)

    def lt(self, a, b):
        return self._out(self._ns.lt, a.handle, b.handle)

    def gt(self, a, b):
        return self._out(self._ns.gt, a.handle, b.handle)

    def gte(self, a, b):
        return self._out(self._ns.gte, a.handle, b.handle)

    def lte(self, a, b):
        return self._out(self._ns.lte, a.handle, b.handle)

    def eq(self, a, b):
        return self._out(self._ns.eq, a.handle, b.handle)

    def where_cond(self, mask, x, y):
        return self._out(self._ns.where_cond, mask.handle, x.handle, y.handle)

    def sin(self, x):
        return self._out(self._ns.sin, x.handle)

    def cos(self, x):
        return self._out(self._ns.cos, x.handle)

    def exp(self, x):
        return self._out(self._ns.exp, x.handle)

    def log(self, x):
        return self._out(self._ns.log, x.handle)

    def floor(self, x):
        return self._out(self._ns.floor, x.handle)

    def round(self, x):
        return self._out(self._ns.round, x.handle)

    def neg(self, x):
        return self._out(self._ns.neg, x.handle)

    def broadcast(self, x, shape):
        d, r = _dims(shape)
        return self._out(self._ns.broadcast, x.handle, d, r)

    def reshape(self, x, new_shape):
        d, r = _dims(new_shape)
        return self._out(self._ns.reshape, x.handle, d, r)

    def transpose(self, x, dim0, dim1):
        return self._out(self._ns.transpose, x.handle, int(dim0), int(dim1))

    def max(self, x):
        return self._out(self._ns.max, x.handle)

    def sum(self, x):
        return self._out(self._ns.sum, x.handle)

    def argmax(self, x):
        return self._out(self._ns.argmax, x.handle)

    def topk(self, x, k):
        v, i = C.c_void_p(), C.c_void_p()
        self._check(self._ns.topk(self._ctx, x.handle, int(k), C.byref(v), C.byref(i)))
        return Tensor(self, v), Tensor(self, i)

    def compare(self, a, b):
        out = C.c_int()
        self._check(self._ns.compare(self._ctx, a.handle, b.handle, C.byref(out)))
        return bool(out.value)

    def concat(self, x, y, dim):
        return self._out(self._ns.concat, x.handle, y.handle, int(dim))

    def index(self, x, dim, indices):
        return self._out(self._ns.index, x.handle, int(dim), indices.handle)

    def slice(self, x, dim, start, length):
        return self._out(self._ns.slice, x.handle, int(dim), int(start), int(length))

    def to_bool(self, x):
        out = C.c_int()
        self._check(self._ns.to_bool(self._ctx, x.handle, C.byref(out)))
        return bool(out.value)

    def to_vec(self, x):
        """Flat row-major contents (TaggedVec); bf16/fp8 come back as bit patterns."""
        return self.to_numpy(x).reshape(-1)

    def format_tensor(self, x):
        buf = C.create_string_buffer(4096)
        self._check(self._ns.format(self._ctx, x.handle, buf, len(buf)))
        return buf.value.decode()

    # -- numpy convenience ------------------------------------------------------------------------
    def to_numpy(self, x):
        shape = x.shape
        arr = np.empty(shape, dtype=_NP_STORAGE[x.dtype])
        self._check(self._ns.to_vec(self._ctx, x.handle, arr.ctypes.data_as(C.c_void_p), arr.nbytes))
        return arr

    def to_f32(self, x):
        """Contents as float32 whatever the float dtype (bf16 widened exactly)."""
        a = self.to_numpy(x)
        if x.dtype == Dtype.BF16:
            return bf16_bits_to_f32(a).reshape(a.shape)
        return a.astype(np.float32)

    def from_numpy(self, arr, dtype=None):
        """float32/uint32/float16 arrays map to their dtype; dtype=BF16 rounds a float32 array to bf16."""
        arr = np.asarray(arr)
        if dtype is None:
            dtype = {np.dtype(np.float32): Dtype.F32, np.dtype(np.uint32): Dtype.U32,
                     np.dtype(np.float16): Dtype.F16}[arr.dtype]
        dtype = Dtype(dtype)
        if dtype == Dtype.F32:
            return self.ndarray_from_vec_f32(arr, arr.shape)
        if dtype == Dtype.U32:
            return self.ndarray_from_vec_u32(arr, arr.shape)
        if dtype == Dtype.F16:
            return self.ndarray_from_vec_f16(arr, arr.shape)
        if dtype == Dtype.BF16:
            bits = arr if arr.dtype == np.uint16 else f32_to_bf16_bits(arr)
            return self.ndarray_from_vec_bf16(bits, arr.shape)
        if dtype == Dtype.F8:
            return self.ndarray_from_vec_fp8(arr, arr.shape)
        raise ValueError(dtype)

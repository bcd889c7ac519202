"""Terms and the interpreter over the C ABI.

Mirrors, on the host side, the pieces of catgrad a caller touches to run a term:
`TermBuilder` ~ the `Builder`/`Var` DSL of catgrad/src/category/lang/ops.rs:74-428 (same function names and
argument orders), `Parameters` ~ interpreter/parameters.rs, `Interpreter.run` ~ interpreter.rs:33-36.
The enum values equal those of `cg::NodeType`, `cg::OpKind`, `cg::ScalarOp` in csrc/host/ir.h.
"""
import ctypes as C
import enum

from . import _ffi
from .backend import Dtype, Tensor


class NodeType(enum.IntEnum):
    Nat = 0
    Dtype = 1
    NdArrayType = 2
    Shape = 3
    Tensor = 4


class ScalarOp(enum.IntEnum):
    Add = 0
    Sub = 1
    Mul = 2
    Div = 3
    Neg = 4
    Pow = 5
    LT = 6
    GT = 7
    GTE = 8
    LTE = 9
    EQ = 10
    Cos = 11
    Sin = 12
    Exp = 13
    Log = 14
    Floor = 15
    Round = 16
    Where = 17


class OpKind(enum.IntEnum):
    TypePack = 0
    TypeUnpack = 1
    TypeShape = 2
    TypeDtype = 3
    NatConstant = 4
    NatMul = 5
    NatAdd = 6
    DtypeConstant = 7
    Map = 8
    NatToU32 = 9
    Cast = 10
    MatMul = 11
    ScalarF32 = 12
    ScalarU32 = 13
    Sum = 14
    Max = 15
    Argmax = 16
    TopK = 17
    Probe = 18
    Broadcast = 19
    Reshape = 20
    Transpose = 21
    Slice = 22
    Concat = 23
    Arange = 24
    Index = 25
    If = 26
    Copy = 27
    Load = 28


class Term:
    def __init__(self, backend, handle):
        self._be = backend
        self._h = handle

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and self._be._ns is not None:
            self._be._ns.term_free(h)

    @property
    def handle(self):
        return self._h

    @property
    def plan_state(self):
        """0: not run yet; 1: cg_interp_run recognised it and runs it as the fused Llama plan; 2: it runs op by op.
        Always 0 on a backend without the recogniser (the CPU oracle)."""
        fn = getattr(self._be._ns, "term_plan_state", None)
        return int(fn(self._h)) if fn is not None else 0

    def stats(self):
        """dict(nodes, edges, tensor_ops, layers)"""
        c = (C.c_uint64 * 4)()
        self._be._check(self._be._ns.term_stats(self._h, c), ctx=False)
        return dict(nodes=int(c[0]), edges=int(c[1]), tensor_ops=int(c[2]), layers=int(c[3]))


class Var:
    """A wire of the term under construction.  Arithmetic operators build Map edges like the reference's
    `Var` (lang/ops.rs:60-96)."""

    def __init__(self, builder, vid, ty):
        self.b, self.id, self.ty = builder, vid, ty

    def __add__(self, o):
        return self.b.map2(ScalarOp.Add, self, o)

    def __sub__(self, o):
        return self.b.map2(ScalarOp.Sub, self, o)

    def __mul__(self, o):
        return self.b.map2(ScalarOp.Mul, self, o)

    def __truediv__(self, o):
        return self.b.map2(ScalarOp.Div, self, o)

    def __neg__(self):
        return self.b.map1(ScalarOp.Neg, self)


class TermBuilder:
    def __init__(self, backend):
        self._be = backend
        h = C.c_void_p()
        backend._check(backend._ns.builder_new(C.byref(h)), ctx=False)
        self._h = h

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and self._be._ns is not None:
            self._be._ns.builder_free(h)

    # -- raw ------------------------------------------------------------------------------------
    def source(self, ty=NodeType.Tensor):
        v = C.c_int()
        self._be._check(self._be._ns.builder_source(self._h, int(ty), C.byref(v)), ctx=False)
        return Var(self, v.value, NodeType(ty))

    def op(self, kind, inputs, out_types, *, sop=ScalarOp.Add, nat=0, dtype=Dtype.F32, f32=0.0, u32=0, s=None,
           then_term=None, else_term=None):
        n_in, n_out = len(inputs), len(out_types)
        ins = (C.c_int * max(n_in, 1))(*[v.id for v in inputs])
        outs_t = (C.c_int * max(n_out, 1))(*[int(t) for t in out_types])
        outs = (C.c_int * max(n_out, 1))()
        self._be._check(self._be._ns.builder_op(
            self._h, int(kind), int(sop), int(nat), int(dtype), float(f32), int(u32),
            s.encode() if s is not None else None,
            then_term.handle if then_term is not None else None,
            else_term.handle if else_term is not None else None,
            ins, n_in, outs_t, n_out, outs), ctx=False)
        return [Var(self, outs[i], NodeType(out_types[i])) for i in range(n_out)]

    def finish(self, targets):
        t = (C.c_int * max(len(targets), 1))(*[v.id for v in targets])
        h = C.c_void_p()
        self._be._check(self._be._ns.builder_finish(self._h, t, len(targets), C.byref(h)), ctx=False)
        return Term(self._be, h)

    # -- DSL, argument orders of lang/ops.rs ------------------------------------------------------
    def _nat(self, x):
        return x if isinstance(x, Var) else self.nat(x)

    def nat(self, n):
        return self.op(OpKind.NatConstant, [], [NodeType.Nat], nat=n)[0]

    def dtype_constant(self, d):
        return self.op(OpKind.DtypeConstant, [], [NodeType.Dtype], dtype=d)[0]

    def lit(self, x):
        """f32 for Python floats, u32 for ints (Literal::{F32,U32})."""
        if isinstance(x, float):
            return self.op(OpKind.ScalarF32, [], [NodeType.Tensor], f32=x)[0]
        return self.op(OpKind.ScalarU32, [], [NodeType.Tensor], u32=x)[0]

    def param(self, path):
        return self.op(OpKind.Load, [], [NodeType.Tensor], s=path)[0]

    def pack(self, extents):
        return self.op(OpKind.TypePack, [self._nat(e) for e in extents], [NodeType.Shape])[0]

    def unpack(self, shape, n):
        return self.op(OpKind.TypeUnpack, [shape], [NodeType.Nat] * n)

    def shape(self, x):
        return self.op(OpKind.TypeShape, [x], [NodeType.Shape])[0]

    def dtype(self, x):
        return self.op(OpKind.TypeDtype, [x], [NodeType.Dtype])[0]

    def map1(self, sop, x):
        return self.op(OpKind.Map, [x], [NodeType.Tensor], sop=sop)[0]

    def map2(self, sop, x, y):
        return self.op(OpKind.Map, [x, y], [NodeType.Tensor], sop=sop)[0]

    def pow(self, x, y):
        return self.map2(ScalarOp.Pow, x, y)

    def sin(self, x):
        return self.map1(ScalarOp.Sin, x)

    def cos(self, x):
        return self.map1(ScalarOp.Cos, x)

    def exp(self, x):
        return self.map1(ScalarOp.Exp, x)

    def log(self, x):
        return self.map1(ScalarOp.Log, x)

    def floor(self, x):
        return self.map1(ScalarOp.Floor, x)

    def round(self, x):
        return self.map1(ScalarOp.Round, x)

    def lt(self, x, y):
        return self.map2(ScalarOp.LT, x, y)

    def gt(self, x, y):
        return self.map2(ScalarOp.GT, x, y)

    def gte(self, x, y):
        return self.map2(ScalarOp.GTE, x, y)

    def lte(self, x, y):
        return self.map2(ScalarOp.LTE, x, y)

    def eq(self, x, y):
        return self.map2(ScalarOp.EQ, x, y)

    def where_cond(self, mask, x, y):
        return self.op(OpKind.Map, [mask, x, y], [NodeType.Tensor], sop=ScalarOp.Where)[0]

    def broadcast(self, s, x):
        return self.op(OpKind.Broadcast, [x, s], [NodeType.Tensor])[0]

    def reshape(self, s, x):
        return self.op(OpKind.Reshape, [s, x], [NodeType.Tensor])[0]

    def transpose(self, dim0, dim1, x):
        return self.op(OpKind.Transpose, [x, self._nat(dim0), self._nat(dim1)], [NodeType.Tensor])[0]

    def index(self, dim, idx, x):
        return self.op(OpKind.Index, [x, self._nat(dim), idx], [NodeType.Tensor])[0]

    def slice(self, dim, start, length, x):
        return self.op(OpKind.Slice, [x, self._nat(dim), self._nat(start), self._nat(length)], [NodeType.Tensor])[0]

    def concat(self, dim, x, y):
        return self.op(OpKind.Concat, [x, y, self._nat(dim)], [NodeType.Tensor])[0]

    def arange(self, end):
        return self.op(OpKind.Arange, [self._nat(end)], [NodeType.Tensor])[0]

    def max(self, x):
        return self.op(OpKind.Max, [x], [NodeType.Tensor])[0]

    def sum(self, x):
        return self.op(OpKind.Sum, [x], [NodeType.Tensor])[0]

    def argmax(self, x):
        return self.op(OpKind.Argmax, [x], [NodeType.Tensor])[0]

    def topk(self, k, x):
        r = self.op(OpKind.TopK, [x, self._nat(k)], [NodeType.Tensor, NodeType.Tensor])
        return r[0], r[1]

    def nat_to_u32(self, n):
        return self.op(OpKind.NatToU32, [n], [NodeType.Tensor])[0]

    def matmul(self, f, g):
        return self.op(OpKind.MatMul, [f, g], [NodeType.Tensor])[0]

    def cast(self, x, dtype):
        d = dtype if isinstance(dtype, Var) else self.dtype_constant(dtype)
        return self.op(OpKind.Cast, [x, d], [NodeType.Tensor])[0]

    def nat_add(self, x, y):
        return self.op(OpKind.NatAdd, [self._nat(x), self._nat(y)], [NodeType.Nat])[0]

    def nat_mul(self, x, y):
        return self.op(OpKind.NatMul, [self._nat(x), self._nat(y)], [NodeType.Nat])[0]

    def probe(self, label, x):
        self.op(OpKind.Probe, [x], [], s=label)

    def cond(self, condition, then_term, else_term, args, out_types):
        return self.op(OpKind.If, [condition] + list(args), out_types, then_term=then_term, else_term=else_term)

    def constant(self, x, s):
        """stdlib/ops.rs:21-24"""
        return self.broadcast(s, self.lit(x))


class Parameters:
    """path -> tensor (interpreter/parameters.rs)."""

    def __init__(self, backend, tensors=None):
        self._be = backend
        h = C.c_void_p()
        backend._check(backend._ns.params_new(C.byref(h)), ctx=False)
        self._h = h
        self._keep = {}
        for k, v in (tensors or {}).items():
            self[k] = v

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and self._be._ns is not None:
            self._be._ns.params_free(h)

    def __setitem__(self, path, tensor):
        self._be._check(self._be._ns.params_set(self._h, path.encode(), tensor.handle), ctx=False)
        self._keep[path] = tensor

    def __getitem__(self, path):
        return self._keep[path]

    def keys(self):
        return self._keep.keys()

    @property
    def handle(self):
        return self._h


class Interpreter:
    """`Interpreter<B>` (interpreter.rs:13-37): a backend plus parameters; `run` evaluates a term."""

    def __init__(self, backend, parameters=None):
        self.backend = backend
        self.parameters = parameters

    def run(self, term, args, max_outputs=16):
        """args: Tensors, ints (Nat), Dtype, or tuples (Shape).  Returns the same kinds."""
        be = self.backend
        n = len(args)
        ins = (_ffi.ValueStruct * max(n, 1))()
        for i, a in enumerate(args):
            if isinstance(a, Tensor):
                ins[i].kind, ins[i].tensor = 4, a.handle
            elif isinstance(a, Dtype):
                ins[i].kind, ins[i].dtype = 2, int(a)
            elif isinstance(a, (tuple, list)):
                ins[i].kind, ins[i].rank = 3, len(a)
                for j, d in enumerate(a):
                    ins[i].dims[j] = int(d)
            else:
                ins[i].kind, ins[i].nat = 1, int(a)
        outs = (_ffi.ValueStruct * max_outputs)()
        n_out = C.c_int()
        be._check(be._ns.interp_run(be._ctx, term.handle, self.parameters.handle if self.parameters else None,
                                    ins, n, outs, max_outputs, C.byref(n_out)))
        res = []
        for i in range(n_out.value):
            v = outs[i]
            if v.kind == 4:
                res.append(Tensor(be, C.c_void_p(v.tensor)))
            elif v.kind == 3:
                res.append(tuple(int(v.dims[j]) for j in range(v.rank)))
            elif v.kind == 2:
                res.append(Dtype(v.dtype))
            else:
                res.append(int(v.nat))
        return res

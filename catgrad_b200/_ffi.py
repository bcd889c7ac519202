"""ctypes signatures of the C ABI declared in include/catgrad_b200.h.

`bind(cdll, prefix)` attaches argtypes/restypes for every entry point the library exports under
`prefix` and returns a namespace whose attributes are the un-prefixed names (`ns.add`, `ns.matmul`, ...).
The shipped library uses the prefix ``cg_``.
"""
import ctypes as C
import os

MAX_RANK = 8

c_void_pp = C.POINTER(C.c_void_p)
u64p = C.POINTER(C.c_uint64)
i64p = C.POINTER(C.c_int64)
intp = C.POINTER(C.c_int)


class LlamaConfigStruct(C.Structure):
    """cg_llama_config"""
    _fields_ = [
        ("hidden_size", C.c_uint64),
        ("intermediate_size", C.c_uint64),
        ("num_hidden_layers", C.c_uint64),
        ("num_attention_heads", C.c_uint64),
        ("num_key_value_heads", C.c_uint64),
        ("vocab_size", C.c_uint64),
        ("rope_theta", C.c_float),
        ("rms_norm_eps", C.c_float),
        ("tie_word_embeddings", C.c_int),
        ("rope_scaling_type", C.c_int),
        ("rope_factor", C.c_float),
        ("rope_low_freq_factor", C.c_float),
        ("rope_high_freq_factor", C.c_float),
        ("rope_original_max_position", C.c_uint64),
    ]


class ValueStruct(C.Structure):
    """cg_value"""
    _fields_ = [
        ("kind", C.c_int),
        ("nat", C.c_uint64),
        ("dtype", C.c_int),
        ("dims", C.c_uint64 * MAX_RANK),
        ("rank", C.c_int),
        ("tensor", C.c_void_p),
    ]


_T = C.c_void_p  # cg_tensor*
_CTX = C.c_void_p

# name -> (restype, argtypes).  Functions marked core exist in every build of c_api.cc; the rest only in
# the CUDA library.
CORE = {
    "init": (C.c_int, [C.c_int, c_void_pp]),
    "destroy": (None, [_CTX]),
    "last_error": (C.c_char_p, [_CTX]),
    "synchronize": (C.c_int, [_CTX]),
    "backend_name": (C.c_char_p, [_CTX]),
    "retain": (None, [_T]),
    "release": (None, [_T]),
    "rank": (C.c_int, [_T]),
    "shape": (C.c_int, [_T, u64p, intp]),
    "dtype_of": (C.c_int, [_T]),
    "is_contiguous": (C.c_int, [_T]),
    "data_ptr": (C.c_void_p, [_T]),
    "strides": (C.c_int, [_T, i64p, intp]),
    "zeros": (C.c_int, [_CTX, u64p, C.c_int, C.c_int, c_void_pp]),
    "from_vec_f32": (C.c_int, [_CTX, C.c_void_p, C.c_uint64, u64p, C.c_int, c_void_pp]),
    "from_vec_f16": (C.c_int, [_CTX, C.c_void_p, C.c_uint64, u64p, C.c_int, c_void_pp]),
    "from_vec_bf16": (C.c_int, [_CTX, C.c_void_p, C.c_uint64, u64p, C.c_int, c_void_pp]),
    "from_vec_fp8": (C.c_int, [_CTX, C.c_void_p, C.c_uint64, u64p, C.c_int, c_void_pp]),
    "from_vec_u32": (C.c_int, [_CTX, C.c_void_p, C.c_uint64, u64p, C.c_int, c_void_pp]),
    "arange": (C.c_int, [_CTX, C.c_uint64, c_void_pp]),
    "cast": (C.c_int, [_CTX, _T, C.c_int, c_void_pp]),
    "matmul": (C.c_int, [_CTX, _T, _T, c_void_pp]),
    "where_cond": (C.c_int, [_CTX, _T, _T, _T, c_void_pp]),
    "broadcast": (C.c_int, [_CTX, _T, u64p, C.c_int, c_void_pp]),
    "reshape": (C.c_int, [_CTX, _T, u64p, C.c_int, c_void_pp]),
    "transpose": (C.c_int, [_CTX, _T, C.c_uint64, C.c_uint64, c_void_pp]),
    "max": (C.c_int, [_CTX, _T, c_void_pp]),
    "sum": (C.c_int, [_CTX, _T, c_void_pp]),
    "argmax": (C.c_int, [_CTX, _T, c_void_pp]),
    "topk": (C.c_int, [_CTX, _T, C.c_uint64, c_void_pp, c_void_pp]),
    "compare": (C.c_int, [_CTX, _T, _T, intp]),
    "concat": (C.c_int, [_CTX, _T, _T, C.c_uint64, c_void_pp]),
    "index": (C.c_int, [_CTX, _T, C.c_uint64, _T, c_void_pp]),
    "slice": (C.c_int, [_CTX, _T, C.c_uint64, C.c_uint64, C.c_uint64, c_void_pp]),
    "to_bool": (C.c_int, [_CTX, _T, intp]),
    "to_vec": (C.c_int, [_CTX, _T, C.c_void_p, C.c_uint64]),
    "format": (C.c_int, [_CTX, _T, C.c_char_p, C.c_uint64]),
    "builder_new": (C.c_int, [c_void_pp]),
    "builder_free": (None, [C.c_void_p]),
    "builder_source": (C.c_int, [C.c_void_p, C.c_int, intp]),
    "builder_op": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_uint64, C.c_int, C.c_float, C.c_uint32, C.c_char_p,
                             C.c_void_p, C.c_void_p, intp, C.c_int, intp, C.c_int, intp]),
    "builder_finish": (C.c_int, [C.c_void_p, intp, C.c_int, c_void_pp]),
    "term_free": (None, [C.c_void_p]),
    "term_stats": (C.c_int, [C.c_void_p, u64p]),
    "llama_term": (C.c_int, [C.POINTER(LlamaConfigStruct), C.c_int, c_void_pp]),
    "params_new": (C.c_int, [c_void_pp]),
    "params_free": (None, [C.c_void_p]),
    "params_set": (C.c_int, [C.c_void_p, C.c_char_p, _T]),
    "interp_run": (C.c_int, [_CTX, C.c_void_p, C.c_void_p, C.POINTER(ValueStruct), C.c_int, C.POINTER(ValueStruct),
                             C.c_int, intp]),
    "op_stats_set_mode": (None, [C.c_int]),
    "op_stats_reset": (None, []),
    "op_stats": (C.c_int, [C.c_char_p, C.c_uint64, C.POINTER(C.c_uint64)]),
}
for _name in ("add", "sub", "mul", "div", "pow", "lt", "gt", "gte", "lte", "eq"):
    CORE[_name] = (C.c_int, [_CTX, _T, _T, c_void_pp])
for _name in ("sin", "cos", "exp", "log", "floor", "round", "neg"):
    CORE[_name] = (C.c_int, [_CTX, _T, c_void_pp])

CUDA_ONLY = {
    "llama_create": (C.c_int, [_CTX, C.POINTER(LlamaConfigStruct), C.c_int, C.c_void_p, C.c_uint64, C.c_uint64,
                               c_void_pp]),
    "llama_free": (None, [C.c_void_p]),
    "llama_create_tp": (C.c_int, [_CTX, C.POINTER(LlamaConfigStruct), C.c_int, C.c_void_p, C.c_uint64, C.c_uint64,
                                  C.c_void_p, C.c_uint64, c_void_pp]),
    "random_normal": (C.c_int, [_CTX, C.c_uint64, C.c_float, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64,
                                C.c_int, c_void_pp]),
    "softmax": (C.c_int, [_CTX, C.c_void_p, c_void_pp]),
    "comm_create": (C.c_int, [_CTX, C.c_int, C.c_int, C.c_uint64, c_void_pp]),
    "comm_handle": (C.c_int, [C.c_void_p, C.c_void_p]),
    "comm_attach": (C.c_int, [C.c_void_p, C.c_void_p]),
    "comm_attach_local": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "comm_set_timeout_ms": (C.c_int, [C.c_void_p, C.c_uint64]),
    "comm_write": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64]),
    "comm_read": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p, C.c_uint64]),
    "comm_data": (C.c_int, [C.c_void_p, c_void_pp, C.POINTER(C.c_uint64)]),
    "comm_allreduce": (C.c_int, [C.c_void_p, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_int]),
    "comm_free": (None, [C.c_void_p]),
    "llama_reset": (C.c_int, [C.c_void_p, C.c_uint64]),
    "llama_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p]),
    "llama_decode": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p]),
    "llama_last_logits": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64]),
    "term_plan_state": (C.c_int, [C.c_void_p]),
    "interp_set_planning": (None, [C.c_int]),
    "llama_set_persistent": (C.c_int, [C.c_void_p, C.c_int]),
    "llama_persistent_active": (C.c_int, [C.c_void_p]),
    "llama_context_len": (C.c_uint64, [C.c_void_p]),
    "llama_launch_count": (C.c_uint64, [C.c_void_p]),
    "runner_create": (C.c_int, [C.POINTER(C.c_int), C.c_int, C.POINTER(LlamaConfigStruct), C.c_int, C.c_uint64, C.c_uint64,
                                c_void_pp]),
    "runner_size": (C.c_int, [C.c_void_p]),
    "runner_ctx": (C.c_void_p, [C.c_void_p, C.c_int]),
    "runner_set_params": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "runner_generate": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p]),
    "runner_last_error": (C.c_char_p, [C.c_void_p]),
    "runner_free": (None, [C.c_void_p]),
    "event_record": (C.c_int, [_CTX, C.c_int]),
    "event_elapsed_ms": (C.c_int, [_CTX, C.c_int, C.c_int, C.POINTER(C.c_float)]),
    "ctx_stats": (C.c_int, [_CTX, u64p]),
    "flush_l2": (C.c_int, [_CTX, C.c_uint64]),
    "argmax_rows_noalloc": (C.c_int, [C.c_void_p, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p]),
}


class Namespace:
    pass


def bind(cdll, prefix="cg_", require_cuda_entry_points=True):
    """Returns a namespace of typed functions.  Raises AttributeError if a declared symbol is missing."""
    ns = Namespace()
    ns.cdll = cdll
    ns.prefix = prefix
    tables = [CORE] + ([CUDA_ONLY] if require_cuda_entry_points else [])
    for table in tables:
        for name, (restype, argtypes) in table.items():
            fn = getattr(cdll, prefix + name)
            fn.restype = restype
            fn.argtypes = argtypes
            setattr(ns, name, fn)
    return ns


def library_path():
    """Location of the in-tree CUDA library built by `__graft_entry__.build()`."""
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "_lib", "libcatgrad_b200.so")

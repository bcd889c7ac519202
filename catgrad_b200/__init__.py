"""catgrad_b200 — a B200-native tensor backend for catgrad's interpreter.

The product is the C-ABI shared library `catgrad_b200/_lib/libcatgrad_b200.so` (hand-written sm_100a CUDA
kernels plus a C++ host layer; header: include/catgrad_b200.h).  This package is the thin host-side mirror of
catgrad's `Backend` trait, of its term builder/interpreter and of the Llama generate loop over that ABI.
"""
from .backend import Backend, BackendError, Dtype, Status, Tensor, bf16_bits_to_f32, f32_to_bf16_bits  # noqa: F401
from .ir import Interpreter, NodeType, OpKind, Parameters, ScalarOp, Term, TermBuilder  # noqa: F401
from .llama import (LLAMA_1B, LLAMA_8B, TINY, LlamaConfig, LlamaRunner, bench_table, empty_state_cache,  # noqa: F401
                    generate_with_interpreter, llama_term, random_weights, upload_weights)
from . import safetensors, tp  # noqa: F401,E402

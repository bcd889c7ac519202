"""Tensor-parallel execution of the fused Llama plan (`cg_comm_*`, `cg_llama_create_tp`).

The reference has no multi-GPU path.  The split follows the usual column/row scheme over the projections of
catgrad-llm's Llama (catgrad-llm-models/src/models/llama.rs:303-385): q/k/v and gate/up are split by output rows
(whole heads / FFN columns per rank), o_proj and down_proj by input columns, and the partial products of those two are
summed across ranks into the residual stream.  Norm gains, the embedding and the lm_head are replicated.
"""
import ctypes as C

import numpy as np

from .backend import BackendError, Status

ROW_SHARDED = ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
               "mlp.gate_proj.weight", "mlp.up_proj.weight")
COL_SHARDED = ("self_attn.o_proj.weight", "mlp.down_proj.weight")


def check_divisible(cfg, size):
    if size < 1 or size > 8:
        raise ValueError("tensor-parallel size must be 1..8")
    if cfg.num_key_value_heads % size or cfg.num_attention_heads % size or cfg.intermediate_size % size:
        raise ValueError(f"heads ({cfg.num_attention_heads}/{cfg.num_key_value_heads}) and intermediate size "
                         f"({cfg.intermediate_size}) must divide by the tensor-parallel size {size}")


def shard_slice(n, rank, size):
    """Rows (or columns) [lo, hi) of an axis of length n that rank `rank` of `size` owns."""
    if n % size:
        raise ValueError(f"axis of {n} does not divide by {size}")
    step = n // size
    return rank * step, (rank + 1) * step


def shard_weights(cfg, weights, rank, size):
    """dict key -> array holding rank's share of `weights` (safetensors names, `[out, in]` matrices)."""
    check_divisible(cfg, size)
    out = {}
    for key, w in weights.items():
        if key.endswith(ROW_SHARDED):
            lo, hi = shard_slice(w.shape[0], rank, size)
            out[key] = np.ascontiguousarray(w[lo:hi])
        elif key.endswith(COL_SHARDED):
            lo, hi = shard_slice(w.shape[1], rank, size)
            out[key] = np.ascontiguousarray(w[:, lo:hi])
        else:
            out[key] = w
    return out


SHARD_BLOCKS = 8   # a sharded axis is drawn in 8 independent blocks, so every size in {1, 2, 4, 8} sees the same model


def _normal_bf16_bits(shape, seed_key, std):
    """N(0, std) drawn as float32 and rounded to bf16 bit patterns (uint16), ~16 M values at a time."""
    import zlib
    rng = np.random.Generator(np.random.SFC64(zlib.crc32(seed_key.encode())))
    n = int(np.prod(shape))
    out = np.empty(n, dtype=np.uint16)
    step = 1 << 24
    for lo in range(0, n, step):
        a = rng.standard_normal(min(step, n - lo), dtype=np.float32)
        a *= np.float32(std)
        u = a.view(np.uint32)
        u += np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
        out[lo:lo + a.size] = (u >> np.uint32(16)).astype(np.uint16)
    return out.reshape(shape)


def random_shard_bf16(cfg, rank, size, seed=0, std=0.02):
    """This rank's shard of a random-init bf16 model (bit patterns as uint16; gains are 1.0), generated without ever
    materialising the whole model: a sharded axis is drawn block by block from seeds that depend only on (seed,
    key, block), so the ranks of any tensor-parallel size in {1, 2, 4, 8} hold slices of one and the same model."""
    check_divisible(cfg, size)
    if SHARD_BLOCKS % size:
        raise ValueError("tensor-parallel size must divide 8")
    per = SHARD_BLOCKS // size
    blocks = range(rank * per, (rank + 1) * per)
    out = {}
    for key, shape in cfg.param_shapes():
        if len(shape) == 1:
            out[key] = np.full(shape, 0x3F80, dtype=np.uint16)
        elif key.endswith(ROW_SHARDED):
            rows = shape[0] // SHARD_BLOCKS
            out[key] = np.concatenate([_normal_bf16_bits((rows, shape[1]), f"{seed}/{key}/{b}", std) for b in blocks], 0)
        elif key.endswith(COL_SHARDED):
            cols = shape[1] // SHARD_BLOCKS
            out[key] = np.ascontiguousarray(
                np.concatenate([_normal_bf16_bits((shape[0], cols), f"{seed}/{key}/{b}", std) for b in blocks], 1))
        else:
            out[key] = _normal_bf16_bits(shape, f"{seed}/{key}", std)
    return out


def random_shard_device(backend, cfg, rank, size, dtype, seed=0, std=0.02):
    """Parameters holding this rank's shard of a random-init model, drawn on the device (`cg_random_normal`): each
    element depends only on (seed, key, its position in the unsharded matrix), so all ranks of any size hold slices
    of the same model and nothing model-sized ever exists on the host.  Norm gains are 1."""
    import zlib
    from .ir import Parameters
    check_divisible(cfg, size)
    params = Parameters(backend)
    for key, shape in cfg.param_shapes():
        if len(shape) == 1:
            params[key] = backend.from_numpy(np.ones(shape, dtype=np.float32), dtype)
            continue
        rows, cols = shape
        row0 = col0 = 0
        if key.endswith(ROW_SHARDED):
            row0, hi = shard_slice(rows, rank, size)
            rows = hi - row0
        elif key.endswith(COL_SHARDED):
            col0, hi = shard_slice(cols, rank, size)
            cols = hi - col0
        tseed = (int(seed) << 32) | zlib.crc32(key.encode())
        params[key] = backend._out(backend._ns.random_normal, tseed, float(std), rows, cols, row0, col0, shape[1],
                                   int(dtype))
    return params


def comm_bytes(cfg, max_tokens, element_size):
    """Size of the symmetric data area a tensor-parallel runner needs."""
    one = (max_tokens * cfg.hidden_size * element_size + 255) // 256 * 256
    return 2 * one


class TpComm:
    """This rank's symmetric buffer plus the mappings of its peers' buffers."""

    def __init__(self, backend, rank, size, data_bytes):
        if not hasattr(backend._ns, "comm_create"):
            raise BackendError(Status.CUDA, "tensor parallelism exists only in the CUDA library")
        self._be = backend
        self.rank, self.size = rank, size
        h = C.c_void_p()
        backend._check(backend._ns.comm_create(backend._ctx, rank, size, int(data_bytes), C.byref(h)))
        self.handle = h

    def ipc_handle(self):
        buf = (C.c_ubyte * 64)()
        self._be._check(self._be._ns.comm_handle(self.handle, buf))
        return bytes(buf)

    def attach(self, handles):
        """handles: list of `size` 64-byte strings in rank order (as gathered from `ipc_handle()` of every rank)."""
        if len(handles) != self.size or any(len(h) != 64 for h in handles):
            raise ValueError("need one 64-byte handle per rank")
        blob = b"".join(handles)
        self._be._check(self._be._ns.comm_attach(self.handle, blob))

    def attach_local(self, comms):
        """Same-process attach: `comms` = the TpComm of every rank, in rank order."""
        arr = (C.c_void_p * self.size)(*[c.handle.value for c in comms])
        self._be._check(self._be._ns.comm_attach_local(self.handle, arr))

    def set_timeout_ms(self, ms):
        self._be._check(self._be._ns.comm_set_timeout_ms(self.handle, int(ms)))

    def allreduce(self, dtype, x_off, part_off, n, residual):
        self._be._check(self._be._ns.comm_allreduce(self.handle, int(dtype), x_off, part_off, n, int(residual)))

    def write(self, off, arr):
        arr = np.ascontiguousarray(arr)
        self._be._check(self._be._ns.comm_write(self.handle, off, arr.ctypes.data_as(C.c_void_p), arr.nbytes))

    def read(self, off, n, dtype):
        out = np.empty(n, dtype=dtype)
        self._be._check(self._be._ns.comm_read(self.handle, off, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def data_ptr(self):
        p, n = C.c_void_p(), C.c_uint64()
        self._be._check(self._be._ns.comm_data(self.handle, C.byref(p), C.byref(n)))
        return p.value, n.value

    def close(self):
        h, self.handle = self.handle, None
        if h and self._be._ns is not None:
            self._be._ns.comm_free(h)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def connect(backend, data_bytes, group=None):
    """Creates the communicator of this process's rank in the `torch.distributed` group and attaches it to all
    peers (handles travel through `all_gather_object`, which is also the barrier the protocol needs)."""
    import torch.distributed as dist
    rank, size = dist.get_rank(group), dist.get_world_size(group)
    comm = TpComm(backend, rank, size, data_bytes)
    if size > 1:
        handles = [None] * size
        dist.all_gather_object(handles, comm.ipc_handle(), group=group)
        comm.attach(handles)
        dist.barrier(group)
    return comm

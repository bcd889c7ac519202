"""Multi-GPU runner: independent sequences are sharded batch-wise across ranks (one process per GPU).

The reference has no distributed code (single device, batch 1: examples/llama/main.rs:947-951); its Llama term is
batch-polymorphic (llama.rs:159,271), which is what makes this split legal: every sequence's result is independent
of which rank ran it and of the other sequences in its batch.  There is no collective on the data path; the
generated ids are gathered once at the end.
"""
import ctypes as C

import numpy as np


def shard_range(n_items, world_size, rank):
    """Contiguous share [lo, hi) of rank `rank`; the first n_items % world_size ranks hold one extra item."""
    if not (0 <= rank < world_size):
        raise ValueError("rank out of range")
    base, extra = divmod(n_items, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def gather_rows(local, n_total, dist=None, device=None):
    """All ranks contribute their [n_local, k] uint32 rows (in shard_range order); every rank gets [n_total, k].
    `dist` is torch.distributed (already initialised) or None for a single process."""
    local = np.ascontiguousarray(local, dtype=np.uint32)
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        assert local.shape[0] == n_total
        return local
    import torch
    world = dist.get_world_size()
    k = local.shape[1]
    counts = [shard_range(n_total, world, r)[1] - shard_range(n_total, world, r)[0] for r in range(world)]
    width = max(counts)
    padded = np.zeros((width, k), dtype=np.int64)          # equal-sized pieces for all_gather
    padded[:local.shape[0]] = local
    t = torch.from_numpy(padded)
    if device is not None:
        t = t.to(device)
    pieces = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(pieces, t)
    rows = [p.cpu().numpy()[:c] for p, c in zip(pieces, counts)]
    return np.concatenate(rows, axis=0).astype(np.uint32)


def generate_sharded(make_runner, prompts, steps, dist=None, device=None):
    """Greedy generation of all prompts [N, S]: this rank runs its contiguous share through `make_runner(batch)`
    (an object with .generate(prompts, steps) -> [batch, steps]) and the ids of all ranks are gathered."""
    prompts = np.ascontiguousarray(prompts, dtype=np.uint32)
    world = dist.get_world_size() if dist is not None and dist.is_initialized() else 1
    rank = dist.get_rank() if world > 1 else 0
    lo, hi = shard_range(prompts.shape[0], world, rank)
    if hi > lo:
        local = make_runner(hi - lo).generate(prompts[lo:hi], steps)
    else:
        local = np.zeros((0, steps), dtype=np.uint32)
    return gather_rows(local, prompts.shape[0], dist, device)


class DeviceRunner:
    """`cg_runner_*`: one process driving several GPUs, one context + weight replica + fused Llama runner per device
    on its own host thread, sequences split by `shard_range`, ids gathered on the host.

        r = DeviceRunner([0, 1, 2, 3], cfg, Dtype.BF16, max_batch_per_device=64, max_positions=256)
        for i in range(r.size):
            r.set_params(i, upload_weights(r.backend(i), weights, Dtype.BF16))
        ids = r.generate(prompts, steps)                 # [n_seq, steps]
    """

    def __init__(self, devices, cfg, dtype, max_batch_per_device, max_positions):
        from . import _ffi
        from .backend import BackendError
        self._ns = _ffi.bind(C.CDLL(_ffi.library_path()))
        self._err = BackendError
        devs = (C.c_int * len(devices))(*[int(d) for d in devices])
        st = cfg.to_struct()
        h = C.c_void_p()
        code = self._ns.runner_create(devs, len(devices), C.byref(st), int(dtype), int(max_batch_per_device), int(max_positions),
                                      C.byref(h))
        if code != 0:
            raise BackendError(code, self._ns.last_error(None).decode())
        self._h = h
        self._keep = {}

    @property
    def size(self):
        return int(self._ns.runner_size(self._h))

    def backend(self, i):
        """A `Backend` over replica i's context (owned by the runner): upload that replica's parameters through it."""
        from .backend import Backend
        ctx = self._ns.runner_ctx(self._h, int(i))
        if not ctx:
            raise IndexError(i)
        return Backend(_borrowed_ctx=C.c_void_p(ctx))

    def set_params(self, i, params):
        code = self._ns.runner_set_params(self._h, int(i), params.handle)
        if code != 0:
            raise self._err(code, self._ns.last_error(None).decode())
        self._keep[i] = params

    def generate(self, prompts, steps):
        prompts = np.ascontiguousarray(prompts, dtype=np.uint32)
        n, s = prompts.shape
        out = np.zeros((n, steps), dtype=np.uint32)
        code = self._ns.runner_generate(self._h, prompts.ctypes.data_as(C.c_void_p), n, s, int(steps), out.ctypes.data_as(C.c_void_p))
        if code != 0:
            raise self._err(code, self._ns.runner_last_error(self._h).decode() or self._ns.last_error(None).decode())
        return out

    def close(self):
        h, self._h = getattr(self, "_h", None), None
        self._keep = {}
        if h:
            self._ns.runner_free(h)

    def __del__(self):
        self.close()

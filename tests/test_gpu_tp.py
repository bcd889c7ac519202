"""Tensor-parallel runner on the GPU.  With one GPU: a single-rank communicator must reproduce the plain runner bit
for bit (same kernels, the residual add moved into the all-reduce kernel), the all-reduce entry point computes what
its header says, and a wait on a peer that never arrives ends with CG_ERR_TIMEOUT and a usable context.  With two
or more GPUs: two processes, one per GPU, against the unsharded model (tests/tp_worker.py)."""
import os
import socket
import subprocess
import sys
import time

import numpy as np
import pytest

import catgrad_b200 as cb
from catgrad_b200 import BackendError, Dtype, Status, tp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _device_count():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("dtype,batch", [(Dtype.F32, 1), (Dtype.F32, 20), (Dtype.BF16, 3), (Dtype.BF16, 40)])
def test_single_rank_communicator_reproduces_the_plain_runner(gpu, dtype, batch):
    cfg = cb.LlamaConfig(512, 1536, 2, 8, 2, 4096, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=True)
    w = cb.random_weights(cfg, seed=0)
    params = cb.upload_weights(gpu, w, dtype)
    ids = np.random.default_rng(2).integers(0, cfg.vocab_size, size=(batch, 17), dtype=np.uint32)
    plain = cb.LlamaRunner(gpu, cfg, params, dtype, max_batch=batch, max_positions=32)
    plain.set_persistent(False)          # the tensor-parallel runner always takes the kernel-per-sub-graph plan
    want = plain.generate(ids, 8)
    want_logits = plain.last_logits()
    es = 4 if dtype == Dtype.F32 else 2
    comm = tp.TpComm(gpu, 0, 1, tp.comm_bytes(cfg, batch * 17, es))
    sharded = cb.LlamaRunner(gpu, cfg, params, dtype, max_batch=batch, max_positions=32, comm=comm,
                             max_tokens=batch * 17)
    got = sharded.generate(ids, 8)
    np.testing.assert_array_equal(got, want)
    np.testing.assert_array_equal(sharded.last_logits().view(np.uint32), want_logits.view(np.uint32))
    with pytest.raises(BackendError):     # more tokens than the symmetric buffer was sized for
        sharded.reset(batch)
        sharded.forward(np.zeros((batch, 18), dtype=np.uint32))


def test_allreduce_entry_point_single_rank(gpu):
    n = 3 * 4096
    comm = tp.TpComm(gpu, 0, 1, 2 * n * 4)
    ptr, nbytes = comm.data_ptr()
    assert ptr and nbytes == 2 * n * 4
    rng = np.random.default_rng(0)
    x, part = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    comm.write(0, x)
    comm.write(n * 4, part)
    comm.allreduce(Dtype.F32, 0, n * 4, n, residual=True)
    comm.allreduce(Dtype.F32, 0, n * 4, n, residual=True)
    np.testing.assert_array_equal(comm.read(0, n, np.float32), (x + part) + part)
    comm.allreduce(Dtype.F32, 0, n * 4, n, residual=False)
    np.testing.assert_array_equal(comm.read(0, n, np.float32), part)
    # bf16: the sum is rounded once, then added to x and rounded again
    xb, pb = cb.f32_to_bf16_bits(x), cb.f32_to_bf16_bits(part)
    comm.write(0, xb)
    comm.write(n * 4, pb)
    comm.allreduce(Dtype.BF16, 0, n * 4, n, residual=True)
    want = cb.f32_to_bf16_bits(cb.bf16_bits_to_f32(xb) + cb.bf16_bits_to_f32(pb))
    np.testing.assert_array_equal(comm.read(0, n, np.uint16), want)
    with pytest.raises(BackendError):
        comm.allreduce(Dtype.F32, 0, n * 4, 2 * n, residual=True)     # outside the buffer


def test_device_drawn_shards_are_slices_of_one_model(gpu):
    cfg = cb.LlamaConfig(128, 384, 1, 8, 4, 512, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)
    whole = tp.random_shard_device(gpu, cfg, 0, 1, Dtype.F32, seed=7)
    for size in (2, 4):
        shards = [tp.random_shard_device(gpu, cfg, r, size, Dtype.F32, seed=7) for r in range(size)]
        for key, _ in cfg.param_shapes():
            full = whole[key].numpy()
            parts = [s[key].numpy() for s in shards]
            if key.endswith(tp.ROW_SHARDED):
                np.testing.assert_array_equal(np.concatenate(parts, 0), full)
            elif key.endswith(tp.COL_SHARDED):
                np.testing.assert_array_equal(np.concatenate(parts, 1), full)
            else:
                np.testing.assert_array_equal(parts[0], full)
    g = whole["model.layers.0.mlp.gate_proj.weight"].numpy()
    assert abs(float(g.std()) - 0.02) < 0.001 and abs(float(g.mean())) < 0.001
    assert np.unique(g).size > 0.9 * g.size
    other = tp.random_shard_device(gpu, cfg, 0, 1, Dtype.F32, seed=8)["model.layers.0.mlp.gate_proj.weight"].numpy()
    assert not np.array_equal(other, g)
    np.testing.assert_array_equal(whole["model.norm.weight"].numpy(), np.ones(128, dtype=np.float32))


def test_peer_that_never_arrives_times_out_and_the_context_survives(gpu):
    """Two communicators of one process on one GPU; only rank 0 ever launches.  Its wait on rank 1's flag (which
    nothing sets) gives up after the 200 ms limit: the next synchronising call reports CG_ERR_TIMEOUT, later calls on
    the dead communicator return at once, and the context keeps working."""
    n = 4096
    c0 = tp.TpComm(gpu, 0, 2, 2 * n * 4)
    c1 = tp.TpComm(gpu, 1, 2, 2 * n * 4)
    c0.attach_local([c0, c1])
    c1.attach_local([c0, c1])
    c0.set_timeout_ms(200)
    t0 = time.time()
    c0.allreduce(Dtype.F32, 0, n * 4, n, residual=True)
    with pytest.raises(BackendError) as ei:
        gpu.synchronize()
    assert ei.value.status == Status.TIMEOUT
    assert time.time() - t0 < 5.0
    t0 = time.time()
    for _ in range(3):
        c0.allreduce(Dtype.F32, 0, n * 4, n, residual=True)      # dead communicator: no waiting
    gpu.synchronize()
    assert time.time() - t0 < 0.15
    a = gpu.from_numpy(np.arange(8, dtype=np.float32))
    np.testing.assert_array_equal(gpu.add(a, a).numpy(), 2 * np.arange(8, dtype=np.float32))


def test_two_ranks_on_two_gpus_match_the_unsharded_model():
    if _device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "tp_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1200)
    print(r.stdout[-4000:])                     # the per-case figures ("-s" or a failure shows them)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count(": ok") == 6, r.stdout[-3000:]

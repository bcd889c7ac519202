"""Batch-sharded runner logic on CPU ranks (gloo, world_size 2 and 3): every sequence lands on exactly one rank, the
gather restores the original order, ragged splits work, and a rank that never joins is reported by the timeout
instead of hanging the others."""
import datetime
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from catgrad_b200.runner import gather_rows, generate_sharded, shard_range


class FakeRunner:
    """Stands in for LlamaRunner on CPU: the 'generated ids' are a deterministic function of each prompt alone,
    like greedy decoding of independent sequences."""

    def __init__(self, batch):
        self.batch = batch

    def generate(self, prompts, steps):
        assert prompts.shape[0] == self.batch
        base = prompts.astype(np.uint64).sum(axis=1, keepdims=True) * 2654435761 % 4294967291
        return ((base + np.arange(steps, dtype=np.uint64)[None, :] * 40503) % 128256).astype(np.uint32)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_seq, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    prompts = np.random.default_rng(1).integers(0, 128256, size=(n_seq, 16), dtype=np.uint32)
    ids = generate_sharded(FakeRunner, prompts, 8, dist)
    np.save(os.path.join(out_dir, f"ids_{rank}.npy"), ids)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n_seq", [(2, 256), (2, 7), (3, 10)])
def test_sharded_generation_equals_single_process(tmp_path, world, n_seq):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, n_seq, str(tmp_path)), nprocs=world, join=True)
    prompts = np.random.default_rng(1).integers(0, 128256, size=(n_seq, 16), dtype=np.uint32)
    want = FakeRunner(n_seq).generate(prompts, 8)
    for r in range(world):
        np.testing.assert_array_equal(np.load(tmp_path / f"ids_{r}.npy"), want)


def test_shard_ranges_partition_the_batch():
    for n in (0, 1, 7, 256, 257):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)
    assert gather_rows(np.zeros((3, 2), np.uint32), 3).shape == (3, 2)


def _absent_worker(rank, world, port, out_dir):
    # rank 1 never joins: rank 0's rendezvous must give up with an error, not hang
    if rank == 1:
        return
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
        outcome = "joined"
    except Exception as e:  # noqa: BLE001
        outcome = type(e).__name__
    with open(os.path.join(out_dir, "outcome.txt"), "w") as f:
        f.write(outcome)


def test_missing_rank_is_an_error_not_a_hang(tmp_path):
    mp.spawn(_absent_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / "outcome.txt").read() != "joined"

"""Host side of tensor parallelism on CPU: the shard slicing of `catgrad_b200.tp`, the algebra it relies on (sum of
the ranks' partial o_proj/down_proj products = the unsharded layer, checked on an independent float64 Llama), and
the exchange of communicator handles between gloo ranks."""
import datetime
import os
import socket

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

import catgrad_b200 as cb
from catgrad_b200 import tp
from llama_numpy import forward, rmsnorm, rope


def small_cfg():
    return cb.LlamaConfig(128, 384, 2, 8, 4, 512, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)


def forward_sharded(cfg, shards, ids):
    """The prefill of llama_numpy.forward with every projection computed rank by rank on `shards` and the partial
    products of o_proj / down_proj summed: what the tensor-parallel runner does on the GPUs."""
    size = len(shards)
    w = [{k: v.astype(np.float64) for k, v in s.items()} for s in shards]
    b, s = ids.shape
    nh, nkv, hd = cfg.num_attention_heads // size, cfg.num_key_value_heads // size, cfg.head_dim
    x = w[0]["model.embed_tokens.weight"][ids]
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        h = rmsnorm(x, w[0][p + "input_layernorm.weight"], cfg.rms_norm_eps)
        part = 0.0
        for r in range(size):
            q = (h @ w[r][p + "self_attn.q_proj.weight"].T).reshape(b, s, nh, hd).transpose(0, 2, 1, 3)
            k = (h @ w[r][p + "self_attn.k_proj.weight"].T).reshape(b, s, nkv, hd).transpose(0, 2, 1, 3)
            v = (h @ w[r][p + "self_attn.v_proj.weight"].T).reshape(b, s, nkv, hd).transpose(0, 2, 1, 3)
            q, k = rope(q, 0, cfg.rope_theta), rope(k, 0, cfg.rope_theta)
            kk, vv = np.repeat(k, nh // nkv, 1), np.repeat(v, nh // nkv, 1)
            sc = q @ kk.transpose(0, 1, 3, 2) / np.sqrt(hd)
            sc = np.where(np.arange(s)[None, :] > np.arange(s)[:, None], -np.inf, sc)
            sc = np.exp(sc - sc.max(-1, keepdims=True))
            a = ((sc / sc.sum(-1, keepdims=True)) @ vv).transpose(0, 2, 1, 3).reshape(b, s, nh * hd)
            part = part + a @ w[r][p + "self_attn.o_proj.weight"].T
        x = x + part
        h = rmsnorm(x, w[0][p + "post_attention_layernorm.weight"], cfg.rms_norm_eps)
        part = 0.0
        for r in range(size):
            g = h @ w[r][p + "mlp.gate_proj.weight"].T
            u = h @ w[r][p + "mlp.up_proj.weight"].T
            part = part + ((g / (1 + np.exp(-g))) * u) @ w[r][p + "mlp.down_proj.weight"].T
        x = x + part
    x = rmsnorm(x, w[0]["model.norm.weight"], cfg.rms_norm_eps)
    return x @ w[0]["lm_head.weight"].T


@pytest.mark.parametrize("size", [1, 2, 4])
def test_sharded_layers_sum_to_the_unsharded_model(size):
    cfg = small_cfg()
    w = cb.random_weights(cfg, seed=3)
    ids = np.random.default_rng(4).integers(0, cfg.vocab_size, size=(2, 9))
    shards = [tp.shard_weights(cfg, w, r, size) for r in range(size)]
    want, _ = forward(cfg, w, ids)
    got = forward_sharded(cfg, shards, ids)
    assert np.abs(got - want).max() <= 1e-9 * max(1.0, np.abs(want).max())


def test_shard_shapes_and_coverage():
    cfg = small_cfg()
    w = cb.random_weights(cfg, seed=3)
    size = 4
    shards = [tp.shard_weights(cfg, w, r, size) for r in range(size)]
    hd = cfg.head_dim
    for key, full in w.items():
        parts = [s[key] for s in shards]
        if key.endswith(tp.ROW_SHARDED):
            np.testing.assert_array_equal(np.concatenate(parts, 0), full)
            assert parts[0].flags.c_contiguous
        elif key.endswith(tp.COL_SHARDED):
            np.testing.assert_array_equal(np.concatenate(parts, 1), full)
            assert parts[0].flags.c_contiguous
        else:
            for p in parts:
                assert p is full
    assert shards[1]["model.layers.0.self_attn.q_proj.weight"].shape == (cfg.num_attention_heads // size * hd, 128)
    assert shards[1]["model.layers.0.self_attn.k_proj.weight"].shape == (cfg.num_key_value_heads // size * hd, 128)
    assert shards[1]["model.layers.0.mlp.down_proj.weight"].shape == (128, 384 // size)
    assert tp.comm_bytes(cfg, 10, 2) == 2 * 2560


def test_block_seeded_shards_are_slices_of_one_model():
    cfg = small_cfg()    # 8 heads / 4 kv heads / FFN 384: every sharded axis divides by 8 blocks
    whole = tp.random_shard_bf16(cfg, 0, 1, seed=5)
    for size in (2, 4):
        shards = [tp.random_shard_bf16(cfg, r, size, seed=5) for r in range(size)]
        for key, full in whole.items():
            parts = [s[key] for s in shards]
            if key.endswith(tp.ROW_SHARDED):
                np.testing.assert_array_equal(np.concatenate(parts, 0), full)
            elif key.endswith(tp.COL_SHARDED):
                np.testing.assert_array_equal(np.concatenate(parts, 1), full)
                assert parts[0].flags.c_contiguous
            else:
                np.testing.assert_array_equal(parts[0], full)
    q = cb.bf16_bits_to_f32(whole["model.layers.0.mlp.gate_proj.weight"])
    assert abs(float(q.std()) - 0.02) < 0.002 and abs(float(q.mean())) < 0.002
    assert whole["model.norm.weight"][0] == 0x3F80


def test_indivisible_configs_are_refused():
    cfg = small_cfg()   # 4 kv heads
    with pytest.raises(ValueError):
        tp.check_divisible(cfg, 8)
    with pytest.raises(ValueError):
        tp.check_divisible(cfg, 3)
    with pytest.raises(ValueError):
        tp.check_divisible(cfg, 0)
    with pytest.raises(ValueError):
        tp.shard_slice(10, 0, 4)


class FakeBackend:
    """Records what `tp.connect` asks the library for; the 'IPC handle' of rank r is 64 bytes of r + 1."""

    class _NS:
        def __init__(self, log):
            self.log = log

        def comm_create(self, ctx, rank, size, nbytes, out):
            self.log.append(("create", rank, size, nbytes))
            self.rank = rank
            return 0

        def comm_handle(self, h, buf):
            for i in range(64):
                buf[i] = self.rank + 1
            return 0

        def comm_attach(self, h, blob):
            self.log.append(("attach", bytes(blob)))
            return 0

        def comm_free(self, h):
            return None

    def __init__(self):
        self.log = []
        self._ns = FakeBackend._NS(self.log)
        self._ctx = None

    def _check(self, status):
        assert status == 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _connect_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    be = FakeBackend()
    comm = tp.connect(be, 4096)
    assert (comm.rank, comm.size) == (rank, world)
    attach = [e for e in be.log if e[0] == "attach"]
    assert len(attach) == 1
    with open(os.path.join(out_dir, f"blob_{rank}.bin"), "wb") as f:
        f.write(attach[0][1])
    dist.barrier()
    dist.destroy_process_group()


def test_handles_reach_every_rank_in_rank_order(tmp_path):
    world = 2
    mp.spawn(_connect_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    want = b"".join(bytes([r + 1]) * 64 for r in range(world))
    for r in range(world):
        assert (tmp_path / f"blob_{r}.bin").read_bytes() == want

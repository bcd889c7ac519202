"""One rank of the 2-GPU tensor-parallel parity test (launched by tests/test_gpu_tp.py through torch.distributed.run).

Every rank runs its shard of the same model on its own GPU; rank 0 also runs the unsharded model on its GPU and
compares.  Exit code 0 = all checks passed."""
import datetime
import os
import sys

import numpy as np
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import catgrad_b200 as cb  # noqa: E402
from catgrad_b200 import Dtype, tp  # noqa: E402
import helpers  # noqa: E402

REL_F32 = 1e-4      # f32 logits, relative to the largest logit
ABS_BF16 = 2e-2     # bf16 logits, max-abs


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def run_case(be, rank, size, cfg, weights, dtype, batch, prompt, steps, what, sem=None):
    """sem: a bf16-semantics fixture (tests/helpers.py); then bf16 logits are held to the bar derived from it instead
    of the small-model 2e-2."""
    es = 4 if dtype == Dtype.F32 else 2
    ids = np.random.default_rng(21).integers(0, cfg.vocab_size, size=(batch, prompt), dtype=np.uint32)
    max_tokens = batch * prompt
    comm = tp.connect(be, tp.comm_bytes(cfg, max_tokens, es))
    shard = cb.upload_weights(be, tp.shard_weights(cfg, weights, rank, size), dtype)
    runner = cb.LlamaRunner(be, cfg, shard, dtype, max_batch=batch, max_positions=prompt + steps + 1, comm=comm,
                            max_tokens=max_tokens)
    runner.reset(batch)
    first = runner.forward(ids)
    logits0 = runner.last_logits()
    rest = runner.decode(steps)               # captured graph: the all-reduce replays inside it
    logits1 = runner.last_logits()
    out = np.concatenate([first[:, None], rest], 1)
    # every rank must hold the same ids
    gathered = [None] * size
    dist.all_gather_object(gathered, out.tobytes())
    assert all(g == gathered[0] for g in gathered), f"{what}: ranks disagree on the generated ids"
    if rank == 0:
        full = cb.upload_weights(be, weights, dtype)
        ref = cb.LlamaRunner(be, cfg, full, dtype, max_batch=batch, max_positions=prompt + steps + 1)
        ref.reset(batch)
        rfirst = ref.forward(ids)
        rlogits0 = ref.last_logits()
        if dtype == Dtype.F32:
            e = rel_err(logits0, rlogits0)
            assert e <= REL_F32, f"{what}: prefill logits rel err {e}"
            np.testing.assert_array_equal(first, rfirst)
            rrest = ref.decode(steps)
            np.testing.assert_array_equal(rest, rrest)
            e = rel_err(logits1, ref.last_logits())
            assert e <= REL_F32, f"{what}: decode logits rel err {e}"
        else:
            # the bar for bf16 is the f32 model on the same (bf16-representable) weights; the unsharded bf16 run is
            # held to the same bar and printed for comparison
            full32 = cb.upload_weights(be, weights, Dtype.F32)
            ref32 = cb.LlamaRunner(be, cfg, full32, Dtype.F32, max_batch=batch, max_positions=prompt + steps + 1)
            ref32.reset(batch)
            ref32.forward(ids)
            want0 = ref32.last_logits()
            e_tp, e_plain = float(np.abs(logits0 - want0).max()), float(np.abs(rlogits0 - want0).max())
            m_tp, m_plain = float(np.abs(logits0 - want0).mean()), float(np.abs(rlogits0 - want0).mean())
            print(f"[tp_worker] {what}: prefill max-abs vs f32: sharded {e_tp:.4f}, unsharded {e_plain:.4f}; "
                  f"mean-abs: sharded {m_tp:.4f}, unsharded {m_plain:.4f}", flush=True)
            if sem is None:
                assert e_tp <= ABS_BF16 and e_plain <= ABS_BF16, f"{what}: prefill logits max-abs {e_tp} / {e_plain}"
            else:
                helpers.check_bf16_against_f32(sem, None, logits0, want0, small_bar=ABS_BF16, max_factor=2.0)
                helpers.check_bf16_against_f32(sem, None, rlogits0, want0, small_bar=ABS_BF16, max_factor=2.0)
            # teacher-force the f32 run with the sharded run's ids so both see the same history
            tok = first
            for s in range(steps):
                ref32.forward(tok.reshape(batch, 1))
                tok = rest[:, s]
            e = float(np.abs(logits1 - ref32.last_logits()).max())
            me = float(np.abs(logits1 - ref32.last_logits()).mean())
            print(f"[tp_worker] {what}: decode max-abs vs f32: sharded {e:.4f}; mean-abs {me:.4f}", flush=True)
            if sem is None:
                assert e <= ABS_BF16, f"{what}: decode logits max-abs {e}"
            else:
                helpers.check_bf16_against_f32(sem, None, logits1, ref32.last_logits(), small_bar=ABS_BF16, max_factor=2.0)
        print(f"[tp_worker] {what}: ok", flush=True)
    dist.barrier()
    del runner
    comm.close()


def main():
    rank, size = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=size, timeout=datetime.timedelta(seconds=120))
    be = cb.Backend(int(os.environ.get("LOCAL_RANK", rank)))
    tiny = cb.LlamaConfig(256, 688, 2, 4, 4, 1024, rope_theta=10000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)
    w = cb.random_weights(tiny, seed=0)
    run_case(be, rank, size, tiny, w, Dtype.F32, 1, 24, 6, "tiny f32 batch 1 (GEMV path, one-shot all-reduce)")
    run_case(be, rank, size, tiny, w, Dtype.F32, 20, 12, 4, "tiny f32 batch 20 (GEMM path)")
    # Llama-3 proportions (GQA 2:1, head_dim 128, theta 5e5) at 2 layers / hidden 512; the prefill of 48 x 24 tokens
    # moves 1.1 MiB per all-reduce, which takes the two-shot path
    small = cb.LlamaConfig(512, 1536, 2, 4, 2, 4096, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)
    wb = cb.random_weights(small, seed=1)
    wb = {k: cb.bf16_bits_to_f32(cb.f32_to_bf16_bits(v)).reshape(v.shape) for k, v in wb.items()}
    run_case(be, rank, size, small, wb, Dtype.BF16, 2, 40, 5, "small bf16 batch 2 (GEMV path)")
    run_case(be, rank, size, small, wb, Dtype.BF16, 48, 24, 4, "small bf16 batch 48 (tcgen05 GEMM path, two-shot)")
    run_case(be, rank, size, small, wb, Dtype.F32, 48, 24, 2, "small f32 batch 48 (two-shot)")
    del w, wb
    # the dimensions of the tensor-parallel benchmark configuration (Llama-3-8B: hidden 4096, 32 query / 8 kv heads x 128,
    # FFN 14336, untied 128256-row head) at two of its 32 layers, batch 32 like the benchmark; the bf16 bar at this size
    # comes from the reference semantics' own distance to f32 on two of these very sequences
    # (tests/golden/llama8b2l_tp_bf16_semantics.json: same weights, rows 0 and 1 of this prompt matrix, same steps)
    big = cb.LlamaConfig(4096, 14336, 2, 32, 8, 128256, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False)
    w8 = cb.random_weights(big, seed=3)
    w8 = {k: cb.bf16_bits_to_f32(cb.f32_to_bf16_bits(v)).reshape(v.shape) for k, v in w8.items()}
    run_case(be, rank, size, big, w8, Dtype.BF16, 32, 16, 3, "8B dimensions x 2 layers, bf16 batch 32 (tcgen05 GEMM path)",
             sem=helpers.bf16_semantics("llama8b2l_tp"))
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException as e:   # the launcher keeps only the tail of stderr: say what failed on stdout too
        import traceback
        print(f"[tp_worker] rank {os.environ.get('RANK')} FAILED: {type(e).__name__}: {e}\n{traceback.format_exc()[-1500:]}", flush=True)
        raise

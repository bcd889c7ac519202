"""Benchmark of the hot path: greedy Llama decoding (and prefill) through the C ABI.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload auto|c3|c4|c5|tiny|sweep]

One "step" is one decode step of the whole batch (one new token per sequence).
  Every N: baseline config 4, the configuration the metric is quoted on ("1/2/4/8 B200"): Llama-3.2-1B shape, bf16,
           256 sequences x 128-token prompt, split evenly over the N ranks (one process per GPU, no collective on the
           data path; the generated ids are gathered once at the end).  Total work is fixed: strong scaling.
  N = 1  : additionally times baseline config 3 (batch 1, 512-token prompt: the configuration the 70 %-of-roofline
           target is stated on) and reports it under "c3" with its own roofline; `--workload c3` makes it the line.
`value` is decode tokens/s with everything resident on the device (CUDA-graph replay, or the persistent decode
kernel for a few sequences; ids fed back on the device): the median of `--repeats` timed blocks of exactly
`--steps` steps, each after a fresh prefill and the warm-up steps so that every block sees the same context
range.  `e2e` is the same loop driven like the reference's runner, one host round trip per token: the token
ids are copied host->device, the step runs, the new ids are read back (examples/llama/main.rs:1016-1037).
`ids_match`: the generated ids are checked, not just summed: every timed block must reproduce the first one's ids,
with more than one rank rank 0 re-runs rank 1's shard and compares it with what rank 1 sent (batch sharding), or all
ranks must hold the same ids (tensor parallelism); `ids_sha1` hashes each sequence's ids so that runs at different
N can be compared row by row.
Weights are synthetic (N(0,0.02), seed 0), prompts are uniform random ids (seed 1); the 2.47 GB of weights read
per step exceed the 126 MB L2, so no flush is needed between steps.

`--workload c5` (any N in 1, 2, 4, 8): baseline config 5, the Llama-3-8B shape run tensor-parallel over the N ranks
(q/k/v/gate/up split by rows, o/down by columns, their partial products all-reduced over NVLink by the library's own
peer-memory kernel), batch 32, 1024-token prompt; weights are drawn on the device, shard by shard.

`--impl reference` times the CPU restatement of the reference's ndarray path (oracle/ndarray_ref.cc,
single-threaded like the reference's tensor ops) on a bounded sample of the same workload.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import catgrad_b200 as cb  # noqa: E402

HBM_NOMINAL_GBS = 8000.0
# DRAM bytes per step from ncu captures (constants, not measured in this run).  Batch 1, kernel-per-sub-graph plan:
# (8.44 + 67.18 + 33.62 + 12.66) MB x 16 layers + 525.3 MB lm_head, measured per launch.
TRAFFIC_PER_STEP_B1 = int((8.44e6 + 67.18e6 + 33.62e6 + 12.66e6) * 16 + 525.3e6)
# batch 1, persistent kernel: one captured launch of 4 steps at context ~520 read 9 964 379 904 B and wrote 77 484 544 B
TRAFFIC_PER_STEP_B1_PERSISTENT = (9964379904 + 77484544) // 4
# batch 256 on one GPU: per layer [q;k;v] 12.73 + o_proj 8.67 + down_proj 34.23 MB (ncu, split-K summary), [gate;up]
# 67.11 MB and lm_head 525.3 MB (not captured: their weight bytes), attention 70.1 MB (ncu, context ~135)
TRAFFIC_PER_STEP_C4 = int((12.73e6 + 8.67e6 + 34.23e6 + 67.11e6 + 70.1e6) * 16 + 525.3e6)
L2_BYTES = 126 * 1024 * 1024


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), float(p.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.rows, self.proc = device, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def event_ms(be, a, b):
    out = ctypes.c_float()
    be._check(be._ns.event_elapsed_ms(be._ctx, a, b, ctypes.byref(out)))
    return out.value


def build_model(be, cfg, dtype):
    t0 = time.time()
    w = cb.random_weights(cfg, seed=0)
    params = cb.upload_weights(be, w, dtype)
    be.synchronize()
    return params, w, time.time() - t0


def decode_bytes(cfg, batch, ctx_len):
    """Algorithmic HBM bytes of one decode step: every weight once (the tied head counted once, the embedding
    rows actually gathered are negligible) + the KV cache read + the new KV rows written."""
    n_weights = cfg.num_params()
    kv_per_tok = 2 * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim * 2
    return 2 * n_weights + batch * kv_per_tok * ctx_len + batch * kv_per_tok


def run_decode_workload(be, cfg, params, batch, prompt_len, steps, warmup, dev_index, e2e_steps=None, name="",
                        comm=None, persistent=True, repeats=3, prompts=None):
    """`repeats` times: prefill, W warm-up steps, K timed decode steps (device-resident); then the same loop through
    host round trips.  Returns timings and the ids [batch, steps] of the first timed block."""
    warmup = max(warmup, 3)
    P = prompt_len + warmup + steps + 2 * (3 + (e2e_steps or steps)) + 16
    runner = cb.LlamaRunner(be, cfg, params, cb.Dtype.BF16, max_batch=batch, max_positions=P, comm=comm,
                            max_tokens=batch * prompt_len)
    if not persistent:
        runner.set_persistent(False)
    if prompts is None:
        prompts = np.random.default_rng(1).integers(0, cfg.vocab_size, size=(batch, prompt_len), dtype=np.uint32)
    res = {}
    sampler = ClockSampler(dev_index)
    sampler.start()          # nvidia-smi needs ~0.1 s to come up: start it before the first block
    time.sleep(0.2)
    pre_ms, dec_ms, ids0, same = [], [], None, True
    for rep in range(repeats + 1):                      # block 0 is a dry run (kernel loading, graph capture)
        runner.reset(batch)
        be._ns.event_record(be._ctx, 0)
        runner.forward(prompts, read=False)
        be._ns.event_record(be._ctx, 1)
        runner.decode(warmup)
        l0 = runner.launch_count
        ctx0 = runner.context_len
        be.synchronize()
        be._ns.event_record(be._ctx, 2)
        ids = runner.decode(steps)
        be._ns.event_record(be._ctx, 3)
        be.synchronize()
        if rep == 0:
            continue
        pre_ms.append(event_ms(be, 0, 1))
        dec_ms.append(event_ms(be, 2, 3))
        res["launches"] = runner.launch_count - l0
        res["ctx_mid"] = ctx0 + steps / 2
        if ids0 is None:
            ids0 = ids
        else:
            same = same and bool((ids == ids0).all())
    res["clocks"] = sampler.stop()
    res["prefill_ms"] = float(np.median(pre_ms))
    res["prefill_tok_s"] = batch * prompt_len / (res["prefill_ms"] / 1e3)
    res["ms"] = float(np.median(dec_ms))
    res["ms_all"] = [round(v, 4) for v in dec_ms]
    res["ids"] = ids0
    res["repeat_ids_equal"] = same
    res["persistent"] = runner.persistent_active
    # ---- end to end: one host round trip per token, like the reference runner ----
    k = e2e_steps or steps
    tok = ids[:, -1].copy().reshape(batch, 1)
    for _ in range(3):
        tok = runner.forward(tok).reshape(batch, 1)
    t0 = time.perf_counter()
    for _ in range(k):
        tok = runner.forward(tok).reshape(batch, 1)
    res["e2e_ms"] = (time.perf_counter() - t0) * 1e3
    res["e2e_steps"] = k
    res["batch"] = batch
    del runner
    return res


def ids_digest(ids):
    """sha1 over each sequence's generated ids (first 12 hex digits), and one over all of them."""
    import hashlib
    rows = [hashlib.sha1(np.ascontiguousarray(r, dtype=np.uint32).tobytes()).hexdigest()[:12] for r in ids]
    return rows, hashlib.sha1("".join(rows).encode()).hexdigest()[:16]


def interpreter_path_tok_s(be, cfg, params, prompt_len=64, steps=8):
    """The same model through cg_interp_run on the Llama term, the route catgrad's own `interpreter.run(term)` takes,
    with the KV cache threaded as a value (helpers/cache.rs:13-75), twice: op by op (one kernel per IR edge, the cache
    re-stacked every step) and with the term recognised and executed as the fused plan (the default)."""
    ids = np.random.default_rng(1).integers(0, cfg.vocab_size, size=(1, prompt_len), dtype=np.uint32)
    res = {"prompt_len": prompt_len, "steps": steps}
    for name, planning in (("op_by_op", 0), ("planned", 1)):
        be._ns.interp_set_planning(planning)
        try:
            term = cb.llama_term(be, cfg)
            interp = cb.Interpreter(be, params)
            in_k, in_v = cb.empty_state_cache(be, cfg, 1, cb.Dtype.BF16)
            x = ids
            times, launches = [], []
            for i in range(steps + 2):
                stats0 = be.stats()[3]
                t0 = time.perf_counter()
                r = interp.run(term, [be.ndarray_from_vec_u32(x, x.shape), in_k, in_v, prompt_len + steps + 3])
                last = be.to_numpy(r[0])[:, -1, 0]
                times.append(time.perf_counter() - t0)
                launches.append(be.stats()[3] - stats0)
                in_k, in_v = r[1], r[2]
                x = last.reshape(1, 1).astype(np.uint32)
            dec = times[2:]                              # skip the prefill call and the first decode call
            res[name] = {"decode_tok_s": len(dec) / sum(dec), "ms_per_step": 1e3 * sum(dec) / len(dec),
                         "backend_calls_per_step": int(launches[-1]), "plan_state": term.plan_state}
            del in_k, in_v, r, term, interp
        finally:
            be._ns.interp_set_planning(1)
    return res


def cpu_baseline_sample(cfg, weights_f32, prompt_len=8, steps=2, batch=1):
    """The oracle (CPU restatement of the reference's ndarray path, 1 thread) on a bounded sample of the workload:
    a short prefill, then `steps` decode steps through the op-by-op interpreter, f32 (the ndarray backend has no
    bf16).  Returns decode tokens/s."""
    so = os.path.join(ROOT, "oracle", "_build", "libndarray_ref.so")
    if not os.path.exists(so):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle")], check=True, capture_output=True)
    oracle = cb.Backend(_cdll=ctypes.CDLL(so), _prefix="ref_")
    params = cb.upload_weights(oracle, weights_f32, cb.Dtype.F32)
    term = cb.llama_term(oracle, cfg)
    interp = cb.Interpreter(oracle, params)
    ids = np.random.default_rng(1).integers(0, cfg.vocab_size, size=(batch, prompt_len), dtype=np.uint32)
    in_k, in_v = cb.empty_state_cache(oracle, cfg, batch, cb.Dtype.F32)
    x = ids
    times = []
    for i in range(steps + 1):
        t0 = time.perf_counter()
        r = interp.run(term, [oracle.ndarray_from_vec_u32(x, x.shape), in_k, in_v, prompt_len + steps + 1])
        last = oracle.to_numpy(r[0])[:, -1, 0]
        times.append(time.perf_counter() - t0)
        in_k, in_v = r[1], r[2]
        x = last.reshape(batch, 1).astype(np.uint32)
    dec = times[1:]
    return {"value": batch * len(dec) / sum(dec), "unit": "tok/s", "cores": 1, "kind": "port",
            "sample": f"oracle/ndarray_ref (1 thread, f32): {batch} sequence(s), prefill of {prompt_len} tokens "
                      f"({times[0]:.1f} s) then {steps} decode steps of the same model ({sum(dec):.1f} s)",
            "prefill_tok_s": batch * prompt_len / times[0]}


def timed_op(be, fn, iters=10, flush_bytes=256 << 20):
    """Median CUDA-event time of fn() over `iters` runs, L2 flushed (256 MiB written) before each."""
    for _ in range(3):
        fn()
    ms = []
    for _ in range(iters):
        be._ns.flush_l2(be._ctx, flush_bytes)
        be._ns.event_record(be._ctx, 10)
        out = fn()
        be._ns.event_record(be._ctx, 11)
        be.synchronize()
        ms.append(event_ms(be, 10, 11))
        del out
    return float(np.median(ms))


def run_op_sweep(be):
    """Baseline config 2: op-level sweep on random tensors (seed 2), f32 and bf16, through the Backend entry
    points.  Bytes are the algorithmic ones: inputs read once + output written once; a broadcast operand counts
    its source only."""
    rng = np.random.default_rng(2)
    hbm, tflops_peak, _ = measured_peaks()
    rows = []
    x_np = rng.uniform(-4, 4, (4096, 8192)).astype(np.float32)
    v_np = rng.uniform(-4, 4, (8192,)).astype(np.float32)
    r_np = rng.uniform(-4, 4, (8192, 4096)).astype(np.float32)
    table_np = rng.standard_normal((32000, 2048)).astype(np.float32)
    idx_np = rng.integers(0, 32000, 4096, dtype=np.uint32)
    am_np = rng.standard_normal((64, 32000)).astype(np.float32)
    a_np = rng.standard_normal((16, 1024, 1024)).astype(np.float32)
    b_np = rng.standard_normal((16, 1024, 1024)).astype(np.float32)
    for dt, es, name in ((cb.Dtype.F32, 4, "f32"), (cb.Dtype.BF16, 2, "bf16")):
        x, v = be.from_numpy(x_np, dt), be.from_numpy(v_np, dt)
        vb = be.broadcast(v, x.shape)                      # explicit Broadcast: the trait never broadcasts implicitly
        n = x_np.size

        def add_row(op, ms, nbytes, flops=None):
            row = {"op": op, "dtype": name, "ms": ms, "GB/s": nbytes / ms / 1e6, "frac_hbm_measured": nbytes / ms / 1e6 / hbm}
            if flops:
                row["TFLOP/s"] = flops / ms / 1e9
                if name == "bf16":
                    row["frac_bf16_tensor_measured"] = flops / ms / 1e9 / tflops_peak
            rows.append(row)

        add_row("exp [4096,8192]", timed_op(be, lambda: be.exp(x)), 2 * n * es)
        for op in ("add", "mul", "div"):
            add_row(f"{op} [4096,8192] x row vector", timed_op(be, lambda: getattr(be, op)(x, vb)), 2 * n * es + 8192 * es)
        r = be.from_numpy(r_np, dt)
        add_row("sum [8192,4096]", timed_op(be, lambda: be.sum(r)), (r_np.size + 8192) * es)
        add_row("max [8192,4096]", timed_op(be, lambda: be.max(r)), (r_np.size + 8192) * es)

        def softmax_graph():
            xf = be.cast(r, cb.Dtype.F32)
            m = be.max(xf)
            e = be.exp(be.sub(xf, be.broadcast(m, xf.shape)))
            s = be.sum(e)
            return be.cast(be.div(e, be.broadcast(s, xf.shape)), dt)
        add_row("softmax [8192,4096] (nn::softmax op graph)", timed_op(be, softmax_graph), 2 * r_np.size * es)
        add_row("softmax [8192,4096] (fused kernel, cg_softmax)", timed_op(be, lambda: be.softmax(r)), 2 * r_np.size * es)
        a, b = be.from_numpy(a_np, dt), be.from_numpy(b_np, dt)
        add_row("matmul [16,1024,1024]x[16,1024,1024]", timed_op(be, lambda: be.matmul(a, b)), 3 * a_np.size * es,
                flops=2 * 16 * 1024 ** 3)
        bt = be.transpose(be.from_numpy(np.ascontiguousarray(b_np.transpose(0, 2, 1)), dt), 1, 2)
        add_row("matmul [16,1024,1024]x[16,1024,1024], right operand stored K-contiguous",
                timed_op(be, lambda: be.matmul(a, bt)), 3 * a_np.size * es, flops=2 * 16 * 1024 ** 3)
        if name == "bf16":
            # a compute-bound product in the prefill's layout (x @ W^T, both K-contiguous): 4096 output tiles
            big_x = be.from_numpy(rng.standard_normal((8192, 4096)).astype(np.float32), dt)
            big_w = be.transpose(be.from_numpy(rng.standard_normal((8192, 4096)).astype(np.float32), dt), 0, 1)
            add_row("matmul [8192,4096]x[4096,8192], right operand stored K-contiguous",
                    timed_op(be, lambda: be.matmul(big_x, big_w)), 3 * 8192 * 4096 * es + 8192 * 8192 * es - 8192 * 4096 * es,
                    flops=2 * 8192 * 8192 * 4096)
            del big_x, big_w
        table, idx = be.from_numpy(table_np, dt), be.from_numpy(idx_np)
        add_row("index 4096 rows of [32000,2048]", timed_op(be, lambda: be.index(table, 0, idx)), 2 * 4096 * 2048 * es + 16384)
        am = be.from_numpy(am_np, dt)
        add_row("argmax [64,32000]", timed_op(be, lambda: be.argmax(am)), am_np.size * es)
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeats", type=int, default=3, help="timed blocks of --steps steps; the median is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto", "c3", "c4", "c5", "tiny", "sweep"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="profiling aid: override the number of sequences (c3/c4)")
    ap.add_argument("--prompt", type=int, default=0, help="profiling aid: override the prompt length (c3/c4)")
    ap.add_argument("--no-persistent", action="store_true",
                    help="small batches: take the graph of per-sub-graph kernels instead of the persistent decode kernel")
    ap.add_argument("--skip-c4", action="store_true", help="with --workload c3: do not time config 4 as well")
    ap.add_argument("--skip-c3", action="store_true", help="N=1 only: do not time config 3 (batch 1) as well")
    ap.add_argument("--no-interpreter-path", action="store_true", help="N=1 only: skip the op-by-op interpreter timing")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    args.repeats = max(args.repeats, 1)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = cb.TINY if args.workload == "tiny" else (cb.LLAMA_8B if args.workload == "c5" else cb.LLAMA_1B)
    model_name = {"tiny": "tiny-llama", "c5": "Llama-3-8B shape"}.get(args.workload, "Llama-3.2-1B shape")

    if args.workload == "sweep":
        # the op-level sweep on random tensors; not the headline metric, printed as its own JSON line
        if rank == 0:
            be = cb.Backend(local_rank)
            hbm, tfl, src = measured_peaks()
            print(json.dumps({"metric": "op sweep", "unit": "GB/s", "data": "synthetic", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tfl, "source": src},
                              "timing": "median of 10 CUDA-event timings, 256 MiB written between runs to evict L2",
                              "ops": run_op_sweep(be)}))
        return
    if args.impl == "reference":
        if rank != 0:
            return
        # The reference's tensor ops are single-threaded and its runner is batch 1: the bounded sample is ONE sequence of
        # the workload (sequences are independent), a short prompt and two decode steps; tokens/s of that sequence.
        w = cb.random_weights(cfg, seed=0)
        nsteps = max(1, min(args.steps, 2))
        base = cpu_baseline_sample(cfg, w, prompt_len=8, steps=nsteps, batch=1)
        line = {"impl": "reference", "metric": "decode tokens/s", "value": base["value"], "unit": "tok/s",
                "n_gpus": args.gpus, "steps": nsteps, "warmup": 0,
                "ms_per_step": 1e3 / base["value"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": f"{model_name}: ONE sequence of the workload (the reference runner is batch 1 and single-threaded), "
                                       f"8-token prompt then {nsteps} greedy decode steps on the host CPU, f32 (ndarray-path restatement)",
                           "like_for_like_with": "the `c3` block of the GPU arm's line (one sequence); the GPU arm's headline runs 256 "
                                                 "sequences at once, so a ratio against it compares 256 sequences with one"},
                "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    be = cb.Backend(local_rank)
    hbm_peak, _, peak_src = measured_peaks()
    single = world == 1
    workload = args.workload if args.workload != "auto" else "c4"
    tensor_parallel = workload == "c5"
    comm = None
    if tensor_parallel:
        from catgrad_b200 import tp
        batch_total, prompt_len = 32, 1024
        batch = batch_total                       # every rank sees the whole batch
        t0 = time.time()
        params, w = tp.random_shard_device(be, cfg, rank, world, cb.Dtype.BF16, seed=0), None
        be.synchronize()
        load_s = time.time() - t0
        nbytes = tp.comm_bytes(cfg, batch_total * prompt_len, 2)
        if dist is not None:
            comm = tp.connect(be, nbytes)
        else:
            comm = tp.TpComm(be, 0, 1, nbytes)
    else:
        params, w, load_s = build_model(be, cfg, cb.Dtype.BF16)
        if workload in ("c3", "tiny"):
            batch_total, prompt_len = 1, (512 if workload == "c3" else 64)
        else:
            batch_total, prompt_len = 256, 128
        if args.batch:
            batch_total = args.batch
        if args.prompt:
            prompt_len = args.prompt
        assert batch_total % world == 0
        batch = batch_total // world

    # every rank draws the whole batch of prompts and takes its contiguous share (catgrad_b200.runner.shard_range)
    from catgrad_b200 import runner as sharding
    all_prompts = np.random.default_rng(1).integers(0, cfg.vocab_size, size=(batch_total, prompt_len), dtype=np.uint32)
    lo, hi = (0, batch_total) if tensor_parallel else sharding.shard_range(batch_total, world, rank)
    if dist is not None:
        dist.barrier()
    r = run_decode_workload(be, cfg, params, batch, prompt_len, args.steps, args.warmup, local_rank, comm=comm,
                            persistent=not args.no_persistent, repeats=args.repeats, prompts=all_prompts[lo:hi])
    ms, e2e_ms, pre_ms = r["ms"], r["e2e_ms"], r["prefill_ms"]
    ids_match = r["repeat_ids_equal"]
    all_ids = r["ids"]
    if dist is not None:
        import torch
        t = torch.tensor([ms, e2e_ms, pre_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)      # max over ranks
        ms, e2e_ms, pre_ms = [float(v) for v in t.tolist()]
        if tensor_parallel:
            # every rank ran the whole batch: all must hold the same ids
            pieces = [None] * world
            dist.all_gather_object(pieces, r["ids"].tobytes())
            ids_match = ids_match and all(p == pieces[0] for p in pieces)
        else:
            # the one collective of this workload: the final gather of the generated ids [256, steps]
            all_ids = sharding.gather_rows(r["ids"], batch_total, dist, device="cuda")
            flags = [None] * world
            dist.all_gather_object(flags, bool(r["repeat_ids_equal"]))
            ids_match = all(flags)
            if rank == 0:
                # rank 0 re-runs rank 1's shard (same batch size, hence the same kernels) and compares with what rank 1 sent
                lo1, hi1 = sharding.shard_range(batch_total, world, 1)
                chk = cb.LlamaRunner(be, cfg, params, cb.Dtype.BF16, max_batch=hi1 - lo1, max_positions=prompt_len + args.warmup + args.steps + 8)
                if args.no_persistent:
                    chk.set_persistent(False)
                chk.reset(hi1 - lo1)
                chk.forward(all_prompts[lo1:hi1], read=False)
                chk.decode(args.warmup)
                ids_match = ids_match and bool((chk.decode(args.steps) == all_ids[lo1:hi1]).all())
                del chk
        dist.barrier()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    tok_per_step = batch_total
    value = tok_per_step * args.steps / (ms / 1e3)
    e2e_value = tok_per_step * r["e2e_steps"] / (e2e_ms / 1e3)
    if tensor_parallel:
        # per GPU: its share of the layer weights + the replicated embedding row gather (negligible) and lm_head,
        # its share of the KV cache (heads are split)
        layer_params = cfg.num_params() - 2 * cfg.vocab_size * cfg.hidden_size
        kv_per_tok = 2 * cfg.num_hidden_layers * cfg.num_key_value_heads * cfg.head_dim * 2 // world
        bytes_step = 2 * (layer_params // world + cfg.vocab_size * cfg.hidden_size) + batch * kv_per_tok * (r["ctx_mid"] + 1)
    else:
        bytes_step = decode_bytes(cfg, batch, r["ctx_mid"])
    achieved = bytes_step / (ms / args.steps / 1e3) / 1e9
    rows_sha, all_sha = ids_digest(all_ids)
    if tensor_parallel:
        kernel = "one decode step of one rank: tcgen05 GEMMs over its weight shard, attention, 64 all-reduces"
    elif r["persistent"]:
        kernel = "llama_decode_persistent_kernel: one launch runs up to 64 decode steps (weights streamed through shared memory)"
    elif batch <= 16:
        kernel = "one decode step = 65 gemv_fused_kernel launches (79 % of the device time) + attention + greedy pick"
    else:
        kernel = "one decode step = 64 gemm_tcgen05 launches (62 % of the device time) + attention + norms + greedy pick"
    traffic = ((TRAFFIC_PER_STEP_B1_PERSISTENT if r["persistent"] else TRAFFIC_PER_STEP_B1)
               if (batch_total == 1 and workload == "c3" and not args.prompt) else
               TRAFFIC_PER_STEP_C4 if (workload == "c4" and batch == 256 and not args.prompt) else None)
    line = {
        "metric": "decode tokens/s", "value": value, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong" if workload in ("c4", "c5") else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{model_name} bf16, {batch_total} sequence(s) x {prompt_len}-token prompt, greedy decode, "
                               f"context {int(r['ctx_mid'] - args.steps / 2)}..{int(r['ctx_mid'] + args.steps / 2)}",
                   "global_batch": batch_total, "prompt_len": prompt_len,
                   "parallelism": f"tensor-parallel x{world}" if tensor_parallel else f"batch-sharded x{world}",
                   "l2": "inputs larger than L2 (weights read per step exceed 126 MB many times over)"},
        "timing": {"blocks": args.repeats, "ms_per_step_each_block_rank0": [v / args.steps for v in r["ms_all"]],
                   "how": "median over the blocks, each exactly `steps` steps after a fresh prefill and the warm-up steps; CUDA events "
                          "on the launching stream, max over ranks"},
        "per_sequence_tok_s": value / batch_total,
        "ids_match": bool(ids_match), "ids_sha1": all_sha, "ids_sha1_per_sequence": rows_sha,
        "prefill": {"tok_s": batch_total * prompt_len / (pre_ms / 1e3), "ms": pre_ms,
                    "note": "lm_head on the last position of each sequence only"},
        "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": 4 * batch * (world if tensor_parallel else 1),
                "d2h_bytes_per_step": 4 * batch * (world if tensor_parallel else 1),
                "steps": r["e2e_steps"], "how": "cg_llama_forward per token with host id buffers (copy in, step, copy out)"},
        "gpu_launches": r["launches"],
        "clocks": r["clocks"],
        "roofline": {"bound": "hbm", "kernel": kernel,
                     "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "peak_source": peak_src, "frac_of_8TBs_nominal": achieved / HBM_NOMINAL_GBS,
                     "bytes_per_step": bytes_step,
                     "how": "algorithmic bytes of a step on one GPU (every weight it holds once + KV cache read + new KV "
                            "rows) / CUDA-event time of a step on the launching stream",
                     "traffic": traffic,
                     "traffic_how": "constant from ncu captures of the launches of one step (dram__bytes_read.sum + "
                                    "dram__bytes_write.sum), part of it assumed equal to the weight bytes; not measured in this run"},
        "load_s": load_s,
    }
    if single and workload == "c4" and args.workload == "auto" and not args.skip_c3:
        # one sequence, 512-token prompt: the configuration the 70 %-of-HBM-roofline target is stated on
        c3_steps = min(max(args.steps, 32), 128)
        r3 = run_decode_workload(be, cfg, params, 1, 512, c3_steps, args.warmup, local_rank, persistent=not args.no_persistent,
                                 repeats=args.repeats)
        b3 = decode_bytes(cfg, 1, r3["ctx_mid"])
        a3 = b3 / (r3["ms"] / c3_steps / 1e3) / 1e9
        line["c3"] = {"workload": "1 sequence x 512-token prompt on one GPU", "decode_tok_s": c3_steps / (r3["ms"] / 1e3),
                      "ms_per_step": r3["ms"] / c3_steps, "ms_per_step_each_block": [v / c3_steps for v in r3["ms_all"]],
                      "prefill_tok_s": r3["prefill_tok_s"], "prefill_ms": r3["prefill_ms"],
                      "e2e_tok_s": r3["e2e_steps"] / (r3["e2e_ms"] / 1e3), "gpu_launches": r3["launches"],
                      "ids_match": bool(r3["repeat_ids_equal"]), "ids_sha1": ids_digest(r3["ids"])[1],
                      "roofline": {"bound": "hbm",
                                   "kernel": "llama_decode_persistent_kernel (one launch runs up to 64 steps)" if r3["persistent"]
                                   else "65 gemv_fused_kernel launches per step (79 % of the device time)",
                                   "achieved": a3, "peak": hbm_peak,
                                   "unit": "GB/s", "frac": a3 / hbm_peak, "peak_source": peak_src,
                                   "frac_of_8TBs_nominal": a3 / HBM_NOMINAL_GBS, "bytes_per_step": b3,
                                   "traffic": TRAFFIC_PER_STEP_B1_PERSISTENT if r3["persistent"] else TRAFFIC_PER_STEP_B1,
                                   "traffic_how": "constant from one ncu capture of this kernel (dram__bytes_read.sum + "
                                                  "dram__bytes_write.sum per step); not measured in this run"}}
        if not args.no_interpreter_path:
            line["c3"]["interpreter_path"] = interpreter_path_tok_s(be, cfg, params)
        # the same two figures in the reference benchmark mode's own table (stderr: stdout carries the one JSON line)
        for row in cb.bench_table("llama-3.2-1b shape (synthetic weights)", cfg.num_params() * 2 / 2 ** 30, cfg.num_params() / 1e6,
                                  "b200", 512, r3["prefill_ms"] / 1e3, c3_steps, r3["ms"] / 1e3):
            print(row, file=sys.stderr)
    if tensor_parallel:
        del comm
    if single and workload == "c3" and not args.skip_c4:
        # the batch-sharded workload on one GPU: the N=1 point of the scaling runs
        c4_steps = min(args.steps, 64)
        r4 = run_decode_workload(be, cfg, params, 256, 128, c4_steps, args.warmup, local_rank, e2e_steps=8, repeats=args.repeats)
        line["c4"] = {"decode_tok_s": 256 * c4_steps / (r4["ms"] / 1e3), "ms_per_step": r4["ms"] / c4_steps,
                      "prefill_tok_s": r4["prefill_tok_s"], "e2e_tok_s": 256 * r4["e2e_steps"] / (r4["e2e_ms"] / 1e3),
                      "workload": "256 sequences x 128-token prompt on one GPU"}
    if single and workload == "c3" and not args.no_interpreter_path:
        line["interpreter_path"] = interpreter_path_tok_s(be, cfg, params)
    if single and not args.no_cpu_baseline and not tensor_parallel:
        del params
        wf = {k: cb.bf16_bits_to_f32(cb.f32_to_bf16_bits(v)).reshape(v.shape) for k, v in w.items()}
        line["cpu_baseline"] = cpu_baseline_sample(cfg, wf, prompt_len=8, steps=2, batch=1)
        line["cpu_baseline"]["host"] = {"nproc": os.cpu_count()}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

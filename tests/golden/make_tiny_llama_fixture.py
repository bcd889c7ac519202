"""Writes tests/golden/tiny_llama_c1.json: greedy ids and a slice of the prefill logits of baseline config 1
(tiny Llama, f32, weights N(0,0.02) from seed 0 with unit norm gains, 64 prompt ids from seed 1, 33 generated
tokens = 1 from the prefill + 32 decode steps), computed by the CPU oracle (oracle/ndarray_ref.cc) through the
interpreter.  The reference itself cannot be run (no Rust toolchain), so this fixture pins the oracle's output
against regressions; its agreement with a textbook float64 Llama is checked in tests/test_host_cpu.py."""
import ctypes
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import catgrad_b200 as cb  # noqa: E402

be = cb.Backend(_cdll=ctypes.CDLL(os.path.join(ROOT, "oracle", "_build", "libndarray_ref.so")), _prefix="ref_")
cfg = cb.TINY
w = cb.random_weights(cfg, 0)
ids = np.random.default_rng(1).integers(0, cfg.vocab_size, size=(1, 64), dtype=np.uint32)
term = cb.llama_term(be, cfg, tap_logits=True)
out, logits = cb.generate_with_interpreter(be, term, cb.upload_weights(be, w, cb.Dtype.F32), cfg, ids, 33, cb.Dtype.F32,
                                           97, tap=True)
fx = {"weight_seed": 0, "prompt_seed": 1, "prompt_head": ids[0, :8].tolist(), "ids": out[0].tolist(),
      "prefill_logits_head": [float(v) for v in logits[0][0, -1, :16]]}
with open(os.path.join(ROOT, "tests", "golden", "tiny_llama_c1.json"), "w") as f:
    json.dump(fx, f, indent=1)
print(fx["ids"])

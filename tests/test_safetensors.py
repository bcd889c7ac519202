"""safetensors loader on the CPU oracle backend: round trip through a file, dtype conversion rules, sharded
checkpoints, error cases; a loaded tiny Llama generates the ids of the in-memory one."""
import json
import os
import struct

import numpy as np
import pytest

import catgrad_b200 as cb
from catgrad_b200 import Dtype, safetensors as st


def test_round_trip_f32_and_bf16(tmp_path, oracle):
    rng = np.random.default_rng(0)
    w = {"a.weight": rng.standard_normal((3, 5)).astype(np.float32), "b.c.bias": rng.standard_normal(7).astype(np.float32)}
    st.save_file(tmp_path / "m.safetensors", w)
    p, n = st.load_parameters(oracle, str(tmp_path / "m.safetensors"), Dtype.F32)
    assert n == 22 and sorted(p.keys()) == sorted(w)
    for k in w:
        np.testing.assert_array_equal(oracle.to_numpy(p[k]), w[k])
    st.save_file(tmp_path / "h.safetensors", w, bf16=True)
    p16, _ = st.load_parameters(oracle, str(tmp_path / "h.safetensors"), Dtype.F32)     # BF16 file -> f32 model: exact widening
    for k in w:
        np.testing.assert_array_equal(oracle.to_numpy(p16[k]), cb.bf16_bits_to_f32(cb.f32_to_bf16_bits(w[k])).reshape(w[k].shape))
    pb, _ = st.load_parameters(oracle, str(tmp_path / "m.safetensors"), Dtype.BF16)     # F32 file -> bf16 model: rounds
    assert pb["a.weight"].dtype == Dtype.BF16


def test_sharded_checkpoint_and_skipped_i64(tmp_path, oracle):
    a = {"x": np.ones((2, 2), dtype=np.float32)}
    b = {"y": np.full((4,), 2.0, dtype=np.float32)}
    st.save_file(tmp_path / "1.safetensors", a)
    st.save_file(tmp_path / "2.safetensors", b)
    # a file with an I64 tensor (skipped, utils/mod.rs:341-344) next to an F32 one
    hdr = {"steps": {"dtype": "I64", "shape": [1], "data_offsets": [0, 8]},
           "z": {"dtype": "F32", "shape": [2], "data_offsets": [8, 16]}}
    h = json.dumps(hdr).encode()
    with open(tmp_path / "3.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(h)) + h + struct.pack("<q", 7) + np.array([1.5, 2.5], dtype="<f4").tobytes())
    p, n = st.load_parameters(oracle, [str(tmp_path / f"{i}.safetensors") for i in (1, 2, 3)], Dtype.F32)
    assert sorted(p.keys()) == ["x", "y", "z"] and n == 4 + 4 + 2
    np.testing.assert_array_equal(oracle.to_numpy(p["z"]), [1.5, 2.5])


def test_malformed_files_are_refused(tmp_path, oracle):
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes(b"\\x01\\x02")
    with pytest.raises(st.SafetensorsError):
        st.load_parameters(oracle, str(bad), Dtype.F32)
    bad.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(st.SafetensorsError):
        st.load_parameters(oracle, str(bad), Dtype.F32)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}).encode()
    bad.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\\0" * 8)
    with pytest.raises(st.SafetensorsError):
        st.load_parameters(oracle, str(bad), Dtype.F32)
    hdr = json.dumps({"t": {"dtype": "F64", "shape": [1], "data_offsets": [0, 8]}}).encode()
    bad.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\\0" * 8)
    with pytest.raises(st.SafetensorsError):
        st.load_parameters(oracle, str(bad), Dtype.F32)
    with pytest.raises(st.SafetensorsError):
        st.load_parameters(oracle, str(bad), Dtype.U32)


def test_loaded_tiny_llama_generates_the_same_ids(tmp_path, oracle):
    cfg = cb.TINY
    w = cb.random_weights(cfg, seed=0)
    st.save_file(tmp_path / "tiny.safetensors", w)
    loaded, n = st.load_parameters(oracle, str(tmp_path / "tiny.safetensors"), Dtype.F32)
    assert n == cfg.num_params()
    ids = np.random.default_rng(1).integers(0, cfg.vocab_size, size=(1, 8), dtype=np.uint32)
    term = cb.llama_term(oracle, cfg)
    a = cb.generate_with_interpreter(oracle, term, loaded, cfg, ids, 3, Dtype.F32, 16)
    b = cb.generate_with_interpreter(oracle, term, cb.upload_weights(oracle, w, Dtype.F32), cfg, ids, 3, Dtype.F32, 16)
    np.testing.assert_array_equal(a[0], b[0])


def test_config_json_and_checkpoint_directory(tmp_path, oracle):
    """config.json -> LlamaConfig (llama.rs:9-27 field for field, llama3 rope scaling kept, unimplemented features
    refused) and a Hugging Face style directory -> (config, parameters) that generate like the in-memory model."""
    hf = {"architectures": ["LlamaForCausalLM"], "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
          "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 256, "rope_theta": 500000.0, "rms_norm_eps": 1e-5,
          "tie_word_embeddings": True, "head_dim": 16, "torch_dtype": "bfloat16",
          "rope_scaling": {"factor": 32.0, "high_freq_factor": 4.0, "low_freq_factor": 1.0,
                           "original_max_position_embeddings": 8192, "rope_type": "llama3"}}
    cfg = cb.LlamaConfig.from_hf_config(hf)
    assert (cfg.hidden_size, cfg.intermediate_size, cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads,
            cfg.vocab_size, cfg.tie_word_embeddings) == (64, 128, 2, 4, 2, 256, True)
    assert cfg.rope_theta == 500000.0 and cfg.rope_scaling["rope_type"] == "llama3" and cfg.rope_scaling["factor"] == 32.0
    assert cfg.to_struct().rope_scaling_type == 1
    for bad in ({"no_rope_layer_interval": 4}, {"partial_rotary_factor": 0.5}, {"quantization_config": {"format": "x"}},
                {"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, {"head_dim": 32}):
        with pytest.raises(ValueError):
            cb.LlamaConfig.from_hf_config({**hf, **bad})
    assert cb.LlamaConfig.from_hf_config({k: v for k, v in hf.items() if k != "num_key_value_heads"}).num_key_value_heads == 4

    w = cb.random_weights(cfg, seed=2)
    keys = sorted(w)
    (tmp_path / "config.json").write_text(json.dumps(hf))
    st.save_file(tmp_path / "model-00001-of-00002.safetensors", {k: w[k] for k in keys[:5]})
    st.save_file(tmp_path / "model-00002-of-00002.safetensors", {k: w[k] for k in keys[5:]})
    cfg2, params, n = st.load_model(oracle, str(tmp_path), Dtype.F32)
    assert cfg2 == cfg and n == cfg.num_params()
    ids = np.random.default_rng(3).integers(0, cfg.vocab_size, size=(1, 6), dtype=np.uint32)
    term = cb.llama_term(oracle, cfg)
    a = cb.generate_with_interpreter(oracle, term, params, cfg, ids, 3, Dtype.F32, 12)
    b = cb.generate_with_interpreter(oracle, term, cb.upload_weights(oracle, w, Dtype.F32), cfg, ids, 3, Dtype.F32, 12)
    np.testing.assert_array_equal(a[0], b[0])
    # a directory whose files lack a tensor of the configured model is refused
    os.remove(tmp_path / "model-00002-of-00002.safetensors")
    with pytest.raises(st.SafetensorsError):
        st.load_model(oracle, str(tmp_path), Dtype.F32)

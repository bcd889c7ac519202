"""safetensors files -> Parameters on a backend (the loader of catgrad-llm/src/utils/mod.rs:321-449 for dense
models).

Behaviour kept from the reference: every file of a (possibly sharded) checkpoint is read; F32 and BF16 tensors are
converted to the model dtype the caller asks for (f32, f16 or bf16), F8_E4M3 tensors are kept as fp8, I64 tensors are
skipped, any other dtype is an error; keys are the safetensors names split at '.', which for Llama are already the
names the term loads (`model.layers.N.self_attn.q_proj.weight`, ...), so no key mapping is needed.  Packed
mixture-of-experts tensors (utils/mod.rs:347-395) are out of scope like the MoE models themselves.

The format (8-byte little-endian header length, JSON header with dtype/shape/data_offsets per tensor, raw
little-endian data) is parsed here directly; files are memory-mapped, so a tensor is converted and uploaded without
a second host copy of the file.
"""
import json
import mmap
import struct

import numpy as np

from .backend import Dtype, bf16_bits_to_f32, f32_to_bf16_bits
from .ir import Parameters

_SIZES = {"F32": 4, "BF16": 2, "F16": 2, "F8_E4M3": 1, "I64": 8, "U32": 4}


class SafetensorsError(ValueError):
    pass


def read_header(buf):
    """(header dict, offset of the data section) of a safetensors byte buffer."""
    if len(buf) < 8:
        raise SafetensorsError("file shorter than its length prefix")
    (n,) = struct.unpack("<Q", buf[:8])
    if n > len(buf) - 8:
        raise SafetensorsError("header length exceeds the file")
    try:
        header = json.loads(bytes(buf[8:8 + n]).decode("utf-8"))
    except (UnicodeDecodeError, json.JSONDecodeError) as e:
        raise SafetensorsError(f"bad header: {e}")
    return header, 8 + n


def iter_tensors(path):
    """Yields (name, dtype string, shape, raw bytes view) for every tensor of one file, in header order."""
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    header, base = read_header(mm)
    for name, info in header.items():
        if name == "__metadata__":
            continue
        dt, shape = info["dtype"], [int(d) for d in info["shape"]]
        lo, hi = info["data_offsets"]
        n = int(np.prod(shape)) if shape else 1
        if dt not in _SIZES:
            raise SafetensorsError(f"{name}: unsupported dtype {dt}")
        if hi - lo != n * _SIZES[dt] or base + hi > len(mm):
            raise SafetensorsError(f"{name}: data_offsets do not match dtype and shape")
        yield name, dt, shape, memoryview(mm)[base + lo:base + hi]


def load_parameters(backend, paths, dtype):
    """Parameters holding every tensor of the files `paths` in `dtype` (Dtype.F32, F16 or BF16), plus the element
    count (utils/mod.rs:451-470 `load_model_weights` returns the same pair)."""
    dtype = Dtype(dtype)
    if dtype not in (Dtype.F32, Dtype.F16, Dtype.BF16):
        raise SafetensorsError(f"unsupported model dtype {dtype.name}")
    params = Parameters(backend)
    total = 0
    for path in ([paths] if isinstance(paths, (str, bytes)) else list(paths)):
        for name, dt, shape, raw in iter_tensors(path):
            if dt == "I64":
                continue
            if dt == "F8_E4M3":
                params[name] = backend.ndarray_from_vec_fp8(np.frombuffer(raw, dtype=np.uint8), shape)
            elif dt == "BF16":
                bits = np.frombuffer(raw, dtype="<u2")
                if dtype == Dtype.BF16:
                    params[name] = backend.ndarray_from_vec_bf16(bits, shape)
                else:
                    params[name] = backend.from_numpy(bf16_bits_to_f32(bits).reshape(shape).astype(
                        np.float16 if dtype == Dtype.F16 else np.float32), dtype)
            elif dt == "F32":
                arr = np.frombuffer(raw, dtype="<f4").reshape(shape)
                if dtype == Dtype.F16:
                    arr = arr.astype(np.float16)
                params[name] = backend.from_numpy(arr, dtype)
            else:
                raise SafetensorsError(f"{name}: unsupported dtype {dt}")
            total += int(np.prod(shape)) if shape else 1
    return params, total


def load_model(backend, directory, dtype):
    """A checkpoint directory in the Hugging Face layout (config.json + *.safetensors, sharded or not) ->
    (LlamaConfig, Parameters, element count): what `get_model_files` + `load_model` hand the runner
    (catgrad-llm/src/utils/mod.rs:321-470), for the dense Llama family."""
    import glob
    import os
    from .llama import LlamaConfig
    cfg = LlamaConfig.from_hf_config(os.path.join(directory, "config.json"))
    files = sorted(glob.glob(os.path.join(directory, "*.safetensors")))
    if not files:
        raise SafetensorsError(f"no .safetensors file in {directory}")
    params, n = load_parameters(backend, files, dtype)
    missing = [k for k, _ in cfg.param_shapes() if k not in params.keys()]
    if missing:
        raise SafetensorsError(f"checkpoint lacks {len(missing)} tensors of the configured model, e.g. {missing[0]}")
    return cfg, params, n


def save_file(path, tensors, bf16=False):
    """Writes float32 arrays as F32 (or, with bf16=True, rounded to BF16): used by tests and for exporting synthetic
    models."""
    header, blobs, off = {}, [], 0
    for name, arr in tensors.items():
        arr = np.ascontiguousarray(arr, dtype=np.float32)
        data = f32_to_bf16_bits(arr).astype("<u2").tobytes() if bf16 else arr.astype("<f4").tobytes()
        header[name] = {"dtype": "BF16" if bf16 else "F32", "shape": list(arr.shape), "data_offsets": [off, off + len(data)]}
        blobs.append(data)
        off += len(data)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)

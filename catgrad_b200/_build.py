"""Builds the in-tree CUDA library `catgrad_b200/_lib/libcatgrad_b200.so` with nvcc for sm_100a.

Run as `python -m catgrad_b200._build` or through `__graft_entry__.build()`.  No GPU is needed to build.
The runtime is linked statically (`-cudart static`) and the driver API is reached through
`cudaGetDriverEntryPoint`, so the library loads on a machine without a GPU driver (its entry points then
return CG_ERR_CUDA).
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_lib")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
LIB = os.path.join(OUT_DIR, "libcatgrad_b200.so")

SOURCES = [
    "kernels/elementwise.cu",
    "kernels/reduce.cu",
    "kernels/matmul.cu",
    "kernels/gemm_tcgen05.cu",
    "kernels/gemm_f32x3.cu",
    "kernels/argmax_noalloc.cu",
    "host/cuda_backend.cu",
    "host/llama_engine.cu",
    "host/tp_comm.cu",
    "host/device_runner.cu",
    "host/c_api.cc",
    "host/interp.cc",
    "host/llama_term.cc",
]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo", "-fmad=false",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default", "-DCG_PREFIX=cg_",
              "-I", os.path.join(os.path.dirname(HERE), "include")]


def _newer(src, obj):
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    deps = [src]
    for root, _, files in os.walk(CSRC):
        deps += [os.path.join(root, f) for f in files if f.endswith((".h", ".cuh"))]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "catgrad_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def _compile(src):
    path = os.path.join(CSRC, src)
    obj = os.path.join(OBJ_DIR, src.replace("/", "_") + ".o")
    if not _newer(path, obj):
        return obj, ""
    cmd = ["nvcc"] + NVCC_FLAGS + (["-x", "cu"] if src.endswith(".cc") else []) + ["-c", path, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(verbose=False):
    os.makedirs(OBJ_DIR, exist_ok=True)
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        results = list(ex.map(_compile, SOURCES))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log.strip():
                print(log, file=sys.stderr)
    if (not os.path.exists(LIB)) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "static", "-o", LIB] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(verbose=True))

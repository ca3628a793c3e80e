"""Builds the CUDA library of the llama path for sm_100a, in-tree.

    python enzyme-jax_b200/build.py [--force] [--verbose]

Every ``csrc/*.cu`` is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` and linked into
``enzyme-jax_b200/lib/libb200_llama.so``.  nvcc cross-compiles, so this runs on
a machine without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")
LIB = os.path.join(LIBDIR, "libb200_llama.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "-Xptxas", "-v",
]
# Only the bf16 tensor-core kernels (2e-2 bar) are built with fast math.  The files that serve the fp32
# configuration (FFMA GEMM, fp32 attention, RMSNorm and the other elementwise kernels; 1e-4 / 1e-5 bar and
# equal argmax) keep IEEE division and square roots, denormals, and the accurate expf.
FAST_MATH_FILES = {"attention_mma.cu", "attention_bwd_tc.cu", "attention_decode.cu", "gemm_tc.cu", "gemm_tc2.cu",
                   "comm.cu", "gemv_decode.cu"}


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _newest(paths) -> float:
    return max(os.path.getmtime(p) for p in paths)


def _xla_ffi_include():
    """Directory holding xla/ffi/api/ffi.h (jaxlib ships it), or None.  B200_XLA_FFI_INCLUDE overrides."""
    cand = [os.environ.get("B200_XLA_FFI_INCLUDE")]
    try:
        import importlib.util
        spec = importlib.util.find_spec("jaxlib")
        if spec and spec.submodule_search_locations:
            cand.append(os.path.join(list(spec.submodule_search_locations)[0], "include"))
    except Exception:
        pass
    for c in cand:
        if c and os.path.exists(os.path.join(c, "xla", "ffi", "api", "ffi.h")):
            return c
    return None


def _compile(src: str, obj: str, log: str):
    fast = ["--use_fast_math", "-DB200_FAST_MATH=1"] if os.path.basename(src) in FAST_MATH_FILES else []
    if src.endswith(".cc"):  # the XLA FFI shim: handlers are compiled in only where the XLA FFI headers exist
        inc = _xla_ffi_include()
        fast = ["-I", inc] if inc else []
    cmd = [_nvcc(), *NVCC_FLAGS, *fast, "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return r.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu"))) + sorted(glob.glob(os.path.join(CSRC, "ffi", "*.cc")))
    hdrs = sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + [os.path.join(HERE, "..", "include", "b200_llama.h")]
    if not srcs:
        raise RuntimeError("no CUDA sources found")
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    hdr_time = _newest(hdrs)
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(OBJDIR, os.path.splitext(os.path.basename(s))[0] + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_time):
            jobs.append((s, o, o[:-2] + ".log"))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for (s, _, _), out in zip(jobs, ex.map(lambda j: _compile(*j), jobs)):
                if verbose:
                    print(f"--- {os.path.basename(s)}\n{out}")
    if jobs or not os.path.exists(LIB):
        tmp = LIB + ".linking"
        cmd = [_nvcc(), "-shared", "-o", tmp, *objs, "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB)  # a reader never sees a half-written library
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)

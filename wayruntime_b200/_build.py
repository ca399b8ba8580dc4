"""Build libwr_cuda.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libwr_cuda.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

SOURCES = ["kv_cache.cu", "attn_decode.cu", "attn_decode_static.cu", "attn_prefill.cu", "attn_exchange.cu",
           "model_glue.cu", "attn_step_small.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(INCLUDE, "wr_cuda.h")]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the CUDA sources into wayruntime_b200/lib/libwr_cuda.so."""
    if not force and not _stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-I", CSRC]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES] + ["-o", LIB_PATH]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed:\n{res.stdout}")
    if verbose:
        print(res.stdout)
    return LIB_PATH


DROPIN_PATH = os.path.join(LIB_DIR, "libwayruntime_b200.so")


def build_dropin(ref_root: str) -> str | None:
    """Link lib/libwayruntime_b200.so: the reference library (compiled from the
    checkout at `ref_root`, unmodified) with this package's session objects and
    engine gate in place of its session.c / batch.c / engine entry points.
    Returns None when there is no checkout (the GPU box uses the prebuilt file)."""
    if not os.path.exists(os.path.join(ref_root, "src", "core", "kernels.c")):
        return None
    build()
    res = subprocess.run(["make", "-C", os.path.join(PKG, "host"), f"REF={ref_root}"],
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"drop-in link failed:\n{res.stdout}")
    return DROPIN_PATH

"""Compile csrc/ into lib/libtensor_ash.so for sm_100a with nvcc.

One object per translation unit (compiled in parallel, rebuilt only when the
source or a header is newer), then one link.  cudart is linked statically and
the driver API is reached through cudaGetDriverEntryPoint, so the library has
no load-time dependency beyond libstdc++ and loads on machines without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libtensor_ash.so")
BIN_DIR = os.path.join(HERE, "bin")
LLAMA_ASH = os.path.join(BIN_DIR, "llama_ash")     # CLI over the C ABI (csrc/llama_ash_main.cpp)
TOOLS = {"llama_ash": "llama_ash_main.cpp", "ml_bench": "ml_bench_main.cpp"}

SOURCES = [
    "ta_host.cpp",
    "gguf.cpp",
    "ta_runtime.cu",
    "ta_graph.cu",
    "ta_capi.cu",
    "ta_comm.cu",
    "ta_host_stream.cu",
    "llama_ash.cu",
    "k_gemm_ffma.cu",
    "k_gemm_tf32x3.cu",
    "k_gemm_tf32x3_2cta.cu",
    "k_gemm_f16w.cu",
    "k_gemv.cu",
    "k_gemv_umma.cu",
    "k_attention.cu",
    "k_ops.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function",
    "--expt-relaxed-constexpr",
    "-x", "cu",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA toolkit is required to build this library")
    return exe


def _headers_mtime() -> float:
    m = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "include")):
        for name in os.listdir(root):
            if name.endswith((".hpp", ".cuh", ".h")):
                m = max(m, os.path.getmtime(os.path.join(root, name)))
    return m


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    if os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(path), _headers_mtime()):
        return obj
    cmd = [nvcc(), *NVCC_FLAGS, "-c", path, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    if verbose:
        sys.stderr.write(r.stderr)
    return obj


def build(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    if force:
        for f in os.listdir(OBJ):
            os.remove(os.path.join(OBJ, f))
    with cf.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), SOURCES))
    if not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        # link beside the target and rename: a reader never sees a half-written library
        tmp = LIB + ".partial"
        cmd = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp, *objs,
               "-Xlinker", "--exclude-libs,ALL", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB)
    build_tools()
    return LIB


def build_tools() -> str:
    """llama_ash and ml_bench: plain C++ against the public headers; they find the library next to
    themselves (rpath $ORIGIN/../lib)."""
    os.makedirs(BIN_DIR, exist_ok=True)
    cxx = shutil.which("g++") or "g++"
    for name, source in TOOLS.items():
        src, exe = os.path.join(CSRC, source), os.path.join(BIN_DIR, name)
        if os.path.exists(exe) and os.path.getmtime(exe) >= max(os.path.getmtime(src), os.path.getmtime(LIB),
                                                               _headers_mtime()):
            continue
        cmd = [cxx, "-O2", "-std=c++17", "-Wall", "-pthread", src, "-o", exe, "-L", LIB_DIR, "-ltensor_ash",
               "-Wl,-rpath,$ORIGIN/../lib"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"building {name} failed:\n{r.stdout}\n{r.stderr}")
    return LLAMA_ASH


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))

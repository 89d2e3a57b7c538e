"""Builds ``libsimp_gpu.so`` (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m simplang_b200.build [--force] [--verbose] [--trace]

One object per ``csrc/*.cu`` (compiled in parallel, skipped when up to date), linked into
``simplang_b200/libsimp_gpu.so``.  nvcc cross-compiles without a GPU.
``--trace`` builds a second, instrumented library ``libsimp_gpu_trace.so`` (-DSIMP_W4_TRACE: the W4 projection and
attention kernels of a decode step write %globaltimer marks from thread 0 of every block); load it with
``SIMP_GPU_LIB=simplang_b200/libsimp_gpu_trace.so python -m simplang_b200.opbench --only decode3b_marks``.
It is a measurement aid: its timings are not the product's.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libsimp_gpu.so")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
HOST_CXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-ccbin", HOST_CXX, "-Xcompiler", "-fPIC,-fvisibility=hidden,-O3",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _compile(src, force, verbose, obj_dir=None, extra=()):
    obj = os.path.join(obj_dir or OBJ, os.path.basename(src)[:-3] + ".o")
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.hpp")) + \
        glob.glob(os.path.join(ROOT, "include", "*.h"))
    if not force and _newer(obj, [src] + headers):
        return obj, ""
    cmd = [NVCC] + FLAGS + list(extra) + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    return obj, r.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, force, verbose), srcs))
    objs = [o for o, _ in results]
    if verbose:
        for _, log in results:
            if log:
                print(log)
    if force or not _newer(LIB, objs):
        cmd = [NVCC, "-shared", "-ccbin", HOST_CXX, "-o", LIB] + objs + ["-lcudart_static", "-ldl", "-lpthread", "-lrt"]  # NCCL is dlopen-ed
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    build_host()
    return LIB


def build_trace() -> str:
    """The instrumented library (see the module docstring)."""
    obj_dir = os.path.join(HERE, "build_trace")
    os.makedirs(obj_dir, exist_ok=True)
    lib = os.path.join(HERE, "libsimp_gpu_trace.so")
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = [o for o, _ in ex.map(lambda s: _compile(s, False, False, obj_dir, ("-DSIMP_W4_TRACE",)), srcs)]
    r = subprocess.run([NVCC, "-shared", "-ccbin", HOST_CXX, "-o", lib] + objs + ["-lcudart_static", "-ldl", "-lpthread", "-lrt"],
                       capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib


def build_host() -> str:
    """Compiles the C++ host example (plain g++, links only -ldl: it dlopen()s the runtime library)."""
    host_dir = os.path.join(HERE, "host")
    src = os.path.join(host_dir, "bench_int8_gemm_host.cpp")
    exe = os.path.join(host_dir, "bench_int8_gemm_host")
    if not _newer(exe, [src, os.path.join(host_dir, "gpu_kernel_runner.hpp")]):
        r = subprocess.run([HOST_CXX, "-O2", "-std=c++17", "-o", exe, src, "-ldl"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"host build failed:\n{r.stdout}\n{r.stderr}")
    return exe


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--trace" in sys.argv:
        print(build_trace())

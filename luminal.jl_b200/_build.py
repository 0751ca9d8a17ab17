"""Builds libluminal_b200.so in-tree with nvcc for sm_100a (no JIT cache, no torch extension)."""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libluminal_b200.so")
SOURCES = ["api.cu", "gemv.cu", "attention.cu", "model.cu", "prims.cu", "flash.cu", "flash_tc.cu", "flash_tc_f32.cu", "prefill.cu", "whisper_enc.cu", "noalloc.cu", "match.cu", "wide.cu"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(HERE, "..", "include", "luminal_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


TRACE_LIB = os.path.join(HERE, "build_trace", "libluminal_b200_trace.so")


def build_library(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """Compile every .cu under csrc/ and link the shared library.  Returns its path.

    trace=True builds a second library, build_trace/libluminal_b200_trace.so, with -DLMB_GEMV_TRACE:
    the GEMV kernels then stamp the SM clock at their phase boundaries into a device array that
    lmb200_debug_gemv_trace copies out
    (luminal.jl_b200/trace.py reads them).  The product library never carries the stamps."""
    lib = TRACE_LIB if trace else LIB
    if not trace and not force and not _stale():
        return LIB
    objdir = os.path.join(HERE, "build_trace" if trace else "build")
    os.makedirs(objdir, exist_ok=True)
    nvcc = _nvcc()
    extra = ["-DLMB_GEMV_TRACE"] if trace else []

    def compile_one(src):
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=8) as pool:
        objs = list(pool.map(compile_one, _sources()))
    cmd = [nvcc, "-shared", "-o", lib, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
           "-Xcompiler", "-fPIC", "-lcudart_static", "-ldl", "-lpthread", "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv))

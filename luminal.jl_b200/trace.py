"""Phase stamps of the decode GEMV kernels (tuning aid).

    python luminal.jl_b200/_build.py --trace          # builds build_trace/libluminal_b200_trace.so
    python -m luminal_jl_b200.trace 768x4096 4096x512  # rows x K of the matrices to run (batch 32)

Runs lmb200_linear_gemv of the trace build on random data and prints, per phase, the median and the
maximum over the CTAs of the time since the CTA's entry: setup (barriers, TMEM), dep_ok (the wait
for the previous kernel), first_data (first stage landed), mma_done (last MMA issued), acc_ready
(accumulators read), sent (partial stored / sent to the cluster), gathered (cluster barrier or fold
wait passed), epi_done, exit.  The product library carries no stamps; this module refuses to run on
it."""
from __future__ import annotations

import ctypes as C
import os
import sys

import numpy as np

NAMES = ["entry", "setup", "dep_ok", "first_data", "mma_done", "acc_ready", "sent", "gathered", "epi_done", "exit",
         "ns0", "ns1", "fold_fetch", "fold_sum"]


def gemv_phase_trace(shapes, batch=32, out=sys.stdout):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    import luminal_jl_b200 as L
    from luminal_jl_b200 import _build, _lib
    if not os.path.exists(_build.TRACE_LIB):
        raise SystemExit(f"{_build.TRACE_LIB} is missing: run `python luminal.jl_b200/_build.py --trace`")
    _lib.LIB_PATH = _build.TRACE_LIB
    dev = L.get_device()
    lib = C.CDLL(_build.TRACE_LIB)
    for rows, K in shapes:
        rng = np.random.default_rng(0)
        w = rng.standard_normal((rows, K), dtype=np.float32) * np.float32(0.02)
        x = rng.standard_normal((batch, K), dtype=np.float32)
        for _ in range(3):
            L.linear_gemv(dev, w, x, "bf16")
        buf = np.zeros((160, 16), np.int64)
        if lib.lmb200_debug_gemv_trace(buf.ctypes.data_as(C.c_void_p)) != 0:
            raise SystemExit("lmb200_debug_gemv_trace failed")
        t = buf[:148]
        t = t[t[:, 0] != 0]
        span_ns = t[:, 11].max() - t[:, 10].min()
        cyc_per_ns = float(np.median((t[:, 9] - t[:, 0]) / np.maximum(1, (t[:, 11] - t[:, 10]))))
        print(f"--- rows {rows} K {K} ({rows * K * 2 / 1e6:.1f} MB, batch {batch}): kernel span {span_ns / 1e3:.2f} us, "
              f"{len(t)} CTAs, start skew {(t[:, 10].max() - t[:, 10].min()) / 1e3:.2f} us", file=out)
        for i, name in enumerate(NAMES):
            if i in (0, 10, 11):
                continue
            ok = t[:, i] != 0
            if not ok.any():
                continue
            d = ((t[:, i] - t[:, 0]) / cyc_per_ns / 1e3)[ok]
            print(f"  {name:10s} n={int(ok.sum()):3d}  median {np.median(d):7.2f}  max {d.max():7.2f} us", file=out)


if __name__ == "__main__":
    args = sys.argv[1:] or ["6144x4096", "4096x4096", "28672x4096", "4096x14336"]
    gemv_phase_trace([tuple(int(v) for v in a.split("x")) for a in args])

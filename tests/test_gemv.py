"""The decode GEMV kernels one by one (float32 ring, bf16 mma.sync, bf16 tcgen05) against NumPy:
shapes that exercise padding of rows and K, split-K folds across CTAs, and the three batch
paddings."""
import numpy as np
import pytest

import luminal_oracle as O

pytestmark = pytest.mark.gpu

SHAPES = [(16, 32, 1), (100, 72, 3), (128, 128, 16), (384, 1024, 17), (1000, 2816, 32), (4096, 512, 32),
          (2816, 1024, 5), (130, 4100, 32)]


@pytest.mark.parametrize("rows,K,batch", SHAPES)
@pytest.mark.parametrize("kernel", ["f32", "bf16-mma", "bf16-tcgen05"])
def test_linear_gemv(lib_built, device, rows, K, batch, kernel):
    L = lib_built
    w = O.synth_normal(1, rows * 7 + K, (rows, K), 0.05)
    x = O.synth_normal(2, batch, (batch, K), 1.0)
    if kernel == "f32":
        got = L.linear_gemv(device, w, x, "f32")
        ref = x.astype(np.float64) @ w.astype(np.float64).T
        tol = 1e-5
    else:
        wq, xq = O.bf16_round(w), O.bf16_round(x)
        got = L.linear_gemv(device, wq, xq, "bf16", 0 if kernel.endswith("tcgen05") else 1)
        ref = xq.astype(np.float64) @ wq.astype(np.float64).T       # bf16 operands, exact products
        tol = 2e-5
    assert got.shape == ref.shape
    assert np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max()) * np.sqrt(K / 32.0)

"""The C ABI used from plain C: tests/cabi_driver.c is compiled with gcc as strict C99 against
include/luminal_b200.h and linked to the shared library.  Without a GPU it must fail loudly at
lmb200_init; on a B200 its greedy tokens must equal the CPU oracle's."""
import json
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def driver(lib_built, tmp_path_factory):
    from importlib import import_module
    lib = import_module("luminal_jl_b200._build").LIB
    exe = str(tmp_path_factory.mktemp("cabi") / "cabi_driver")
    cmd = ["gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-O1", os.path.join(ROOT, "tests", "cabi_driver.c"),
           "-I", os.path.join(ROOT, "include"), "-L", os.path.dirname(lib), "-lluminal_b200",
           "-Wl,-rpath," + os.path.dirname(lib), "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_header_is_plain_c_and_driver_fails_loudly_without_a_gpu(driver):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the GPU test runs the driver")
    r = subprocess.run([driver, "0", "1", "4", "2", "1234"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 2 and "lmb200_init" in r.stderr and r.stdout == ""
    assert subprocess.run([driver], capture_output=True).returncode == 64


@pytest.mark.gpu
@pytest.mark.parametrize("batch,prompt,steps", [(1, 32, 24), (3, 9, 12)])
def test_c_driver_tokens_match_the_oracle(driver, batch, prompt, steps):
    import luminal_oracle as O
    r = subprocess.run([driver, "0", str(batch), str(prompt), str(steps), "1234"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    got = json.loads(r.stdout)
    cfg = O.CONFIGS["small_llama"]
    w = O.synth_llama_weights(cfg, seed=1234)
    toks = np.array([[(7 * i + 3 + 11 * b) % cfg["vocab"] for i in range(prompt)] for b in range(batch)], dtype=np.int64)
    ref_tok, _ = O.CachedLlama(w, cfg, batch, prompt + steps + 1).greedy(toks, steps + 1)
    ref_tok = np.asarray(ref_tok)                     # [batch, steps + 1]: the prompt's prediction, then one per step
    assert got["position"] == prompt + steps
    assert got["first"] == ref_tok[:, 0].tolist()
    assert np.array_equal(np.array(got["tokens"]).reshape(steps, batch).T, ref_tok[:, 1:])


@pytest.mark.gpu
def test_c_driver_bf16_runs(driver):
    r = subprocess.run([driver, "1", "2", "16", "8", "7"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    got = json.loads(r.stdout)
    assert got["position"] == 24 and len(got["tokens"]) == 16 and all(0 <= t < 1024 for t in got["tokens"])

"""Prompt phase as tensor-core GEMMs + flash attention (bf16) against the oracle and against the
same prompt fed token by token through the decode step: logits of the last position, the cache
it leaves behind (checked through the decode steps that follow), grouped kv heads of width 128
and 96, ragged sizes that do not fill the 128-token tiles."""
import os

import numpy as np
import pytest

import luminal_oracle as O

pytestmark = pytest.mark.gpu


def make(L, device, cfg, w, batch, max_ctx):
    model = L.Model(device, n_layers=cfg["n_layers"], hidden=cfg["hidden"], n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"],
                    intermediate=cfg["intermediate"], vocab=cfg["vocab"], eps=cfg["eps"], rope_base=cfg["rope_base"], dtype="bf16")
    if w is None:
        model.init_random(seed=11, sigma=0.02)
    else:
        model.set_weights(w)
    return model, L.Session(model, batch, max_ctx)


def run(sess, prompt, steps, mode):
    if mode == "steps":
        os.environ["LMB200_PREFILL"] = "steps"
    try:
        logits = [sess.prefill(prompt)]
    finally:
        os.environ.pop("LMB200_PREFILL", None)
    tok = logits[0].argmax(-1).astype(np.int32)
    for _ in range(steps):
        tok_next, lg = sess.decode_step(tok, want_logits=True)
        logits.append(lg)
        tok = lg.argmax(-1).astype(np.int32)
    return np.stack(logits, 0)


@pytest.mark.parametrize("name,batch,n", [("tiny_gqa128", 3, 40), ("tiny_gqa96", 2, 130), ("mid_gqa", 5, 77)])
def test_gemm_prefill_matches_oracle_and_stepwise(lib_built, device, name, batch, n):
    L = lib_built
    cfg = O.CONFIGS[name]
    w = {k: O.bf16_round(v) if v.ndim == 2 else v for k, v in O.synth_llama_weights(cfg, seed=21).items()}
    prompt = O.synth_tokens(21, 3, (batch, n), cfg["vocab"]).astype(np.int32)
    ref = O.CachedLlama(w, cfg, batch, n + 8)
    ref_logits = ref.forward(prompt)[:, -1, :]
    model, sess = make(L, device, cfg, w, batch, n + 8)
    fast = run(sess, prompt, 3, "gemm")
    sess.reset()
    slow = run(sess, prompt, 3, "steps")
    scale = np.linalg.norm(ref_logits)
    assert np.linalg.norm(fast[0] - ref_logits) / scale <= 4e-2
    assert np.linalg.norm(slow[0] - ref_logits) / scale <= 4e-2
    # the cache the GEMM path leaves behind serves the decode steps as well as the stepwise one
    # (teacher-forced only through each path's own argmax, so compare where the tokens agree)
    for i in range(1, 4):
        if np.array_equal(fast[i - 1].argmax(-1), slow[i - 1].argmax(-1)):
            assert np.linalg.norm(fast[i] - slow[i]) / np.linalg.norm(slow[i]) <= 4e-2
        else:
            break
    sess.close(); model.close()


def test_gemm_prefill_phi3_width(lib_built, device):
    """Two layers at the Phi-3-mini width (hidden 3072, 32 q / 8 kv heads of 96, MLP 8192, vocab 32064),
    512-token prompts: GEMM path against the stepwise path."""
    L = lib_built
    cfg = dict(O.CONFIGS["phi3_mini"], n_layers=2)
    model, sess = make(L, device, cfg, None, 2, 1024)
    prompt = O.synth_tokens(5, 3, (2, 512), cfg["vocab"]).astype(np.int32)
    fast = run(sess, prompt, 2, "gemm")
    sess.reset()
    slow = run(sess, prompt, 2, "steps")
    for i in range(3):
        assert np.linalg.norm(fast[i] - slow[i]) / np.linalg.norm(slow[i]) <= 4e-2, i
        if not np.array_equal(fast[i].argmax(-1), slow[i].argmax(-1)):
            break
    sess.close(); model.close()


@pytest.mark.parametrize("rows,K,tokens", [(128, 128, 128), (100, 72, 37), (384, 1024, 300), (1000, 2816, 129), (4608, 3072, 512),
                                            (256, 256, 256), (512, 4096, 1000), (768, 64, 257)])
def test_prefill_gemm_matches_float64(lib_built, device, rows, K, tokens):
    L = lib_built
    rng = np.random.default_rng(rows + tokens)
    w = O.bf16_round(rng.standard_normal((rows, K), dtype=np.float32) * np.float32(0.05))
    x = O.bf16_round(rng.standard_normal((tokens, K), dtype=np.float32))
    got = L.prefill_gemm(device, w, x)
    ref = x.astype(np.float64) @ w.astype(np.float64).T
    assert got.shape == ref.shape
    assert np.abs(got - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max()) * np.sqrt(K / 32.0)


def test_prefill_gemm_single_cta_kernel(lib_built, device):
    """Shapes of whole 256-row groups and at least 256 tokens run on CTA pairs (tcgen05.mma cta_group::2); the
    single-CTA kernel then serves the other shapes.  LMB200_GEMM_PAIR=0 (read once per process) sends the pair
    shapes through it too: run those in a child process against float64."""
    import subprocess
    import sys
    code = r'''
import numpy as np, sys
sys.path.insert(0, "."); sys.path.insert(0, "oracle")
import luminal_jl_b200 as L
import luminal_oracle as O
dev = L.get_device()
for rows, K, tokens in [(256, 256, 256), (512, 4096, 1000), (4608, 3072, 512)]:
    rng = np.random.default_rng(rows + tokens)
    w = O.bf16_round(rng.standard_normal((rows, K), dtype=np.float32) * np.float32(0.05))
    x = O.bf16_round(rng.standard_normal((tokens, K), dtype=np.float32))
    got = L.prefill_gemm(dev, w, x)
    ref = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(got - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max()) * np.sqrt(K / 32.0), (rows, K, tokens)
print("single ok")
'''
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-c", code], cwd=root, env=dict(os.environ, LMB200_GEMM_PAIR="0"), capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0 and "single ok" in r.stdout, r.stdout + r.stderr

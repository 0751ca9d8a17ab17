"""Full-size shapes of the benchmark configurations (Llama-3-8B, Phi-3-mini, the [4,32,4096,128]
attention case), checked through properties that do not need the oracle to run the whole size:
exact homogeneity of the GEMV under a power-of-two scale, run-to-run bit identity, sampled rows
against float64, sampled (sequence, head) pairs of the 8192-key cache regenerated from the
counter-based generator, and sampled lm_head rows against the captured last hidden state."""
import ctypes as C

import numpy as np
import pytest

import luminal_oracle as O

pytestmark = pytest.mark.gpu


def _bf16(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).bfloat16().float().numpy()


# (rows, K, batch): fused qkv, o, fused gate/up, down, lm_head of Llama-3-8B (batch 32) and Phi-3-mini (batch 16)
GEMV_SHAPES = [(6144, 4096, 32), (4096, 4096, 32), (28672, 4096, 32), (4096, 14336, 32), (128256, 4096, 32),
               (4608, 3072, 16), (16384, 3072, 16), (3072, 8192, 16), (32064, 3072, 16)]


@pytest.mark.parametrize("rows,K,batch", GEMV_SHAPES)
def test_full_size_gemv_properties(lib_built, device, rows, K, batch):
    L = lib_built
    rng = np.random.default_rng(rows + K)
    w = _bf16(rng.standard_normal((rows, K), dtype=np.float32) * np.float32(0.02))
    x = _bf16(rng.standard_normal((batch, K), dtype=np.float32))
    got = L.linear_gemv(device, w, x, "bf16")
    again = L.linear_gemv(device, w, x, "bf16")
    assert np.array_equal(got, again), "two runs differ: the split-K fold is not deterministic"
    doubled = L.linear_gemv(device, w, x * np.float32(2.0), "bf16")
    assert np.array_equal(doubled, got * np.float32(2.0)), "W(2x) != 2 W(x) bit for bit"
    sample = rng.choice(rows, size=96, replace=False)
    ref = x.astype(np.float64) @ w[sample].astype(np.float64).T
    assert np.abs(got[:, sample] - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max()) * np.sqrt(K / 32.0)
    blas = x @ w.T                                    # every row, float32 BLAS
    assert np.abs(got - blas).max() <= 1e-3 * np.abs(blas).max()


def _kv_slice(seed, layer, which, b, kv, KV, max_ctx, D, T):
    base = ((b * KV + kv) * max_ctx) * D
    idx = base + np.arange(T * D, dtype=np.uint64)
    return O.synth_normal_at(seed, 0x100000 + 2 * layer + which, idx, 1.0).reshape(T, D)


def test_llama3_8b_width_decode_properties(lib_built, device):
    """Two layers at the full Llama-3-8B width, vocabulary, batch and cache length."""
    import torch
    L = lib_built
    cfg = dict(O.CONFIGS["llama3_8b"], n_layers=2)
    H, KV, hid, V = cfg["n_heads"], cfg["n_kv_heads"], cfg["hidden"], cfg["vocab"]
    D, G, B, max_ctx, start = hid // H, H // KV, 32, 8192, 8000
    model = L.Model(device, n_layers=2, hidden=hid, n_heads=H, n_kv_heads=KV, intermediate=cfg["intermediate"],
                    vocab=V, rope_base=cfg["rope_base"], dtype="bf16")
    model.init_random(seed=1234, sigma=0.02)
    sess = L.Session(model, B, max_ctx)
    sess.fill_kv_random(start, seed=77)
    first = O.synth_tokens(3, 1, (B,), V).astype(np.int32)

    # attention over 8000 keys: sampled (sequence, kv head) pairs against float64
    q = _bf16(O.synth_normal(5, 77, (B, H, D), 1.0))
    order = [kvh + KV * g for kvh in range(KV) for g in range(G)]
    q_dev = torch.tensor(q[:, order, :], device="cuda").bfloat16().contiguous()
    out_dev = torch.empty_like(q_dev)
    torch.cuda.synchronize()
    sess.decode_attention(1, q_dev.data_ptr(), out_dev.data_ptr(), start)
    device.sync()
    got = np.empty_like(q)
    got[:, order, :] = out_dev.float().cpu().numpy()
    for b, kvh in [(0, 0), (17, 5), (31, 7)]:
        k = _bf16(_kv_slice(77, 1, 0, b, kvh, KV, max_ctx, D, start)).astype(np.float64)
        v = _bf16(_kv_slice(77, 1, 1, b, kvh, KV, max_ctx, D, start)).astype(np.float64)
        for g in range(G):
            h = kvh + KV * g
            s = k @ q[b, h].astype(np.float64) / np.sqrt(D)
            p = np.exp(s - s.max())
            ref = (p / p.sum()) @ v
            assert np.abs(got[b, h] - ref).max() <= 2e-2 * np.abs(ref).max(), (b, h)

    # graph replay == step-by-step launches, and a second replay from the same state is identical
    toks_graph = sess.decode_n(first, 6)
    sess.set_position(start)
    assert np.array_equal(sess.decode_n(first, 6), toks_graph)
    sess.set_position(start)
    sess.set_capture(True)
    tok, steps = first, []
    for _ in range(6):
        tok, logits = sess.decode_step(tok, want_logits=True)
        steps.append(tok.copy())
    assert np.array_equal(np.stack(steps, 0), toks_graph)

    # lm_head at the full vocabulary: sampled rows from the captured last hidden state
    hidden = sess.layer_output(1)                                         # [B, hidden] float32
    norm_w = O.synth_normal(1234, O.GLOBAL_IDS["model.norm.weight"], (hid,), 0.02, 1.0)
    xq = _bf16(O.rms_norm(hidden, norm_w, cfg["eps"])).astype(np.float64)
    rows = np.random.default_rng(0).choice(V, size=128, replace=False)
    idx = rows[:, None].astype(np.uint64) * np.uint64(hid) + np.arange(hid, dtype=np.uint64)[None, :]
    wq = _bf16(O.synth_normal_at(1234, O.GLOBAL_IDS["lm_head.weight"], idx, 0.02)).astype(np.float64)
    ref = xq @ wq.T
    assert np.abs(logits[:, rows] - ref).max() <= 2e-2 * np.abs(ref).max()
    assert np.array_equal(logits.argmax(-1), tok)
    sess.close(); model.close()


@pytest.mark.parametrize("causal", [False, True])
def test_full_size_flash_attention_sampled_rows(lib_built, device, causal):
    """Q, K, V [4, 32, 4096, 128] bf16: sampled query rows of sampled heads against float64, and the
    causal result's first row equals V's first row (its softmax has one term)."""
    import torch
    from importlib import import_module
    _lib = import_module("luminal_jl_b200._lib")
    B, H, S, D = 4, 32, 4096, 128
    gen = torch.Generator(device="cuda").manual_seed(7)
    q, k, v = (torch.randn((B, H, S, D), device="cuda", generator=gen).bfloat16() for _ in range(3))
    out = torch.empty_like(q)
    torch.cuda.synchronize()
    scale = 1.0 / np.sqrt(D)
    p = lambda t: C.c_void_p(t.data_ptr())
    _lib.call("lmb200_flash_attention", device.handle, p(out), p(q), p(k), p(v), _lib.BF16, B, H, S, D, scale, int(causal))
    device.sync()
    rows = [0, 1, 63, 64, 127, 128, 2047, 2048, 4000, 4095]
    for b, h in [(0, 0), (1, 13), (3, 31)]:
        kk = k[b, h].float().cpu().numpy().astype(np.float64)
        vv = v[b, h].float().cpu().numpy().astype(np.float64)
        qq = q[b, h, rows].float().cpu().numpy().astype(np.float64)
        got = out[b, h, rows].float().cpu().numpy()
        for i, r in enumerate(rows):
            n = r + 1 if causal else S
            s = kk[:n] @ qq[i] * scale
            pr = np.exp(s - s.max())
            ref = (pr / pr.sum()) @ vv[:n]
            assert np.abs(got[i] - ref).max() <= 2e-2 * max(np.abs(ref).max(), 0.05), (b, h, r)
    if causal:
        assert torch.equal(out[:, :, 0], v[:, :, 0])


@pytest.mark.parametrize("causal", [False, True])
def test_full_size_flash_attention_fp32_sampled_rows(lib_built, device, causal):
    """The same [4, 32, 4096, 128] case with float32 tensors (the reference's own precision): tensor cores with bf16
    hi + lo operands.  Sampled rows against float64 at rtol 1e-4 of the row's largest magnitude."""
    import torch
    from importlib import import_module
    _lib = import_module("luminal_jl_b200._lib")
    B, H, S, D = 4, 32, 4096, 128
    gen = torch.Generator(device="cuda").manual_seed(11)
    q, k, v = (torch.randn((B, H, S, D), device="cuda", generator=gen) for _ in range(3))
    out = torch.empty_like(q)
    torch.cuda.synchronize()
    scale = 1.0 / np.sqrt(D)
    p = lambda t: C.c_void_p(t.data_ptr())
    _lib.call("lmb200_flash_attention", device.handle, p(out), p(q), p(k), p(v), _lib.F32, B, H, S, D, scale, int(causal))
    device.sync()
    rows = [0, 1, 63, 64, 127, 128, 2047, 2048, 4000, 4095]
    for b, h in [(0, 0), (2, 17), (3, 31)]:
        kk = k[b, h].cpu().numpy().astype(np.float64)
        vv = v[b, h].cpu().numpy().astype(np.float64)
        qq = q[b, h, rows].cpu().numpy().astype(np.float64)
        got = out[b, h, rows].cpu().numpy()
        for i, r in enumerate(rows):
            n = r + 1 if causal else S
            s = kk[:n] @ qq[i] * scale
            pr = np.exp(s - s.max())
            ref = (pr / pr.sum()) @ vv[:n]
            assert np.abs(got[i] - ref).max() <= 1e-4 * np.abs(ref).max(), (b, h, r, float(np.abs(got[i] - ref).max() / np.abs(ref).max()))

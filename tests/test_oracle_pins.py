"""The oracle against every numeric known-answer test the reference holds for this path
(the reference's own tests are named beside each case), plus its internal consistency:
the KV-cached decode equals the reference's full-prefix recompute."""
import numpy as np

import luminal_oracle as O


def test_linear_known_answer():
    # tests/test_nn_layers.jl:8-32
    x = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    w_in_out = np.array([[1, 2, 3, 4], [5, 6, 7, 8], [9, 10, 11, 12]], np.float32)
    bias = np.array([0.1, 0.2, 0.3, 0.4], np.float32)
    got = O.linear(x, w_in_out.T, bias)            # weight is stored [out, in]
    assert np.allclose(got, x @ w_in_out + bias)


def test_embedding_known_answer():
    # tests/test_nn_layers.jl:34-52: ids [2, 0] are 0-based rows
    m = np.array([[1, 2, 3, 4], [5, 6, 7, 8], [9, 10, 11, 12]], np.float32)
    got = O.embedding(m, np.array([2, 0], np.float32))
    assert np.array_equal(got, np.array([[9, 10, 11, 12], [1, 2, 3, 4]], np.float32))


def test_layernorm_property():
    # tests/test_nn_layers.jl:54-69: mean 0, rms 1 per row (atol 1e-5)
    out = O.layer_norm(np.array([[1, 2, 3], [4, 5, 6]], np.float32))
    for row in out:
        assert abs(row.sum() / 3) < 1e-5
        assert abs(np.sqrt((row ** 2).sum() / 3) - 1.0) < 1e-5


def test_mul_add_and_fused_ops():
    # tests/test_gpu_execution.jl:8-24 and :54-76
    a, b, c = (np.array(v, np.float32) for v in ([1, 2, 3], [4, 5, 6], [7, 8, 9]))
    assert np.array_equal(O.add(O.mul(a, b), c), np.array([11, 18, 27], np.float32))
    rng = np.random.default_rng(0)
    a, b, c = (rng.random(10, dtype=np.float32) for _ in range(3))
    assert np.allclose(O.fused_mul_add(a, b, c), a * b + c)
    # tests/test_fusion.jl:7-56: (a+b)*c and relu(x*w+bias)
    a, b, c = (rng.random((3, 3), dtype=np.float32) for _ in range(3))
    assert np.allclose(O.mul(O.add(a, b), c), (a + b) * c)
    x, w = rng.random((2, 2), dtype=np.float32), rng.random((2, 2), dtype=np.float32)
    bias = rng.random((2, 2), dtype=np.float32) - np.float32(0.5)
    assert np.allclose(O.relu(O.add(O.mul(x, w), bias)), np.maximum(x * w + bias, 0))
    assert np.allclose(O.fused_add_relu(O.mul(x, w), bias), np.maximum(x * w + bias, 0))


def test_matmul_add_known_answer():
    # tests/test.jl:17-43
    a = np.array([[1, 2], [3, 4]], np.float32)
    b = np.array([[5, 6], [7, 8]], np.float32)
    c = np.ones((2, 2), np.float32)
    assert np.array_equal(O.add(O.matmul(a, b), c), a @ b + c)


def test_unfold_windows():
    # tests/test_whisper_components.jl:5-23
    a = np.arange(1, 15, dtype=np.float32).reshape(1, 2, 7)
    res = O.unfold1d(a, 3, 2, 1)
    assert res.shape == (1, 2, 3, 3)
    assert np.array_equal(res[0, 0], [[1, 2, 3], [3, 4, 5], [5, 6, 7]])
    assert np.array_equal(res[0, 1], [[8, 9, 10], [10, 11, 12], [12, 13, 14]])


def _manual_attention(q, k, v, scale, causal):
    w = O.mul(O.matmul(q, O.permute(k, [1, 2, 4, 3])), np.float32(scale))
    if causal:
        S = q.shape[2]
        h = O.expand(O.arange(S), 1, S)
        v_idx = O.expand(O.arange(S), 2, S)
        mask = O.less_than(h, O.add(v_idx, np.float32(1.0)))        # `v_idx + 1 > h`
        w = O.add(w, O.mul(O.add(O.mul(mask, np.float32(-1.0)), np.float32(1.0)), np.float32(-1.0e9)))
    return O.matmul(O.softmax(w, 4), v)


def test_flash_attention_vs_manual():
    # tests/test_flash_attention_verification.jl:24-94, B,H,S,D = 1,1,8,16
    rng = np.random.default_rng(1)
    q, k, v = (rng.standard_normal((1, 1, 8, 16), dtype=np.float32) for _ in range(3))
    scale = np.float32(1.0) / np.sqrt(np.float32(16))
    flash = O.flash_attn_cpu(q, k, v, scale, False)
    assert np.allclose(flash, _manual_attention(q, k, v, scale, False), rtol=1e-4, atol=1e-6)
    assert np.allclose(O.flash_attn_fast(q, k, v, scale, False), flash, rtol=1e-5, atol=1e-6)
    causal = O.flash_attn_cpu(q, k, v, scale, True)
    assert np.allclose(causal, _manual_attention(q, k, v, scale, True), rtol=0.15, atol=0.05)
    assert np.allclose(O.flash_attn_fast(q, k, v, scale, True), causal, rtol=1e-5, atol=1e-6)
    assert np.all(np.abs(np.diagonal(causal[0, 0])) > 0.0)


def test_column_major_conventions():
    """Head split f = h + H*d, GQA q -> q mod KV, RoPE pairs (i, i + D/2): consequences of the
    reference's column-major Reshape (src/NN.jl:274-276, 305-317, 347-354)."""
    B, S, H, D = 1, 1, 4, 8
    x = np.arange(H * D, dtype=np.float32).reshape(B, S, H * D)
    heads = O.permute(O.reshape(x, [B, S, H, D]), [1, 3, 2, 4])
    for h in range(H):
        for d in range(D):
            assert heads[0, h, 0, d] == h + H * d
    kv = np.arange(2 * 3, dtype=np.float32).reshape(1, 2, 1, 3)
    rep = O.repeat_kv(kv, 2)
    for qh in range(4):
        assert np.array_equal(rep[0, qh], kv[0, qh % 2])
    # RoPE at position 0 is the identity; at position p it rotates (i, i + D/2)
    x = np.random.default_rng(2).standard_normal((1, 1, 1, 8), dtype=np.float32)
    assert np.allclose(O.apply_rotary_embeddings(x, 0), x, atol=1e-6)
    y = O.apply_rotary_embeddings(x, 3, base=10000.0)
    inv = O.rope_inv_freqs(8, 10000.0)
    for i in range(4):
        a = 3 * inv[i]
        assert np.allclose(y[0, 0, 0, i], x[0, 0, 0, i] * np.cos(a) - x[0, 0, 0, i + 4] * np.sin(a), atol=1e-5)
        assert np.allclose(y[0, 0, 0, i + 4], x[0, 0, 0, i] * np.sin(a) + x[0, 0, 0, i + 4] * np.cos(a), atol=1e-5)


def test_cached_decode_equals_full_recompute():
    """The KV-cached oracle is the same function as the reference's only defined generation
    (whole prefix re-run with prev_seq = 0, examples/llama.jl:39-80)."""
    for name in ("small_llama", "tiny_gqa128", "tiny_gqa96"):
        cfg = O.CONFIGS[name]
        w = O.synth_llama_weights(cfg, seed=3)
        prompt = O.synth_tokens(3, 1000, (2, 7), cfg["vocab"])
        tok_a, log_a = O.greedy_generate_recompute(prompt, w, cfg, 4)
        tok_b, log_b = O.CachedLlama(w, cfg, 2, 16).greedy(prompt, 4)
        assert np.array_equal(tok_a, tok_b)
        assert np.abs(log_a - log_b).max() < 2e-5


def test_generator_golden_values():
    """The counter-based generator is shared bit for bit with the CUDA fill kernels; these values
    pin the host side (tests/golden/synth_golden.json was written by tests/golden/make_golden.py)."""
    import json, os
    path = os.path.join(os.path.dirname(__file__), "golden", "synth_golden.json")
    g = json.load(open(path))
    got = O.synth_normal(g["seed"], g["tensor_id"], (g["n"],), g["sigma"])
    assert got.view(np.uint32).tolist() == g["bits"]
    assert O.synth_tokens(g["seed"], g["tensor_id"], (8,), 1024).tolist() == g["tokens"]


def test_readme_quick_start():
    # README.md:10-34: c = matmul(a [3,1], b [1,4]) with a = [1;2;3], b = [1 2 3 4] -- the outer product, through the
    # oracle's batch_matmul and through the graph builders evaluated node by node
    import luminal_jl_b200 as L
    from plan_eval import eval_graph
    a_val = np.array([[1.0], [2.0], [3.0]], np.float32)
    b_val = np.array([[1.0, 2.0, 3.0, 4.0]], np.float32)
    want = np.array([[1, 2, 3, 4], [2, 4, 6, 8], [3, 6, 9, 12]], np.float32)
    assert np.array_equal(O.matmul(a_val, b_val), want)
    g = L.Graph()
    a, b = L.tensor(g, (3, 1)), L.tensor(g, (1, 4))
    c = L.graph.matmul(a, b)
    (res,) = eval_graph(g, {a.id: a_val, b.id: b_val}, [c.id])
    assert res.shape == (3, 4) and np.array_equal(res, want)

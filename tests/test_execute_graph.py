"""Op-by-op path: the graph API mirror + execute()/compile() on the B200 device against the CPU
oracle, including the reference's own known-answer cases run through the device."""
import ctypes as C

import numpy as np
import pytest

import luminal_oracle as O

pytestmark = pytest.mark.gpu


def test_reference_known_answers_on_device(lib_built, device):
    L = lib_built
    G, nn = L.graph, L.nn
    # tests/test_nn_layers.jl:8-32 (Linear with bias on a 2-D input)
    g = L.Graph()
    x = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    w = np.array([[1, 2, 3, 4], [5, 6, 7, 8], [9, 10, 11, 12]], np.float32)
    b = np.array([0.1, 0.2, 0.3, 0.4], np.float32)
    a = L.tensor(g, x.shape)
    lin = nn.Linear(3, 4, g, bias=True)
    res = L.execute(g, lin(a).id, {a.id: x, lin.weight.id: w.T.copy(), lin.bias.id: b}, device)
    assert np.allclose(res, x @ w + b)
    # tests/test_nn_layers.jl:34-52 (Embedding rows [2, 0])
    g = L.Graph()
    m = np.array([[1, 2, 3, 4], [5, 6, 7, 8], [9, 10, 11, 12]], np.float32)
    idx = L.tensor(g, [2])
    emb = nn.Embedding(3, 4, g)
    res = L.execute(g, emb(idx).id, {idx.id: np.array([2, 0], np.float32), emb.weight.id: m}, device)
    assert np.array_equal(res, [[9, 10, 11, 12], [1, 2, 3, 4]])
    # tests/test_nn_layers.jl:54-69 (LayerNorm: mean 0, rms 1)
    g = L.Graph()
    a = L.tensor(g, [2, 3])
    ln = nn.LayerNorm(3, g, weight=False, bias=False)
    res = L.execute(g, ln(a).id, {a.id: np.array([[1, 2, 3], [4, 5, 6]], np.float32)}, device)
    assert np.allclose(res.sum(axis=1) / 3, 0, atol=1e-5) and np.allclose(np.sqrt((res ** 2).sum(axis=1) / 3), 1, atol=1e-5)
    # tests/test_gpu_execution.jl:8-24 and :54-76
    g = L.Graph()
    a, b_, c = (L.tensor(g, [3]) for _ in range(3))
    out = a * b_ + c
    fma = G.add_op(g, G.FusedMulAdd(), [(a.id, 0, a.shape), (b_.id, 0, b_.shape), (c.id, 0, c.shape)], [3])
    far = G.add_op(g, G.FusedAddReLU(), [(a.id, 0, a.shape), (c.id, 0, c.shape)], [3])
    vals = {a.id: [1, 2, 3], b_.id: [4, 5, 6], c.id: [7, 8, -9]}
    res = L.execute(g, [out.id, fma.id, far.id], vals, device)
    assert np.array_equal(res[out.id], [11, 18, 9]) and np.array_equal(res[fma.id], [11, 18, 9])
    assert np.array_equal(res[far.id], [8, 10, 0])
    # tests/test.jl:17-43 (matmul + add, exact)
    g = L.Graph()
    a, b_, c = (L.tensor(g, [2, 2]) for _ in range(3))
    e = G.matmul(a, b_) + c
    res = L.execute(g, e.id, {a.id: [[1, 2], [3, 4]], b_.id: [[5, 6], [7, 8]], c.id: np.ones((2, 2))}, device)
    assert np.array_equal(res, [[20, 23], [44, 51]])
    # tests/test_fusion.jl:7-56 through compile(): (a+b)*c and relu(x*w+bias)
    g = L.Graph()
    a, b_, c = (L.tensor(g, [3, 3]) for _ in range(3))
    d = (a + b_) * c
    r = G.relu(a * b_ + c)
    rng = np.random.default_rng(0)
    av, bv, cv = (rng.random((3, 3), dtype=np.float32) - np.float32(0.3) for _ in range(3))
    cg = L.compile(g, device)
    bufs = cg({a.id: av, b_.id: bv, c.id: cv})
    assert np.allclose(bufs[d.id].numpy(), (av + bv) * cv)
    assert np.allclose(bufs[r.id].numpy(), np.maximum(av * bv + cv, 0))
    with pytest.raises(ValueError):
        cg({a.id: np.zeros(4, np.float32)})       # input size mismatch (src/Compiler.jl:83-88)


def test_flash_op_vs_manual_attention_graph(lib_built, device):
    """tests/test_flash_attention_verification.jl:24-94 on the device."""
    L = lib_built
    G = L.graph
    B, H, S, D = 1, 1, 8, 16
    rng = np.random.default_rng(1)
    qv, kv, vv = (rng.standard_normal((B, H, S, D), dtype=np.float32) for _ in range(3))
    for causal in (False, True):
        g = L.Graph()
        q, k, v = (L.tensor(g, [B, H, S, D]) for _ in range(3))
        scale = np.float32(1.0) / np.sqrt(np.float32(D))
        flash = G.flash_attention(q, k, v, causal=causal)
        w = G.matmul(q, G.permute(k, [1, 2, 4, 3])) * scale
        if causal:
            h = G.expand(G.arange(g, S), 1, S)
            v_idx = G.expand(G.arange(g, S), 2, S)
            mask = v_idx + np.float32(1.0) > h
            w = w + (mask * np.float32(-1.0) + np.float32(1.0)) * np.float32(-1.0e9)
        manual = G.matmul(G.softmax(w, 4), v)
        res = L.execute(g, [flash.id, manual.id], {q.id: qv, k.id: kv, v.id: vv}, device)
        if causal:
            assert np.allclose(res[flash.id], res[manual.id], rtol=0.15, atol=0.05)
        else:
            assert np.allclose(res[flash.id], res[manual.id], rtol=1e-4, atol=1e-6)
        assert np.allclose(res[flash.id], O.flash_attn_cpu(qv, kv, vv, scale, causal), rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("name,batch,seq", [("tiny_gqa128", 2, 5), ("small_llama", 1, 7)])
def test_llama_graph_op_by_op_matches_oracle(lib_built, device, name, batch, seq):
    """NN.Llama built with the mirror API and run node by node on the device (about 230 primitive
    nodes per layer) against the oracle's replay of the same op sequence."""
    L = lib_built
    cfg = O.CONFIGS[name]
    w = O.synth_llama_weights(cfg, seed=5)
    toks = O.synth_tokens(5, 1000, (batch, seq), cfg["vocab"])
    g = L.Graph()
    reg = {}
    model = L.nn.Llama(g, reg, vocab_size=cfg["vocab"], hidden=cfg["hidden"], n_layers=cfg["n_layers"],
                       n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"], intermediate=cfg["intermediate"])
    model.ROPE_BASE = cfg["rope_base"]
    inp = L.tensor(g, [batch, seq])
    out = model(inp, 0)
    inputs = {t.id: w[n] for n, t in reg.items()}
    inputs[inp.id] = toks.astype(np.float32)
    got = L.execute(g, out.id, inputs, device)
    ref = O.llama_forward(toks, w, cfg, 0)
    assert got.shape == ref.shape
    assert np.abs(got - ref).max() <= 1e-3
    assert np.array_equal(got.argmax(-1), ref.argmax(-1))


def test_primitives_match_oracle(lib_built, device):
    L = lib_built
    G = L.graph
    rng = np.random.default_rng(7)
    g = L.Graph()
    a = L.tensor(g, [2, 3, 4, 5])
    b = L.tensor(g, [4, 5])
    av = rng.standard_normal((2, 3, 4, 5), dtype=np.float32)
    bv = rng.standard_normal((4, 5), dtype=np.float32) + np.float32(2.0)
    cases = {
        "add_bcast": (a + b, O.add(av, bv)),
        "mul_scalar": (a * 3.0, O.mul(av, np.float32(3.0))),
        "mod": (a % b, O.mod(av, bv)),
        "lt": (a < b, O.less_than(av, bv)),
        "div": (a / b, O.div(av, bv)),
        "exp": (G.exp(a), O.exp(av)),
        "sin": (G.sin(a), O.sin(av)),
        "cos": (G.cos(a), O.cos(av)),
        "sqrt": (G.sqrt(b), O.sqrt(bv)),
        "log2": (G.log2(b), O.log2(bv)),
        "swish": (G.swish(a), O.swish(av)),
        "gelu": (G.gelu(a), O.gelu(av)),
        "sum2": (G.sum_(a, 2), O.sum_reduce(av, 2)),
        "sum4": (G.sum_(a, 4), O.sum_reduce(av, 4)),
        "max1": (G.max_reduce(a, 1), O.max_reduce(av, 1)),
        "softmax3": (G.softmax(a, 3), O.softmax(av, 3)),
        "permute": (G.permute(a, [3, 1, 4, 2]), O.permute(av, [3, 1, 4, 2])),
        "reshape_cm": (G.reshape(a, [6, 20]), O.reshape(av, [6, 20])),
        "reshape_cm2": (G.reshape(a, [5, 4, 6]), O.reshape(av, [5, 4, 6])),
        "expand": (G.expand(b, 2, 3), O.expand(bv, 2, 3)),
        "slice": (G.slice_along(a, 3, 1, 3), O.slice_along(av, 3, 1, 3)),
        "pad": (G.pad_along(a, 2, 1, 2), O.pad_along(av, 2, 1, 2)),
        "concat": (G.concat_along(a, a, 4), O.concat_along(av, av, 4)),
        "mean_norm": (G.mean_norm(a, 4), O.mean_norm(av, 4)),
        "std_norm": (G.std_norm(a, 4), O.std_norm(av, 4)),
        "arange": (G.arange(g, 9), O.arange(9)),
        "triu": (G.triu(g, 6, 1), O.triu(6, 1)),
        "mm4": (G.matmul(a, G.permute(a, [1, 2, 4, 3])), O.matmul(av, O.permute(av, [1, 2, 4, 3]))),
        "mm_3d2d": (G.matmul(G.reshape(a, [6, 4, 5]), G.permute(b, [2, 1])),
                    O.matmul(O.reshape(av, [6, 4, 5]), O.permute(bv, [2, 1]))),
    }
    res = L.execute(g, [t.id for t, _ in cases.values()], {a.id: av, b.id: bv}, device)
    for name, (t, ref) in cases.items():
        got = res[t.id]
        assert got.shape == np.asarray(ref).shape, name
        assert np.allclose(got, ref, rtol=2e-5, atol=2e-6), name
    # gather with an out-of-range id -> zeros (src/Execution.jl:587-592); broadcasting error
    g = L.Graph()
    table, ids = L.tensor(g, [5, 3]), L.tensor(g, [2, 2])
    tv = rng.standard_normal((5, 3), dtype=np.float32)
    got = L.execute(g, G.gather(table, ids).id, {table.id: tv, ids.id: [[4, 0], [7, 1]]}, device)
    assert np.array_equal(got[0], tv[[4, 0]]) and np.array_equal(got[1, 1], tv[1]) and not got[1, 0].any()
    with pytest.raises(ValueError):
        _ = L.tensor(g, [2, 3]) + L.tensor(g, [4, 3])


def test_colmajor_upload_download_roundtrip(lib_built, device):
    L = lib_built
    a = np.arange(2 * 3 * 4, dtype=np.float32).reshape(2, 3, 4)
    for dtype in (L.F32, L.BF16):
        d = device.upload(a, dtype, L.COLMAJOR)          # host image in Julia order
        assert np.array_equal(d.numpy(L.ROWMAJOR), a)
        out = d.numpy(L.COLMAJOR)
        assert out.flags.f_contiguous and np.array_equal(out, a)


def test_fused_layer_ops(lib_built, device):
    import torch
    L = lib_built
    from importlib import import_module
    _lib = import_module("luminal_jl_b200._lib")
    rng = np.random.default_rng(3)
    x = rng.standard_normal((5, 96), dtype=np.float32)
    w = rng.standard_normal(96, dtype=np.float32)
    b = rng.standard_normal(96, dtype=np.float32)
    dx, dw, db = device.upload(x), device.upload(w), device.upload(b)
    out = device.empty(x.shape)
    p = lambda a: C.c_void_p(a.ptr)
    _lib.call("lmb200_rmsnorm_scale", device.handle, p(out), p(dx), p(dw), 5, 96, 1e-5)
    assert np.allclose(out.numpy(), O.rms_norm(x, w), rtol=1e-5, atol=1e-6)
    _lib.call("lmb200_layernorm", device.handle, p(out), p(dx), p(dw), p(db), 5, 96, 1e-5)
    assert np.allclose(out.numpy(), O.layer_norm(x, w, b), rtol=1e-5, atol=1e-5)
    _lib.call("lmb200_silu_gate", device.handle, p(out), p(dx), p(dx), x.size)
    assert np.allclose(out.numpy(), O.mul(O.silu(x), x), rtol=1e-5, atol=1e-6)
    xr = rng.standard_normal((2, 3, 4, 32), dtype=np.float32)
    dxr, outr = device.upload(xr), device.empty(xr.shape)
    _lib.call("lmb200_rope", device.handle, p(outr), p(dxr), 2, 3, 4, 32, 17, 10000.0)
    assert np.allclose(outr.numpy(), O.apply_rotary_embeddings(xr, 17, 10000.0), rtol=1e-4, atol=1e-5)
    ids = torch.empty(5, dtype=torch.int32, device="cuda")
    _lib.call("lmb200_argmax", device.handle, C.c_void_p(ids.data_ptr()), p(dx), 5, 96)
    device.sync()
    assert np.array_equal(ids.cpu().numpy(), x.argmax(axis=1))


# float32 with head_dim 64 / 96 / 128 runs on the tensor cores with bf16 hi + lo operands (three MMAs per product):
# 1e-4 is the reference's own pin for this op (tests/test_flash_attention_verification.jl:24-50); head_dim 32 stays on
# the CUDA-core kernel
@pytest.mark.parametrize("dtype,tol", [("f32", 1e-4), ("bf16", 2e-2)])
@pytest.mark.parametrize("shape", [(2, 3, 200, 64), (1, 2, 333, 128), (1, 4, 77, 32), (1, 1, 130, 96), (1, 2, 64, 128), (2, 1, 1, 64)])
@pytest.mark.parametrize("causal", [False, True])
def test_flash_attention_op(lib_built, device, dtype, tol, shape, causal):
    import torch
    L = lib_built
    from importlib import import_module
    _lib = import_module("luminal_jl_b200._lib")
    B, H, S, D = shape
    q, k, v = (O.synth_normal(9, i, shape, 1.0) for i in range(3))
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    if dtype == "bf16":
        q, k, v = O.bf16_round(q), O.bf16_round(k), O.bf16_round(v)
    tq, tk, tv = (torch.tensor(a, device="cuda").to(tdt).contiguous() for a in (q, k, v))
    out = torch.empty_like(tq)
    torch.cuda.synchronize()
    scale = 1.0 / np.sqrt(D)
    _lib.call("lmb200_flash_attention", device.handle, C.c_void_p(out.data_ptr()), C.c_void_p(tq.data_ptr()),
              C.c_void_p(tk.data_ptr()), C.c_void_p(tv.data_ptr()), _lib.BF16 if dtype == "bf16" else _lib.F32,
              B, H, S, D, scale, int(causal))
    device.sync()
    ref = O.flash_attn_fast(q, k, v, scale, causal)
    got = out.float().cpu().numpy()
    assert np.abs(got - ref).max() / np.abs(ref).max() <= tol


def test_fused_session_from_the_same_graph_inputs(lib_built, device):
    """One nn.Llama, one registry, one input dict: run op by op with execute() (recomputing the whole
    prefix per token, as the reference generates) and through compile_fused() with the KV cache."""
    L = lib_built
    cfg = O.CONFIGS["tiny_gqa128"]
    w = O.synth_llama_weights(cfg, seed=8)
    batch, seq, steps = 2, 6, 3
    toks = O.synth_tokens(8, 1000, (batch, seq), cfg["vocab"])
    g, reg = L.Graph(), {}
    model = L.nn.Llama(g, reg, vocab_size=cfg["vocab"], hidden=cfg["hidden"], n_layers=cfg["n_layers"],
                       n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"], intermediate=cfg["intermediate"])
    model.ROPE_BASE = cfg["rope_base"]
    weights = {t.id: w[n] for n, t in reg.items()}
    sess = L.compile_fused(model, reg, weights, device, batch=batch, max_ctx=32)
    logits = sess.prefill(toks.astype(np.int32))
    seqs = toks.copy()
    for step in range(steps):
        gi, ri = L.Graph(), {}
        mi = L.nn.Llama(gi, ri, vocab_size=cfg["vocab"], hidden=cfg["hidden"], n_layers=cfg["n_layers"],
                        n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"], intermediate=cfg["intermediate"])
        mi.ROPE_BASE = cfg["rope_base"]
        inp = L.tensor(gi, list(seqs.shape))
        out = mi(inp, 0)
        inputs = {t.id: w[n] for n, t in ri.items()}
        inputs[inp.id] = seqs.astype(np.float32)
        full = L.execute(gi, out.id, inputs, device)[:, -1, :]
        assert np.abs(full - logits).max() <= 1e-3
        nxt = full.argmax(-1)
        assert np.array_equal(nxt, logits.argmax(-1))
        seqs = np.concatenate([seqs, nxt[:, None]], axis=1)
        _, logits = sess.decode_step(nxt.astype(np.int32), want_logits=True)
    sess.close()

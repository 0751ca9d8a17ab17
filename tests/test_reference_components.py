"""The reference's own component tests restated on this backend, testset for testset, with the reference's sizes:
tests/test_llama.jl:23-113 (RMSNorm, Mlp, RoPE, Attention, top-level Llama), tests/test_whisper_components.jl:47-118
(Conv1D, AudioEncoder, TextDecoder at the whisper-tiny constants of src/Whisper.jl:195-206) and tests/test_kv_cache.jl
(KVCacheState, IncrementalDecodeGraph, _kv_scatter, the cached attention graphs, decode_step! over three steps).

The reference asserts shapes, the absence of NaNs and one RoPE property on random inputs.  Here each graph is built
by the graph builders, evaluated node by node with the oracle's primitives on the CPU (the reference's assertions,
plus the values against the oracle's direct restatement of the layer), and, on the GPU, run through execute() and
compile() against that CPU evaluation."""
import numpy as np
import pytest

import luminal_jl_b200 as L
import luminal_oracle as O
import whisper_oracle as W
from luminal_jl_b200 import graph as G, nn as NN, whisper as WG
from plan_eval import eval_graph

TINY = dict(d_model=384, heads=6, enc_layers=4, dec_layers=4, ffn=1536, vocab=51864, n_mels=80, max_positions=448)
TOL = 2e-4          # float32 graphs, device against the CPU evaluation (relative to the largest magnitude)


def fill_inputs(graph, given, seed):
    """execute_with_random_inputs of tests/test_llama.jl:7-21: random data for every input tensor not given."""
    inputs = dict(given)
    for nid, node in enumerate(graph.nodes, start=1):
        if isinstance(node.op, G.Function) and node.op.name == "InputTensor" and nid not in inputs and (nid, 1) not in graph.tensors:
            inputs[nid] = O.synth_normal(seed, nid, graph.shapes[nid - 1], 0.05)
    return inputs


def close(a, b, tol=TOL):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return a.shape == b.shape and np.abs(a - b).max() <= tol * max(1.0, np.abs(b).max())


# ----------------------------------------------------------------------------------------------------------------
# graphs of tests/test_llama.jl; each returns (graph, output id, inputs, the oracle's value)
# ----------------------------------------------------------------------------------------------------------------
def case_rmsnorm():
    g = G.Graph()
    ln = NN.RMSNorm(128, g, epsilon=1e-5)
    x = G.tensor(g, [2, 128])
    out = ln(x)
    inputs = fill_inputs(g, {x.id: O.synth_normal(1, 900, (2, 128), 1.0)}, 1)
    return g, out.id, inputs, O.rms_norm(inputs[x.id], inputs[ln.weight.id], 1e-5), (2, 128)


def case_mlp():
    g = G.Graph()
    mlp = NN.Mlp(128, 256, g)
    x = G.tensor(g, [2, 128])
    out = mlp(x)
    inputs = fill_inputs(g, {x.id: O.synth_normal(2, 900, (2, 128), 1.0)}, 2)
    want = O.mlp(inputs[x.id], inputs[mlp.gate_proj.weight.id], inputs[mlp.up_proj.weight.id], inputs[mlp.down_proj.weight.id])
    return g, out.id, inputs, want, (2, 128)


def case_rope():
    g = G.Graph()
    x = G.tensor(g, [1, 4, 10, 32])
    out = NN.apply_rotary_embeddings(x, 0)
    inputs = {x.id: O.synth_normal(3, 900, (1, 4, 10, 32), 1.0)}
    return g, out.id, inputs, O.apply_rotary_embeddings(inputs[x.id], 0), (1, 4, 10, 32)


def case_attention():
    g = G.Graph()
    sa = NN.SelfAttention(128, 4, 4, g)
    x = G.tensor(g, [1, 8, 128])
    out = sa(x, 0)
    inputs = fill_inputs(g, {x.id: O.synth_normal(4, 900, (1, 8, 128), 1.0)}, 4)
    want = O.self_attention(inputs[x.id], inputs[sa.q_proj.weight.id], inputs[sa.k_proj.weight.id], inputs[sa.v_proj.weight.id],
                            inputs[sa.o_proj.weight.id], 4, 4, 0)
    return g, out.id, inputs, want, (1, 8, 128)


def case_llama():
    g, reg = G.Graph(), {}
    cfg = dict(n_layers=2, hidden=64, n_heads=4, n_kv_heads=4, intermediate=128, vocab=1000, eps=1e-5, rope_base=NN.Llama.ROPE_BASE)
    llama = NN.Llama(g, reg, vocab_size=1000, hidden=64, n_layers=2, n_heads=4, n_kv_heads=4, intermediate=128)
    x = G.tensor(g, [1, 8])
    out = llama(x, 0)
    tokens = O.synth_tokens(5, 900, (1, 8), 1000)
    w = O.synth_llama_weights(cfg, seed=5)
    inputs = {t.id: w[name] for name, t in reg.items()}
    inputs[x.id] = tokens.astype(np.float32)
    return g, out.id, inputs, O.llama_forward(tokens, w, cfg, 0), (1, 8, 1000)


LLAMA_CASES = dict(rmsnorm=case_rmsnorm, mlp=case_mlp, rope=case_rope, attention=case_attention, llama=case_llama)


@pytest.mark.parametrize("name", list(LLAMA_CASES))
def test_llama_components_on_the_cpu(name):
    g, out_id, inputs, want, shape = LLAMA_CASES[name]()
    (res,) = eval_graph(g, inputs, [out_id])
    assert res.shape == shape                                    # @test size(result) == ...
    assert not np.isnan(res).any()                               # @test all(!isnan, result)
    assert close(res, want, 1e-5)
    if name == "rope":                                           # tests/test_llama.jl:69-72: the pair keeps its norm
        x = next(iter(inputs.values()))
        assert abs(np.hypot(x[0, 0, 0, 0], x[0, 0, 0, 1]) - np.hypot(res[0, 0, 0, 0], res[0, 0, 0, 1])) <= 1e-5
        # ... and, at every position, the pair the column-major split really rotates: (d, d + head_dim / 2)
        assert np.allclose(np.hypot(x[..., :16], x[..., 16:]), np.hypot(res[..., :16], res[..., 16:]), atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(LLAMA_CASES))
def test_llama_components_on_the_device(lib_built, device, name):
    g, out_id, inputs, _, shape = LLAMA_CASES[name]()
    (want,) = eval_graph(g, inputs, [out_id])
    res = L.execute(g, out_id, inputs, device)
    assert res.shape == shape and not np.isnan(res).any()
    assert close(res, want)
    cg = L.compile(g, device)
    assert close(cg(inputs)[out_id].numpy(), want)


# ----------------------------------------------------------------------------------------------------------------
# tests/test_whisper_components.jl:47-118
# ----------------------------------------------------------------------------------------------------------------
def conv1d_case():
    g, reg = G.Graph(), {}
    a = G.tensor(g, [1, 2, 7])
    conv = WG.Conv1D(2, 3, 3, g, reg, "conv", stride=2, padding=1)
    out = conv(a)
    a_data = np.array([[1, 2, 3, 4, 5, 6, 7], [8, 9, 10, 11, 12, 13, 14]], np.float32).reshape(1, 2, 7)
    inputs = {a.id: a_data, conv.weight.id: np.ones((3, 6), np.float32), conv.bias.id: np.full(3, 0.5, np.float32)}
    return g, out.id, inputs


def test_conv1d_on_the_cpu():
    g, out_id, inputs = conv1d_case()
    (res,) = eval_graph(g, inputs, [out_id])
    assert res.shape == (1, 3, 4)                                # @test size(res) == (1, 3, 4)
    # all-ones weights: every output channel is the sum of the zero-padded stride-2 windows of both rows + 0.5
    assert np.array_equal(res, np.broadcast_to(np.array([20.5, 39.5, 51.5, 40.5], np.float32), (1, 3, 4)))


def encoder_case():
    g, reg = G.Graph(), {}
    enc = WG.AudioEncoder(g, reg, d_model=TINY["d_model"], heads=TINY["heads"], layers=TINY["enc_layers"], ffn=TINY["ffn"],
                          n_mels=TINY["n_mels"])
    a = G.tensor(g, [1, 80, 50])
    out = enc(a)
    w = W.synth_weights(dict(TINY, vocab=8, dec_layers=1), seed=6)       # the encoder has no use for the decoder's tables
    inputs = {t.id: w[name] for name, t in reg.items()}
    inputs[a.id] = O.synth_normal(6, 900, (1, 80, 50), 1.0)
    return g, out.id, inputs, w, a.id


def decoder_case():
    g, reg = G.Graph(), {}
    dec = WG.TextDecoder(g, reg, d_model=TINY["d_model"], heads=TINY["heads"], layers=TINY["dec_layers"], ffn=TINY["ffn"],
                         vocab=TINY["vocab"], max_positions=TINY["max_positions"])
    enc_out = G.tensor(g, [1, 25, 384])
    tokens = G.tensor(g, [1, 10])
    out = dec(enc_out, tokens)
    w = W.synth_weights(dict(TINY, vocab=8), seed=7)
    # the 51864-row table from NumPy's generator: the counter-based one is slow at 20 M elements and nothing here
    # compares with the device generator
    w["model.decoder.embed_tokens.weight"] = (np.random.default_rng(7).standard_normal((TINY["vocab"], TINY["d_model"]), dtype=np.float32)
                                              * np.float32(0.02))
    inputs = {t.id: w[name] for name, t in reg.items()}
    inputs[enc_out.id] = O.synth_normal(7, 900, (1, 25, 384), 1.0)
    inputs[tokens.id] = np.ones((1, 10), np.float32)             # "dummy tokens", tests/test_whisper_components.jl:102
    return g, out.id, inputs, w, enc_out.id, tokens.id


def test_audio_encoder_on_the_cpu():
    g, out_id, inputs, w, a_id = encoder_case()
    (res,) = eval_graph(g, inputs, [out_id])
    assert res.shape == (1, 25, 384)                             # @test size(res) == (1, 25, 384)
    assert close(res, W.encoder(inputs[a_id], w, TINY), 1e-5)


def test_text_decoder_on_the_cpu():
    g, out_id, inputs, w, enc_id, tok_id = decoder_case()
    (res,) = eval_graph(g, inputs, [out_id])
    assert res.shape == (1, 10, 51864)                           # @test size(res) == (1, 10, 51864)
    assert close(res, W.decoder_full(inputs[tok_id].astype(np.int64), inputs[enc_id], w, TINY), 1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["conv1d", "encoder", "decoder"])
def test_whisper_components_on_the_device(lib_built, device, which):
    g, out_id, inputs = {"conv1d": conv1d_case, "encoder": encoder_case, "decoder": decoder_case}[which]()[:3]
    (want,) = eval_graph(g, inputs, [out_id])
    res = L.execute(g, out_id, inputs, device)
    assert res.shape == want.shape and close(res, want)
    assert close(L.compile(g, device)(inputs)[out_id].numpy(), want)


# ----------------------------------------------------------------------------------------------------------------
# tests/test_kv_cache.jl (TEST_BATCH 1, TEST_ENC_SEQ 8, TEST_MAX_SEQ 10, TEST_STEPS 3)
# ----------------------------------------------------------------------------------------------------------------
BATCH, ENC_SEQ, MAX_SEQ, STEPS = 1, 8, 10, 3
HEADS, HEAD_DIM, D_MODEL = TINY["heads"], TINY["d_model"] // TINY["heads"], TINY["d_model"]


def test_kv_cache_state_allocation():                            # tests/test_kv_cache.jl:12-27
    cache = WG.KVCacheState(BATCH, 1, HEADS, HEAD_DIM, ENC_SEQ, max_seq=MAX_SEQ)
    assert cache.step_pos == 0 and cache.max_seq == MAX_SEQ
    assert len(cache.self_cache) == 1 and len(cache.cross_cache) == 1
    sk, sv = cache.self_cache[0]
    assert sk.shape == (BATCH, HEADS, MAX_SEQ, HEAD_DIM) and not sk.any() and sv.shape == sk.shape
    ck, cv = cache.cross_cache[0]
    assert ck.shape == (BATCH, HEADS, ENC_SEQ, HEAD_DIM) and cv.shape == ck.shape


def tiny_decoder(g, reg, layers=None):
    return WG.TextDecoder(g, reg, d_model=D_MODEL, heads=HEADS, layers=layers or TINY["dec_layers"], ffn=TINY["ffn"], vocab=TINY["vocab"],
                          max_positions=TINY["max_positions"])


def test_incremental_decode_graph_structure():                   # tests/test_kv_cache.jl:29-53
    g = G.Graph()
    idg = WG.build_decode_step(tiny_decoder(g, {}), g, ENC_SEQ, 0, max_seq=MAX_SEQ, batch=BATCH)
    assert idg.token_input_id > 0 and idg.logits_id > 0 and idg.step_pos == 0
    assert len(idg.cross_k_ids) == len(idg.self_k_ids) == len(idg.new_self_k_ids) == TINY["dec_layers"]
    assert g.shapes[idg.logits_id - 1] == (BATCH, 1, TINY["vocab"])


@pytest.mark.parametrize("step_pos", [0, 1, 3])
def test_kv_scatter_places_the_slot(step_pos):                   # tests/test_kv_cache.jl:55-72
    g = G.Graph()
    past, new = G.tensor(g, [1, 1, 4, 2]), G.tensor(g, [1, 1, 1, 2])
    upd = WG._kv_scatter(past, new, step_pos)
    assert upd.shape[2] == 4                                     # @test realized_dims(updated.shape)[3] == 4
    p = np.arange(8, dtype=np.float32).reshape(1, 1, 4, 2) + 1
    n = np.array([-1, -2], np.float32).reshape(1, 1, 1, 2)
    (res,) = eval_graph(g, {past.id: p, new.id: n}, [upd.id])
    want = p.copy()
    want[0, 0, step_pos] = n[0, 0, 0]
    assert np.array_equal(res, want)


def test_cached_attention_graph_shapes():                        # tests/test_kv_cache.jl:74-115
    g, reg = G.Graph(), {}
    sa = WG.WhisperSelfAttention(D_MODEL, HEADS, g, reg, "test.attn")
    x = G.tensor(g, [BATCH, 1, D_MODEL])
    past_k, past_v = (G.tensor(g, [BATCH, HEADS, MAX_SEQ, HEAD_DIM]) for _ in range(2))
    out, new_k, new_v = WG.whisper_self_attn_cached(sa, x, 0, past_k, past_v)
    assert all(isinstance(t, G.GraphTensor) for t in (out, new_k, new_v))
    assert out.shape == (BATCH, 1, D_MODEL)
    assert new_k.shape[2] == MAX_SEQ and new_k.shape[3] == HEAD_DIM and new_v.shape == new_k.shape
    ca = WG.WhisperCrossAttention(D_MODEL, HEADS, g, reg, "test.cross_attn")
    enc_k, enc_v = (G.tensor(g, [BATCH, HEADS, ENC_SEQ, HEAD_DIM]) for _ in range(2))
    assert WG.whisper_cross_attn_cached(ca, x, enc_k, enc_v).shape == (BATCH, 1, D_MODEL)


@pytest.mark.gpu
@pytest.mark.parametrize("compiled", [False, True])
def test_decode_step_host_loop(lib_built, device, compiled):
    """decode_step! (src/Whisper.jl:760-801) over TEST_STEPS positions, through execute() and through compile(): one
    graph per position, the cache's self K/V replaced by each step's outputs; the logits against the oracle's cached
    decoder and, at the last step, against the un-cached TextDecoder over the whole prefix."""
    cfg = dict(TINY, dec_layers=1, vocab=2048)
    w = W.synth_weights(cfg, seed=8)
    enc_out = O.synth_normal(8, 900, (BATCH, ENC_SEQ, D_MODEL), 1.0)
    cross = W.project_cross_kv(enc_out, w, cfg)
    ref = W.CachedDecoder(w, cfg, BATCH, cross)
    cache = WG.KVCacheState(BATCH, 1, HEADS, HEAD_DIM, ENC_SEQ, max_seq=MAX_SEQ)
    tok = np.array([[3.0]], np.float32)
    fed = []
    for step in range(STEPS):
        g, reg = G.Graph(), {}
        td = WG.TextDecoder(g, reg, d_model=D_MODEL, heads=HEADS, layers=1, ffn=cfg["ffn"], vocab=cfg["vocab"], max_positions=cfg["max_positions"])
        idg = WG.build_decode_step(td, g, ENC_SEQ, step, max_seq=MAX_SEQ, batch=BATCH)
        for name, t in reg.items():
            g.tensors[(t.id, 1)] = w[name]                       # load_weights!, src/Weights.jl:60-91
        assert cache.step_pos == step
        logits = WG.decode_step(L.compile(g, device) if compiled else g, idg, cache, tok, cross, device)
        fed.append(int(tok[0, 0]))
        want = ref.step(np.array([fed[-1]]))
        assert logits.shape == (BATCH, 1, cfg["vocab"])
        assert close(logits[:, 0], want)
        tok = np.array([[float(np.argmax(want[0]))]], np.float32)
    assert cache.step_pos == STEPS
    full = W.decoder_full(np.array([fed]), enc_out, w, cfg)
    assert close(logits[:, 0], full[:, -1], 1e-3)


# ----------------------------------------------------------------------------------------------------------------
# tests/test_greedy_decode.jl: the greedy loop of src/Decoding.jl:33-136 (the tokenizer replaced by its ids)
# ----------------------------------------------------------------------------------------------------------------
TEST_CFG = W.CONFIGS["whisper_test"]
SOT_SEQUENCE = [301, 302, 303, 304]        # stand-ins for <|startoftranscript|><|en|><|transcribe|><|notimestamps|>


def reference_loop(w, cfg, enc_out, start, eot, max_len):
    """The loop of src/Decoding.jl:91-130 on the oracle's cached decoder: only the last start id is fed, at position
    len(start) - 1, over a zeroed cache."""
    ref = W.CachedDecoder(w, cfg, enc_out.shape[0], W.project_cross_kv(enc_out, w, cfg))
    tokens = list(start)
    for _ in range(max_len):
        pos = len(tokens) - 1
        if pos >= cfg["max_positions"] - 1:
            break
        ref.pos = pos
        tokens.append(int(np.argmax(ref.step(np.array([tokens[-1]]))[0])))
        if tokens[-1] == eot:
            break
    return tokens


def test_greedy_loop_start_matches_the_step_graphs():
    """The loop's first steps graph by graph (build_decode_step! at position len(start) - 1 over zeroed self K/V,
    evaluated with the oracle's primitives) against the cached oracle started at that position."""
    cfg, batch, enc_seq = TEST_CFG, 1, 8
    w = W.synth_weights(cfg, seed=12)
    enc_out = O.synth_normal(12, 900, (batch, enc_seq, cfg["d_model"]), 1.0)
    cross = W.project_cross_kv(enc_out, w, cfg)
    want = reference_loop(w, cfg, enc_out, SOT_SEQUENCE, -1, 3)
    H, D = cfg["heads"], cfg["d_model"] // cfg["heads"]
    cache = WG.KVCacheState(batch, cfg["dec_layers"], H, D, enc_seq, max_seq=cfg["max_positions"])
    tokens = list(SOT_SEQUENCE)
    for _ in range(3):
        pos = len(tokens) - 1
        g, reg = G.Graph(), {}
        td = WG.TextDecoder(g, reg, d_model=cfg["d_model"], heads=H, layers=cfg["dec_layers"], ffn=cfg["ffn"], vocab=cfg["vocab"],
                            max_positions=cfg["max_positions"])
        idg = WG.build_decode_step(td, g, enc_seq, pos, batch=batch)
        inputs = {t.id: w[name] for name, t in reg.items()}
        inputs[idg.token_input_id] = np.array([[tokens[-1]]], np.float32)
        for l in range(cfg["dec_layers"]):
            inputs[idg.cross_k_ids[l]], inputs[idg.cross_v_ids[l]] = cross[l]
            inputs[idg.self_k_ids[l]], inputs[idg.self_v_ids[l]] = cache.self_cache[l]
        out = eval_graph(g, inputs, [idg.logits_id] + idg.new_self_k_ids + idg.new_self_v_ids)
        L_ = cfg["dec_layers"]
        cache.self_cache = list(zip(out[1:1 + L_], out[1 + L_:]))
        tokens.append(int(np.argmax(out[0][0, 0])))
    assert tokens == want


@pytest.mark.gpu
def test_greedy_decode_flow(lib_built, device):
    cfg, enc_seq = TEST_CFG, 8
    w = W.synth_weights(cfg, seed=12)
    enc_out = O.synth_normal(12, 900, (1, enc_seq, cfg["d_model"]), 1.0)
    kw = dict(d_model=cfg["d_model"], heads=cfg["heads"], layers=cfg["dec_layers"], ffn=cfg["ffn"], vocab=cfg["vocab"],
              max_positions=cfg["max_positions"], device=device)
    longest = reference_loop(w, cfg, enc_out, SOT_SEQUENCE, -1, 1000)
    never = next(i for i in range(cfg["vocab"]) if i not in longest)          # an end-of-text id nobody produces
    # "Using a very small max_len for speed": max_len 5
    (ids,) = WG.greedy_decode(w, enc_out, SOT_SEQUENCE, never, max_len=5, **kw)
    assert len(ids) > 0 and ids[0] == SOT_SEQUENCE[0]            # tests/test_greedy_decode.jl:88-89
    assert ids == longest[:len(SOT_SEQUENCE) + 5]
    # the end-of-text exit: the loop stops with the step that produced it
    eot = longest[len(SOT_SEQUENCE) + 6]
    stop = longest.index(eot, len(SOT_SEQUENCE)) + 1
    (ids,) = WG.greedy_decode(w, enc_out, SOT_SEQUENCE, eot, max_len=12, **kw)
    assert ids == longest[:stop] == reference_loop(w, cfg, enc_out, SOT_SEQUENCE, eot, 12)
    # the position cap: the loop ends when the position reaches max_positions - 1
    (ids,) = WG.greedy_decode(w, enc_out, SOT_SEQUENCE, never, max_len=1000, **kw)
    assert len(longest) == cfg["max_positions"] and ids == longest
    # a batch: every sequence runs the same loop on its own encoder output
    enc2 = O.synth_normal(13, 900, (2, enc_seq, cfg["d_model"]), 1.0)
    both = WG.greedy_decode(w, enc2, SOT_SEQUENCE, never, max_len=6, **kw)
    for b in range(2):
        assert both[b] == reference_loop(w, cfg, enc2[b:b + 1], SOT_SEQUENCE, never, 6)


# ----------------------------------------------------------------------------------------------------------------
# tests/test_compilation.jl: compile(), the captured CUDA graph in the compiled graph's cache, replays
# ----------------------------------------------------------------------------------------------------------------
@pytest.mark.gpu
def test_graph_compilation_and_capture(lib_built, device):
    rng = np.random.default_rng(0)
    g = G.Graph()
    a, b = G.tensor(g, [3, 3]), G.tensor(g, [3, 3])
    c = a + b
    exec_fn = L.compile(g, device)
    a_val, b_val = rng.random((3, 3), np.float32), rng.random((3, 3), np.float32)
    assert np.allclose(exec_fn({a.id: a_val, b.id: b_val}, device)[c.id].numpy(), a_val + b_val)
    assert exec_fn.cache.get("cuda_exec") is not None            # @test haskey(exec_fn.cache, :cuda_exec)
    # every later call is one replay of that graph, on the new inputs
    before = device.launch_count()
    a2, b2 = rng.random((3, 3), np.float32), rng.random((3, 3), np.float32)
    assert np.allclose(exec_fn({a.id: a2, b.id: b2}, device)[c.id].numpy(), a2 + b2)
    assert device.launch_count() - before == exec_fn.kernel_count() == 1
    exec_fn.close()
    # Mul + Add + ReLU
    g2 = G.Graph()
    x, w, bias = (G.tensor(g2, [2, 2]) for _ in range(3))
    z = G.relu((x * w) + bias)
    exec_fn2 = L.compile(g2, device)
    for _ in range(3):
        xv, wv, bv = rng.random((2, 2), np.float32), rng.random((2, 2), np.float32), rng.random((2, 2), np.float32) - 0.5
        got = exec_fn2({x.id: xv, w.id: wv, bias.id: bv}, device)[z.id].numpy()
        assert np.allclose(got, np.maximum(xv * wv + bv, 0))
    exec_fn2.close()


@pytest.mark.gpu
def test_captured_llama_graph_replays_on_new_tokens(lib_built, device):
    """The 2-layer Llama of tests/test_llama_compiled.jl: the first call runs step by step, the later ones replay the
    recorded graph; each against execute() on the same inputs, and against an uncaptured compile()."""
    g, out_id, inputs, _, shape = case_llama()
    tok_id = next(i for i, v in inputs.items() if v.shape == (1, 8))
    cg, plain = L.compile(g, device), L.compile(g, device, capture=False)
    for seed in range(3):
        inputs[tok_id] = O.synth_tokens(40 + seed, 900, (1, 8), 1000).astype(np.float32)
        want = L.execute(g, out_id, inputs, device)
        got = cg(inputs)[out_id].numpy()
        assert got.shape == shape and np.array_equal(got, plain(inputs)[out_id].numpy())
        assert close(got, want)
        assert cg.cache.get("cuda_exec") is not None and "cuda_exec" not in plain.cache
    cg.close()


@pytest.mark.gpu
def test_capture_with_flash_attention_and_refused_calls(lib_built, device):
    """A graph with the float32 FlashAttentionOp (its scratch is sized by the first, unrecorded call) replays; calls
    that cannot be recorded are refused with an error during a capture and the context works on afterwards."""
    g = G.Graph()
    q, k, v = (G.tensor(g, [1, 2, 128, 64]) for _ in range(3))
    out = G.flash_attention(q, k, v, causal=True) * np.float32(2.0)
    cg = L.compile(g, device)
    for seed in range(3):
        vals = {t.id: O.synth_normal(50 + seed, t.id, t.shape, 1.0) for t in (q, k, v)}
        want = 2.0 * O.flash_attn_fast(vals[q.id], vals[k.id], vals[v.id], 1.0 / 8.0, True)
        assert np.abs(cg(vals)[out.id].numpy() - want).max() <= 1e-3
    assert cg.cache.get("cuda_exec") is not None
    # a larger call makes the scratch grow while the recorded graph still reads the old block: both keep working
    g2 = G.Graph()
    q2, k2, v2 = (G.tensor(g2, [1, 2, 256, 64]) for _ in range(3))
    out2 = G.flash_attention(q2, k2, v2, causal=False)
    vals2 = {t.id: O.synth_normal(60, t.id, t.shape, 1.0) for t in (q2, k2, v2)}
    want2 = O.flash_attn_fast(vals2[q2.id], vals2[k2.id], vals2[v2.id], 1.0 / 8.0, False)
    assert np.abs(L.execute(g2, out2.id, vals2, device) - want2).max() <= 1e-3
    assert np.abs(cg(vals)[out.id].numpy() - want).max() <= 1e-3
    cg.close()

    def bad():
        device.upload(np.zeros(4, np.float32))                   # a host copy: cannot be recorded
    with pytest.raises(L.LuminalB200Error):
        device.capture(bad)
    cache = {}
    L.device.execute_with_capture(device, bad, cache)            # runs it, then finds it cannot be recorded
    assert cache["cuda_exec"] is None and "capture" in cache["cuda_exec_error"]
    x = device.upload(np.arange(6, dtype=np.float32))
    assert np.array_equal(x.numpy(), np.arange(6, dtype=np.float32))
    # a session call inside a recording is refused too, and the session is usable afterwards
    cfg = O.CONFIGS["tiny_gqa128"]
    model = L.Model(device, n_layers=cfg["n_layers"], hidden=cfg["hidden"], n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"],
                    intermediate=cfg["intermediate"], vocab=cfg["vocab"], eps=cfg["eps"], rope_base=cfg["rope_base"], dtype="f32")
    model.init_random(1, 0.02)
    sess = L.Session(model, 1, 8)
    with pytest.raises(L.LuminalB200Error, match="cannot be recorded"):
        device.capture(lambda: sess.decode_step(np.zeros(1, np.int32)))
    assert sess.position() == 0
    sess.decode_step(np.zeros(1, np.int32))
    assert sess.position() == 1
    sess.close(); model.close()
    # misuse of the entry points is an error, not a fault
    import ctypes as C
    from luminal_jl_b200 import _lib
    h = C.c_uint64(0)
    with pytest.raises(L.LuminalB200Error, match="no capture is open"):
        _lib.call("lmb200_capture_end", device.handle, C.byref(h))
    with pytest.raises(L.LuminalB200Error, match="invalid graph handle"):
        _lib.call("lmb200_graph_launch", device.handle, C.c_uint64(0))

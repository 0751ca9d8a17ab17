"""The node-list text form and the structural matcher: a graph built by the nn mirror of src/NN.jl is
exported, read back with no model object or weight names, and recognised; graphs that deviate are refused.
The GPU case runs the recognised graph through the fused session and op by op, and compares."""
import json

import numpy as np
import pytest

import luminal_jl_b200 as L
from luminal_jl_b200 import graph as G, match as M, nn


def build(cls=nn.Llama, seq=4, batch=2, kv=2, layers=3, prev_seq=0, hidden=32, heads=4, inter=48, vocab=64, base=None):
    g, reg = G.Graph(), {}
    model = cls(g, reg, vocab_size=vocab, hidden=hidden, n_layers=layers, n_heads=heads, n_kv_heads=kv, intermediate=inter)
    if base is not None:
        model.ROPE_BASE = base
    tok = G.tensor(g, [batch, seq])
    out = model(tok, prev_seq)
    return g, reg, tok, out


@pytest.mark.parametrize("cls,seq,kv,base", [(nn.Llama, 5, 2, 500000.0), (nn.Phi3, 1, 4, 10000.0), (nn.Llama, 3, 1, 500000.0),
                                             (nn.Llama, 2, 4, 1000000.0)])
def test_roundtrip_and_match(cls, seq, kv, base):
    g, reg, tok, out = build(cls, seq=seq, kv=kv, base=base)
    text = json.dumps(M.export_graph(g))
    g2 = M.import_graph(text)
    assert g2.nodes == g.nodes and g2.shapes == g.shapes
    m = M.match_decoder(g2, out.id)
    assert (m.n_layers, m.hidden, m.n_heads, m.n_kv_heads, m.head_dim, m.intermediate, m.vocab) == (3, 32, 4, kv, 8, 48, 64)
    assert (m.batch, m.seq, m.prev_seq, m.tokens) == (2, seq, 0, tok.id)
    assert m.rope_base == base and np.float32(m.eps) == np.float32(1e-5)
    assert m.weights == {name: t.id for name, t in reg.items()}


def test_prev_seq_is_recovered_and_refused_by_compile():
    g, _, _, out = build(seq=2, prev_seq=7)
    assert M.match_decoder(g, out.id).prev_seq == 7
    with pytest.raises(M.MatchError, match="prev_seq"):
        M.compile_b200(g, out.id, {})


def test_import_rejects_malformed_lists():
    g, _, _, _ = build(layers=1)
    doc = M.export_graph(g)
    bad = json.loads(json.dumps(doc))
    bad["nodes"][5]["op"] = "Tanh"
    with pytest.raises(ValueError, match="unknown op"):
        M.import_graph(bad)
    bad = json.loads(json.dumps(doc))
    k = next(i for i, n in enumerate(bad["nodes"]) if n["inputs"])
    bad["nodes"][k]["inputs"][0][0] = len(bad["nodes"]) + 3
    with pytest.raises(ValueError, match="earlier node"):
        M.import_graph(bad)
    with pytest.raises(ValueError, match="node list"):
        M.import_graph({"nodes": []})


def _mutate(g, pick, new_op):
    """Replaces the op of the first node (searching from the end) for which pick(op) is true."""
    for i in range(len(g.nodes) - 1, -1, -1):
        if pick(g.nodes[i].op):
            g.nodes[i] = G.Node(new_op(g.nodes[i].op), g.nodes[i].inputs)
            return i + 1
    raise AssertionError("nothing to mutate")


@pytest.mark.parametrize("pick,new_op", [
    (lambda o: isinstance(o, G.Exp2), lambda o: G.Log2()),                                       # another activation / softmax
    (lambda o: isinstance(o, G.Constant) and o.value == -1e9, lambda o: G.Constant(-1e4)),       # another mask value
    (lambda o: isinstance(o, G.Sin), lambda o: G.Cos()),                                         # another rotation
    (lambda o: isinstance(o, G.SumReduce) and o.dim == 3, lambda o: G.MaxReduce(3)),             # not an RMS
    (lambda o: isinstance(o, G.Permute) and o.dims == (2, 1), lambda o: G.Permute((1, 2))),      # weight not transposed
    (lambda o: isinstance(o, G.Constant) and abs(o.value - 8 ** -0.5) < 1e-6, lambda o: G.Constant(0.5)),   # another score scale
    (lambda o: isinstance(o, G.Slice), lambda o: G.Slice(o.ranges[:-1] + ((0, 2),))),            # another pair split
])
def test_deviating_graphs_are_refused(pick, new_op):
    g, _, _, out = build(seq=3)
    _mutate(g, pick, new_op)
    with pytest.raises(M.MatchError, match="node "):
        M.match_decoder(g, out.id)


def test_other_structures_are_refused():
    # a bias on the head; a mean-centring LayerNorm instead of the final RMSNorm
    g = G.Graph()
    x = G.tensor(g, [2, 16])
    with pytest.raises(M.MatchError):
        M.match_decoder(g, nn.Linear(16, 8, g, bias=True)(x).id)
    g = G.Graph()
    x = G.tensor(g, [2, 3, 16])
    head = nn.Linear(16, 8, g, bias=False)
    with pytest.raises(M.MatchError, match="Linear's MatMul"):      # the centred tensor is a sum, but not a block's
        M.match_decoder(g, head(nn.LayerNorm(16, g, bias=False)(x)).id)
    with pytest.raises(M.MatchError, match="no node"):
        M.match_decoder(g, 10 ** 6)


def test_layers_must_agree():
    g, reg = G.Graph(), {}
    a = nn.Llama(g, reg, vocab_size=64, hidden=32, n_layers=1, n_heads=4, n_kv_heads=2, intermediate=48)
    odd = nn.TransformerBlock(32, 4, 4, 48, g, reg, "model.layers.1")        # other kv head count
    tok = G.tensor(g, [1, 2])
    x = a.embedding(tok)
    x = odd(a.layers[0](x, 0, rope_base=500000.0), 0, rope_base=500000.0)
    with pytest.raises(M.MatchError, match="block 1 differs"):
        M.match_decoder(g, a.head(a.norm(x)).id)


@pytest.mark.gpu
def test_compile_b200_from_a_node_list(lib_built, device):
    """Node list as text -> import -> match -> fused session; against execute() of the same graph."""
    import luminal_oracle as O
    cfg = O.CONFIGS["tiny_gqa128"]
    w = O.synth_llama_weights(cfg, seed=21)
    batch, seq = 2, 5
    toks = O.synth_tokens(21, 1000, (batch, seq), cfg["vocab"])
    g, reg = G.Graph(), {}
    model = nn.Llama(g, reg, vocab_size=cfg["vocab"], hidden=cfg["hidden"], n_layers=cfg["n_layers"], n_heads=cfg["n_heads"],
                     n_kv_heads=cfg["n_kv_heads"], intermediate=cfg["intermediate"])
    model.ROPE_BASE = cfg["rope_base"]
    inp = G.tensor(g, [batch, seq])
    out = model(inp, 0)
    by_id = {t.id: w[n] for n, t in reg.items()}
    g2 = M.import_graph(json.dumps(M.export_graph(g)))
    sess, m = M.compile_b200(g2, out.id, by_id, device, max_ctx=16)
    assert m.rope_base == cfg["rope_base"] and m.n_layers == cfg["n_layers"]
    logits = sess.prefill(toks.astype(np.int32))
    full = L.execute(g, out.id, {**by_id, inp.id: toks.astype(np.float32)}, device)[:, -1, :]
    ref = O.llama_forward(toks, w, cfg)[:, -1, :]
    assert np.abs(full - logits).max() <= 1e-3 and np.abs(ref - logits).max() <= 1e-3
    assert np.array_equal(full.argmax(-1), logits.argmax(-1))
    sess.close()


def test_flat_node_list_and_error_code():
    """The array form the library's matcher reads (lmb200_node_list): offsets, op codes and op fields of a small
    graph; a refusal is LMB200_ENOMATCH (-8), a malformed list LMB200_ENOMATCH with the offending node named."""
    import ctypes as C
    from luminal_jl_b200 import _lib
    g = G.Graph()
    x = G.tensor(g, [2, 6])
    y = G.slice_along(G.permute(x, [2, 1]), 1, 1, G.BIG) * np.float32(3.0)
    nl = M.flatten_graph(g)
    assert nl.n_nodes == len(g.nodes)
    ops = [nl.op[i] for i in range(nl.n_nodes)]
    assert ops[0] == 25 and 18 in ops and 21 in ops and 24 in ops and ops[y.id - 1] == 9
    k = ops.index(21)
    args = [nl.arg[i] for i in range(nl.arg_off[k], nl.arg_off[k + 1])]
    assert args[:3] == [1.0, 6.0, 0.0] and args[3] >= 2.0
    assert [nl.in_node[i] for i in range(nl.in_off[y.id - 1], nl.in_off[y.id])] == [i for i, _, _ in g.nodes[y.id - 1].inputs]
    assert [nl.shape[i] for i in range(nl.shape_off[y.id - 1], nl.shape_off[y.id])] == list(g.shapes[y.id - 1])
    with pytest.raises(_lib.LuminalB200Error) as e:
        _lib.call("lmb200_match_decoder", C.byref(nl), y.id, None, None, None, 0, None, 0)
    assert e.value.code == -8 and "Linear's MatMul" in str(e.value)
    nl.in_node[nl.in_off[y.id - 1]] = y.id + 5                  # an input that is not an earlier node
    with pytest.raises(M.MatchError, match="earlier node"):
        try:
            _lib.call("lmb200_match_decoder", C.byref(nl), y.id, None, None, None, 0, None, 0)
        except _lib.LuminalB200Error as err:
            M._raise_match(err)


def test_matchers_over_a_sweep_of_shapes():
    """Seeded sweep over widths, head splits, batches, sequence lengths and positions: whatever the builders build, the
    three matchers give back exactly the configuration and the weight roles it was built with, and each refuses the
    other two builders' graphs."""
    from luminal_jl_b200 import whisper as WG
    rng = np.random.default_rng(20240)
    for _ in range(12):
        heads = int(rng.choice([1, 2, 4, 6, 8]))
        kv = int(rng.choice([k for k in (1, 2, 3, 4, 6, 8) if heads % k == 0]))
        D = int(rng.choice([2, 4, 8, 16]))
        layers, batch, seq = int(rng.integers(1, 4)), int(rng.integers(1, 5)), int(rng.integers(1, 7))
        inter, vocab, prev = int(rng.integers(3, 40)), int(rng.integers(5, 90)), int(rng.choice([0, 0, 3]))
        cls = nn.Llama if rng.integers(2) else nn.Phi3
        g, reg, tok, out = build(cls, seq=seq, batch=batch, kv=kv, layers=layers, prev_seq=prev, hidden=heads * D, heads=heads,
                                 inter=inter, vocab=vocab)
        m = M.match_decoder(g, out.id)
        assert (m.n_layers, m.hidden, m.n_heads, m.n_kv_heads, m.head_dim, m.intermediate, m.vocab) == (
            layers, heads * D, heads, kv, D, inter, vocab)
        assert (m.batch, m.seq, m.prev_seq, m.tokens, m.rope_base) == (batch, seq, prev, tok.id, cls.ROPE_BASE)
        assert m.weights == {name: t.id for name, t in reg.items()}
        for other in (M.match_whisper_step, M.match_whisper_encoder):
            with pytest.raises(M.MatchError):
                other(g, out.id)
    for _ in range(8):
        heads, D = int(rng.choice([1, 2, 4])), int(rng.choice([8, 16, 64]))
        d, layers, ffn = heads * D, int(rng.integers(1, 4)), int(rng.integers(2, 9)) * 8
        batch, enc_seq, max_seq = int(rng.integers(1, 4)), int(rng.integers(3, 30)), int(rng.integers(4, 20))
        step = int(rng.integers(0, max_seq))
        vocab, n_mels, frames = int(rng.integers(10, 80)), int(rng.integers(1, 5)) * 8, int(rng.integers(4, 50))
        g, reg = G.Graph(), {}
        td = WG.TextDecoder(g, reg, d_model=d, heads=heads, layers=layers, ffn=ffn, vocab=vocab, max_positions=max_seq + 3)
        idg = WG.build_decode_step(td, g, enc_seq, step, max_seq=max_seq, batch=batch)
        m = M.match_whisper_step(g, idg.logits_id)
        assert (m.n_layers, m.d_model, m.heads, m.ffn, m.vocab, m.max_positions) == (layers, d, heads, ffn, vocab, max_seq + 3)
        assert (m.batch, m.step_pos, m.max_seq, m.enc_seq, m.tokens) == (batch, step, max_seq, enc_seq, idg.token_input_id)
        assert m.weights == {n: t.id for n, t in reg.items() if "encoder_attn.k_proj" not in n and "encoder_attn.v_proj" not in n}
        assert (m.self_k_ids, m.new_self_v_ids) == (idg.self_k_ids, idg.new_self_v_ids)
        g, reg = G.Graph(), {}
        enc = WG.AudioEncoder(g, reg, d_model=d, heads=heads, layers=layers, ffn=ffn, n_mels=n_mels)
        mel = G.tensor(g, [batch, n_mels, frames])
        out = enc(mel)
        e = M.match_whisper_encoder(g, out.id)
        assert (e.d_model, e.heads, e.layers, e.ffn, e.n_mels, e.batch, e.frames, e.mel) == (d, heads, layers, ffn, n_mels, batch, frames, mel.id)
        assert e.weights == {n: t.id for n, t in reg.items()}
        for other in (M.match_decoder, M.match_whisper_step):
            with pytest.raises(M.MatchError):
                other(g, out.id)


def test_corrupted_node_lists_get_a_status_not_a_fault():
    """tests/fuzz_node_lists.py in a child process: 3 graphs x 150 random corruptions x 3 matchers."""
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.dirname(here), here, os.environ.get("PYTHONPATH", "")]))
    r = subprocess.run([sys.executable, os.path.join(here, "fuzz_node_lists.py"), "7", "150"], capture_output=True, text=True, env=env,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    accepted, refused = (int(x) for x in r.stdout.split()[1::2])
    assert accepted + refused == 3 * 150 * 3 and refused > accepted          # a changed list is, as a rule, not the graph

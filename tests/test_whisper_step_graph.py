"""The Whisper TextDecoder's incremental decode-step graph (src/Whisper.jl:541-742): the graph builder evaluated node
by node with the oracle's primitives against the oracle's cached decoder; the library's structural matcher on such
graphs (accepts every step position, refuses deviating graphs); and, on the GPU, a step graph compiled into a cached
session through lmb200_compile_node_list against the oracle."""
import numpy as np
import pytest

import luminal_jl_b200 as L
import luminal_oracle as O
import whisper_oracle as W
from luminal_jl_b200 import graph as G, match as M, whisper as WG
from plan_eval import run_op

CFG = W.CONFIGS["whisper_test"]


def build(step, batch, enc_seq, layers=None, max_seq=None):
    g, reg = G.Graph(), {}
    td = WG.TextDecoder(g, reg, d_model=CFG["d_model"], heads=CFG["heads"], layers=layers or CFG["dec_layers"], ffn=CFG["ffn"],
                        vocab=CFG["vocab"], max_positions=max_seq or CFG["max_positions"])
    return g, reg, WG.build_decode_step(td, g, enc_seq, step, batch=batch)


def evaluate(g, inputs, want):
    vals = {}
    for n, (node, shp) in enumerate(zip(g.nodes, g.shapes), start=1):
        op = node.op
        if isinstance(op, G.Function) and op.name == "InputTensor":
            if n in inputs:
                vals[n] = np.asarray(inputs[n], np.float32)
        elif isinstance(op, G.Constant):
            vals[n] = np.float32(op.value)
        else:
            vals[n] = run_op(op, [vals[i] for i, _, _ in node.inputs], shp)
    return [vals[i] for i in want]


def test_step_graph_matches_cached_oracle():
    """decode_step! driven as the reference drives it (src/Whisper.jl:757-801): one graph per position, the updated
    self K/V of one step fed to the next.  Batch 1, the only batch the reference's Linear bias broadcast is right for."""
    batch, enc_seq, steps = 1, 23, 4
    w = W.synth_weights(CFG, seed=4)
    enc = O.synth_normal(4, 2, (batch, enc_seq, CFG["d_model"]), 1.0)
    kv = W.project_cross_kv(enc, w, CFG)
    ref = W.CachedDecoder(w, CFG, batch, kv)
    H, D, T = CFG["heads"], CFG["d_model"] // CFG["heads"], CFG["max_positions"]
    self_k = [np.zeros((batch, H, T, D), np.float32) for _ in range(CFG["dec_layers"])]
    self_v = [np.zeros((batch, H, T, D), np.float32) for _ in range(CFG["dec_layers"])]
    tok = O.synth_tokens(4, 3, (batch,), CFG["vocab"])
    for step in range(steps):
        g, reg, idg = build(step, batch, enc_seq)
        inputs = {t.id: w[name] for name, t in reg.items()}
        inputs[idg.token_input_id] = tok.reshape(batch, 1).astype(np.float32)
        for l in range(CFG["dec_layers"]):
            inputs[idg.cross_k_ids[l]], inputs[idg.cross_v_ids[l]] = kv[l]
            inputs[idg.self_k_ids[l]], inputs[idg.self_v_ids[l]] = self_k[l], self_v[l]
        out = evaluate(g, inputs, [idg.logits_id] + idg.new_self_k_ids + idg.new_self_v_ids)
        logits = out[0][:, 0]
        self_k, self_v = out[1:1 + CFG["dec_layers"]], out[1 + CFG["dec_layers"]:]
        want = ref.step(tok)
        assert np.abs(logits - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
        assert np.array_equal(self_k[0][:, :, :step + 1], ref.k[0][:, :, :step + 1])
        tok = np.argmax(want, axis=-1)


@pytest.mark.parametrize("step", [0, 1, 9, CFG["max_positions"] - 1])
@pytest.mark.parametrize("batch", [1, 3])
def test_matcher_recognises_every_step_position(step, batch):
    g, reg, idg = build(step, batch, 31)
    m = M.match_whisper_step(g, idg.logits_id)
    assert (m.n_layers, m.d_model, m.heads, m.ffn, m.vocab, m.max_positions) == (
        CFG["dec_layers"], CFG["d_model"], CFG["heads"], CFG["ffn"], CFG["vocab"], CFG["max_positions"])
    assert (m.batch, m.step_pos, m.max_seq, m.enc_seq, m.tokens) == (batch, step, CFG["max_positions"], 31, idg.token_input_id)
    assert np.float32(m.eps) == np.float32(1e-5)
    # the cross attention's k_proj / v_proj act once on the encoder output (project_cross_kv): not part of the step
    assert m.weights == {n: t.id for n, t in reg.items() if "encoder_attn.k_proj" not in n and "encoder_attn.v_proj" not in n}
    assert (m.cross_k_ids, m.cross_v_ids, m.self_k_ids, m.self_v_ids) == (idg.cross_k_ids, idg.cross_v_ids, idg.self_k_ids, idg.self_v_ids)
    assert (m.new_self_k_ids, m.new_self_v_ids) == (idg.new_self_k_ids, idg.new_self_v_ids)


def _mutate(g, pick, new_op):
    for i in range(len(g.nodes) - 1, -1, -1):
        if pick(g.nodes[i].op):
            g.nodes[i] = G.Node(new_op(g.nodes[i].op), g.nodes[i].inputs)
            return
    raise AssertionError("nothing to mutate")


@pytest.mark.parametrize("pick,new_op", [
    (lambda o: isinstance(o, G.Constant) and abs(o.value - 0.044715) < 1e-6, lambda o: G.Constant(0.05)),        # another activation
    (lambda o: isinstance(o, G.Constant) and o.value == 2.0, lambda o: G.Constant(3.0)),                         # not a tanh
    (lambda o: isinstance(o, G.Slice) and len(o.ranges) == 4 and o.ranges[2] == (0, 4), lambda o: G.Slice(o.ranges[:2] + ((0, 3),) + o.ranges[3:])),   # a shorter context than the cache position
    (lambda o: isinstance(o, G.Pad) and o.padding[2] == (3, 0), lambda o: G.Pad(o.padding[:2] + ((2, 1),) + o.padding[3:])),   # slot written elsewhere
    (lambda o: isinstance(o, G.Slice) and len(o.ranges) == 2, lambda o: G.Slice(((5, 6), o.ranges[1]))),           # another position row
    (lambda o: isinstance(o, G.SumReduce), lambda o: G.MaxReduce(o.dim)),                                         # not a LayerNorm / softmax
    (lambda o: isinstance(o, G.Permute) and o.dims == (1, 2, 4, 3), lambda o: G.Permute((1, 2, 3, 4))),           # keys not transposed
])
def test_deviating_step_graphs_are_refused(pick, new_op):
    g, _, idg = build(3, 2, 17)
    _mutate(g, pick, new_op)
    with pytest.raises(M.MatchError, match="node "):
        M.match_whisper_step(g, idg.logits_id)


def test_other_graphs_are_refused_by_the_step_matcher():
    from luminal_jl_b200 import nn
    g, reg = G.Graph(), {}
    model = nn.Llama(g, reg, vocab_size=64, hidden=32, n_layers=1, n_heads=4, n_kv_heads=2, intermediate=48)
    out = model(G.tensor(g, [1, 3]), 0)
    with pytest.raises(M.MatchError):
        M.match_whisper_step(g, out.id)
    g, _, idg = build(2, 1, 9)
    with pytest.raises(M.MatchError):
        M.match_decoder(g, idg.logits_id)
    with pytest.raises(M.MatchError):                       # the updated cache is not a logits node
        M.match_whisper_step(g, idg.new_self_k_ids[0])


@pytest.mark.gpu
@pytest.mark.parametrize("step,batch", [(0, 1), (5, 3)])
def test_step_graph_compiles_to_cached_session(lib_built, device, step, batch):
    """compile_b200 on ONE step graph (any position) gives the cached session: its greedy tokens over 10 steps from
    position 0 equal the oracle's, with the weights and the encoder K/V taken from the graph's inputs."""
    enc_seq = 45
    w = W.synth_weights(CFG, seed=12)
    enc = O.synth_normal(12, 2, (batch, enc_seq, CFG["d_model"]), 1.0)
    kv = W.project_cross_kv(enc, w, CFG)
    g, reg, idg = build(step, batch, enc_seq)
    inputs = {t.id: w[name] for name, t in reg.items()}
    for l in range(CFG["dec_layers"]):
        inputs[idg.cross_k_ids[l]], inputs[idg.cross_v_ids[l]] = kv[l]
    sess, m = L.compile_b200(g, idg.logits_id, inputs, device=device)
    assert isinstance(m, M.WhisperStepMatch) and m.step_pos == step and sess.max_ctx == CFG["max_positions"]
    first = O.synth_tokens(12, 6, (batch,), CFG["vocab"])
    ref_tok, ref_log = W.CachedDecoder(w, CFG, batch, kv).greedy(first, 10)
    tok, logs, toks = first.astype(np.int32), [], []
    for _ in range(10):
        tok, lg = sess.decode_step(tok, want_logits=True)
        toks.append(tok.copy()); logs.append(lg)
    assert np.abs(np.stack(logs, 1) - ref_log).max() <= 1e-3
    assert np.array_equal(np.stack(toks, 1), ref_tok)
    sess.close(); sess.model.close()

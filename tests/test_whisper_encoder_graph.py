"""The Whisper AudioEncoder's graph (src/Whisper.jl:354-404) through the library's structural matcher: accepted at every
batch and length, refused when it deviates anywhere, and, on the GPU, compiled into the tensor-core encoder through
lmb200_compile_encoder_node_list against the oracle."""
import numpy as np
import pytest

import luminal_jl_b200 as L
import luminal_oracle as O
import whisper_oracle as W
from luminal_jl_b200 import graph as G, match as M, whisper as WG

CFG = W.CONFIGS["whisper_test"]


def build(batch, frames, layers=None):
    g, reg = G.Graph(), {}
    enc = WG.AudioEncoder(g, reg, d_model=CFG["d_model"], heads=CFG["heads"], layers=layers or CFG["enc_layers"], ffn=CFG["ffn"],
                          n_mels=CFG["n_mels"])
    mel = G.tensor(g, [batch, CFG["n_mels"], frames])
    return g, reg, mel, enc(mel)


@pytest.mark.parametrize("batch,frames,layers", [(1, 50, 1), (2, 61, 2), (8, 300, 3)])
def test_matcher_recognises_the_encoder(batch, frames, layers):
    g, reg, mel, out = build(batch, frames, layers)
    m = M.match_whisper_encoder(g, out.id)
    assert (m.d_model, m.heads, m.layers, m.ffn, m.n_mels) == (CFG["d_model"], CFG["heads"], layers, CFG["ffn"], CFG["n_mels"])
    assert (m.batch, m.frames, m.mel) == (batch, frames, mel.id) and np.float32(m.eps) == np.float32(1e-5)
    assert m.weights == {n: t.id for n, t in reg.items()} and len(m.weights) == 6 + 15 * layers
    inc = np.log(10000.0) / (CFG["d_model"] / 2 - 1)
    assert np.allclose(g.tensors[(m.rates, 1)], np.exp(-inc * np.arange(CFG["d_model"] // 2)), rtol=1e-6)


def _mutate(g, pick, new_op):
    for i in range(len(g.nodes) - 1, -1, -1):
        if pick(g.nodes[i].op):
            g.nodes[i] = G.Node(new_op(g.nodes[i].op), g.nodes[i].inputs)
            return
    raise AssertionError("nothing to mutate")


@pytest.mark.parametrize("pick,new_op", [
    (lambda o: isinstance(o, G.Constant) and abs(o.value - 0.044715) < 1e-6, lambda o: G.Constant(0.05)),     # another activation
    (lambda o: isinstance(o, G.Unfold), lambda o: G.Unfold(o.kernel_shape, o.stride_shape, [2])),             # a dilated stem
    (lambda o: isinstance(o, G.Pad) and len(o.padding) == 3, lambda o: G.Pad(o.padding[:2] + ((2, 0),))),     # one-sided padding
    (lambda o: isinstance(o, G.SumReduce), lambda o: G.MaxReduce(o.dim)),                                     # not a LayerNorm / softmax
    (lambda o: isinstance(o, G.Permute) and o.dims == (1, 3, 4, 2), lambda o: G.Permute((1, 3, 2, 4))),       # keys not transposed
    (lambda o: isinstance(o, G.Sin), lambda o: G.Exp2()),                                                     # not a sinusoid table
    (lambda o: isinstance(o, G.Permute) and o.dims == (1, 3, 2), lambda o: G.Permute((1, 2, 3))),             # stem output not turned token-major
])
def test_deviating_encoder_graphs_are_refused(pick, new_op):
    g, _, _, out = build(2, 40)
    _mutate(g, pick, new_op)
    with pytest.raises(M.MatchError):
        M.match_whisper_encoder(g, out.id)


def test_other_graphs_are_refused_by_the_encoder_matcher():
    from luminal_jl_b200 import nn
    g, reg = G.Graph(), {}
    model = nn.Llama(g, reg, vocab_size=64, hidden=32, n_layers=1, n_heads=4, n_kv_heads=2, intermediate=48)
    out = model(G.tensor(g, [1, 3]), 0)
    with pytest.raises(M.MatchError):
        M.match_whisper_encoder(g, out.id)
    g, reg = G.Graph(), {}
    td = WG.TextDecoder(g, reg, d_model=CFG["d_model"], heads=CFG["heads"], layers=1, ffn=CFG["ffn"], vocab=CFG["vocab"],
                        max_positions=CFG["max_positions"])
    idg = WG.build_decode_step(td, g, 9, 2)
    with pytest.raises(M.MatchError):
        M.match_whisper_encoder(g, idg.logits_id)
    g, _, mel, out = build(1, 20)
    with pytest.raises(M.MatchError):                       # the encoder's graph is neither decoder
        M.match_decoder(g, out.id)
    with pytest.raises(M.MatchError):
        M.match_whisper_step(g, out.id)
    with pytest.raises(M.MatchError):                       # an inner node is not the encoder's output
        M.match_whisper_encoder(g, out.id - 3)
    # the same encoder with a causal (decoder-style) mask in its self attention is not the encoder
    g, reg = G.Graph(), {}
    enc = WG.AudioEncoder(g, reg, d_model=CFG["d_model"], heads=CFG["heads"], layers=1, ffn=CFG["ffn"], n_mels=CFG["n_mels"])
    x = G.permute(G.gelu(enc.conv2(G.gelu(enc.conv1(G.tensor(g, [1, CFG["n_mels"], 20]))))), [1, 3, 2])
    x = x + G.expand(WG.sinusoids(CFG["d_model"], x.shape[1], g), 1, 1)
    for layer in enc.layers:
        x = x + layer.attn(layer.attn_norm(x), True)
        x = x + layer.ff2(G.gelu(layer.ff1(layer.ff_norm(x))))
    with pytest.raises(M.MatchError, match="queries x keys"):
        M.match_whisper_encoder(g, enc.post_ln(x).id)


@pytest.mark.gpu
@pytest.mark.parametrize("batch,frames", [(2, 60), (1, 301)])
def test_encoder_graph_compiles_to_the_fused_encoder(lib_built, device, batch, frames):
    w = W.synth_weights(CFG, seed=27)
    g, reg, mel, out = build(batch, frames)
    inputs = {t.id: w[name] for name, t in reg.items()}
    enc, m = M.compile_encoder_b200(g, out.id, inputs, device=device)
    assert isinstance(m, M.WhisperEncoderMatch) and (m.batch, m.frames) == (batch, frames)
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))
    x = O.synth_normal(27, 5, (batch, CFG["n_mels"], frames), 1.0)
    assert rel(enc.run(x), W.encoder(x, w, CFG)) <= 2e-2
    # the compiled encoder is not tied to the traced shape
    x2 = O.synth_normal(28, 5, (3, CFG["n_mels"], 77), 1.0)
    assert rel(enc.run(x2), W.encoder(x2, w, CFG)) <= 2e-2
    # ... and agrees with the same graph run node by node (float32) within the bf16 tolerance
    inputs[mel.id] = x
    assert rel(enc.run(x), L.execute(g, out.id, inputs, device)) <= 2e-2
    enc.close()
    # other sinusoid rates: not the graph the fused encoder stands for
    g.tensors[(m.rates, 1)] = g.tensors[(m.rates, 1)] * np.float32(1.5)
    with pytest.raises(M.MatchError, match="rate"):
        M.compile_encoder_b200(g, out.id, inputs, device=device)
    # a weight without data
    g2, reg2, _, out2 = build(batch, frames)
    some = {t.id: w[name] for name, t in reg2.items() if "conv2.bias" not in name}
    with pytest.raises(KeyError, match="conv2.bias"):
        M.compile_encoder_b200(g2, out2.id, some, device=device)

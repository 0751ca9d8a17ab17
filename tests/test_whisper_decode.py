"""Whisper decoder with cached self attention and cross attention (src/Whisper.jl:584-801) on the
GPU against the CPU oracle: float32 greedy tokens identical and logits within 1e-3; bf16 layer
outputs within relative error 2e-2 (teacher-forced)."""
import numpy as np
import pytest

import luminal_oracle as O
import whisper_oracle as W

pytestmark = pytest.mark.gpu


def build(L, device, cfg, w, batch, cross_kv, dtype, T):
    model = L.WhisperDecoderModel(device, d_model=cfg["d_model"], heads=cfg["heads"], layers=cfg["dec_layers"],
                                  ffn=cfg["ffn"], vocab=cfg["vocab"], max_positions=cfg["max_positions"],
                                  cross_len=T, dtype=dtype)
    for name, a in w.items():
        model.set_weight(name, a)
    sess = L.Session(model, batch, cfg["max_positions"])
    for i, (k, v) in enumerate(cross_kv):
        sess.set_cross_kv(i, k, v)
    return model, sess


@pytest.mark.parametrize("batch,frames", [(1, 40), (3, 150)])
def test_whisper_decode_fp32_matches_oracle(lib_built, device, batch, frames):
    L = lib_built
    cfg = W.CONFIGS["whisper_test"]
    w = W.synth_weights(cfg, seed=9)
    mel = O.synth_normal(9, 5, (batch, cfg["n_mels"], frames), 1.0)
    enc = W.encoder(mel, w, cfg)
    kv = W.project_cross_kv(enc, w, cfg)
    first = O.synth_tokens(9, 6, (batch,), cfg["vocab"])
    ref_tok, ref_log = W.CachedDecoder(w, cfg, batch, kv).greedy(first, 12)
    model, sess = build(L, device, cfg, w, batch, kv, "f32", enc.shape[1])
    tok = first.astype(np.int32)
    toks, logs = [], []
    for _ in range(12):
        tok, lg = sess.decode_step(tok, want_logits=True)
        toks.append(tok.copy()); logs.append(lg)
    assert np.abs(np.stack(logs, 1) - ref_log).max() <= 1e-3
    assert np.array_equal(np.stack(toks, 1), ref_tok)
    sess.reset()
    assert np.array_equal(sess.decode_n(first, 12).T, ref_tok)       # CUDA-graph loop
    sess.close(); model.close()


def test_whisper_decode_bf16_layer_outputs(lib_built, device):
    L = lib_built
    cfg = W.CONFIGS["whisper_test"]
    batch = 8
    w = W.synth_weights(cfg, seed=4)
    mel = O.synth_normal(4, 5, (batch, cfg["n_mels"], 130), 1.0)
    enc = W.encoder(mel, w, cfg)
    kv = W.project_cross_kv(enc, w, cfg)
    ref = W.CachedDecoder(w, cfg, batch, kv)
    model, sess = build(L, device, cfg, w, batch, kv, "bf16", enc.shape[1])
    sess.set_capture(True)
    tok = O.synth_tokens(4, 6, (batch,), cfg["vocab"])
    for step in range(6):
        ref_logits, ref_hidden = ref.step(tok, return_hidden=True)
        _, logits = sess.decode_step(tok, want_logits=True)
        for l in range(cfg["dec_layers"]):
            got = sess.layer_output(l)
            err = np.linalg.norm(got - ref_hidden[l]) / np.linalg.norm(ref_hidden[l])
            assert err <= 2e-2, f"step {step} layer {l}: {err}"
        assert np.linalg.norm(logits - ref_logits) / np.linalg.norm(ref_logits) <= 4e-2
        tok = ref_logits.argmax(-1)          # teacher forcing with the oracle's tokens
    sess.close(); model.close()


def test_unfold_matches_oracle(lib_built, device):
    L = lib_built
    x = O.synth_normal(2, 1, (2, 3, 23), 1.0)
    for k, st, dil in [(3, 1, 1), (3, 2, 1), (4, 3, 2), (1, 1, 1)]:
        g = L.Graph()
        t = L.tensor(g, x.shape)
        u = L.graph.unfold(t, [k], [st], [dil])
        got = L.execute(g, u.id, {t.id: x}, device)
        o = (23 - dil * (k - 1) - 1) // st + 1
        ref = np.stack([x[..., dil * j: dil * j + st * (o - 1) + 1: st] for j in range(k)], -1)
        assert got.shape == ref.shape and np.array_equal(got, ref)


def test_whisper_encoder_graph_matches_oracle(lib_built, device):
    """AudioEncoder + project_cross_kv built as a graph and run node by node on the device against
    the oracle's encoder; then the whole chain encoder -> cross K/V upload -> greedy decode."""
    L = lib_built
    cfg = W.CONFIGS["whisper_test"]
    batch, frames = 2, 60
    w = W.synth_weights(cfg, seed=13)
    mel = O.synth_normal(13, 5, (batch, cfg["n_mels"], frames), 1.0)
    ref_enc = W.encoder(mel, w, cfg)
    ref_kv = W.project_cross_kv(ref_enc, w, cfg)
    enc, kv = L.whisper.encode_cross_kv(device, w, mel, d_model=cfg["d_model"], heads=cfg["heads"],
                                        enc_layers=cfg["enc_layers"], dec_layers=cfg["dec_layers"], ffn=cfg["ffn"],
                                        n_mels=cfg["n_mels"])
    assert enc.shape == ref_enc.shape
    assert np.abs(enc - ref_enc).max() <= 1e-3
    for (k, v), (rk, rv) in zip(kv, ref_kv):
        assert np.abs(k - rk).max() <= 1e-3 and np.abs(v - rv).max() <= 1e-3
    first = O.synth_tokens(13, 6, (batch,), cfg["vocab"])
    ref_tok, ref_log = W.CachedDecoder(w, cfg, batch, ref_kv).greedy(first, 10)
    model, sess = build(L, device, cfg, w, batch, kv, "f32", enc.shape[1])
    tok = first.astype(np.int32)
    toks, logs = [], []
    for _ in range(10):
        tok, lg = sess.decode_step(tok, want_logits=True)
        toks.append(tok.copy()); logs.append(lg)
    assert np.abs(np.stack(logs, 1) - ref_log).max() <= 1e-3
    assert np.array_equal(np.stack(toks, 1), ref_tok)
    sess.close(); model.close()


def _fast_weights(cfg, seed):
    """Whisper-base is 70 M parameters: a NumPy generator instead of the counter-based one."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in sorted(W.weight_shapes(cfg).items()):
        a = rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
        w[name] = a + np.float32(1.0) if name.endswith("layer_norm.weight") else a
    return w


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_whisper_base_full_size_decoder(lib_built, device, dtype):
    """The Whisper-base decoder at its full size (d_model 512, 8 heads, 6 layers, FFN 2048, vocab
    51865, batch 8, 1500 encoder positions): the oracle is small enough to run it whole."""
    L = lib_built
    cfg = W.CONFIGS["whisper_base"]
    batch, T, steps = 8, 1500, 5
    w = _fast_weights(cfg, 17)
    if dtype == "bf16":
        w = {k: (O.bf16_round(v) if v.ndim == 2 and "embed_positions" not in k else v) for k, v in w.items()}
    rng = np.random.default_rng(3)
    D = cfg["d_model"] // cfg["heads"]
    kv = [(rng.standard_normal((batch, cfg["heads"], T, D), dtype=np.float32) * np.float32(0.5),
           rng.standard_normal((batch, cfg["heads"], T, D), dtype=np.float32)) for _ in range(cfg["dec_layers"])]
    if dtype == "bf16":
        kv = [(O.bf16_round(k), O.bf16_round(v)) for k, v in kv]
    first = O.synth_tokens(17, 6, (batch,), cfg["vocab"])
    ref = W.CachedDecoder(w, cfg, batch, kv)
    model, sess = build(L, device, cfg, w, batch, kv, dtype, T)
    tok = first.astype(np.int32)
    for step in range(steps):
        ref_logits = ref.step(tok)
        nxt, logits = sess.decode_step(tok, want_logits=True)
        if dtype == "f32":
            assert np.abs(logits - ref_logits).max() <= 1e-3, step
            assert np.array_equal(nxt, ref_logits.argmax(-1)), step
        else:
            assert np.linalg.norm(logits - ref_logits) / np.linalg.norm(ref_logits) <= 4e-2, step
        tok = ref_logits.argmax(-1).astype(np.int32)          # teacher forcing with the oracle's tokens
    # the CUDA-graph loop reproduces the stepwise tokens
    sess.reset()
    tok = first.astype(np.int32)
    stepwise = []
    for _ in range(steps):
        tok = sess.decode_step(tok)
        stepwise.append(tok.copy())
    sess.reset()
    assert np.array_equal(sess.decode_n(first, steps), np.stack(stepwise, 0))
    sess.close(); model.close()


@pytest.mark.parametrize("batch,frames", [(2, 60), (3, 301)])
def test_fused_encoder_matches_oracle(lib_built, device, batch, frames):
    """AudioEncoder + cross K/V projection on the tensor cores (bf16) against the float32 oracle, then
    the decoder on the cross cache the fused path wrote."""
    L = lib_built
    cfg = W.CONFIGS["whisper_test"]
    w = W.synth_weights(cfg, seed=23)
    mel = O.synth_normal(23, 5, (batch, cfg["n_mels"], frames), 1.0)
    ref_enc = W.encoder(mel, w, cfg)
    ref_kv = W.project_cross_kv(ref_enc, w, cfg)
    enc = L.whisper.FusedEncoder(device, d_model=cfg["d_model"], heads=cfg["heads"], enc_layers=cfg["enc_layers"],
                                 dec_layers=cfg["dec_layers"], ffn=cfg["ffn"], n_mels=cfg["n_mels"])
    enc.set_weights(w)
    out = enc.run(mel)
    assert out.shape == ref_enc.shape
    assert np.linalg.norm(out - ref_enc) / np.linalg.norm(ref_enc) <= 2e-2
    T = ref_enc.shape[1]
    model = L.WhisperDecoderModel(device, d_model=cfg["d_model"], heads=cfg["heads"], layers=cfg["dec_layers"], ffn=cfg["ffn"],
                                  vocab=cfg["vocab"], max_positions=cfg["max_positions"], cross_len=T, dtype="bf16")
    for name, a in w.items():
        model.set_weight(name, a)
    sess = L.Session(model, batch, cfg["max_positions"])
    enc.cross_kv_into(sess)
    ref = W.CachedDecoder(w, cfg, batch, ref_kv)
    tok = O.synth_tokens(23, 6, (batch,), cfg["vocab"])
    for step in range(5):
        ref_logits = ref.step(tok)
        _, logits = sess.decode_step(tok, want_logits=True)
        assert np.linalg.norm(logits - ref_logits) / np.linalg.norm(ref_logits) <= 4e-2, step
        tok = ref_logits.argmax(-1)
    sess.close(); model.close(); enc.close()

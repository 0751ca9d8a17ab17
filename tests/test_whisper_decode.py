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

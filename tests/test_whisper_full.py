"""Whisper at the widths of the benchmark configuration (d_model 512, 8 heads, 6 + 6 layers, FFN 2048):
the fused tensor-core encoder at the full input size against the oracle, and the whole chain
encoder -> cross K/V -> greedy decoding in float32 with tokens identical to the oracle's."""
import numpy as np
import pytest

import luminal_oracle as O
import whisper_oracle as W

from test_whisper_decode import _fast_weights, build

pytestmark = pytest.mark.gpu


def test_fused_encoder_at_full_size_matches_oracle(lib_built, device):
    """mel [8, 80, 3000] through the fused encoder; the oracle runs sequence 0 alone (the sequences of a batch do not
    interact), all 1500 output positions compared."""
    L = lib_built
    cfg = W.CONFIGS["whisper_base"]
    w = _fast_weights(cfg, 29)
    rng = np.random.default_rng(5)
    mel = rng.standard_normal((8, cfg["n_mels"], 3000), dtype=np.float32)
    enc = L.whisper.FusedEncoder(device, d_model=cfg["d_model"], heads=cfg["heads"], enc_layers=cfg["enc_layers"],
                                 dec_layers=cfg["dec_layers"], ffn=cfg["ffn"], n_mels=cfg["n_mels"])
    enc.set_weights(w)
    out = enc.run(mel)
    assert out.shape == (8, 1500, cfg["d_model"])
    again = enc.run(mel)
    assert np.array_equal(out, again)
    for b in (0, 7):
        ref = W.encoder(mel[b:b + 1], w, cfg)[0]
        err = np.linalg.norm(out[b] - ref) / np.linalg.norm(ref)
        assert err <= 2e-2, (b, err)
        row_err = np.linalg.norm(out[b] - ref, axis=1) / np.linalg.norm(ref, axis=1)
        assert row_err.max() <= 5e-2, (b, float(row_err.max()))
    enc.close()


def test_whisper_chain_fp32_tokens_identical(lib_built, device):
    """Encoder graph -> project_cross_kv -> 48 greedy steps, float32, the base model's widths with a reduced
    vocabulary and a 600-frame input: the device's tokens equal the oracle's, logits within 1e-3."""
    L = lib_built
    cfg = dict(W.CONFIGS["whisper_base"], vocab=2048)
    w = _fast_weights(cfg, 31)
    batch, frames, steps = 2, 600, 48
    mel = np.random.default_rng(6).standard_normal((batch, cfg["n_mels"], frames), dtype=np.float32)
    ref_enc = W.encoder(mel, w, cfg)
    ref_kv = W.project_cross_kv(ref_enc, w, cfg)
    first = O.synth_tokens(31, 6, (batch,), cfg["vocab"])
    ref_tok, ref_log = W.CachedDecoder(w, cfg, batch, ref_kv).greedy(first, steps)
    enc, kv = L.whisper.encode_cross_kv(device, w, mel, d_model=cfg["d_model"], heads=cfg["heads"],
                                        enc_layers=cfg["enc_layers"], dec_layers=cfg["dec_layers"], ffn=cfg["ffn"],
                                        n_mels=cfg["n_mels"])
    assert np.abs(enc - ref_enc).max() <= 2e-3
    model, sess = build(L, device, cfg, w, batch, kv, "f32", enc.shape[1])
    tok = first.astype(np.int32)
    toks, worst = [], 0.0
    for s in range(steps):
        tok, lg = sess.decode_step(tok, want_logits=True)
        toks.append(tok.copy())
        worst = max(worst, float(np.abs(lg - ref_log[:, s]).max()))
    assert np.array_equal(np.stack(toks, 1), ref_tok)
    assert worst <= 1e-3
    sess.reset()
    assert np.array_equal(sess.decode_n(first, steps).T, ref_tok)          # the CUDA-graph loop
    sess.close(); model.close()


def test_whisper_base_pipeline_bf16(lib_built, device):
    """The benchmark configuration as one chain: mel [8, 80, 3000] -> fused encoder -> cross K/V into the session ->
    128 greedy steps at batch 8, bf16.  Checked: the decoder's logits over the fused cross cache against the oracle's
    decoder over the oracle's cross K/V of the SAME encoder output (teacher-forced, 4 steps), and that two runs of
    the chain give the same 128 x 8 tokens."""
    L = lib_built
    cfg = W.CONFIGS["whisper_base"]
    w = _fast_weights(cfg, 37)
    wq = {k: (O.bf16_round(v) if v.ndim == 2 and "embed_positions" not in k else v) for k, v in w.items()}
    batch, steps = 8, 128
    mel = np.random.default_rng(7).standard_normal((batch, cfg["n_mels"], 3000), dtype=np.float32)
    enc = L.whisper.FusedEncoder(device, d_model=cfg["d_model"], heads=cfg["heads"], enc_layers=cfg["enc_layers"],
                                 dec_layers=cfg["dec_layers"], ffn=cfg["ffn"], n_mels=cfg["n_mels"])
    enc.set_weights(wq)
    enc_out = enc.run(mel)
    model = L.WhisperDecoderModel(device, d_model=cfg["d_model"], heads=cfg["heads"], layers=cfg["dec_layers"], ffn=cfg["ffn"],
                                  vocab=cfg["vocab"], max_positions=cfg["max_positions"], cross_len=enc_out.shape[1], dtype="bf16")
    for name, a in wq.items():
        if name.startswith("model.decoder."):
            model.set_weight(name, a)
    sess = L.Session(model, batch, cfg["max_positions"])
    enc.cross_kv_into(sess)
    first = np.full(batch, 50258, dtype=np.int32)
    ref = W.CachedDecoder(wq, cfg, batch, W.project_cross_kv(enc_out, wq, cfg))
    tok = first
    for s in range(4):
        ref_logits = ref.step(tok)
        _, logits = sess.decode_step(tok, want_logits=True)
        assert np.linalg.norm(logits - ref_logits) / np.linalg.norm(ref_logits) <= 4e-2, s
        tok = ref_logits.argmax(-1).astype(np.int32)
    sess.reset()
    a = sess.decode_n(first, steps)
    enc.run(mel, want_output=False)
    enc.cross_kv_into(sess)
    sess.reset()
    b = sess.decode_n(first, steps)
    assert a.shape == (steps, batch) and np.array_equal(a, b)
    sess.close(); model.close(); enc.close()

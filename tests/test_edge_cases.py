"""Edge shapes of the decode path against the oracle: a batch of one, a one-token prompt, decoding into the last slot
of the context, multi-query attention (one kv head), a vocabulary and an MLP width that fill no tile, out-of-range
token ids (the reference's gather kernel returns a zero row for them, src/Execution.jl:587-592)."""
import numpy as np
import pytest

import luminal_oracle as O

pytestmark = pytest.mark.gpu

LOGIT_TOL = 1e-3
ODD = dict(n_layers=2, hidden=256, n_heads=4, n_kv_heads=1, intermediate=200, vocab=1001, eps=1e-5, rope_base=10000.0)


def make_model(L, device, cfg, w, dtype):
    model = L.Model(device, n_layers=cfg["n_layers"], hidden=cfg["hidden"], n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"],
                    intermediate=cfg["intermediate"], vocab=cfg["vocab"], eps=cfg["eps"], rope_base=cfg["rope_base"], dtype=dtype)
    model.set_weights(w)
    return model


@pytest.mark.parametrize("batch,prompt_len", [(1, 1), (1, 7), (32, 1), (5, 3)])
def test_odd_shapes_fp32_tokens_identical(lib_built, device, batch, prompt_len):
    L = lib_built
    w = O.synth_llama_weights(ODD, seed=5)
    prompt = O.synth_tokens(5, 1000, (batch, prompt_len), ODD["vocab"])
    steps = 6
    ref_tok, ref_log = O.CachedLlama(w, ODD, batch, prompt_len + steps).greedy(prompt, steps)
    model = make_model(L, device, ODD, w, "f32")
    sess = L.Session(model, batch, prompt_len + steps - 1)        # the last step writes the last slot of the context
    tok, log = L.greedy_generate(sess, prompt, steps, want_logits=True)
    assert np.abs(log - ref_log).max() <= LOGIT_TOL
    assert np.array_equal(tok, ref_tok)
    sess.close(); model.close()


def test_odd_shapes_bf16_within_tolerance(lib_built, device):
    L = lib_built
    batch, n = 3, 10
    w = {k: O.bf16_round(v) if v.ndim == 2 else v for k, v in O.synth_llama_weights(ODD, seed=6).items()}
    prompt = O.synth_tokens(6, 1000, (batch, n), ODD["vocab"])
    ref_logits, ref_hidden = O.CachedLlama(w, ODD, batch, 32).forward(prompt, return_hidden=True)
    model = make_model(L, device, ODD, w, "bf16")
    sess = L.Session(model, batch, 32)
    sess.set_capture(True)
    logits = sess.prefill(prompt)
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))
    for l in range(ODD["n_layers"]):
        assert rel(sess.layer_output(l), ref_hidden[l][:, -1, :]) <= 2e-2, f"layer {l}"
    assert rel(logits, ref_logits[:, -1, :]) <= 4e-2
    sess.close(); model.close()


def test_out_of_range_token_reads_a_zero_row(lib_built, device):
    """Token ids outside the table give a zero embedding row, as _gather_kernel! does: the step then equals the one
    for a row of zeros, whatever the id."""
    L = lib_built
    w = O.synth_llama_weights(ODD, seed=8)
    model = make_model(L, device, ODD, w, "f32")
    outs = []
    for bad in (ODD["vocab"], ODD["vocab"] + 12345, -3):
        sess = L.Session(model, 2, 8)
        _, lg = sess.decode_step(np.array([bad, 5], dtype=np.int32), want_logits=True)
        outs.append(lg)
        sess.close()
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][0], outs[2][0])
    assert np.array_equal(outs[0][1], outs[1][1])                       # the valid sequence is unaffected
    # the oracle on an all-zero embedding row for sequence 0
    w0 = dict(w)
    emb = w["model.embed_tokens.weight"].copy()
    emb[7] = 0.0
    w0["model.embed_tokens.weight"] = emb
    ref = O.CachedLlama(w0, ODD, 2, 8)
    ref_log = ref.forward(np.array([[7], [5]]))[:, -1, :]
    assert np.abs(outs[0] - ref_log).max() <= LOGIT_TOL
    model.close()


@pytest.mark.parametrize("batch", [40, 70])
def test_batch_above_32_matches_oracle(lib_built, device, batch):
    """The reference's Llama takes any batch (src/NN.jl:448-455); here a batch above 32 runs as sub-sessions of at most
    32 sequences over one model.  float32: tokens identical and logits <= 1e-3 through every entry point a session has."""
    L = lib_built
    cfg = O.CONFIGS["tiny_gqa128"]
    w = O.synth_llama_weights(cfg, seed=31)
    steps = 5
    prompt = O.synth_tokens(31, 1000, (batch, 6), cfg["vocab"])
    ref_tok, ref_log = O.CachedLlama(w, cfg, batch, 32).greedy(prompt, steps)
    model = make_model(L, device, cfg, w, "f32")
    sess = L.Session(model, batch, 32)
    tok, log = L.greedy_generate(sess, prompt, steps, want_logits=True)
    assert np.abs(log - ref_log).max() <= LOGIT_TOL
    assert np.array_equal(tok, ref_tok)
    assert sess.position() == 6 + steps - 1 and list(sess.positions()) == [6 + steps - 1] * batch
    # the device-resident loop
    sess.reset()
    first = sess.prefill(prompt).argmax(-1).astype(np.int32)
    assert np.array_equal(sess.decode_n(first, steps - 1).T, ref_tok[:, 1:])
    # the loop with its end-of-text exit: an id that only some sequences produce
    sess.reset()
    first = sess.prefill(prompt).argmax(-1).astype(np.int32)
    free = ref_tok[:, 1:]
    eot = int(free[batch - 1, 1])                        # the last sub-session's last sequence produces it at its 2nd step
    got = sess.decode_until(first, steps - 1, eot)
    want = free.copy()
    for b in range(batch):
        hit = np.nonzero(free[b] == eot)[0]
        if hit.size:
            want[b, hit[0]:] = eot
    n = got.shape[0]
    assert 2 <= n <= steps - 1 and np.array_equal(got.T, want[:, :n])
    assert (want[:, n:] == eot).all()                    # nothing but end-of-text ids was cut
    # prompts of different lengths, one per sequence
    sess.reset()
    lens = [2 + (b * 5) % 7 for b in range(batch)]
    prompts = [O.synth_tokens(32, 100 + b, (n_,), cfg["vocab"]) for b, n_ in enumerate(lens)]
    logits = sess.prefill_ragged(prompts)
    assert list(sess.positions()) == lens
    for b in (0, 31, 32, batch - 1):
        alone = O.CachedLlama(w, cfg, 1, 32).forward(prompts[b][None, :])[:, -1, :]
        assert np.abs(logits[b] - alone[0]).max() <= LOGIT_TOL, b
    # what a row of sub-sessions cannot offer is refused, not approximated
    with pytest.raises(L.LuminalB200Error):
        sess.kv_layer(0)
    assert sess.step_bytes(8) > 0
    sess.close(); model.close()


def test_batch_above_32_is_refused_where_it_is_not_built(lib_built, device):
    import whisper_oracle as W
    L = lib_built
    cfg = W.CONFIGS["whisper_test"]
    model = L.WhisperDecoderModel(device, d_model=cfg["d_model"], heads=cfg["heads"], layers=cfg["dec_layers"], ffn=cfg["ffn"],
                                  vocab=cfg["vocab"], max_positions=cfg["max_positions"], cross_len=16)
    with pytest.raises(L.LuminalB200Error, match="Llama / Phi-3 only"):
        L.Session(model, 33, 8)
    model.close()


def test_batch_above_32_bf16_layer_outputs(lib_built, device):
    L = lib_built
    cfg, batch = O.CONFIGS["mid_gqa"], 48
    w = O.synth_llama_weights(cfg, seed=33)
    prompt = O.synth_tokens(33, 1000, (batch, 10), cfg["vocab"])
    ref_logits, ref_hidden = O.CachedLlama(w, cfg, batch, 32).forward(prompt, return_hidden=True)
    model = make_model(L, device, cfg, w, "bf16")
    sess = L.Session(model, batch, 32)
    sess.set_capture(True)
    logits = sess.prefill(prompt)
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))
    for l in range(cfg["n_layers"]):
        got = sess.layer_output(l)
        assert got.shape == (batch, cfg["hidden"]) and rel(got, ref_hidden[l][:, -1, :]) <= 2e-2, l
    assert rel(logits, ref_logits[:, -1, :]) <= 4e-2
    sess.close(); model.close()

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

"""GPU parity of the decode session against the CPU oracle (reference semantics of
src/NN.jl:343-455 replayed op by op).  fp32: identical greedy tokens, logits max-abs-err <= 1e-3.
bf16: layer outputs within relative error 2e-2 of the fp32 oracle."""
import numpy as np
import pytest

import luminal_oracle as O

pytestmark = pytest.mark.gpu

LOGIT_TOL = 1e-3      # fp32 logits, max abs error (north-star tolerance)
BF16_REL_TOL = 2e-2   # bf16 layer outputs, relative error (north-star tolerance)


def make_model(L, device, cfg, w, dtype):
    m = L.Model(device, n_layers=cfg["n_layers"], hidden=cfg["hidden"], n_heads=cfg["n_heads"],
                n_kv_heads=cfg["n_kv_heads"], intermediate=cfg["intermediate"], vocab=cfg["vocab"],
                eps=cfg["eps"], rope_base=cfg["rope_base"], dtype=dtype)
    if w is None:
        m.init_random(1234, 0.02)
    else:
        m.set_weights(w)
    return m


def rel_err(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) /
                 (np.linalg.norm(b.astype(np.float64)) + 1e-30))


def test_small_llama_fp32_greedy_matches_oracle(lib_built, device):
    """BASELINE config 1: 4 layers, hidden 256, 8x32 heads, MLP 688, vocab 1024; batch 1,
    32-token prompt, 64 greedy steps with KV cache; weights from the shared generator."""
    L = lib_built
    cfg = O.CONFIGS["small_llama"]
    w = O.synth_llama_weights(cfg, seed=1234)
    prompt = O.synth_tokens(1234, 1000, (1, 32), cfg["vocab"])
    ref_tok, ref_log = O.CachedLlama(w, cfg, 1, 128).greedy(prompt, 64)

    model = make_model(L, device, cfg, None, "f32")          # device-side generator
    sess = L.Session(model, 1, 128)
    tok, log = L.greedy_generate(sess, prompt, 64, want_logits=True)
    assert np.array_equal(tok, ref_tok)
    assert np.abs(log - ref_log).max() <= LOGIT_TOL
    # ... and against the committed fixture of the same run (tests/golden/make_golden.py)
    import os
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "small_llama_golden.npz"))
    assert np.array_equal(prompt, gold["prompt"])
    assert np.array_equal(tok, gold["tokens"])
    assert np.abs(log[:, 0] - gold["logits_first"]).max() <= LOGIT_TOL
    assert np.abs(log[:, -1] - gold["logits_last"]).max() <= LOGIT_TOL

    # the same weights pushed through set_weight (row-major and Julia column-major images)
    for layout in (L.ROWMAJOR, L.COLMAJOR):
        m2 = L.Model(device, n_layers=cfg["n_layers"], hidden=cfg["hidden"], n_heads=cfg["n_heads"],
                     n_kv_heads=cfg["n_kv_heads"], intermediate=cfg["intermediate"], vocab=cfg["vocab"],
                     eps=cfg["eps"], rope_base=cfg["rope_base"], dtype="f32")
        m2.set_weights(w, layout)
        s2 = L.Session(m2, 1, 128)
        lg = s2.prefill(prompt)
        assert np.abs(lg - ref_log[:, 0]).max() <= LOGIT_TOL
        s2.close(); m2.close()

    # device-resident loop (CUDA graph replay) gives the same tokens as the stepwise calls
    sess.reset()
    sess.prefill(prompt[:, :-1], want_logits=False)
    toks = sess.decode_n(prompt[:, -1], 64)
    assert np.array_equal(toks.T, ref_tok)
    sess.close(); model.close()


@pytest.mark.parametrize("name,batch", [("tiny_gqa128", 3), ("tiny_gqa96", 2), ("small_llama", 9), ("tiny_gqa128", 17),
                                        ("mid_gqa", 2)])
def test_gqa_fp32_matches_oracle(lib_built, device, name, batch):
    """Reduced shapes of the Llama-3-8B (head_dim 128, GQA) and Phi-3 (head_dim 96) paths and
    the three batch tilings (<=8, <=16, <=32)."""
    L = lib_built
    cfg = O.CONFIGS[name]
    w = O.synth_llama_weights(cfg, seed=7)
    prompt = O.synth_tokens(7, 1000, (batch, 9), cfg["vocab"])
    ref = O.CachedLlama(w, cfg, batch, 64)
    ref_tok, ref_log = ref.greedy(prompt, 6)
    model = make_model(L, device, cfg, w, "f32")
    sess = L.Session(model, batch, 40)
    tok, log = L.greedy_generate(sess, prompt, 6, want_logits=True)
    assert np.abs(log - ref_log).max() <= LOGIT_TOL
    assert np.array_equal(tok, ref_tok)
    sess.close(); model.close()


@pytest.mark.parametrize("name,batch", [("tiny_gqa128", 4), ("tiny_gqa96", 16), ("small_llama", 32),
                                        ("mid_gqa", 32), ("mid_gqa", 5)])
def test_bf16_layer_outputs_within_tolerance(lib_built, device, name, batch):
    L = lib_built
    cfg = O.CONFIGS[name]
    w = O.synth_llama_weights(cfg, seed=11)
    prompt = O.synth_tokens(11, 1000, (batch, 12), cfg["vocab"])
    ref = O.CachedLlama(w, cfg, batch, 64)
    ref_logits, ref_hidden = ref.forward(prompt, return_hidden=True)

    model = make_model(L, device, cfg, w, "bf16")
    sess = L.Session(model, batch, 64)
    sess.set_capture(True)
    logits = sess.prefill(prompt)
    for l in range(cfg["n_layers"]):
        got = sess.layer_output(l)
        assert rel_err(got, ref_hidden[l][:, -1, :]) <= BF16_REL_TOL, f"layer {l}"
    assert rel_err(logits, ref_logits[:, -1, :]) <= 2 * BF16_REL_TOL
    sess.close(); model.close()


def test_decode_past_max_ctx_is_an_error(lib_built, device):
    L = lib_built
    cfg = O.CONFIGS["tiny_gqa128"]
    model = make_model(L, device, cfg, None, "f32")
    sess = L.Session(model, 1, 4)
    sess.prefill(np.zeros((1, 4), dtype=np.int32), want_logits=False)
    with pytest.raises(L.LuminalB200Error):
        sess.decode_step(np.zeros(1, dtype=np.int32))
    with pytest.raises(L.LuminalB200Error):
        L.Session(model, 0, 8)
    sess.close(); model.close()


def test_decode_until_stops_at_end_of_text(lib_built, device):
    """The generation loop's two exits (src/Decoding.jl:93-95, 126-129) for a batch: every sequence follows the
    oracle until its first end-of-text token and emits that token from then on; the loop ends with the step in which
    the last sequence finished, or at the position cap."""
    L = lib_built
    cfg = O.CONFIGS["tiny_gqa128"]
    w = O.synth_llama_weights(cfg, seed=7)
    batch, steps = 3, 12
    prompt = O.synth_tokens(7, 1000, (batch, 9), cfg["vocab"])
    ref_tok, _ = O.CachedLlama(w, cfg, batch, 64).greedy(prompt, steps + 1)     # [B, steps + 1]; column 0 comes from the prompt
    model = make_model(L, device, cfg, w, "f32")
    sess = L.Session(model, batch, 64)
    first = sess.prefill(prompt).argmax(-1).astype(np.int32)
    assert np.array_equal(first, ref_tok[:, 0])
    free = ref_tok[:, 1:]                                                       # what an unstopped loop produces
    # an id nobody produces: the loop runs to max_steps
    unused = int(np.setdiff1d(np.arange(cfg["vocab"]), free)[0])
    got = sess.decode_until(first, steps, unused)
    assert got.shape == (steps, batch) and np.array_equal(got.T, free)
    # the id sequence 1 produces at step 4 ends that sequence there; the others run on (or stop at their own first hit)
    eot = int(free[1, 4])
    want = free.copy()
    last = 0
    for b in range(batch):
        hits = np.nonzero(free[b] == eot)[0]
        if len(hits):
            want[b, hits[0]:] = eot
            last = max(last, hits[0])
        else:
            last = steps - 1
    sess.reset()
    sess.prefill(prompt, want_logits=False)
    got = sess.decode_until(first, steps, eot)
    assert got.shape[0] == last + 1 and np.array_equal(got.T, want[:, :last + 1])
    assert sess.position() == 9 + last + 1
    # the position cap: 64 - 9 positions are left however many steps are asked for
    sess.reset()
    sess.prefill(prompt, want_logits=False)
    assert sess.decode_until(first, 1000, unused).shape[0] == 64 - 9
    sess.close(); model.close()

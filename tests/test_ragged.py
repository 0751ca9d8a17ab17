"""Prompts of different lengths in one batch (per-sequence positions): every sequence must behave as if it ran
alone -- its logits at its own last prompt position and its greedy continuation equal the oracle run on that
sequence by itself."""
import numpy as np
import pytest

import luminal_oracle as O

from test_decode_parity import make_model

pytestmark = pytest.mark.gpu


def _oracle_alone(w, cfg, prompt, steps):
    tok, log = O.CachedLlama(w, cfg, 1, 64).greedy(np.asarray(prompt)[None, :], steps)
    return tok[0], log[0]


@pytest.mark.parametrize("name,lens", [("tiny_gqa128", [5, 9, 2]), ("tiny_gqa96", [1, 7]), ("small_llama", [12, 3, 8, 8])])
def test_ragged_prompts_fp32_match_per_sequence_oracle(lib_built, device, name, lens):
    L = lib_built
    cfg = O.CONFIGS[name]
    w = O.synth_llama_weights(cfg, seed=21)
    steps = 6
    prompts = [O.synth_tokens(21, 500 + b, (n,), cfg["vocab"]) for b, n in enumerate(lens)]
    refs = [_oracle_alone(w, cfg, p, steps) for p in prompts]
    model = make_model(L, device, cfg, w, "f32")
    sess = L.Session(model, len(lens), 64)
    logits = sess.prefill_ragged(prompts)
    assert list(sess.positions()) == lens
    for b, (rt, rl) in enumerate(refs):
        assert np.abs(logits[b] - rl[0]).max() <= 1e-3, b
    tok = logits.argmax(-1).astype(np.int32)
    got = [tok.copy()]
    for _ in range(steps - 1):
        tok = sess.decode_step(tok)
        got.append(tok.copy())
    got = np.stack(got, axis=1)
    for b, (rt, _) in enumerate(refs):
        assert np.array_equal(got[b], rt), b
    # the device-resident loop from the same ragged state gives the same tokens
    sess.reset()
    first = sess.prefill_ragged(prompts).argmax(-1).astype(np.int32)
    loop = sess.decode_n(first, steps - 1)
    assert np.array_equal(loop.T, got[:, 1:])
    assert list(sess.positions()) == [n + steps - 1 for n in lens]
    sess.close(); model.close()


@pytest.mark.parametrize("lens", [[20, 9, 33], [8, 8, 30, 17]])
def test_ragged_prompts_bf16_through_the_prompt_gemms(lib_built, device, lens):
    """bf16, prompts of 8 or more tokens: all positions at once through the GEMM prompt phase, the last-position rows
    taken per sequence; logits within the bf16 tolerance of the per-sequence oracle, teacher-forced decode after it."""
    L = lib_built
    cfg = O.CONFIGS["mid_gqa"]
    w = O.synth_llama_weights(cfg, seed=22)
    prompts = [O.synth_tokens(22, 600 + b, (n,), cfg["vocab"]) for b, n in enumerate(lens)]
    refs = [_oracle_alone(w, cfg, p, 4) for p in prompts]
    model = make_model(L, device, cfg, w, "bf16")
    sess = L.Session(model, len(lens), 64)
    logits = sess.prefill_ragged(prompts)
    assert list(sess.positions()) == lens
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))
    for b, (rt, rl) in enumerate(refs):
        assert rel(logits[b], rl[0]) <= 4e-2, b
    for s in range(3):                                   # feed the oracle's tokens, compare the next logits
        tok = np.array([rt[s] for rt, _ in refs], dtype=np.int32)
        _, lg = sess.decode_step(tok, want_logits=True)
        for b, (_, rl) in enumerate(refs):
            assert rel(lg[b], rl[s + 1]) <= 4e-2, (s, b)
    sess.close(); model.close()


def test_ragged_whisper_positions(lib_built, device):
    """The Whisper decoder reads its learned position embedding per sequence too: two sequences moved to different
    positions decode as two single-sequence sessions at those positions do."""
    import whisper_oracle as W
    L = lib_built
    cfg = W.CONFIGS["whisper_test"]
    w = W.synth_weights(cfg, seed=9)
    mel = O.synth_normal(9, 5, (2, cfg["n_mels"], 40), 1.0)
    kv = W.project_cross_kv(W.encoder(mel, w, cfg), w, cfg)
    from test_whisper_decode import build
    model, sess = build(L, device, cfg, w, 2, kv, "f32", kv[0][0].shape[2])
    tok = O.synth_tokens(9, 6, (2,), cfg["vocab"]).astype(np.int32)
    # sequence 0 takes 3 steps alone-equivalent, sequence 1 takes 1: run both 3 steps, then rewind sequence 1 to position 1
    hist = []
    t = tok
    for _ in range(3):
        t, lg = sess.decode_step(t, want_logits=True)
        hist.append((t.copy(), lg.copy()))
    sess.set_positions([3, 1])
    nxt, lg = sess.decode_step(np.array([hist[2][0][0], hist[0][0][1]], dtype=np.int32), want_logits=True)
    # sequence 1 at position 1 with the token it produced at step 0 must repeat its own step-1 result
    assert np.abs(lg[1] - hist[1][1][1]).max() <= 1e-4
    assert nxt[1] == hist[1][0][1]
    sess.close(); model.close()

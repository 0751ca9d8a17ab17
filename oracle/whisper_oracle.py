"""CPU oracle for the Whisper path of Luminal.jl (encoder, cross-KV projection, cached decoder
step, greedy loop).  TEST INFRASTRUCTURE ONLY -- see luminal_oracle.py for the rules.

PARITY UNPINNED: the reference's Whisper tests check shapes only (tests/test_kv_cache.jl:55-72,
tests/test_greedy_decode.jl:88-90) and Unfold windows (tests/test_whisper_components.jl:5-23,
reproduced in tests/test_oracle_pins.py).  This file follows src/Whisper.jl and src/NN.jl op by op.

The reference hard-codes whisper-tiny constants (src/Whisper.jl:195-206); here they are a config
dict so that the base shape of BASELINE config 3 (d_model 512, 8 heads, 6+6 layers, FFN 2048,
vocab 51865) and small test shapes run through the same code.  Linear biases on [B,S,out] inputs
are a broadcast over the last dim (the reference's expand is only shape-correct for B == 1,
src/NN.jl:27-33, src/Decoding.jl:43)."""
from __future__ import annotations

import math

import numpy as np

import luminal_oracle as O

F32 = np.float32

CONFIGS = {
    "whisper_base": dict(d_model=512, heads=8, enc_layers=6, dec_layers=6, ffn=2048, vocab=51865,
                         n_mels=80, max_positions=448),
    "whisper_test": dict(d_model=128, heads=2, enc_layers=2, dec_layers=2, ffn=256, vocab=320,
                         n_mels=16, max_positions=48),
}


def attn_scale(cfg):
    # (Float32(hidden) / Float32(HEADS)) ^ -0.25f0      src/Whisper.jl:257
    return F32(F32(F32(cfg["d_model"]) / F32(cfg["heads"])) ** F32(-0.25))


def sinusoids(channels, length):                 # src/Whisper.jl:208-231
    inc = math.log(10000.0) / (channels / 2 - 1)
    inv_ts = np.array([math.exp(-inc * i) for i in range(channels // 2)], dtype=F32)
    scaled = O.mul(O.expand(O.arange(length), 2, channels // 2), O.expand(inv_ts, 1, length))
    return O.concat_along(O.sin(scaled), O.cos(scaled), 2)


def conv1d(x, weight, bias, kernel, stride, padding):      # src/NN.jl:55-104
    """x [B, C, L]; weight [ch_out, C*kernel] with merged index c + C*k (column-major reshape)."""
    x = np.asarray(x, F32)
    rank = x.ndim
    padded = O.pad_along(x, rank, padding, padding) if padding > 0 else x
    unfolded = O.unfold1d(padded, kernel, stride, 1)                       # [B, C, O, K]
    perm = O.permute(unfolded, [1, 3, 2, 4])                               # [B, O, C, K]
    B, Ol, C, K = perm.shape
    merged = O.reshape(perm, [B, Ol, C * K])                               # column-major: c + C*k
    out = O.matmul(merged, O.permute(weight, [2, 1]))                      # [B, O, ch_out]
    out = O.permute(out, [1, 3, 2])                                        # [B, ch_out, O]
    if bias is not None:
        out = O.add(out, np.asarray(bias, F32)[None, :, None])
    return out


def _heads(x, H):
    """[B,S,hidden] -> [B,H,S,D] with the column-major split f = h + H*d (src/Whisper.jl:259-261)."""
    B, S, hid = x.shape
    return O.permute(O.reshape(x, [B, S, H, hid // H]), [1, 3, 2, 4])


def _merge(x):
    B, H, S, D = x.shape
    return O.reshape(O.permute(x, [1, 3, 2, 4]), [B, S, H * D])


def self_attention(x, w, p, cfg, mask):          # src/Whisper.jl:253-276
    H = cfg["heads"]
    scale = attn_scale(cfg)
    q = _heads(O.mul(O.linear(x, w[p + ".q_proj.weight"], w[p + ".q_proj.bias"]), scale), H)
    k = _heads(O.mul(O.linear(x, w[p + ".k_proj.weight"]), scale), H)
    v = _heads(O.linear(x, w[p + ".v_proj.weight"], w[p + ".v_proj.bias"]), H)
    weights = O.matmul(q, O.permute(k, [1, 2, 4, 3]))
    if mask:
        S = x.shape[1]
        m = O.mul(O.triu(S, 1), F32(-1e9))
        weights = O.add(weights, O.expand(O.expand(m, 1, H), 1, x.shape[0]))
    out = _merge(O.matmul(O.softmax(weights, 4), v))
    return O.linear(out, w[p + ".out_proj.weight"], w[p + ".out_proj.bias"])


def cross_attention(x, enc, w, p, cfg):          # src/Whisper.jl:297-316
    H = cfg["heads"]
    scale = attn_scale(cfg)
    q = _heads(O.mul(O.linear(x, w[p + ".q_proj.weight"], w[p + ".q_proj.bias"]), scale), H)
    k = _heads(O.mul(O.linear(enc, w[p + ".k_proj.weight"]), scale), H)
    v = _heads(O.linear(enc, w[p + ".v_proj.weight"], w[p + ".v_proj.bias"]), H)
    out = _merge(O.matmul(O.softmax(O.matmul(q, O.permute(k, [1, 2, 4, 3])), 4), v))
    return O.linear(out, w[p + ".out_proj.weight"], w[p + ".out_proj.bias"])


def _ln(x, w, p):
    return O.layer_norm(x, w[p + ".weight"], w[p + ".bias"], 1e-5, True)


def _mlp(x, w, p1, p2):
    return O.linear(O.gelu(O.linear(x, w[p1 + ".weight"], w[p1 + ".bias"])), w[p2 + ".weight"], w[p2 + ".bias"])


def encoder(mel, w, cfg):                        # src/Whisper.jl:379-404
    """mel [B, n_mels, frames] -> [B, frames/2, d_model]."""
    pfx = "model.encoder"
    x = O.gelu(conv1d(mel, w[pfx + ".conv1.weight"], w[pfx + ".conv1.bias"], 3, 1, 1))
    x = O.gelu(conv1d(x, w[pfx + ".conv2.weight"], w[pfx + ".conv2.bias"], 3, 2, 1))
    x = O.permute(x, [1, 3, 2])
    x = O.add(x, O.expand(sinusoids(cfg["d_model"], x.shape[1]), 1, x.shape[0]))
    for i in range(cfg["enc_layers"]):
        p = f"{pfx}.layers.{i}"
        x = O.add(x, self_attention(_ln(x, w, p + ".self_attn_layer_norm"), w, p + ".self_attn", cfg, False))
        x = O.add(x, _mlp(_ln(x, w, p + ".final_layer_norm"), w, p + ".fc1", p + ".fc2"))
    return _ln(x, w, pfx + ".layer_norm")


def project_cross_kv(enc_out, w, cfg):           # src/Whisper.jl:809-831
    """Per decoder layer: (K [B,H,T,D] already scaled, V [B,H,T,D])."""
    H = cfg["heads"]
    scale = attn_scale(cfg)
    kv = []
    for i in range(cfg["dec_layers"]):
        p = f"model.decoder.layers.{i}.encoder_attn"
        k = _heads(O.mul(O.linear(enc_out, w[p + ".k_proj.weight"]), scale), H)
        v = _heads(O.linear(enc_out, w[p + ".v_proj.weight"], w[p + ".v_proj.bias"]), H)
        kv.append((np.ascontiguousarray(k), np.ascontiguousarray(v)))
    return kv


def decoder_full(tokens, enc_out, w, cfg):       # src/Whisper.jl:483-502 (no cache, causal mask)
    pfx = "model.decoder"
    tokens = np.asarray(tokens)
    x = O.embedding(w[pfx + ".embed_tokens.weight"], tokens.astype(F32))
    S = tokens.shape[1]
    x = O.add(x, O.expand(O.slice_along(w[pfx + ".embed_positions.weight"], 1, 0, S), 1, x.shape[0]))
    for i in range(cfg["dec_layers"]):
        p = f"{pfx}.layers.{i}"
        x = O.add(x, self_attention(_ln(x, w, p + ".self_attn_layer_norm"), w, p + ".self_attn", cfg, True))
        x = O.add(x, cross_attention(_ln(x, w, p + ".encoder_attn_layer_norm"), enc_out, w, p + ".encoder_attn", cfg))
        x = O.add(x, _mlp(_ln(x, w, p + ".final_layer_norm"), w, p + ".fc1", p + ".fc2"))
    out = _ln(x, w, pfx + ".layer_norm")
    return O.matmul(out, O.permute(w[pfx + ".embed_tokens.weight"], [2, 1]))


class CachedDecoder:
    """build_decode_step! / decode_step! (src/Whisper.jl:679-801): one token per sequence, self K/V
    written at step_pos, attention over [0, step_pos], cross attention over the fixed cross K/V."""

    def __init__(self, w, cfg, batch, cross_kv):
        self.w, self.cfg, self.cross = w, cfg, cross_kv
        H, D = cfg["heads"], cfg["d_model"] // cfg["heads"]
        L, T = cfg["dec_layers"], cfg["max_positions"]
        self.k = np.zeros((L, batch, H, T, D), F32)
        self.v = np.zeros((L, batch, H, T, D), F32)
        self.pos = 0

    def step(self, tokens, return_hidden=False):
        w, cfg = self.w, self.cfg
        H = cfg["heads"]
        scale = attn_scale(cfg)
        pfx = "model.decoder"
        tokens = np.asarray(tokens).reshape(-1, 1)
        p0 = self.pos
        x = O.embedding(w[pfx + ".embed_tokens.weight"], tokens.astype(F32))
        x = O.add(x, O.expand(O.slice_along(w[pfx + ".embed_positions.weight"], 1, p0, p0 + 1), 1, x.shape[0]))
        hiddens = []
        for i in range(cfg["dec_layers"]):
            p = f"{pfx}.layers.{i}"
            xn = _ln(x, w, p + ".self_attn_layer_norm")
            a = p + ".self_attn"
            q = _heads(O.mul(O.linear(xn, w[a + ".q_proj.weight"], w[a + ".q_proj.bias"]), scale), H)
            kn = _heads(O.mul(O.linear(xn, w[a + ".k_proj.weight"]), scale), H)
            vn = _heads(O.linear(xn, w[a + ".v_proj.weight"], w[a + ".v_proj.bias"]), H)
            self.k[i, :, :, p0:p0 + 1] = kn
            self.v[i, :, :, p0:p0 + 1] = vn
            kc, vc = self.k[i, :, :, :p0 + 1], self.v[i, :, :, :p0 + 1]
            out = _merge(O.matmul(O.softmax(O.matmul(q, O.permute(kc, [1, 2, 4, 3])), 4), vc))
            x = O.add(x, O.linear(out, w[a + ".out_proj.weight"], w[a + ".out_proj.bias"]))
            xn = _ln(x, w, p + ".encoder_attn_layer_norm")
            c = p + ".encoder_attn"
            q = _heads(O.mul(O.linear(xn, w[c + ".q_proj.weight"], w[c + ".q_proj.bias"]), scale), H)
            ck, cv = self.cross[i]
            out = _merge(O.matmul(O.softmax(O.matmul(q, O.permute(ck, [1, 2, 4, 3])), 4), cv))
            x = O.add(x, O.linear(out, w[c + ".out_proj.weight"], w[c + ".out_proj.bias"]))
            x = O.add(x, _mlp(_ln(x, w, p + ".final_layer_norm"), w, p + ".fc1", p + ".fc2"))
            if return_hidden:
                hiddens.append(x[:, 0])
        out = _ln(x, w, pfx + ".layer_norm")
        logits = O.matmul(O.slice_along(out, 2, 0, 1), O.permute(w[pfx + ".embed_tokens.weight"], [2, 1]))[:, 0]
        self.pos += 1
        return (logits, hiddens) if return_hidden else logits

    def greedy(self, first_tokens, n_steps):
        """Greedy loop of src/Decoding.jl:91-130 (argmax, feed back): tokens [B, n], logits [B, n, V]."""
        tok = np.asarray(first_tokens).reshape(-1)
        toks, lgs = [], []
        for _ in range(n_steps):
            logits = self.step(tok)
            tok = np.argmax(logits, axis=-1)
            toks.append(tok)
            lgs.append(logits)
        return np.stack(toks, 1), np.stack(lgs, 1)


def weight_shapes(cfg):
    d, ffn, V = cfg["d_model"], cfg["ffn"], cfg["vocab"]
    s = {"model.encoder.conv1.weight": (d, cfg["n_mels"] * 3), "model.encoder.conv1.bias": (d,),
         "model.encoder.conv2.weight": (d, d * 3), "model.encoder.conv2.bias": (d,),
         "model.encoder.layer_norm.weight": (d,), "model.encoder.layer_norm.bias": (d,),
         "model.decoder.embed_tokens.weight": (V, d), "model.decoder.embed_positions.weight": (cfg["max_positions"], d),
         "model.decoder.layer_norm.weight": (d,), "model.decoder.layer_norm.bias": (d,)}

    def attn(p):
        s[p + ".q_proj.weight"] = (d, d); s[p + ".q_proj.bias"] = (d,)
        s[p + ".k_proj.weight"] = (d, d)
        s[p + ".v_proj.weight"] = (d, d); s[p + ".v_proj.bias"] = (d,)
        s[p + ".out_proj.weight"] = (d, d); s[p + ".out_proj.bias"] = (d,)

    def ln(p):
        s[p + ".weight"] = (d,); s[p + ".bias"] = (d,)

    def mlp(p):
        s[p + ".fc1.weight"] = (ffn, d); s[p + ".fc1.bias"] = (ffn,)
        s[p + ".fc2.weight"] = (d, ffn); s[p + ".fc2.bias"] = (d,)

    for i in range(cfg["enc_layers"]):
        p = f"model.encoder.layers.{i}"
        attn(p + ".self_attn"); ln(p + ".self_attn_layer_norm"); mlp(p); ln(p + ".final_layer_norm")
    for i in range(cfg["dec_layers"]):
        p = f"model.decoder.layers.{i}"
        attn(p + ".self_attn"); ln(p + ".self_attn_layer_norm")
        attn(p + ".encoder_attn"); ln(p + ".encoder_attn_layer_norm")
        mlp(p); ln(p + ".final_layer_norm")
    return s


def synth_weights(cfg, seed=1234, sigma=0.02):
    """Seeded weights: matrices ~N(0, sigma) (Irwin-Hall), norm gains 1 + N(0, sigma), biases N(0, sigma)."""
    w = {}
    for tid, (name, shape) in enumerate(sorted(weight_shapes(cfg).items())):
        gain = name.endswith("layer_norm.weight")
        w[name] = O.synth_normal(seed, 0x200000 + tid, shape, sigma, 1.0 if gain else 0.0)
    return w

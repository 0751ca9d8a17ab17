"""Model and decode session: thin ctypes wrappers over the session API of libluminal_b200.so.
A `Model` holds the weights of an NN.Llama / NN.Phi3 shaped decoder (src/NN.jl:417-507); a
`Session` owns the KV cache and replaces the per-token generation loop
(examples/llama.jl:73-99, src/Decoding.jl:91-130)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import BF16, COLMAJOR, F32, ROWMAJOR, ModelConfig


def _dtype_code(dtype):
    if dtype in (F32, "f32", "float32", np.float32):
        return F32
    if dtype in (BF16, "bf16", "bfloat16"):
        return BF16
    raise ValueError(f"dtype {dtype!r}: expected 'f32' or 'bf16'")


class Model:
    def __init__(self, device, *, n_layers, hidden, n_heads, n_kv_heads, intermediate, vocab,
                 eps=1e-5, rope_base=10000.0, dtype="f32", tp_size=1, tp_rank=0, arch=0, max_positions=0,
                 cross_len=0):
        self.device = device
        self.cfg = ModelConfig(n_layers=n_layers, hidden=hidden, n_heads=n_heads, n_kv_heads=n_kv_heads,
                               head_dim=hidden // n_heads, intermediate=intermediate, vocab=vocab,
                               rms_eps=eps, rope_base=rope_base, dtype=_dtype_code(dtype),
                               tp_size=tp_size, tp_rank=tp_rank, arch=arch, max_positions=max_positions,
                               cross_len=cross_len)
        h = C.c_uint64(0)
        _lib.call("lmb200_model_create", device.handle, C.byref(self.cfg), C.byref(h))
        self.handle = h

    @classmethod
    def adopt(cls, device, handle, *, n_layers, hidden, n_heads, n_kv_heads, intermediate, vocab, eps, rope_base, dtype,
              arch=0, max_positions=0, cross_len=0):
        """Wraps a model handle the library created (lmb200_compile_node_list)."""
        self = cls.__new__(cls)
        self.device = device
        self.cfg = ModelConfig(n_layers=n_layers, hidden=hidden, n_heads=n_heads, n_kv_heads=n_kv_heads,
                               head_dim=hidden // n_heads, intermediate=intermediate, vocab=vocab, rms_eps=eps,
                               rope_base=rope_base, dtype=_dtype_code(dtype), tp_size=1, tp_rank=0, arch=arch,
                               max_positions=max_positions, cross_len=cross_len)
        self.handle = C.c_uint64(int(handle))
        return self

    def set_weight(self, name, array, layout=ROWMAJOR):
        a = np.asarray(array, dtype=np.float32)
        host = np.asfortranarray(a) if layout == COLMAJOR else np.ascontiguousarray(a)
        _lib.call("lmb200_model_set_weight", self.handle, name.encode(), host.ctypes.data_as(C.c_void_p),
                  a.ndim, _lib.dims(a.shape), layout)

    def missing_weights(self):
        """Registry names of the model's tensors that nothing has set yet."""
        n = C.c_int32(0)
        buf = C.create_string_buffer(1 << 20)
        _lib.call("lmb200_model_missing_weights", self.handle, buf, len(buf), C.byref(n))
        names = [s for s in buf.value.decode().split("\n") if s]
        return names if len(names) == n.value else names + [f"... and {n.value - len(names)} more"]

    def set_weights(self, weights, layout=ROWMAJOR):
        for name, a in weights.items():
            self.set_weight(name, a, layout)

    def init_random(self, seed=1234, sigma=0.02):
        _lib.call("lmb200_model_init_random", self.handle, int(seed), float(sigma))

    def weight_bytes(self):
        n = C.c_int64(0)
        _lib.call("lmb200_model_weight_bytes", self.handle, C.byref(n))
        return n.value

    def close(self):
        if self.handle:
            _lib.call("lmb200_model_destroy", self.handle)
            self.handle = C.c_uint64(0)


def WhisperDecoderModel(device, *, d_model, heads, layers, ffn, vocab, max_positions, cross_len, dtype="f32"):
    """The Whisper TextDecoder (src/Whisper.jl:449-502) for cached decoding: LayerNorm, biases, GELU
    MLP, learned positions, tied-embedding head.  Weights by their registry names
    (model.decoder.*); the cross K/V of every layer go to Session.set_cross_kv."""
    return Model(device, n_layers=layers, hidden=d_model, n_heads=heads, n_kv_heads=heads, intermediate=ffn,
                 vocab=vocab, eps=1e-5, rope_base=10000.0, dtype=dtype, arch=1, max_positions=max_positions,
                 cross_len=cross_len)


class Session:
    def __init__(self, model, batch, max_ctx):
        self.model, self.batch, self.max_ctx = model, int(batch), int(max_ctx)
        h = C.c_uint64(0)
        _lib.call("lmb200_session_create", model.handle, self.batch, self.max_ctx, C.byref(h))
        self.handle = h

    @classmethod
    def adopt(cls, model, handle, batch, max_ctx):
        """Wraps a session handle the library created (lmb200_compile_node_list)."""
        self = cls.__new__(cls)
        self.model, self.batch, self.max_ctx = model, int(batch), int(max_ctx)
        self.handle = C.c_uint64(int(handle))
        return self

    @property
    def vocab(self):
        return self.model.cfg.vocab

    def reset(self):
        _lib.call("lmb200_session_reset", self.handle)

    def position(self):
        p = C.c_int32(0)
        _lib.call("lmb200_session_position", self.handle, C.byref(p))
        return p.value

    def set_position(self, pos):
        _lib.call("lmb200_session_set_position", self.handle, int(pos))

    def positions(self):
        """One position per sequence."""
        p = (C.c_int32 * self.batch)()
        _lib.call("lmb200_session_positions", self.handle, p)
        return np.array(p[:], dtype=np.int32)

    def set_positions(self, pos):
        p = (C.c_int32 * self.batch)(*[int(v) for v in pos])
        _lib.call("lmb200_session_set_positions", self.handle, p)

    def prefill_ragged(self, prompts, want_logits=True):
        """Prompts of different lengths, one per sequence (a list of 1-D id arrays).  Returns, per sequence,
        the logits of its own last prompt position ([batch, vocab]); decoding then goes on with one position
        per sequence."""
        assert len(prompts) == self.batch
        lens = np.array([len(p) for p in prompts], dtype=np.int32)
        n_max = int(lens.max())
        t = np.zeros((self.batch, n_max), dtype=np.int32)
        for b, p in enumerate(prompts):
            t[b, :len(p)] = np.asarray(p, dtype=np.int32)
        logits = np.empty((self.batch, self.vocab), dtype=np.float32) if want_logits else None
        _lib.call("lmb200_prefill_ragged", self.handle, t.ctypes.data_as(C.c_void_p), lens.ctypes.data_as(C.c_void_p), n_max,
                  logits.ctypes.data_as(C.c_void_p) if want_logits else None)
        return logits

    def fill_kv_random(self, n_pos, seed=1234):
        _lib.call("lmb200_session_fill_kv_random", self.handle, int(n_pos), int(seed))

    def set_cross_kv(self, layer, k, v, layout=ROWMAJOR):
        """Whisper: cross-attention K (already scaled) and V of one layer, [batch, heads, T, head_dim]."""
        k = np.asarray(k, dtype=np.float32)
        v = np.asarray(v, dtype=np.float32)
        if layout == COLMAJOR:
            k, v = np.asfortranarray(k), np.asfortranarray(v)
        else:
            k, v = np.ascontiguousarray(k), np.ascontiguousarray(v)
        _lib.call("lmb200_session_set_cross_kv", self.handle, int(layer), k.ctypes.data_as(C.c_void_p),
                  v.ctypes.data_as(C.c_void_p), layout)

    def set_capture(self, enable=True):
        _lib.call("lmb200_session_set_capture", self.handle, int(bool(enable)))

    def layer_output(self, layer):
        out = np.empty((self.batch, self.model.cfg.hidden), dtype=np.float32)
        _lib.call("lmb200_session_read_layer_output", self.handle, int(layer), out.ctypes.data_as(C.c_void_p))
        return out

    def prefill(self, tokens, want_logits=True):
        t = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32))
        assert t.ndim == 2 and t.shape[0] == self.batch, "tokens must be [batch, n]"
        logits = np.empty((self.batch, self.vocab), dtype=np.float32) if want_logits else None
        _lib.call("lmb200_prefill", self.handle, t.ctypes.data_as(C.c_void_p), t.shape[1],
                  logits.ctypes.data_as(C.c_void_p) if want_logits else None)
        return logits

    def decode_step(self, tokens, want_logits=False):
        t = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32).reshape(self.batch))
        nxt = np.empty(self.batch, dtype=np.int32)
        logits = np.empty((self.batch, self.vocab), dtype=np.float32) if want_logits else None
        _lib.call("lmb200_decode_step", self.handle, t.ctypes.data_as(C.c_void_p), nxt.ctypes.data_as(C.c_void_p),
                  logits.ctypes.data_as(C.c_void_p) if want_logits else None)
        return (nxt, logits) if want_logits else nxt

    def decode_step_raw(self, tokens_in_ptr, next_out_ptr):
        """Host buffers by address (pinned memory of the caller): the end-to-end timed call."""
        _lib.call("lmb200_decode_step", self.handle, C.c_void_p(tokens_in_ptr), C.c_void_p(next_out_ptr), None)

    def decode_n(self, first_tokens, n_steps):
        first = None
        if first_tokens is not None:
            first = np.ascontiguousarray(np.asarray(first_tokens, dtype=np.int32).reshape(self.batch))
        out = np.empty((n_steps, self.batch), dtype=np.int32)
        _lib.call("lmb200_decode_n", self.handle, first.ctypes.data_as(C.c_void_p) if first is not None else None,
                  int(n_steps), out.ctypes.data_as(C.c_void_p))
        return out

    def decode_until(self, first_tokens, max_steps, eot_token):
        """Greedy steps until every sequence has produced eot_token or max_steps (or the context) run out:
        greedy_decode's loop (src/Decoding.jl:91-130).  Returns tokens [steps_done, batch]; a sequence
        that finished early is padded with eot_token."""
        first = None
        if first_tokens is not None:
            first = np.ascontiguousarray(np.asarray(first_tokens, dtype=np.int32).reshape(self.batch))
        out = np.empty((max_steps, self.batch), dtype=np.int32)
        done = C.c_int32(0)
        _lib.call("lmb200_decode_until", self.handle, first.ctypes.data_as(C.c_void_p) if first is not None else None,
                  int(max_steps), int(eot_token), out.ctypes.data_as(C.c_void_p), C.byref(done))
        return out[:done.value]

    def decode_n_device(self, first_tokens_dptr, n_steps, tokens_out_dptr=None):
        _lib.call("lmb200_decode_n_device", self.handle, C.c_void_p(first_tokens_dptr or 0), int(n_steps),
                  C.c_void_p(tokens_out_dptr or 0))

    def step_bytes(self, T):
        n = C.c_int64(0)
        _lib.call("lmb200_session_step_bytes", self.handle, int(T), C.byref(n))
        return n.value

    def decode_attention(self, layer, q_dptr, out_dptr, T):
        _lib.call("lmb200_decode_attention_splitkv", self.handle, int(layer), C.c_void_p(q_dptr),
                  C.c_void_p(out_dptr), int(T))

    def kv_layer(self, layer):
        """(device address, batch stride, head stride) of one layer of the tiled KV cache."""
        p, bs, hs = C.c_void_p(0), C.c_int64(0), C.c_int64(0)
        _lib.call("lmb200_session_kv_layer", self.handle, int(layer), C.byref(p), C.byref(bs), C.byref(hs))
        return p.value, bs.value, hs.value

    def close(self):
        if self.handle:
            _lib.call("lmb200_session_destroy", self.handle)
            self.handle = C.c_uint64(0)


def greedy_generate(session, prompt, n_steps, want_logits=False):
    """Prompt then n_steps greedy tokens: what examples/llama.jl's generation loop does, with the
    KV cache the reference lacks for Llama.  Returns tokens [batch, n_steps] (and the logits that
    produced them, [batch, n_steps, vocab])."""
    logits = session.prefill(prompt)
    toks, lgs = [], []
    for step in range(n_steps):
        nxt = np.argmax(logits, axis=-1).astype(np.int32)
        toks.append(nxt)
        lgs.append(logits)
        if step + 1 < n_steps:
            _, logits = _step_logits(session, nxt)
    t = np.stack(toks, axis=1)
    return (t, np.stack(lgs, axis=1)) if want_logits else t


def decode_attention_noalloc(device, dtype, q_dptr, out_dptr, kv_layer_dptr, kv_batch_stride, kv_head_stride,
                             batch, n_kv_heads, group, head_dim, T):
    """Split-KV decode attention whose scratch is an array inside the library: for callers that
    cannot let the library allocate device memory.  Asynchronous; see include/luminal_b200.h."""
    _lib.call("lmb200_decode_attention_noalloc", device.handle, _dtype_code(dtype), C.c_void_p(q_dptr),
              C.c_void_p(out_dptr), C.c_void_p(kv_layer_dptr), int(kv_batch_stride), int(kv_head_stride),
              int(batch), int(n_kv_heads), int(group), int(head_dim), int(T))


def _step_logits(session, tokens):
    # the logits of the step that consumed `tokens`
    nxt, logits = session.decode_step(tokens, want_logits=True)
    return nxt, logits


__all__ = ["Model", "Session", "greedy_generate", "decode_attention_noalloc", "shard_layout", "linear_gemv",
           "WhisperDecoderModel"]


def shard_layout(cfg_kwargs, matrix, tp_size=1, tp_rank=0):
    """Host-only: (rows, cols, row_map, col_map) of this rank's fused matrix `matrix`
    ('qkv', 'o', 'gate_up', 'down', 'head').  row_map[i] = (slot, logical row), col_map[k] =
    logical column; -1 marks padding.  Needs no GPU."""
    idx = {"qkv": 0, "o": 1, "gate_up": 2, "down": 3, "head": 4}[matrix]
    cfg = ModelConfig(n_layers=cfg_kwargs["n_layers"], hidden=cfg_kwargs["hidden"], n_heads=cfg_kwargs["n_heads"],
                      n_kv_heads=cfg_kwargs["n_kv_heads"], head_dim=cfg_kwargs["hidden"] // cfg_kwargs["n_heads"],
                      intermediate=cfg_kwargs["intermediate"], vocab=cfg_kwargs["vocab"], rms_eps=1e-5,
                      rope_base=10000.0, dtype=F32, tp_size=tp_size, tp_rank=tp_rank)
    rows, cols = C.c_int32(0), C.c_int32(0)
    _lib.call("lmb200_shard_extent", C.byref(cfg), idx, C.byref(rows), C.byref(cols))
    s, r, c = C.c_int32(0), C.c_int32(0), C.c_int32(0)
    row_map, col_map = [], []
    for i in range(rows.value):
        _lib.call("lmb200_shard_map", C.byref(cfg), idx, i, 0, C.byref(s), C.byref(r), C.byref(c))
        row_map.append((s.value, r.value))
    for k in range(cols.value):
        _lib.call("lmb200_shard_map", C.byref(cfg), idx, 0, k, C.byref(s), C.byref(r), C.byref(c))
        col_map.append(c.value)
    return rows.value, cols.value, row_map, col_map


def linear_gemv(device, w, x, dtype="bf16", variant=0):
    """out[b, o] = sum_i x[b, i] * w[o, i] through the decode GEMV kernel (host arrays in and out).
    variant is reserved (0)."""
    w = np.ascontiguousarray(np.asarray(w, dtype=np.float32))
    x = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
    rows, K = w.shape
    batch = x.shape[0]
    assert x.shape[1] == K
    out = np.empty((batch, rows), dtype=np.float32)
    _lib.call("lmb200_linear_gemv", device.handle, _dtype_code(dtype), int(variant), rows, K, batch,
              w.ctypes.data_as(C.c_void_p), x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p))
    return out


def prefill_gemm(device, w, x):
    """out[t, o] = sum_i x[t, i] * w[o, i] through the tensor-core prompt GEMM (bf16 operands)."""
    w = np.ascontiguousarray(np.asarray(w, dtype=np.float32))
    x = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
    rows, K = w.shape
    assert x.shape[1] == K
    out = np.empty((x.shape[0], rows), dtype=np.float32)
    _lib.call("lmb200_prefill_gemm", device.handle, rows, K, x.shape[0], w.ctypes.data_as(C.c_void_p),
              x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p))
    return out

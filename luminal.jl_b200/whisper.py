"""Whisper as graph builders: the Python stand-in for src/Whisper.jl:208-404, 406-742, 809-831 and for
NN.Conv1D (src/NN.jl:38-104) -- sinusoids, self attention, encoder blocks, AudioEncoder,
project_cross_kv, TextDecoder and its incremental decode-step graph -- with the model sizes as arguments instead of the reference's hard-coded
whisper-tiny constants (src/Whisper.jl:195-206).  The encoder and the cross-K/V projection run
once per utterance through execute() (one device call per node); the per-token decoder runs in
the fused session (session.WhisperDecoderModel).

One deliberate difference: a Linear bias on a [batch, seq, out] tensor is added as a broadcast
over the last dim.  The reference expands it along dim 1 to the batch size, which only has the
right shape for batch 1 (src/NN.jl:27-33; greedy_decode asserts batch == 1, src/Decoding.jl:43)."""
from __future__ import annotations

import math

import numpy as np

from . import graph as G

F32 = np.float32


class WLinear:
    def __init__(self, in_features, out_features, graph, reg, prefix, bias=True):
        self.weight = G.tensor(graph, [out_features, in_features])
        reg[f"{prefix}.weight"] = self.weight
        self.bias = None
        if bias:
            self.bias = G.tensor(graph, [out_features])
            reg[f"{prefix}.bias"] = self.bias

    def __call__(self, x):
        out = G.matmul(x, G.permute(self.weight, [2, 1]))
        return out + self.bias if self.bias is not None else out


class WLayerNorm:
    def __init__(self, dim, graph, reg, prefix, epsilon=1e-5):
        self.weight = G.tensor(graph, [dim])
        self.bias = G.tensor(graph, [dim])
        reg[f"{prefix}.weight"], reg[f"{prefix}.bias"] = self.weight, self.bias
        self.epsilon = epsilon

    def __call__(self, x):            # src/NN.jl:138-173
        axis = len(x.shape)
        out = G.std_norm(G.mean_norm(x, axis), axis, self.epsilon)
        w, b = self.weight, self.bias
        for i in range(1, len(out.shape)):
            w = G.expand(w, i, out.shape[i - 1])
            b = G.expand(b, i, out.shape[i - 1])
        return out * w + b


class Conv1D:                          # src/NN.jl:38-104
    def __init__(self, ch_in, ch_out, kernel, graph, reg, prefix, stride=1, padding=0):
        self.weight = G.tensor(graph, [ch_out, ch_in * kernel])
        self.bias = G.tensor(graph, [ch_out])
        reg[f"{prefix}.weight"], reg[f"{prefix}.bias"] = self.weight, self.bias
        self.kernel, self.stride, self.padding = kernel, stride, padding

    def __call__(self, x):             # x: [batch, channels, length]
        rank = len(x.shape)
        padded = G.pad_along(x, rank, self.padding, self.padding) if self.padding > 0 else x
        unfolded = G.unfold(padded, [self.kernel], [self.stride], [1])           # [B, C, O, K]
        perm = G.permute(unfolded, [1, 3, 2, 4])                                 # [B, O, C, K]
        B, O, C, K = perm.shape
        merged = G.reshape(perm, [B, O, C * K])                                  # column-major: c + C*k
        out = G.matmul(merged, G.permute(self.weight, [2, 1]))                   # [B, O, ch_out]
        out = G.permute(out, [1, 3, 2])                                          # [B, ch_out, O]
        b = G.expand(G.expand(self.bias, 1, out.shape[0]), 3, out.shape[2])
        return out + b


def sinusoids(channels, length, graph):          # src/Whisper.jl:208-231
    inc = math.log(10000.0) / (channels / 2 - 1)
    inv_ts = np.array([math.exp(-inc * i) for i in range(channels // 2)], dtype=F32)
    inv = G.tensor(graph, [channels // 2])
    graph.tensors[(inv.id, 1)] = inv_ts
    scaled = G.expand(G.arange(graph, length), 2, channels // 2) * G.expand(inv, 1, length)
    return G.concat_along(G.sin(scaled), G.cos(scaled), 2)


class WhisperSelfAttention:                      # src/Whisper.jl:238-276
    def __init__(self, hidden, heads, graph, reg, prefix):
        self.q_proj = WLinear(hidden, hidden, graph, reg, f"{prefix}.q_proj", bias=True)
        self.k_proj = WLinear(hidden, hidden, graph, reg, f"{prefix}.k_proj", bias=False)
        self.v_proj = WLinear(hidden, hidden, graph, reg, f"{prefix}.v_proj", bias=True)
        self.o_proj = WLinear(hidden, hidden, graph, reg, f"{prefix}.out_proj", bias=True)
        self.heads = heads

    def __call__(self, x, mask):
        batch, seq, hidden = x.shape
        H, D = self.heads, hidden // self.heads
        scale = F32(F32(F32(hidden) / F32(H)) ** F32(-0.25))
        q = G.permute(G.reshape(self.q_proj(x) * scale, [batch, seq, H, D]), [1, 3, 2, 4])
        k = G.permute(G.reshape(self.k_proj(x) * scale, [batch, seq, H, D]), [1, 3, 4, 2])
        v = G.permute(G.reshape(self.v_proj(x), [batch, seq, H, D]), [1, 3, 2, 4])
        weights = G.matmul(q, k)
        if mask:
            m = G.triu(x.graph_ref, seq, 1) * F32(-1e9)
            weights = weights + G.expand(G.expand(m, 1, H), 1, batch)
        out = G.matmul(G.softmax(weights, 4), v)
        return self.o_proj(G.reshape(G.permute(out, [1, 3, 2, 4]), [batch, seq, hidden]))


class EncoderTransformerBlock:                   # src/Whisper.jl:322-352
    """Registry names: the checkpoint's (self_attn.*, self_attn_layer_norm.*, fc1.*, fc2.*) by default; with
    reference_names the ones the reference's encoder block registers (attn.*, attn_layer_norm.*, mlp.fc1.*, mlp.fc2.*,
    src/Whisper.jl:330-336).  The library takes either spelling."""

    def __init__(self, hidden, heads, ff, graph, reg, prefix, reference_names=False):
        attn, norm, fc1, fc2 = (("attn", "attn_layer_norm", "mlp.fc1", "mlp.fc2") if reference_names else
                                ("self_attn", "self_attn_layer_norm", "fc1", "fc2"))
        self.attn = WhisperSelfAttention(hidden, heads, graph, reg, f"{prefix}.{attn}")
        self.attn_norm = WLayerNorm(hidden, graph, reg, f"{prefix}.{norm}")
        self.ff1 = WLinear(hidden, ff, graph, reg, f"{prefix}.{fc1}")
        self.ff2 = WLinear(ff, hidden, graph, reg, f"{prefix}.{fc2}")
        self.ff_norm = WLayerNorm(hidden, graph, reg, f"{prefix}.final_layer_norm")

    def __call__(self, x):
        x = x + self.attn(self.attn_norm(x), False)
        return x + self.ff2(G.gelu(self.ff1(self.ff_norm(x))))


class AudioEncoder:                              # src/Whisper.jl:354-404
    def __init__(self, graph, reg, *, d_model, heads, layers, ffn, n_mels, reference_names=False):
        pfx = "model.encoder"
        self.d_model = d_model
        self.conv1 = Conv1D(n_mels, d_model, 3, graph, reg, f"{pfx}.conv1", stride=1, padding=1)
        self.conv2 = Conv1D(d_model, d_model, 3, graph, reg, f"{pfx}.conv2", stride=2, padding=1)
        self.layers = [EncoderTransformerBlock(d_model, heads, ffn, graph, reg, f"{pfx}.layers.{i}", reference_names)
                       for i in range(layers)]
        self.post_ln = WLayerNorm(d_model, graph, reg, f"{pfx}.layer_norm")

    def __call__(self, x):                       # x: [batch, n_mels, frames]
        x = G.gelu(self.conv1(x))
        x = G.gelu(self.conv2(x))
        x = G.permute(x, [1, 3, 2])
        x = x + G.expand(sinusoids(self.d_model, x.shape[1], x.graph_ref), 1, x.shape[0])
        for layer in self.layers:
            x = layer(x)
        return self.post_ln(x)


def project_cross_kv(graph, reg, enc_output, *, d_model, heads, layers):     # src/Whisper.jl:809-831
    """[(K, V)] per decoder layer, each [batch, heads, seq, head_dim]; K carries head_dim^-0.25."""
    batch, seq, _ = enc_output.shape
    D = d_model // heads
    scale = F32(F32(F32(d_model) / F32(heads)) ** F32(-0.25))
    out = []
    for i in range(layers):
        p = f"model.decoder.layers.{i}.encoder_attn"
        k_proj = WLinear(d_model, d_model, graph, reg, f"{p}.k_proj", bias=False)
        v_proj = WLinear(d_model, d_model, graph, reg, f"{p}.v_proj", bias=True)
        k = G.permute(G.reshape(k_proj(enc_output) * scale, [batch, seq, heads, D]), [1, 3, 2, 4])
        v = G.permute(G.reshape(v_proj(enc_output), [batch, seq, heads, D]), [1, 3, 2, 4])
        out.append((k, v))
    return out


# ---------------------------------------------------------------------------------------------
# TextDecoder and its incremental decode-step graph (src/Whisper.jl:406-742)
# ---------------------------------------------------------------------------------------------
class WhisperCrossAttention:                     # src/Whisper.jl:282-316 (parameters; the cached call is below)
    def __init__(self, hidden, heads, graph, reg, prefix):
        self.q_proj = WLinear(hidden, hidden, graph, reg, f"{prefix}.q_proj", bias=True)
        self.k_proj = WLinear(hidden, hidden, graph, reg, f"{prefix}.k_proj", bias=False)
        self.v_proj = WLinear(hidden, hidden, graph, reg, f"{prefix}.v_proj", bias=True)
        self.o_proj = WLinear(hidden, hidden, graph, reg, f"{prefix}.out_proj", bias=True)
        self.heads = heads

    def __call__(self, queries_t, keys_t, values_t):      # src/Whisper.jl:297-316: projects the encoder output itself
        batch, dec_seq, hidden = queries_t.shape
        enc_seq = keys_t.shape[1]
        H, D = self.heads, hidden // self.heads
        scale = F32(F32(F32(hidden) / F32(H)) ** F32(-0.25))
        q = G.permute(G.reshape(self.q_proj(queries_t) * scale, [batch, dec_seq, H, D]), [1, 3, 2, 4])
        k = G.contiguous(G.permute(G.reshape(self.k_proj(keys_t) * scale, [batch, enc_seq, H, D]), [1, 3, 4, 2]))
        v = G.permute(G.reshape(self.v_proj(values_t), [batch, enc_seq, H, D]), [1, 3, 2, 4])
        out = G.matmul(G.softmax(G.matmul(q, k), 4), v)
        return self.o_proj(G.reshape(G.permute(out, [1, 3, 2, 4]), [batch, dec_seq, hidden]))


class DecoderTransformerBlock:                   # src/Whisper.jl:410-432
    def __init__(self, hidden, heads, ff, graph, reg, prefix):
        self.attn = WhisperSelfAttention(hidden, heads, graph, reg, f"{prefix}.self_attn")
        self.attn_norm = WLayerNorm(hidden, graph, reg, f"{prefix}.self_attn_layer_norm")
        self.cross_attn = WhisperCrossAttention(hidden, heads, graph, reg, f"{prefix}.encoder_attn")
        self.cross_attn_norm = WLayerNorm(hidden, graph, reg, f"{prefix}.encoder_attn_layer_norm")
        self.ff1 = WLinear(hidden, ff, graph, reg, f"{prefix}.fc1")
        self.ff2 = WLinear(ff, hidden, graph, reg, f"{prefix}.fc2")
        self.ff_norm = WLayerNorm(hidden, graph, reg, f"{prefix}.final_layer_norm")

    def __call__(self, x, encoded):                       # src/Whisper.jl:433-443: no cache, causal mask
        x = x + self.attn(self.attn_norm(x), True)
        x = x + self.cross_attn(self.cross_attn_norm(x), encoded, encoded)
        return x + self.ff2(G.gelu(self.ff1(self.ff_norm(x))))


class TextDecoder:                               # src/Whisper.jl:449-486
    def __init__(self, graph, reg, *, d_model, heads, layers, ffn, vocab, max_positions):
        pfx = "model.decoder"
        self.d_model, self.heads, self.max_positions = d_model, heads, max_positions
        self.embedding = G.tensor(graph, [vocab, d_model])
        self.pos_embedding = G.tensor(graph, [max_positions, d_model])
        reg[f"{pfx}.embed_tokens.weight"], reg[f"{pfx}.embed_positions.weight"] = self.embedding, self.pos_embedding
        self.layers = [DecoderTransformerBlock(d_model, heads, ffn, graph, reg, f"{pfx}.layers.{i}") for i in range(layers)]
        self.layer_norm = WLayerNorm(d_model, graph, reg, f"{pfx}.layer_norm")

    def __call__(self, enc_output, tokens):               # src/Whisper.jl:488-505: the whole prefix at once
        x = G.gather(self.embedding, tokens)
        cur_seq = tokens.shape[1]
        pos = G.contiguous(G.slice_along(self.pos_embedding, 1, 0, cur_seq))
        x = x + G.expand(pos, 1, x.shape[0])
        for layer in self.layers:
            x = layer(x, enc_output)
        return G.matmul(self.layer_norm(x), G.permute(self.embedding, [2, 1]))


class KVCacheState:                              # src/Whisper.jl:519-541
    """Host-side state of one decode session driven graph by graph: the position and, per layer, the self K/V
    [batch, heads, max_seq, head_dim] (zeroed) and the cross K/V [batch, heads, enc_seq, head_dim]."""

    def __init__(self, batch, n_layers, n_heads, head_dim, enc_seq, max_seq):
        z = lambda s: np.zeros((batch, n_heads, s, head_dim), F32)
        self.step_pos, self.max_seq = 0, max_seq
        self.self_cache = [(z(max_seq), z(max_seq)) for _ in range(n_layers)]
        self.cross_cache = [(z(enc_seq), z(enc_seq)) for _ in range(n_layers)]


def decode_step(exec_obj, idg, cache, token_ids, cross_kv_arrays, device=None):      # src/Whisper.jl:760-801
    """One step of the incremental decode graph `idg` (built for cache.step_pos): exec_obj is the Graph (run through
    execute) or its CompiledGraph; the cache's self K/V are replaced by the step's updated ones and its position
    advances.  Returns the logits [batch, 1, vocab].  The cached session (Session.decode_step) is the fast form of the
    same step; this one is the reference's host loop kept call for call."""
    from .execution import execute
    inputs = {idg.token_input_id: np.asarray(token_ids, F32)}
    for i, (ck, cv) in enumerate(cross_kv_arrays):
        inputs[idg.cross_k_ids[i]], inputs[idg.cross_v_ids[i]] = ck, cv
    for i in range(len(idg.self_k_ids)):
        inputs[idg.self_k_ids[i]], inputs[idg.self_v_ids[i]] = cache.self_cache[i]
    want = [idg.logits_id] + list(idg.new_self_k_ids) + list(idg.new_self_v_ids)
    if isinstance(exec_obj, G.Graph):
        result = execute(exec_obj, want, inputs, device)
    else:
        bufs = exec_obj(inputs, device)
        result = {i: bufs[i].numpy() for i in want}
    for i in range(len(idg.new_self_k_ids)):
        cache.self_cache[i] = (result[idg.new_self_k_ids[i]], result[idg.new_self_v_ids[i]])
    cache.step_pos += 1
    return result[idg.logits_id]


def _kv_scatter(past, new_slot, step_pos):       # src/Whisper.jl:541-570: slice-and-concat write of one cache slot
    max_seq = past.shape[2]
    if step_pos == 0:
        return G.concat_along(new_slot, G.slice_along(past, 3, 1, max_seq), 3)
    head = G.concat_along(G.slice_along(past, 3, 0, step_pos), new_slot, 3)
    if max_seq - step_pos - 1 == 0:
        return head
    return G.concat_along(head, G.slice_along(past, 3, step_pos + 1, max_seq), 3)


def whisper_self_attn_cached(sa, x, step_pos, past_k, past_v):       # src/Whisper.jl:584-625
    batch, _, hidden = x.shape
    H, D = sa.heads, hidden // sa.heads
    scale = F32(F32(F32(hidden) / F32(H)) ** F32(-0.25))
    q = G.permute(G.reshape(sa.q_proj(x) * scale, [batch, 1, H, D]), [1, 3, 2, 4])
    k_new = G.contiguous(G.permute(G.reshape(sa.k_proj(x) * scale, [batch, 1, H, D]), [1, 3, 2, 4]))
    v_new = G.permute(G.reshape(sa.v_proj(x), [batch, 1, H, D]), [1, 3, 2, 4])
    new_k, new_v = _kv_scatter(past_k, k_new, step_pos), _kv_scatter(past_v, v_new, step_pos)
    k_ctx = G.slice_along(new_k, 3, 0, step_pos + 1)
    v_ctx = G.slice_along(new_v, 3, 0, step_pos + 1)
    probs = G.softmax(G.matmul(q, G.contiguous(G.permute(k_ctx, [1, 2, 4, 3]))), 4)
    out = G.reshape(G.permute(G.matmul(probs, v_ctx), [1, 3, 2, 4]), [batch, 1, hidden])
    return sa.o_proj(out), new_k, new_v


def whisper_cross_attn_cached(ca, x, enc_k, enc_v):                  # src/Whisper.jl:633-651
    batch, _, hidden = x.shape
    H, D = ca.heads, hidden // ca.heads
    scale = F32(F32(F32(hidden) / F32(H)) ** F32(-0.25))
    q = G.permute(G.reshape(ca.q_proj(x) * scale, [batch, 1, H, D]), [1, 3, 2, 4])
    probs = G.softmax(G.matmul(q, G.contiguous(G.permute(enc_k, [1, 2, 4, 3]))), 4)
    out = G.reshape(G.permute(G.matmul(probs, enc_v), [1, 3, 2, 4]), [batch, 1, hidden])
    return ca.o_proj(out)


class IncrementalDecodeGraph:                    # src/Whisper.jl:662-672: node ids for driving one step
    def __init__(self, **kw):
        self.__dict__.update(kw)


def build_decode_step(td, graph, enc_seq, step_pos, *, max_seq=None, batch=1):     # src/Whisper.jl:687-742
    """One step of the incremental decode graph for position `step_pos` (baked into the slice positions, so the
    reference builds one graph per position).  Inputs: the token [batch, 1], per layer the cross K/V [batch, heads,
    enc_seq, head_dim] and the past self K/V [batch, heads, max_seq, head_dim]; outputs: logits [batch, 1, vocab] and
    the updated self K/V."""
    max_seq = max_seq or td.max_positions
    H, D, L = td.heads, td.d_model // td.heads, len(td.layers)
    token_in = G.tensor(graph, [batch, 1])
    cross_k = [G.tensor(graph, [batch, H, enc_seq, D]) for _ in range(L)]
    cross_v = [G.tensor(graph, [batch, H, enc_seq, D]) for _ in range(L)]
    self_k = [G.tensor(graph, [batch, H, max_seq, D]) for _ in range(L)]
    self_v = [G.tensor(graph, [batch, H, max_seq, D]) for _ in range(L)]
    x = G.gather(td.embedding, token_in)
    pos_slot = G.contiguous(G.slice_along(td.pos_embedding, 1, step_pos, step_pos + 1))
    x = x + G.expand(pos_slot, 1, batch)
    new_k, new_v = [], []
    for i, layer in enumerate(td.layers):
        attn_out, nk, nv = whisper_self_attn_cached(layer.attn, layer.attn_norm(x), step_pos, self_k[i], self_v[i])
        x = x + attn_out
        new_k.append(nk)
        new_v.append(nv)
        x = x + whisper_cross_attn_cached(layer.cross_attn, layer.cross_attn_norm(x), cross_k[i], cross_v[i])
        x = x + layer.ff2(G.gelu(layer.ff1(layer.ff_norm(x))))
    out = td.layer_norm(x)
    logits = G.matmul(G.contiguous(G.slice_along(out, 2, 0, 1)), G.permute(td.embedding, [2, 1]))
    ids = lambda ts: [t.id for t in ts]
    return IncrementalDecodeGraph(token_input_id=token_in.id, cross_k_ids=ids(cross_k), cross_v_ids=ids(cross_v),
                                  self_k_ids=ids(self_k), self_v_ids=ids(self_v), logits_id=logits.id,
                                  new_self_k_ids=ids(new_k), new_self_v_ids=ids(new_v), step_pos=step_pos)


def encode_cross_kv(device, weights, mel, *, d_model, heads, enc_layers, dec_layers, ffn, n_mels):
    """Runs AudioEncoder + project_cross_kv node by node on the device (execute()).  Returns the
    encoder output and the per-layer cross (K, V) as host arrays, ready for Session.set_cross_kv."""
    from .execution import execute
    g, reg = G.Graph(), {}
    mel = np.asarray(mel, dtype=F32)
    inp = G.tensor(g, mel.shape)
    enc = AudioEncoder(g, reg, d_model=d_model, heads=heads, layers=enc_layers, ffn=ffn, n_mels=n_mels)(inp)
    kv = project_cross_kv(g, reg, enc, d_model=d_model, heads=heads, layers=dec_layers)
    inputs = {t.id: weights[name] for name, t in reg.items()}
    inputs[inp.id] = mel
    ids = [enc.id] + [t.id for pair in kv for t in pair]
    res = execute(g, ids, inputs, device)
    return res[enc.id], [(res[k.id], res[v.id]) for k, v in kv]


def conv_weight_from_checkpoint(a):
    """A Conv1D weight as checkpoints store it, [ch_out, ch_in, kernel], as the [ch_out, ch_in * kernel] matrix NN.Conv1D
    multiplies by (src/NN.jl:55-104): column c + ch_in * k, which is what the reference gets when SafeTensors.jl hands it
    the tensor column-major and load_weights! copies it into the 2-D node by length.  2-D input is returned as it is."""
    a = np.asarray(a, dtype=F32)
    if a.ndim != 3:
        return a
    ch_out, ch_in, kernel = a.shape
    return np.ascontiguousarray(a.transpose(0, 2, 1).reshape(ch_out, kernel * ch_in))


def canonical_name(name):
    """The checkpoint's spelling of a Whisper registry name (lmb200_whisper_canonical_name): the reference's encoder
    blocks register attn.* / attn_layer_norm.* / mlp.fc1.* / mlp.fc2.* for what checkpoints call self_attn.* /
    self_attn_layer_norm.* / fc1.* / fc2.* (src/Whisper.jl:330-336)."""
    import ctypes as C
    from . import _lib
    out = C.create_string_buffer(len(name) + 64)
    _lib.call("lmb200_whisper_canonical_name", name.encode(), out, len(out))
    return out.value.decode()


def greedy_decode(weights, enc_output, sot_sequence, eot_id, *, d_model, heads, layers, ffn, vocab, max_positions=448,
                  max_len=448, dtype="f32", device=None):
    """greedy_decode of src/Decoding.jl:33-136 on the cached session.  The tokenizer stays with the caller: it gives
    `sot_sequence` (the start-of-transcript ids, Decoding.jl:89) and `eot_id`, and turns the returned ids into text.

    As in the reference, the cross K/V are projected once from `enc_output` [batch, enc_seq, d_model] (Decoding.jl:
    52-78), the self cache starts zeroed at max_positions slots, and the loop feeds only the LAST id of the start
    sequence at position len(sot_sequence) - 1 (Decoding.jl:92, 112): the earlier start ids never enter the cache, whose
    first slots stay zero rows that the attention still reads.  Each step takes the argmax, the loop ends after the
    step that produced eot_id, after max_len steps, or when the position reaches max_positions - 1 (Decoding.jl:93-95,
    126-129).  What the reference does with one compiled graph per position runs here as one device-resident loop.

    Returns one id list per sequence (the start sequence included, ending with eot_id if it was produced)."""
    from .device import get_device
    from .execution import execute
    from .session import Session, WhisperDecoderModel
    dev = device or get_device()
    enc_output = np.asarray(enc_output, dtype=F32)
    batch, enc_seq, _ = enc_output.shape
    start = [int(t) for t in sot_sequence]
    assert start, "greedy_decode: empty start sequence"
    g, reg = G.Graph(), {}
    enc_in = G.tensor(g, enc_output.shape)
    kv = project_cross_kv(g, reg, enc_in, d_model=d_model, heads=heads, layers=layers)
    inputs = {t.id: weights[name] for name, t in reg.items()}
    inputs[enc_in.id] = enc_output
    res = execute(g, [t.id for pair in kv for t in pair], inputs, dev)
    pos = len(start) - 1
    steps = min(int(max_len), (max_positions - 1) - pos)
    if steps <= 0:
        return [list(start) for _ in range(batch)]
    model = WhisperDecoderModel(dev, d_model=d_model, heads=heads, layers=layers, ffn=ffn, vocab=vocab, max_positions=max_positions,
                                cross_len=enc_seq, dtype=dtype)
    sess = None
    try:
        for name, a in weights.items():
            if name.startswith("model.decoder."):
                model.set_weight(name, a)
        sess = Session(model, batch, max_positions - 1)
        for i, (k, v) in enumerate(kv):
            sess.set_cross_kv(i, res[k.id], res[v.id])
        sess.set_position(pos)
        out = sess.decode_until(np.full(batch, start[-1], np.int32), steps, int(eot_id))      # [steps done, batch]
    finally:
        if sess is not None:
            sess.close()
        model.close()
    ids = []
    for b in range(batch):
        seq = [int(t) for t in out[:, b]]
        if int(eot_id) in seq:
            seq = seq[:seq.index(int(eot_id)) + 1]
        ids.append(start + seq)
    return ids


class FusedEncoder:
    """AudioEncoder + project_cross_kv on the tensor cores (bf16): the fused counterpart of
    encode_cross_kv.  Weights by the reference's registry names; names it does not use are skipped."""

    def __init__(self, device, *, d_model, heads, enc_layers, dec_layers, ffn, n_mels):
        import ctypes as C
        from . import _lib
        self._lib, self._C = _lib, C
        self.device, self.d_model = device, d_model
        h = C.c_uint64(0)
        _lib.call("lmb200_whisper_encoder_create", device.handle, d_model, heads, enc_layers, ffn, n_mels, dec_layers, C.byref(h))
        self.handle = h

    @classmethod
    def adopt(cls, device, handle, d_model):
        """Wraps an encoder handle the library created (lmb200_compile_encoder_node_list)."""
        import ctypes as C
        from . import _lib
        self = cls.__new__(cls)
        self._lib, self._C, self.device, self.d_model = _lib, C, device, int(d_model)
        self.handle = C.c_uint64(int(handle))
        return self

    def set_weights(self, weights):
        C = self._C
        used = []
        for name, a in weights.items():
            if not (name.startswith("model.encoder.") or ".encoder_attn.k_proj." in name or ".encoder_attn.v_proj." in name):
                continue
            host = np.ascontiguousarray(conv_weight_from_checkpoint(a))
            try:
                self._lib.call("lmb200_whisper_encoder_set_weight", self.handle, name.encode(), host.ctypes.data_as(C.c_void_p),
                               host.ndim, self._lib.dims(host.shape), 0)
            except self._lib.LuminalB200Error as e:
                if e.code != -7:                 # LMB200_ENOTFOUND (a decoder layer this encoder was not built for): skipped
                    raise
                continue
            used.append(name)
        return used

    def run(self, mel, want_output=True):
        """mel [batch, n_mels, frames] -> encoder output [batch, frames // 2 (rounded up), d_model] (or None)."""
        C = self._C
        mel = np.ascontiguousarray(np.asarray(mel, dtype=np.float32))
        batch, _, frames = mel.shape
        seq = (frames - 1) // 2 + 1
        out = np.empty((batch, seq, self.d_model), dtype=np.float32) if want_output else None
        self._lib.call("lmb200_whisper_encoder_run", self.handle, mel.ctypes.data_as(C.c_void_p), batch, frames,
                       out.ctypes.data_as(C.c_void_p) if want_output else None)
        return out

    def cross_kv_into(self, session):
        """Projects the last output to every decoder layer's cross K/V, straight into the session's cache."""
        self._lib.call("lmb200_whisper_encoder_cross_kv", self.handle, session.handle)

    def close(self):
        if self.handle:
            self._lib.call("lmb200_whisper_encoder_destroy", self.handle)
            self.handle = None


def registry_shapes(*, d_model, heads, enc_layers, dec_layers, ffn, vocab, n_mels, max_positions):
    """Registry name -> logical shape of every tensor of a Whisper model of these sizes, under the names
    AudioEncoder / TextDecoder register them with (src/Whisper.jl:354-404, 423-481): what a checkpoint
    has to provide, and what random initialisation fills."""
    del heads
    d = d_model
    s = {"model.encoder.conv1.weight": (d, n_mels * 3), "model.encoder.conv1.bias": (d,),
         "model.encoder.conv2.weight": (d, d * 3), "model.encoder.conv2.bias": (d,),
         "model.encoder.layer_norm.weight": (d,), "model.encoder.layer_norm.bias": (d,),
         "model.decoder.embed_tokens.weight": (vocab, d), "model.decoder.embed_positions.weight": (max_positions, d),
         "model.decoder.layer_norm.weight": (d,), "model.decoder.layer_norm.bias": (d,)}

    def attention(p):                       # k_proj has no bias (src/Whisper.jl:249)
        for n in ("q_proj", "v_proj", "out_proj"):
            s[f"{p}.{n}.weight"], s[f"{p}.{n}.bias"] = (d, d), (d,)
        s[f"{p}.k_proj.weight"] = (d, d)

    def norm(p):
        s[p + ".weight"], s[p + ".bias"] = (d,), (d,)

    def mlp(p):
        s[p + ".fc1.weight"], s[p + ".fc1.bias"] = (ffn, d), (ffn,)
        s[p + ".fc2.weight"], s[p + ".fc2.bias"] = (d, ffn), (d,)

    for i in range(enc_layers):
        p = f"model.encoder.layers.{i}"
        attention(p + ".self_attn"); norm(p + ".self_attn_layer_norm"); mlp(p); norm(p + ".final_layer_norm")
    for i in range(dec_layers):
        p = f"model.decoder.layers.{i}"
        attention(p + ".self_attn"); norm(p + ".self_attn_layer_norm")
        attention(p + ".encoder_attn"); norm(p + ".encoder_attn_layer_norm")
        mlp(p); norm(p + ".final_layer_norm")
    return s


__all__ = ["registry_shapes", "FusedEncoder", "AudioEncoder", "Conv1D", "WhisperSelfAttention", "EncoderTransformerBlock", "sinusoids", "project_cross_kv",
           "encode_cross_kv", "WhisperCrossAttention", "DecoderTransformerBlock", "TextDecoder", "KVCacheState", "decode_step", "greedy_decode", "canonical_name", "conv_weight_from_checkpoint", "build_decode_step",
           "IncrementalDecodeGraph", "whisper_self_attn_cached", "whisper_cross_attn_cached"]

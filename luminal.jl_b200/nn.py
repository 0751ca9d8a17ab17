"""NN layers and models as graph builders: the Python stand-in for src/NN.jl (Linear, Embedding,
LayerNorm/RMSNorm, Mlp, RoPE, repeat_kv, SelfAttention, TransformerBlock, Llama, Phi3), kept
call for call.  Weights are graph input tensors registered under the reference's names."""
from __future__ import annotations

import numpy as np

from . import graph as G

F32 = np.float32


class Linear:                                   # src/NN.jl:11-35
    def __init__(self, in_features, out_features, graph, bias=True, reg=None, prefix=None):
        self.weight = G.tensor(graph, [out_features, in_features])
        self.bias = G.tensor(graph, [out_features]) if bias else None
        if reg is not None:
            reg[f"{prefix}.weight"] = self.weight
            if bias:
                reg[f"{prefix}.bias"] = self.bias

    def __call__(self, x):
        out = G.matmul(x, G.permute(self.weight, [2, 1]))
        if self.bias is not None:
            out = out + G.expand(self.bias, 1, out.shape[0])
        return out


class Embedding:                                # src/NN.jl:107-118
    def __init__(self, vocab_size, embed_dim, graph, reg=None, prefix=None):
        self.weight = G.tensor(graph, [vocab_size, embed_dim])
        if reg is not None:
            reg[f"{prefix}.weight"] = self.weight

    def __call__(self, x):
        return G.gather(self.weight, x)


class LayerNorm:                                # src/NN.jl:121-173
    def __init__(self, dim, graph, weight=True, bias=True, epsilon=1e-5, mean_norm=True, reg=None, prefix=None):
        self.weight = G.tensor(graph, [dim]) if weight else None
        self.bias = G.tensor(graph, [dim]) if bias else None
        self.epsilon, self.mean_norm = float(epsilon), mean_norm
        if reg is not None:
            if weight:
                reg[f"{prefix}.weight"] = self.weight
            if bias:
                reg[f"{prefix}.bias"] = self.bias

    def __call__(self, x):
        axis = len(x.shape)
        out = x
        if self.mean_norm:
            out = G.mean_norm(out, axis)
        out = G.std_norm(out, axis, self.epsilon)
        for param, combine in ((self.weight, lambda a, b: a * b), (self.bias, lambda a, b: a + b)):
            if param is not None:
                p = param
                for i in range(1, len(out.shape)):
                    p = G.expand(p, i, out.shape[i - 1])
                out = combine(out, p)
        return out


def RMSNorm(dim, graph, epsilon=1e-5, reg=None, prefix=None):      # src/NN.jl:134-136
    return LayerNorm(dim, graph, weight=True, bias=False, epsilon=epsilon, mean_norm=False, reg=reg, prefix=prefix)


class Mlp:                                      # src/NN.jl:232-250
    def __init__(self, hidden, intermediate, graph, reg=None, prefix="mlp"):
        self.gate_proj = Linear(hidden, intermediate, graph, bias=False, reg=reg, prefix=f"{prefix}.gate_proj")
        self.down_proj = Linear(intermediate, hidden, graph, bias=False, reg=reg, prefix=f"{prefix}.down_proj")
        self.up_proj = Linear(hidden, intermediate, graph, bias=False, reg=reg, prefix=f"{prefix}.up_proj")

    def __call__(self, x):
        gate = G.silu(self.gate_proj(x))
        up = self.up_proj(x)
        return self.down_proj(gate * up)


def apply_rotary_embeddings(inp, prev_seq, base=10000.0):           # src/NN.jl:253-303
    batch, n_heads, seq, head_dim = inp.shape
    graph = inp.graph_ref
    half = head_dim // 2
    freqs = G.arange(graph, half) * F32(2.0) / F32(head_dim)
    inv_freqs = G.reciprocal(G.exp2(freqs * F32(np.log2(F32(base)))))
    pos = G.arange(graph, seq) + F32(prev_seq)
    emb = G.matmul(G.expand(pos, 2, 1), G.expand(inv_freqs, 1, 1))
    split = G.reshape(inp, [batch, n_heads, seq, half, 2])
    x0 = G.slice_along(split, 5, 0, 1)
    x1 = G.slice_along(split, 5, 1, 2)
    emb_expanded = G.expand(G.expand(emb, 1, n_heads), 1, batch)
    sin_emb = G.sin(emb_expanded)
    cos_emb = G.cos(emb_expanded)
    x0 = G.reshape(G.contiguous(x0), [batch, n_heads, seq, half])
    x1 = G.reshape(G.contiguous(x1), [batch, n_heads, seq, half])
    x0_out = x0 * cos_emb - x1 * sin_emb
    x1_out = x0 * sin_emb + x1 * cos_emb
    res = G.concat_along(G.expand(x0_out, 5, 1), G.expand(x1_out, 5, 1), 5)
    return G.reshape(res, [batch, n_heads, seq, head_dim])


def repeat_kv(keys, groups):                    # src/NN.jl:305-317
    if groups == 1:
        return keys
    batch, kv_heads, seq, head_dim = keys.shape
    return G.reshape(G.expand(keys, 3, groups), [batch, kv_heads * groups, seq, head_dim])


class SelfAttention:                            # src/NN.jl:320-387
    def __init__(self, hidden, n_heads, n_kv_heads, graph, reg=None, prefix="self_attn"):
        head_dim = hidden // n_heads
        self.q_proj = Linear(hidden, hidden, graph, bias=False, reg=reg, prefix=f"{prefix}.q_proj")
        self.k_proj = Linear(hidden, n_kv_heads * head_dim, graph, bias=False, reg=reg, prefix=f"{prefix}.k_proj")
        self.v_proj = Linear(hidden, n_kv_heads * head_dim, graph, bias=False, reg=reg, prefix=f"{prefix}.v_proj")
        self.o_proj = Linear(hidden, hidden, graph, bias=False, reg=reg, prefix=f"{prefix}.o_proj")
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim

    def __call__(self, x, prev_seq, rope_base=10000.0):
        batch, seq, hidden = x.shape
        H, KV, D = self.n_heads, self.n_kv_heads, self.head_dim
        queries = G.permute(G.reshape(self.q_proj(x), [batch, seq, H, D]), [1, 3, 2, 4])
        keys = G.permute(G.reshape(self.k_proj(x), [batch, seq, KV, D]), [1, 3, 2, 4])
        values = G.permute(G.reshape(self.v_proj(x), [batch, seq, KV, D]), [1, 3, 2, 4])
        queries = apply_rotary_embeddings(queries, prev_seq, base=rope_base)
        keys = apply_rotary_embeddings(keys, prev_seq, base=rope_base)
        if KV < H:
            keys = repeat_kv(keys, H // KV)
            values = repeat_kv(values, H // KV)
        weights = G.matmul(queries, G.permute(keys, [1, 2, 4, 3])) * (F32(1.0) / np.sqrt(F32(D)))
        if seq > 1:
            mask = G.triu(x.graph_ref, seq, 1) * F32(-1e9)
            weights = weights + G.expand(G.expand(mask, 1, H), 1, batch)
        probs = G.softmax(weights, 4)
        out = G.matmul(probs, values)
        out = G.reshape(G.permute(out, [1, 3, 2, 4]), [batch, seq, hidden])
        return self.o_proj(out)


class TransformerBlock:                         # src/NN.jl:390-414
    def __init__(self, hidden, n_heads, n_kv_heads, intermediate, graph, reg=None, prefix="block"):
        self.attention = SelfAttention(hidden, n_heads, n_kv_heads, graph, reg, f"{prefix}.self_attn")
        self.attention_norm = RMSNorm(hidden, graph, reg=reg, prefix=f"{prefix}.input_layernorm")
        self.feed_forward = Mlp(hidden, intermediate, graph, reg, f"{prefix}.mlp")
        self.feed_forward_norm = RMSNorm(hidden, graph, reg=reg, prefix=f"{prefix}.post_attention_layernorm")

    def __call__(self, x, prev_seq, rope_base=10000.0):
        x = x + self.attention(self.attention_norm(x), prev_seq, rope_base=rope_base)
        return x + self.feed_forward(self.feed_forward_norm(x))


class Llama:                                    # src/NN.jl:417-455
    ROPE_BASE = 500000.0

    def __init__(self, graph, reg=None, vocab_size=128256, hidden=4096, n_layers=32, n_heads=32, n_kv_heads=8,
                 intermediate=14336):
        self.config = dict(n_layers=n_layers, hidden=hidden, n_heads=n_heads, n_kv_heads=n_kv_heads,
                           intermediate=intermediate, vocab=vocab_size)
        self.layers = [TransformerBlock(hidden, n_heads, n_kv_heads, intermediate, graph, reg, f"model.layers.{i}")
                       for i in range(n_layers)]
        self.embedding = Embedding(vocab_size, hidden, graph, reg, "model.embed_tokens")
        self.norm = RMSNorm(hidden, graph, reg=reg, prefix="model.norm")
        self.head = Linear(hidden, vocab_size, graph, bias=False, reg=reg, prefix="lm_head")

    def __call__(self, inp, prev_seq):
        x = self.embedding(inp)
        for layer in self.layers:
            x = layer(x, prev_seq, rope_base=self.ROPE_BASE)
        return self.head(self.norm(x))


class Phi3(Llama):                              # src/NN.jl:461-507
    ROPE_BASE = 10000.0

    def __init__(self, graph, reg=None, vocab_size=32064, hidden=3072, n_layers=32, n_heads=32, n_kv_heads=8,
                 intermediate=8192):
        super().__init__(graph, reg, vocab_size, hidden, n_layers, n_heads, n_kv_heads, intermediate)


__all__ = ["Linear", "Embedding", "LayerNorm", "RMSNorm", "Mlp", "SelfAttention", "TransformerBlock", "Llama", "Phi3",
           "apply_rotary_embeddings", "repeat_kv"]

"""CPU oracle for the Luminal.jl transformer decode path.  TEST INFRASTRUCTURE ONLY.

This module is a NumPy restatement of what the reference's interpreter `execute()` computes
for the graphs that `NN.jl` builds.  It is the checker for the CUDA path; nothing in the
product package imports it.  Only the tests, the smoke check and the bench's CPU-baseline leg
may call into this directory.

PARITY UNPINNED (for the model-level path): the reference is Julia and cannot be run where this
was written, and its own tests pin RMSNorm / RoPE / attention / Llama only by shape and
no-NaN checks (tests/test_llama.jl:24-113).  What *is* pinned by the reference's tests is
reproduced in tests/test_oracle_pins.py: Linear (tests/test_nn_layers.jl:8-32), Embedding
(:34-52), LayerNorm property (:54-69), a*b+c (tests/test_gpu_execution.jl:8-24), FusedMulAdd
(:54-76), fused chains (tests/test_fusion.jl:7-56), matmul+add (tests/test.jl:17-43), flash vs
manual attention (tests/test_flash_attention_verification.jl:24-94), Unfold windows
(tests/test_whisper_components.jl:5-23).

Conventions
-----------
* Arrays carry the reference's *logical* shapes.  Julia is column-major and `Reshape` keeps the
  column-major linear order (src/Execution.jl:228,287-296); here that is `order="F"`.
* Axis arguments are 1-based, exactly as in the reference's call sites, so the model code below
  reads like src/NN.jl.
* Everything is float32 (src/Compiler.jl:223); token ids are float32 too
  (src/Execution.jl:263).
* Every operator replays the primitive decomposition of src/HighLevelOps.jl in the same order
  (subtraction is `a + b*(-1)`, division is `a * recip(b)`, exp is `exp2(x * 1/ln2)` ...).
"""
from __future__ import annotations

import math

import numpy as np

F32 = np.float32


def _f(x):
    return np.asarray(x, dtype=F32)


# ----------------------------------------------------------------------------------------------
# Primitive ops: src/Execution.jl:207-270 (functional execute_op methods)
# ----------------------------------------------------------------------------------------------

def _align(a, b):
    """align_broadcast_ranks (src/Execution.jl:207-214): the lower-rank operand gets 1-dims
    PREPENDED; after that NumPy and Julia broadcasting agree."""
    a = _f(a)
    b = _f(b)
    if a.ndim < b.ndim:
        a = a.reshape((1,) * (b.ndim - a.ndim) + a.shape)
    elif b.ndim < a.ndim:
        b = b.reshape((1,) * (a.ndim - b.ndim) + b.shape)
    return a, b


def add(a, b):            # src/Execution.jl:216
    a, b = _align(a, b)
    return (a + b).astype(F32)


def mul(a, b):            # src/Execution.jl:217
    a, b = _align(a, b)
    return (a * b).astype(F32)


def mod(a, b):            # src/Execution.jl:218 (Julia % is the truncated remainder)
    a, b = _align(a, b)
    return np.fmod(a, b).astype(F32)


def less_than(a, b):      # src/Execution.jl:219 -> 0/1 floats
    a, b = _align(a, b)
    return (a < b).astype(F32)


def fused_mul_add(a, b, c):   # src/Execution.jl:220
    return (_f(a) * _f(b) + _f(c)).astype(F32)


def fused_add_relu(a, b):     # src/Execution.jl:221
    return np.maximum(_f(a) + _f(b), F32(0)).astype(F32)


def log2(a):   # src/Execution.jl:222
    return np.log2(_f(a)).astype(F32)


def exp2(a):   # src/Execution.jl:223
    return np.exp2(_f(a)).astype(F32)


def sin(a):    # src/Execution.jl:224
    return np.sin(_f(a)).astype(F32)


def sqrt(a):   # src/Execution.jl:226
    return np.sqrt(_f(a)).astype(F32)


def recip(a):  # src/Execution.jl:227
    return (F32(1.0) / _f(a)).astype(F32)


def relu(a):
    return np.maximum(_f(a), F32(0)).astype(F32)


def reshape(a, shape):    # src/Execution.jl:228 column-major reshape
    return np.reshape(_f(a), tuple(shape), order="F")


def permute(a, dims):     # src/Execution.jl:229, dims 1-based
    return np.transpose(_f(a), tuple(d - 1 for d in dims))


def sum_reduce(a, dim):   # src/Execution.jl:232, dim 1-based, dropped
    return np.sum(_f(a), axis=dim - 1, dtype=F32)


def max_reduce(a, dim):   # src/Execution.jl:233
    return np.max(_f(a), axis=dim - 1)


def expand(a, dim, size):  # src/Execution.jl:238-248: insert a new axis at `dim`, repeat
    a = _f(a)
    return np.repeat(np.expand_dims(a, dim - 1), size, axis=dim - 1)


def slice_along(a, axis, start, stop):   # src/HighLevelOps.jl:237-241 + Execution.jl:160-168
    a = _f(a)
    idx = [slice(None)] * a.ndim
    idx[axis - 1] = slice(max(0, start), min(a.shape[axis - 1], stop))
    return a[tuple(idx)].copy()


def pad_along(a, axis, left, right):     # src/HighLevelOps.jl:222-226 + Execution.jl:183-191
    a = _f(a)
    pw = [(0, 0)] * a.ndim
    pw[axis - 1] = (left, right)
    return np.pad(a, pw).astype(F32)


def concat_along(a, b, axis):            # src/HighLevelOps.jl:243-248: pad both, then add
    a = _f(a)
    b = _f(b)
    return add(pad_along(a, axis, 0, b.shape[axis - 1]), pad_along(b, axis, a.shape[axis - 1], 0))


def matmul(a, b):         # batch_matmul, src/Execution.jl:12-54
    a = _f(a)
    b = _f(b)
    if a.ndim == 2 and b.ndim == 2:
        return (a @ b).astype(F32)
    if a.ndim == 3 and b.ndim == 2:
        return np.stack([a[i] @ b for i in range(a.shape[0])]).astype(F32)
    if a.ndim == 3 and b.ndim == 3:
        assert a.shape[0] == b.shape[0]
        return np.matmul(a, b).astype(F32)
    if a.ndim == 4 and b.ndim == 4:
        assert a.shape[:2] == b.shape[:2]
        return np.matmul(a, b).astype(F32)
    raise ValueError(f"Batch matmul not implemented for {a.ndim}D and {b.ndim}D")


def gather(matrix, indexes):   # src/Execution.jl:262-264: rows Int(idx)+1 (0-based ids)
    idx = _f(indexes).astype(np.int64)
    return _f(matrix)[idx, :]


def cumsum_last(a):            # src/Execution.jl:265-266
    return np.cumsum(_f(a), axis=-1, dtype=F32)


def unfold1d(a, kernel, stride, dilation):   # src/Execution.jl:481-550
    a = _f(a)
    L = a.shape[-1]
    O = (L - dilation * (kernel - 1) - 1) // stride + 1
    out = np.zeros(a.shape[:-1] + (O, kernel), dtype=F32)
    for o in range(O):
        for k in range(kernel):
            out[..., o, k] = a[..., o * stride + k * dilation]
    return out


# ----------------------------------------------------------------------------------------------
# High-level decompositions: src/HighLevelOps.jl
# ----------------------------------------------------------------------------------------------

NEG1 = F32(-1.0)
INV_LN2 = F32(F32(1.0) / F32(math.log(2.0)))     # 1.0f0 / log(2.0f0), HighLevelOps.jl:128
HALF_PI = F32(math.pi / 2)                        # Float32(pi/2), HighLevelOps.jl:124


def neg(a):               # HighLevelOps.jl:58
    return mul(a, NEG1)


def sub(a, b):            # HighLevelOps.jl:59-61: a + (b * -1); for a Number b it is a + (-b)
    if np.isscalar(b) or np.ndim(b) == 0:
        return add(a, F32(-F32(b)))
    return add(a, neg(b))


def div(a, b):            # HighLevelOps.jl:63-64
    if np.isscalar(b) or np.ndim(b) == 0:
        return mul(a, F32(F32(1.0) / F32(b)))
    return mul(a, recip(b))


def cos(a):               # HighLevelOps.jl:123-125: sin(Float32(pi/2) - a)
    return sin(add(HALF_PI, neg(a)))


def exp(a):               # HighLevelOps.jl:127-129
    return exp2(mul(a, INV_LN2))


def sigmoid(a):           # HighLevelOps.jl:153-155: 1 / (1 + exp2(-a * 1/ln2))
    inner = add(exp2(mul(neg(a), INV_LN2)), F32(1.0))
    return mul(F32(1.0), recip(inner))


def swish(a):             # HighLevelOps.jl:157-160
    return mul(a, sigmoid(a))


silu = swish


def tanh(a):              # HighLevelOps.jl:166-168
    return sub(mul(sigmoid(mul(a, F32(2.0))), F32(2.0)), 1.0)


def gelu(a):              # HighLevelOps.jl:162-164, left-to-right as Julia parses it
    inner = mul(mul(F32(0.7978845608), a), add(mul(mul(F32(0.044715), a), a), F32(1.0)))
    return mul(mul(a, F32(0.5)), add(tanh(inner), F32(1.0)))


def mean(a, dim):         # HighLevelOps.jl:284-287
    n = _f(a).shape[dim - 1]
    return mul(sum_reduce(a, dim), F32(F32(1.0) / F32(n)))


def mean_norm(a, dim):    # HighLevelOps.jl:292-297
    n = _f(a).shape[dim - 1]
    return sub(a, expand(mean(a, dim), dim, n))


def std_norm(a, dim, epsilon=1e-5):   # HighLevelOps.jl:299-304
    n = _f(a).shape[dim - 1]
    var = mean(mul(a, a), dim)
    inv_std = recip(sqrt(add(var, F32(epsilon))))
    return mul(a, expand(inv_std, dim, n))


def softmax(a, dim):      # HighLevelOps.jl:313-319
    n = _f(a).shape[dim - 1]
    m = max_reduce(a, dim)
    shifted = sub(a, expand(m, dim, n))
    e = exp(shifted)
    return div(e, expand(sum_reduce(e, dim), dim, n))


def arange(to):           # HighLevelOps.jl:332-340
    if to == 1:
        return expand(F32(0.0), 1, 1)
    return sub(cumsum_last(expand(F32(1.0), 1, to)), 1.0)


def triu(size, diagonal=0):   # HighLevelOps.jl:353-361: 1 where column j >= row i + diagonal
    h = expand(arange(size), 1, size)
    v = expand(arange(size), 2, size)
    return less_than(v, sub(h, F32(diagonal - 1)))     # `h - c > v` is `v < h - c`


# ----------------------------------------------------------------------------------------------
# Flash attention op: src/Execution.jl:453-479 (flash_attn_cpu)
# ----------------------------------------------------------------------------------------------

def flash_attn_cpu(q, k, v, scale, causal):
    """Literal restatement of the reference's scalar online-softmax loops.  Small cases only."""
    q, k, v = _f(q), _f(k), _f(v)
    B, H, N, D = q.shape
    scale = F32(scale)
    out = np.empty_like(q)
    for b in range(B):
        for h in range(H):
            for i in range(N):
                m_i = F32(-np.inf)
                l_i = F32(0.0)
                o_row = np.zeros(D, dtype=F32)
                for j in range(N):
                    if causal and j > i:
                        continue
                    dot = F32(np.sum(q[b, h, i, :] * k[b, h, j, :], dtype=F32) * scale)
                    m_next = max(m_i, dot)
                    p = F32(np.exp(F32(dot - m_next)))
                    scale_old = F32(np.exp(F32(m_i - m_next)))
                    if np.isnan(scale_old):
                        scale_old = F32(0.0)
                    o_row = (o_row * scale_old + p * v[b, h, j, :]).astype(F32)
                    l_i = F32(l_i * scale_old + p)
                    m_i = m_next
                out[b, h, i, :] = o_row / l_i
    return out


def flash_attn_fast(q, k, v, scale, causal):
    """Same function as `flash_attn_cpu`, evaluated one (batch, head) at a time with a
    materialised score matrix in float64 (the online softmax is an exact algebraic
    rearrangement of softmax(scale*QK^T)V; causal = keys j>i skipped).  Used where the scalar
    loops would take hours."""
    q, k, v = _f(q), _f(k), _f(v)
    B, H, N, D = q.shape
    out = np.empty_like(q)
    mask = np.triu(np.ones((N, N), dtype=bool), 1) if causal else None
    for b in range(B):
        for h in range(H):
            s = (q[b, h].astype(np.float64) @ k[b, h].astype(np.float64).T) * float(scale)
            if causal:
                s[mask] = -np.inf
            s -= s.max(axis=1, keepdims=True)
            p = np.exp(s)
            out[b, h] = ((p @ v[b, h].astype(np.float64)) / p.sum(axis=1, keepdims=True)).astype(F32)
    return out


# ----------------------------------------------------------------------------------------------
# NN layers: src/NN.jl
# ----------------------------------------------------------------------------------------------

def linear(x, weight, bias=None):
    """NN.jl:22-35.  weight is [out, in]; y = x * permute(W,[2,1]).  The reference expands the
    bias along dim 1 to the first dim of the output, which is shape-correct only for 2-D x (or
    B == 1); for other ranks the bias is defined here as a broadcast over the last dim."""
    out = matmul(x, permute(weight, [2, 1]))
    if bias is not None:
        if out.ndim == 2:
            out = add(out, expand(bias, 1, out.shape[0]))
        else:
            out = add(out, bias)
    return out


def embedding(weight, ids):      # NN.jl:116-118
    return gather(weight, ids)


def layer_norm(x, weight=None, bias=None, epsilon=1e-5, mean_norm_=True):
    """NN.jl:138-173 (RMSNorm is mean_norm=false, bias=nothing)."""
    axis = _f(x).ndim
    out = _f(x)
    if mean_norm_:
        out = mean_norm(out, axis)
    out = std_norm(out, axis, epsilon)
    if weight is not None:
        w = _f(weight)
        for i in range(1, out.ndim):
            w = expand(w, i, out.shape[i - 1])
        out = mul(out, w)
    if bias is not None:
        b = _f(bias)
        for i in range(1, out.ndim):
            b = expand(b, i, out.shape[i - 1])
        out = add(out, b)
    return out


def rms_norm(x, weight, epsilon=1e-5):   # NN.jl:134-136
    return layer_norm(x, weight, None, epsilon, mean_norm_=False)


def mlp(x, gate_w, up_w, down_w):        # NN.jl:246-250
    gate = silu(linear(x, gate_w))
    up = linear(x, up_w)
    return linear(mul(gate, up), down_w)


def rope_inv_freqs(head_dim, base):
    """NN.jl:261-263.  `arange(half)*2.0f0/Float32(D)` parses as (arange*2)*(1/D)."""
    half = head_dim // 2
    freqs = div(mul(arange(half), F32(2.0)), F32(head_dim))
    return recip(exp2(mul(freqs, F32(np.log2(F32(base))))))


def apply_rotary_embeddings(x, prev_seq, base=10000.0):   # NN.jl:253-303
    x = _f(x)
    batch, n_heads, seq, head_dim = x.shape
    half = head_dim // 2
    inv_freqs = rope_inv_freqs(head_dim, base)
    pos = add(arange(seq), F32(prev_seq))
    emb = matmul(expand(pos, 2, 1), expand(inv_freqs, 1, 1))          # (seq, half)
    split = reshape(x, [batch, n_heads, seq, half, 2])
    x0 = slice_along(split, 5, 0, 1)
    x1 = slice_along(split, 5, 1, 2)
    emb_expanded = expand(expand(emb, 1, n_heads), 1, batch)
    sin_emb = sin(emb_expanded)
    cos_emb = cos(emb_expanded)
    x0 = reshape(x0, [batch, n_heads, seq, half])
    x1 = reshape(x1, [batch, n_heads, seq, half])
    x0_out = sub(mul(x0, cos_emb), mul(x1, sin_emb))
    x1_out = add(mul(x0, sin_emb), mul(x1, cos_emb))
    res = concat_along(expand(x0_out, 5, 1), expand(x1_out, 5, 1), 5)
    return reshape(res, [batch, n_heads, seq, head_dim])


def repeat_kv(keys, groups):             # NN.jl:305-317
    if groups == 1:
        return keys
    batch, kv_heads, seq, head_dim = keys.shape
    return reshape(expand(keys, 3, groups), [batch, kv_heads * groups, seq, head_dim])


def self_attention(x, wq, wk, wv, wo, n_heads, n_kv_heads, prev_seq, rope_base=10000.0):
    """NN.jl:343-387."""
    x = _f(x)
    batch, seq, hidden = x.shape
    head_dim = hidden // n_heads
    queries = permute(reshape(linear(x, wq), [batch, seq, n_heads, head_dim]), [1, 3, 2, 4])
    keys = permute(reshape(linear(x, wk), [batch, seq, n_kv_heads, head_dim]), [1, 3, 2, 4])
    values = permute(reshape(linear(x, wv), [batch, seq, n_kv_heads, head_dim]), [1, 3, 2, 4])
    queries = apply_rotary_embeddings(queries, prev_seq, rope_base)
    keys = apply_rotary_embeddings(keys, prev_seq, rope_base)
    if n_kv_heads < n_heads:
        groups = n_heads // n_kv_heads
        keys = repeat_kv(keys, groups)
        values = repeat_kv(values, groups)
    weights = mul(matmul(queries, permute(keys, [1, 2, 4, 3])),
                  F32(F32(1.0) / np.sqrt(F32(head_dim))))
    if seq > 1:
        mask = mul(triu(seq, 1), F32(-1e9))
        weights = add(weights, expand(expand(mask, 1, n_heads), 1, batch))
    probs = softmax(weights, 4)
    out = matmul(probs, values)
    out = reshape(permute(out, [1, 3, 2, 4]), [batch, seq, hidden])
    return linear(out, wo)


def layer_names(i):
    p = f"model.layers.{i}"
    return {
        "attn_norm": f"{p}.input_layernorm.weight",
        "q": f"{p}.self_attn.q_proj.weight",
        "k": f"{p}.self_attn.k_proj.weight",
        "v": f"{p}.self_attn.v_proj.weight",
        "o": f"{p}.self_attn.o_proj.weight",
        "ffn_norm": f"{p}.post_attention_layernorm.weight",
        "gate": f"{p}.mlp.gate_proj.weight",
        "up": f"{p}.mlp.up_proj.weight",
        "down": f"{p}.mlp.down_proj.weight",
    }


def transformer_block(x, w, i, cfg, prev_seq):   # NN.jl:406-414
    n = layer_names(i)
    normed = rms_norm(x, w[n["attn_norm"]], cfg["eps"])
    attn = self_attention(normed, w[n["q"]], w[n["k"]], w[n["v"]], w[n["o"]],
                          cfg["n_heads"], cfg["n_kv_heads"], prev_seq, cfg["rope_base"])
    x = add(x, attn)
    normed = rms_norm(x, w[n["ffn_norm"]], cfg["eps"])
    ff = mlp(normed, w[n["gate"]], w[n["up"]], w[n["down"]])
    return add(x, ff)


def llama_forward(tokens, w, cfg, prev_seq=0, return_hidden=False):
    """NN.jl:448-455 (Llama) / :499-507 (Phi3): logits for ALL positions.  tokens: [B,S] ids."""
    x = embedding(w["model.embed_tokens.weight"], _f(tokens))
    hiddens = []
    for i in range(cfg["n_layers"]):
        x = transformer_block(x, w, i, cfg, prev_seq)
        if return_hidden:
            hiddens.append(x)
    x = rms_norm(x, w["model.norm.weight"], cfg["eps"])
    logits = linear(x, w["lm_head.weight"])
    if return_hidden:
        return logits, hiddens
    return logits


def greedy_generate_recompute(prompt, w, cfg, n_steps):
    """The reference's only defined Llama generation: no KV cache, the whole prefix is re-run
    with prev_seq=0 for every token (examples/llama.jl:39-80 feeds prev_seq=0; NN.jl has no
    cache for Llama).  Returns (tokens [B,n_steps], last-position logits per step)."""
    toks = np.array(prompt, dtype=np.int64)
    out_t, out_l = [], []
    for _ in range(n_steps):
        logits = llama_forward(toks, w, cfg, 0)[:, -1, :]
        nxt = np.argmax(logits, axis=-1)
        out_t.append(nxt)
        out_l.append(logits)
        toks = np.concatenate([toks, nxt[:, None]], axis=1)
    return np.stack(out_t, axis=1), np.stack(out_l, axis=1)


# ----------------------------------------------------------------------------------------------
# KV-cached decode (fast oracle).  Mathematically the same function as the recompute above; the
# tests cross-check it against `llama_forward`.  Head split / GQA / RoPE pairing are the
# reference's column-major conventions: feature f = h + H*d, kv(q) = q mod KV, pairs (i, i+D/2).
# ----------------------------------------------------------------------------------------------

class CachedLlama:
    def __init__(self, w, cfg, batch, max_ctx):
        self.w, self.cfg = w, cfg
        L, KV, D = cfg["n_layers"], cfg["n_kv_heads"], cfg["hidden"] // cfg["n_heads"]
        self.k = np.zeros((L, batch, KV, max_ctx, D), dtype=F32)
        self.v = np.zeros((L, batch, KV, max_ctx, D), dtype=F32)
        self.pos = 0
        self.inv = rope_inv_freqs(D, cfg["rope_base"])

    def _rope(self, x, positions):
        # x: [B, heads, S, D]; positions: [S]
        half = x.shape[-1] // 2
        ang = (positions.astype(F32)[:, None] * self.inv[None, :]).astype(F32)
        s = np.sin(ang).astype(F32)
        c = np.sin((HALF_PI + ang * NEG1).astype(F32)).astype(F32)
        x0, x1 = x[..., :half], x[..., half:]
        o0 = (x0 * c + (x1 * s) * NEG1).astype(F32)
        o1 = (x0 * s + x1 * c).astype(F32)
        return np.concatenate([o0, o1], axis=-1)

    def forward(self, tokens, return_hidden=False):
        """tokens [B,S] appended at positions pos..pos+S-1; returns logits [B,S,V]."""
        cfg, w = self.cfg, self.w
        H, KV = cfg["n_heads"], cfg["n_kv_heads"]
        tokens = np.asarray(tokens)
        B, S = tokens.shape
        D = cfg["hidden"] // H
        p0 = self.pos
        positions = np.arange(p0, p0 + S)
        x = _f(w["model.embed_tokens.weight"])[tokens.astype(np.int64)]
        hiddens = []
        scale = F32(F32(1.0) / np.sqrt(F32(D)))
        for i in range(cfg["n_layers"]):
            n = layer_names(i)
            xn = rms_norm(x, w[n["attn_norm"]], cfg["eps"])
            q = linear(xn, w[n["q"]]).reshape(B, S, D, H).transpose(0, 3, 1, 2)    # f = h + H*d
            k = linear(xn, w[n["k"]]).reshape(B, S, D, KV).transpose(0, 3, 1, 2)
            v = linear(xn, w[n["v"]]).reshape(B, S, D, KV).transpose(0, 3, 1, 2)
            q = self._rope(q, positions)
            k = self._rope(k, positions)
            self.k[i, :, :, p0:p0 + S] = k
            self.v[i, :, :, p0:p0 + S] = v
            T = p0 + S
            kk = self.k[i, :, np.arange(H) % KV, :T].transpose(1, 0, 2, 3)       # kv = q mod KV
            vv = self.v[i, :, np.arange(H) % KV, :T].transpose(1, 0, 2, 3)
            sc = (np.matmul(q, kk.transpose(0, 1, 3, 2)) * scale).astype(F32)   # [B,H,S,T]
            qi = positions[:, None]
            kj = np.arange(T)[None, :]
            sc = np.where(kj > qi, F32(-np.inf), sc)       # causal: keys after the query
            sc = sc - sc.max(axis=-1, keepdims=True)
            pr = np.exp2((sc * INV_LN2).astype(F32)).astype(F32)
            pr = (pr * (F32(1.0) / pr.sum(axis=-1, keepdims=True, dtype=F32))).astype(F32)
            o = np.matmul(pr, vv).astype(F32)                                     # [B,H,S,D]
            o = o.transpose(0, 2, 3, 1).reshape(B, S, D * H)                      # f = h + H*d
            x = add(x, linear(o, w[n["o"]]))
            xn = rms_norm(x, w[n["ffn_norm"]], cfg["eps"])
            x = add(x, mlp(xn, w[n["gate"]], w[n["up"]], w[n["down"]]))
            if return_hidden:
                hiddens.append(x)
        self.pos += S
        x = rms_norm(x, w["model.norm.weight"], cfg["eps"])
        logits = linear(x, w["lm_head.weight"])
        if return_hidden:
            return logits, hiddens
        return logits

    def greedy(self, prompt, n_steps):
        """Prompt [B,P] then n_steps greedy tokens.  Returns (tokens [B,n], logits [B,n,V])."""
        logits = self.forward(np.asarray(prompt))[:, -1, :]
        toks, lg = [], []
        for step in range(n_steps):
            nxt = np.argmax(logits, axis=-1)
            toks.append(nxt)
            lg.append(logits)
            if step + 1 < n_steps:
                logits = self.forward(nxt[:, None])[:, -1, :]
        return np.stack(toks, axis=1), np.stack(lg, axis=1)


# ----------------------------------------------------------------------------------------------
# Synthetic inputs: one counter-based generator shared (bit for bit) with the CUDA init kernel.
# value(seed, tensor_id, i) = (2*sum_of_12_uint16_lanes - 12*65535) * (sigma / 131072)
# The 12 lanes come from three splitmix64 outputs; the sum has mean 0 and standard deviation
# 65536*sqrt(1 - 2^-32) in units of 1/2, i.e. the value is an Irwin-Hall(12) approximation of
# N(0, sigma) computed with integer arithmetic and ONE float32 multiply, so host and device
# agree exactly.
# ----------------------------------------------------------------------------------------------

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
    z = x
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
    return z ^ (z >> np.uint64(31))


def _stream_key(seed, tensor_id):
    with np.errstate(over="ignore"):
        return _splitmix64(np.uint64(seed) * np.uint64(0xD1342543DE82EF95) + np.uint64(tensor_id))


def synth_normal(seed, tensor_id, shape, sigma, offset=0.0):
    """Row-major linear index -> value.  `offset` is added after the multiply (norm gains)."""
    n = int(np.prod(shape))
    return synth_normal_at(seed, tensor_id, np.arange(n, dtype=np.uint64), sigma, offset).reshape(shape)


def synth_normal_at(seed, tensor_id, linear_index, sigma, offset=0.0):
    """The generator's values at the given row-major linear indices (any shape of indices), so a
    slice of a tensor too large to build on the host can be regenerated."""
    idx = np.asarray(linear_index).astype(np.uint64)
    shape = idx.shape
    idx = idx.reshape(-1)
    n = idx.size
    with np.errstate(over="ignore"):
        key = _stream_key(seed, tensor_id)
        total = np.zeros(n, dtype=np.int64)
        for r in range(3):
            h = _splitmix64(key ^ (idx * np.uint64(3) + np.uint64(r)))
            for lane in range(4):
                total += ((h >> np.uint64(16 * lane)) & np.uint64(0xFFFF)).astype(np.int64)
    centred = (2 * total - 12 * 65535).astype(F32)
    val = centred * F32(F32(sigma) / F32(131072.0))
    if offset != 0.0:
        val = (val + F32(offset)).astype(F32)
    return val.astype(F32).reshape(shape)


def synth_tokens(seed, tensor_id, shape, vocab):
    n = int(np.prod(shape))
    idx = np.arange(n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        h = _splitmix64(_stream_key(seed, tensor_id) ^ idx)
    return ((h >> np.uint64(11)) % np.uint64(vocab)).astype(np.int64).reshape(shape)


# Fixed tensor-id scheme shared with the library: id = 16*layer + slot (layer 0xFFFF for globals).
SLOT = {"attn_norm": 0, "q": 1, "k": 2, "v": 3, "o": 4, "ffn_norm": 5, "gate": 6, "up": 7, "down": 8}
GLOBAL_IDS = {"model.embed_tokens.weight": 0xFFFF0, "model.norm.weight": 0xFFFF1,
              "lm_head.weight": 0xFFFF2}


def synth_llama_weights(cfg, seed=1234, sigma=0.02):
    """All weights of a Llama/Phi-3 shaped model, logical [out,in] row-major, float32."""
    H, KV, hid, inter, V = (cfg["n_heads"], cfg["n_kv_heads"], cfg["hidden"],
                            cfg["intermediate"], cfg["vocab"])
    D = hid // H
    shapes = {"attn_norm": (hid,), "q": (H * D, hid), "k": (KV * D, hid), "v": (KV * D, hid),
              "o": (hid, H * D), "ffn_norm": (hid,), "gate": (inter, hid), "up": (inter, hid),
              "down": (hid, inter)}
    w = {}
    for i in range(cfg["n_layers"]):
        names = layer_names(i)
        for key, shp in shapes.items():
            off = 1.0 if key.endswith("norm") else 0.0
            w[names[key]] = synth_normal(seed, 16 * i + SLOT[key], shp, sigma, off)
    w["model.embed_tokens.weight"] = synth_normal(seed, GLOBAL_IDS["model.embed_tokens.weight"], (V, hid), sigma)
    w["model.norm.weight"] = synth_normal(seed, GLOBAL_IDS["model.norm.weight"], (hid,), sigma, 1.0)
    w["lm_head.weight"] = synth_normal(seed, GLOBAL_IDS["lm_head.weight"], (V, hid), sigma)
    return w


def bf16_round(a):
    """Round-to-nearest-even float32 -> bfloat16 -> float32 (for bf16-path comparisons)."""
    u = _f(a).view(np.uint32).astype(np.uint64)
    r = ((u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)) << np.uint64(16)
    return r.astype(np.uint32).view(F32).reshape(np.shape(a))


CONFIGS = {
    # BASELINE configs[0]: the examples/llama.jl shape with BASELINE's explicit numbers
    "small_llama": dict(n_layers=4, hidden=256, n_heads=8, n_kv_heads=8, intermediate=688,
                        vocab=1024, eps=1e-5, rope_base=10000.0),
    # reduced GQA shapes used for fp32 parity of the cfg4 / cfg5 code paths
    "tiny_gqa128": dict(n_layers=2, hidden=512, n_heads=4, n_kv_heads=2, intermediate=1024,
                        vocab=2048, eps=1e-5, rope_base=500000.0),
    "tiny_gqa96": dict(n_layers=2, hidden=384, n_heads=4, n_kv_heads=2, intermediate=768,
                       vocab=1536, eps=1e-5, rope_base=10000.0),
    # wide enough that the GEMV work units span several CTAs per row group and vice versa
    "mid_gqa": dict(n_layers=2, hidden=1024, n_heads=8, n_kv_heads=2, intermediate=2816,
                    vocab=4096, eps=1e-5, rope_base=500000.0),
    # four kv heads: shards over four tensor-parallel ranks
    "mid_gqa_kv4": dict(n_layers=2, hidden=1024, n_heads=8, n_kv_heads=4, intermediate=2816,
                        vocab=4096, eps=1e-5, rope_base=500000.0),
    # eight kv heads: shards over eight tensor-parallel ranks (one kv head and one query head each)
    "mid_gqa_kv8": dict(n_layers=2, hidden=1024, n_heads=8, n_kv_heads=8, intermediate=2816,
                        vocab=4096, eps=1e-5, rope_base=500000.0),
    "phi3_mini": dict(n_layers=32, hidden=3072, n_heads=32, n_kv_heads=8, intermediate=8192,
                      vocab=32064, eps=1e-5, rope_base=10000.0),
    "llama3_8b": dict(n_layers=32, hidden=4096, n_heads=32, n_kv_heads=8, intermediate=14336,
                      vocab=128256, eps=1e-5, rope_base=500000.0),
}

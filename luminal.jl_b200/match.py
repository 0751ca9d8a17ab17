"""Recognising a decoder-only transformer in a bare node list, and the node list's text form.

The reference has no plugin seam other than its graph: a backend sees `Graph.nodes` (src/Graph.jl:4-26), a
flat, topologically ordered list of primitive ops, with every NN layer already decomposed (src/NN.jl,
src/HighLevelOps.jl).  `export_graph` / `import_graph` give that list a JSON form a Julia shim can emit with
a dozen lines (one record per node: op name, op fields, inputs, output shape).  `match_decoder` walks such a
list backwards from the logits node and recovers, by structure alone -- no model object, no weight names --
what src/NN.jl:390-455 built: the layer count, the widths, the head split, the RMSNorm epsilon, the RoPE
base, and which input-tensor node plays which weight's role.  `compile_b200` hands that to the fused
session.  A graph that deviates anywhere (another activation, a bias, a different mask) raises MatchError
naming the node, and the caller falls back to compile(), which runs any graph one kernel per node."""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field, fields
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import graph as G


class MatchError(ValueError):
    pass


# ---------------------------------------------------------------------------------------------
# Text form of a node list
# ---------------------------------------------------------------------------------------------
_OPS = {c.__name__: c for c in (G.Log2, G.Exp2, G.Sin, G.Sqrt, G.Cos, G.Recip, G.Contiguous, G.ReLU, G.Add, G.Mul, G.Mod,
                                G.Max, G.LessThan, G.FusedMulAdd, G.FusedAddReLU, G.MatMul, G.SumReduce, G.MaxReduce,
                                G.Permute, G.Expand, G.Reshape, G.Slice, G.Pad, G.Unfold, G.Constant, G.Function,
                                G.FlashAttentionOp)}


def _plain(v):
    if isinstance(v, tuple):
        return [_plain(x) for x in v]
    return v


def _frozen(v):
    if isinstance(v, list):
        return tuple(_frozen(x) for x in v)
    return v


def export_graph(graph) -> dict:
    """{"nodes": [{"op", "args", "inputs": [[node id, output index, shape]], "shape"}]}; ids are 1-based positions."""
    nodes = []
    for node, shape in zip(graph.nodes, graph.shapes):
        args = {f.name: _plain(getattr(node.op, f.name)) for f in fields(node.op)}
        nodes.append({"op": type(node.op).__name__, "args": args,
                      "inputs": [[int(i), int(o), [int(s) for s in shp]] for i, o, shp in node.inputs],
                      "shape": [int(s) for s in shape]})
    return {"format": "luminal-node-list", "version": 1, "nodes": nodes}


def import_graph(doc) -> G.Graph:
    if isinstance(doc, (str, bytes)):
        doc = json.loads(doc)
    if doc.get("format") != "luminal-node-list":
        raise ValueError("not a luminal node list")
    g = G.Graph()
    for n, rec in enumerate(doc["nodes"], start=1):
        cls = _OPS.get(rec["op"])
        if cls is None:
            raise ValueError(f"node {n}: unknown op {rec['op']}")
        op = cls(**{k: _frozen(v) for k, v in rec.get("args", {}).items()})
        inputs = [(int(i), int(o), tuple(int(s) for s in shp)) for i, o, shp in rec["inputs"]]
        for i, _, _ in inputs:
            if not 1 <= i < n:
                raise ValueError(f"node {n}: input {i} is not an earlier node")
        g.nodes.append(G.Node(op, inputs))
        g.shapes.append(tuple(int(s) for s in rec["shape"]))
    return g


# ---------------------------------------------------------------------------------------------
# Structural walker
# ---------------------------------------------------------------------------------------------
@dataclass
class DecoderMatch:
    """What match_decoder found.  `weights` maps the reference's registry names (src/NN.jl:180-225)
    to input-tensor node ids; `tokens` is the node the token ids enter through."""
    n_layers: int
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    intermediate: int
    vocab: int
    eps: float
    rope_base: float
    prev_seq: int
    batch: int
    seq: int
    tokens: int
    weights: Dict[str, int] = field(default_factory=dict)


class _Walker:
    def __init__(self, graph):
        self.g = graph

    def op(self, i):
        return self.g.nodes[i - 1].op

    def ins(self, i):
        return [j for j, _, _ in self.g.nodes[i - 1].inputs]

    def shape(self, i):
        return self.g.shapes[i - 1]

    def fail(self, i, what):
        raise MatchError(f"node {i} ({type(self.op(i)).__name__}{list(self.shape(i))}): expected {what}")

    def expect(self, i, cls, what=None):
        if not isinstance(self.op(i), cls):
            self.fail(i, what or cls.__name__)
        return self.ins(i)

    def is_input(self, i):
        o = self.op(i)
        return isinstance(o, G.Function) and o.name == "InputTensor"

    def const(self, i):
        o = self.op(i)
        return o.value if isinstance(o, G.Constant) else None

    def with_const(self, i, cls, what):
        """Binary node of type cls with one Constant operand (either side) -> (other operand, value)."""
        a, b = self.expect(i, cls, what)
        if self.const(b) is not None:
            return a, self.const(b)
        if self.const(a) is not None:
            return b, self.const(a)
        self.fail(i, what)

    def skip(self, i, *classes):
        """Steps up through unary nodes of the given classes."""
        while isinstance(self.op(i), classes):
            i = self.ins(i)[0]
        return i

    def ancestors(self, i, stop):
        """All nodes reachable upwards from i without passing through `stop` (stop itself excluded)."""
        seen, todo = set(), [i]
        while todo:
            n = todo.pop()
            if n in seen or n == stop:
                continue
            seen.add(n)
            todo.extend(self.ins(n))
        return seen

    # ---- layer patterns -------------------------------------------------------------------
    def linear(self, i):
        """MatMul(x, Permute[2,1](W)) with W a rank-2 input tensor and no bias (src/NN.jl:23-35) -> (x, W)."""
        x, wt = self.expect(i, G.MatMul, "a Linear's MatMul")
        if not (isinstance(self.op(wt), G.Permute) and self.op(wt).dims == (2, 1)):
            self.fail(wt, "Permute[2,1] of a weight")
        w = self.ins(wt)[0]
        if not (self.is_input(w) and len(self.shape(w)) == 2):
            self.fail(w, "a [out, in] weight input")
        return x, w

    def rmsnorm(self, i):
        """x * expand(recip(sqrt(sum(x*x)*(1/n) + eps))) * expand(g) (src/NN.jl:138-173 with mean_norm off,
        src/HighLevelOps.jl:296-300) -> (x, g, eps)."""
        a, b = self.expect(i, G.Mul, "RMSNorm's scale by the gain")
        g = self.skip(b, G.Expand)
        if not (self.is_input(g) and len(self.shape(g)) == 1):
            a, b = b, a
            g = self.skip(b, G.Expand)
        if not (self.is_input(g) and len(self.shape(g)) == 1):
            self.fail(i, "RMSNorm's scale by a [hidden] gain")
        x, inv = self.expect(a, G.Mul, "x * inv_rms")
        ex = self.expect(inv, G.Expand, "expand(inv_rms)")[0]
        sq = self.expect(ex, G.Recip, "recip(sqrt(...))")[0]
        ms = self.expect(sq, G.Sqrt, "sqrt(mean + eps)")[0]
        mean, eps = self.with_const(ms, G.Add, "mean + eps")
        total, inv_n = self.with_const(mean, G.Mul, "sum * (1/n)")
        n = self.shape(x)[-1]
        if abs(inv_n * n - 1.0) > 1e-5:
            self.fail(mean, f"sum * (1/{n})")
        red = self.op(total)
        if not (isinstance(red, G.SumReduce) and red.dim == len(self.shape(x))):
            self.fail(total, "sum over the last dim")
        p, q = self.expect(self.ins(total)[0], G.Mul, "x * x")
        if not (p == q == x):
            self.fail(self.ins(total)[0], "x * x of the normalised tensor")
        if self.shape(g)[0] != n:
            self.fail(g, f"a gain of length {n}")
        return x, g, float(eps)

    def silu(self, i):
        """a * (1 * recip(1 + exp2(a * -1 * (1/ln 2)))) (src/HighLevelOps.jl:153-160) -> a."""
        a, s = self.expect(i, G.Mul, "silu(gate)")
        r, one = self.with_const(s, G.Mul, "1 / (1 + exp2(..))")
        den = self.expect(r, G.Recip, "recip(1 + exp2(..))")[0]
        e, one2 = self.with_const(den, G.Add, "1 + exp2(..)")
        arg = self.expect(e, G.Exp2, "exp2(-a / ln 2)")[0]
        neg, k = self.with_const(arg, G.Mul, "(-a) * (1/ln 2)")
        src, m1 = self.with_const(neg, G.Mul, "a * -1")
        if not (one == 1.0 and one2 == 1.0 and m1 == -1.0 and abs(k - 1.0 / math.log(2.0)) < 1e-6 and src == a):
            self.fail(i, "silu(gate) with the reference's constants")
        return a

    def arange(self, i):
        """arange(n): cumsum(expand(1, n)) - 1, or expand(0, 1) for n == 1 (src/HighLevelOps.jl:336-345) -> n."""
        if isinstance(self.op(i), G.Expand):
            if self.const(self.ins(i)[0]) == 0.0 and self.shape(i) == (1,):
                return 1
            self.fail(i, "arange(1)")
        c, m1 = self.with_const(i, G.Add, "cumsum(ones) - 1")
        o = self.op(c)
        if not (m1 == -1.0 and isinstance(o, G.Function) and o.name == "CumSum"):
            self.fail(i, "cumsum(ones) - 1")
        ones = self.expect(self.ins(c)[0], G.Expand, "expand(1, n)")[0]
        if self.const(ones) != 1.0 or len(self.shape(c)) != 1:
            self.fail(c, "cumsum over expand(1, n)")
        return self.shape(c)[0]

    def rope(self, i):
        """apply_rotary_embeddings (src/NN.jl:253-303): the half-split rotation of pairs (j, j + D/2) that the
        column-major reshape to [.., D/2, 2] produces -> (input [B, heads, S, D], base, prev_seq)."""
        shp = self.shape(i)
        if len(shp) != 4 or shp[3] % 2:
            self.fail(i, "RoPE output [batch, heads, seq, head_dim]")
        D, half = shp[3], shp[3] // 2
        cat = self.expect(i, G.Reshape, "reshape of the rotated pairs")[0]
        pa, pb = self.expect(cat, G.Add, "concat of the two halves")
        outs = []
        for p, want in ((pa, (0, 1)), (pb, (1, 0))):
            e = self.expect(p, G.Pad, "pad of one half")[0]
            if self.op(p).padding[-1] != want or any(x != (0, 0) for x in self.op(p).padding[:-1]):
                self.fail(p, f"pad {want} along the pair dim")
            outs.append(self.expect(e, G.Expand, "expand(.., 5, 1)")[0])
        # x0' = x0 cos - x1 sin ; x1' = x0 sin + x1 cos
        t0, t1 = self.expect(outs[0], G.Add, "x0*cos - x1*sin")
        x0, cosn = self.expect(t0, G.Mul, "x0 * cos")
        m, neg = self.with_const(t1, G.Mul, "-(x1 * sin)")
        x1, sinn = self.expect(m, G.Mul, "x1 * sin")
        u0, u1 = self.expect(outs[1], G.Add, "x0*sin + x1*cos")
        if neg != -1.0 or self.ins(u0) != [x0, sinn] or not isinstance(self.op(u0), G.Mul) \
                or self.ins(u1) != [x1, cosn] or not isinstance(self.op(u1), G.Mul):
            self.fail(outs[1], "the rotation's second row over the same x0, x1, sin, cos")
        ang = self.expect(sinn, G.Sin, "sin(angle)")[0]
        shifted = self.expect(cosn, G.Sin, "cos as sin(pi/2 - angle)")[0]
        na, hp = self.with_const(shifted, G.Add, "pi/2 - angle")
        a2, m1 = self.with_const(na, G.Mul, "angle * -1")
        if a2 != ang or m1 != -1.0 or abs(hp - math.pi / 2) > 1e-6:
            self.fail(cosn, "sin(pi/2 - angle) of the same angle")
        srcs = []
        for x, rng in ((x0, (0, 1)), (x1, (1, 2))):
            s = self.expect(self.skip(x, G.Contiguous), G.Reshape, "reshape of one pair element")[0]
            if not isinstance(self.op(s), G.Slice) or self.op(s).ranges[-1] != rng:
                self.fail(s, f"slice {rng} of the pair dim")
            sp = self.ins(s)[0]
            if not isinstance(self.op(sp), G.Reshape) or self.shape(sp) != shp[:3] + (half, 2):
                self.fail(sp, "reshape to [.., D/2, 2]")
            srcs.append(self.ins(sp)[0])
        if srcs[0] != srcs[1]:
            self.fail(i, "both pair elements from one tensor")
        emb = self.skip(ang, G.Expand)
        pcol, frow = self.expect(emb, G.MatMul, "positions x inverse frequencies")
        pos, prev = self.with_const(self.expect(pcol, G.Expand, "positions as a column")[0], G.Add, "arange(seq) + prev_seq")
        if self.arange(pos) != shp[2] or prev != int(prev) or prev < 0:
            self.fail(pos, f"arange({shp[2]}) + a whole prev_seq")
        inv = self.expect(self.expect(frow, G.Expand, "frequencies as a row")[0], G.Recip, "1 / base^(2j/D)")[0]
        fr, lb = self.with_const(self.expect(inv, G.Exp2, "exp2(log2(base) * 2j/D)")[0], G.Mul, "freqs * log2(base)")
        f2, inv_d = self.with_const(fr, G.Mul, "(2j) / D")
        ar, two = self.with_const(f2, G.Mul, "2 * j")
        if two != 2.0 or abs(inv_d * D - 1.0) > 1e-5 or self.arange(ar) != half:
            self.fail(fr, f"arange({half}) * 2 / {D}")
        base = float(2.0 ** lb)          # the graph holds log2(base) rounded to fp32: snap back to the whole number it came from
        if base < 2.0 ** 40 and float(np.float32(np.log2(np.float32(round(base))))) == lb:
            base = float(round(base))
        return srcs[0], base, int(prev)

    def causal_mask(self, i, seq):
        """expand(expand(triu(seq, 1) * -1e9)) (src/NN.jl:368-373, src/HighLevelOps.jl:347-361)."""
        m = self.skip(i, G.Expand)
        tri, big = self.with_const(m, G.Mul, "triu * -1e9")
        v, hh = self.expect(tri, G.LessThan, "column index > row index")
        h, zero = self.with_const(hh, G.Add, "row index - 0")
        eh, ev = self.op(h), self.op(v)
        if not (big == -1e9 and zero == 0.0 and isinstance(eh, G.Expand) and isinstance(ev, G.Expand) and (eh.dim, ev.dim) == (1, 2)
                and self.arange(self.ins(h)[0]) == seq and self.arange(self.ins(v)[0]) == seq and self.shape(tri) == (seq, seq)):
            self.fail(i, f"the strict upper-triangular mask of size {seq}")

    def softmax_last(self, i):
        """exp2((a - expand(max a)) / ln 2) * recip(expand(sum ..)) over dim 4 (src/HighLevelOps.jl:318-327) -> a."""
        e, r = self.expect(i, G.Mul, "softmax's e / sum(e)")
        s = self.expect(self.expect(r, G.Recip, "1 / sum(e)")[0], G.Expand, "expand(sum(e))")[0]
        if not (isinstance(self.op(s), G.SumReduce) and self.op(s).dim == 4 and self.ins(s) == [e]):
            self.fail(s, "sum(e) over the key dim")
        d, k = self.with_const(self.expect(e, G.Exp2, "exp2(..)")[0], G.Mul, "(a - max) * (1/ln 2)")
        a, nm = self.expect(d, G.Add, "a - max")
        mx, m1 = self.with_const(nm, G.Mul, "max * -1")
        red = self.expect(mx, G.Expand, "expand(max)")[0]
        if not (abs(k - 1.0 / math.log(2.0)) < 1e-6 and m1 == -1.0 and isinstance(self.op(red), G.MaxReduce)
                and self.op(red).dim == 4 and self.ins(red) == [a]):
            self.fail(i, "a softmax over the key dim")
        return a

    def split_heads(self, i):
        """permute[1,3,2,4](reshape[B,S,heads,D](Linear(x))) -> (weight, heads, D, x)."""
        if not (isinstance(self.op(i), G.Permute) and self.op(i).dims == (1, 3, 2, 4)):
            self.fail(i, "permute [1,3,2,4] of the head split")
        r = self.expect(self.ins(i)[0], G.Reshape, "reshape to [batch, seq, heads, head_dim]")[0]
        x, w = self.linear(r)
        shp = self.shape(self.ins(i)[0])
        return w, shp[2], shp[3], x

    def repeated(self, i, H):
        """repeat_kv (src/NN.jl:305-317): reshape[B,H,S,D](expand(x, 3, groups)), or x itself when groups == 1."""
        if self.shape(i)[1] == H and isinstance(self.op(i), G.Reshape) and isinstance(self.op(self.ins(i)[0]), G.Expand):
            e = self.ins(i)[0]
            if self.op(e).dim != 3 or self.op(e).size * self.shape(self.ins(e)[0])[1] != H:
                self.fail(e, "expand(kv, 3, heads / kv_heads)")
            return self.ins(e)[0]
        return i

    def attention(self, i):
        """SelfAttention's output projection and everything under it down to the tensor the q, k and v
        projections read (src/NN.jl:320-387)."""
        ctx, w_o = self.linear(i)
        B, S, hidden = self.shape(ctx)
        pv = self.expect(ctx, G.Reshape, "reshape to [batch, seq, hidden]")[0]
        if not (isinstance(self.op(pv), G.Permute) and self.op(pv).dims == (1, 3, 2, 4)):
            self.fail(pv, "permute [1,3,2,4] of the attention output")
        probs, vals = self.expect(self.ins(pv)[0], G.MatMul, "probs x values")
        H = self.shape(probs)[1]
        scores = self.softmax_last(probs)
        if S > 1:
            scores, mask = self.expect(scores, G.Add, "scores + causal mask")
            self.causal_mask(mask, S)
        qk, scale = self.with_const(scores, G.Mul, "q.k * 1/sqrt(head_dim)")
        q, kt = self.expect(qk, G.MatMul, "queries x keys^T")
        if not (isinstance(self.op(kt), G.Permute) and self.op(kt).dims == (1, 2, 4, 3)):
            self.fail(kt, "permute [1,2,4,3] of the keys")
        q_in, base_q, prev_q = self.rope(q)
        k_in, base_k, prev_k = self.rope(self.repeated(self.ins(kt)[0], H))
        w_q, Hq, D, xq = self.split_heads(q_in)
        w_k, KV, Dk, xk = self.split_heads(k_in)
        w_v, KVv, Dv, xv = self.split_heads(self.repeated(vals, H))
        if not (xq == xk == xv):
            self.fail(i, "q, k and v projections of one tensor")
        if not (Hq == H and D == Dk == Dv and KV == KVv and H % KV == 0 and H * D == hidden and base_q == base_k and prev_q == prev_k
                and abs(scale * math.sqrt(D) - 1.0) < 1e-5):
            self.fail(i, "consistent head counts, head_dim, RoPE base and 1/sqrt(head_dim) scale")
        return xq, dict(q=w_q, k=w_k, v=w_v, o=w_o, H=H, KV=KV, D=D, base=base_q, prev=prev_q, B=B, S=S)

    def block(self, i):
        """TransformerBlock (src/NN.jl:390-414): x + attn(norm(x)), then + mlp(norm(.)) -> (block input, parts)."""
        h, ff = self.expect(i, G.Add, "residual + mlp")
        act, w_down = self.linear(ff)
        sg, up = self.expect(act, G.Mul, "silu(gate) * up")
        gate = self.silu(sg)
        n2, w_gate = self.linear(gate)
        n2b, w_up = self.linear(up)
        h2, g_post, eps2 = self.rmsnorm(n2)
        if n2 != n2b or h2 != h:
            self.fail(ff, "gate and up projections of one normalised residual")
        x, at = self.expect(h, G.Add, "residual + attention")
        n1, parts = self.attention(at)
        x1, g_in, eps1 = self.rmsnorm(n1)
        if x1 != x or eps1 != eps2:
            self.fail(at, "attention over the normalised block input, one epsilon per block")
        parts.update(gate=w_gate, up=w_up, down=w_down, post=g_post, inp=g_in, eps=eps1)
        return x, parts


_ROLE_NAMES = (("q", "self_attn.q_proj"), ("k", "self_attn.k_proj"), ("v", "self_attn.v_proj"), ("o", "self_attn.o_proj"),
               ("gate", "mlp.gate_proj"), ("up", "mlp.up_proj"), ("down", "mlp.down_proj"),
               ("inp", "input_layernorm"), ("post", "post_attention_layernorm"))


def match_decoder(graph, output_id: int) -> DecoderMatch:
    """Recognises Llama / Phi3 (src/NN.jl:417-507) ending in the logits node `output_id`:
    lm_head(norm(block^L(embedding(tokens)))).  Raises MatchError at the first node that does not fit."""
    w = _Walker(graph)
    if not 1 <= output_id <= len(graph.nodes):
        raise MatchError(f"no node {output_id}")
    normed, w_head = w.linear(output_id)
    x, g_final, eps = w.rmsnorm(normed)
    layers = []
    while not (isinstance(w.op(x), G.Function) and w.op(x).name == "Gather"):
        if not isinstance(w.op(x), G.Add):
            w.fail(x, "a transformer block's residual sum, or the embedding gather")
        x, parts = w.block(x)
        layers.append(parts)
    if not layers:
        raise MatchError("no transformer block between the embedding and the final norm")
    layers.reverse()
    table, tokens = w.ins(x)
    if not (w.is_input(table) and len(w.shape(table)) == 2 and w.is_input(tokens)):
        w.fail(x, "gather(embedding table input, token input)")
    first = layers[0]
    for n, p in enumerate(layers):
        same = all(p[k] == first[k] for k in ("H", "KV", "D", "base", "prev", "B", "S")) and p["eps"] == eps
        dims = all(w.shape(p[a]) == w.shape(first[a]) for a, _ in _ROLE_NAMES)
        if not (same and dims):
            raise MatchError(f"block {n} differs from block 0 in its head split, widths, epsilon or RoPE constants")
    hidden = first["H"] * first["D"]
    inter = w.shape(first["gate"])[0]
    want = {"q": (hidden, hidden), "k": (first["KV"] * first["D"], hidden), "v": (first["KV"] * first["D"], hidden),
            "o": (hidden, hidden), "gate": (inter, hidden), "up": (inter, hidden), "down": (hidden, inter)}
    for role, shp in want.items():
        if w.shape(first[role]) != shp:
            w.fail(first[role], f"{role} weight of shape {list(shp)}")
    vocab = w.shape(w_head)[0]
    if w.shape(table) != (vocab, hidden) or w.shape(w_head) != (vocab, hidden) or w.shape(g_final) != (hidden,):
        w.fail(table, f"[{vocab}, {hidden}] embedding table, lm_head and a [{hidden}] final gain")
    if w.shape(tokens) != (first["B"], first["S"]):
        w.fail(tokens, f"token ids of shape [{first['B']}, {first['S']}]")
    weights = {"model.embed_tokens.weight": table, "model.norm.weight": g_final, "lm_head.weight": w_head}
    for n, p in enumerate(layers):
        for role, name in _ROLE_NAMES:
            weights[f"model.layers.{n}.{name}.weight"] = p[role]
    if len(set(weights.values())) != len(weights):
        raise MatchError("one input tensor plays two weight roles")
    return DecoderMatch(n_layers=len(layers), hidden=hidden, n_heads=first["H"], n_kv_heads=first["KV"], head_dim=first["D"],
                        intermediate=inter, vocab=vocab, eps=eps, rope_base=first["base"], prev_seq=first["prev"],
                        batch=first["B"], seq=first["S"], tokens=tokens, weights=weights)


def compile_b200(graph, output_id, inputs=None, device=None, max_ctx=2048, dtype="f32", batch=None):
    """compile() for a graph match_decoder recognises: returns (Session, DecoderMatch).  The weights come from
    `inputs` (node id -> array, as execute() takes them) or from data pre-loaded into graph.tensors
    (src/Weights.jl:60-114 fills those).  The session keeps a KV cache, so the caller feeds it the tokens
    the graph was traced for (prefill) and then one token per step, instead of re-running a longer graph
    for every position as examples/llama.jl:39-99 does."""
    from .device import DeviceArray, get_device
    from .session import Model, Session
    m = match_decoder(graph, output_id)
    if m.prev_seq != 0:
        raise MatchError("the graph was traced with prev_seq != 0: a cached session starts at position 0")
    dev = device or get_device()
    model = Model(dev, n_layers=m.n_layers, hidden=m.hidden, n_heads=m.n_heads, n_kv_heads=m.n_kv_heads,
                  intermediate=m.intermediate, vocab=m.vocab, eps=m.eps, rope_base=m.rope_base, dtype=dtype)
    inputs = inputs or {}
    for name, node_id in m.weights.items():
        data = inputs.get(node_id)
        if data is None:
            data = graph.tensors.get((node_id, 1))
        if data is None:
            raise KeyError(f"{name} (node {node_id}) has no data")
        model.set_weight(name, data.numpy() if isinstance(data, DeviceArray) else np.asarray(data, dtype=np.float32))
    missing = model.missing_weights()
    if missing:
        model.close()
        raise KeyError(f"the graph leaves {len(missing)} model tensors unset: {missing[:6]}")
    return Session(model, batch or m.batch, max_ctx), m


__all__ = ["MatchError", "DecoderMatch", "export_graph", "import_graph", "match_decoder", "compile_b200"]

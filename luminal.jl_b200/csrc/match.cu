// Recognising a decoder-only transformer in a bare node list (host code only: no kernel here).
//
// The reference's only plugin seam is its graph: a backend sees Graph.nodes (src/Graph.jl:4-26), a flat,
// topologically ordered list of primitive ops with every NN layer already decomposed (src/NN.jl,
// src/HighLevelOps.jl).  lmb200_match_decoder walks such a list backwards from the logits node and recovers, by
// structure alone -- no model object, no weight names -- what src/NN.jl:390-455 built: the layer count, the
// widths, the head split, the RMSNorm epsilon, the RoPE base, and which input-tensor node plays which weight's
// role.  lmb200_compile_node_list hands that to the fused session.  A graph that deviates anywhere (another
// activation, a bias, a different mask) is refused with LMB200_ENOMATCH and a message naming the node; the caller
// then runs it node by node.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <set>
#include <string>
#include <vector>

#include "common.cuh"

namespace {

struct NoMatch {
  std::string what;
};

const char* kOpNames[] = {"Log2", "Exp2", "Sin", "Sqrt", "Cos", "Recip", "Contiguous", "ReLU", "Add", "Mul", "Mod", "Max",
                          "LessThan", "FusedMulAdd", "FusedAddReLU", "MatMul", "SumReduce", "MaxReduce", "Permute", "Expand",
                          "Reshape", "Slice", "Pad", "Unfold", "Constant", "InputTensor", "Gather", "CumSum",
                          "FlashAttentionOp", "Other"};

using Shape = std::vector<int64_t>;

std::string shape_text(const Shape& s) {
  std::string t = "[";
  for (size_t i = 0; i < s.size(); ++i) t += (i ? ", " : "") + std::to_string(s[i]);
  return t + "]";
}

[[noreturn]] void no_match(const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  throw NoMatch{buf};
}

// What one attention + MLP block resolved to: input-tensor node ids by role and the block's constants.
struct Block {
  int q = 0, k = 0, v = 0, o = 0, gate = 0, up = 0, down = 0, inp = 0, post = 0;
  int64_t H = 0, KV = 0, D = 0, B = 0, S = 0;
  double base = 0, eps = 0;
  int64_t prev = 0;
};

struct Walker {
  const lmb200_node_list& g;
  explicit Walker(const lmb200_node_list& list) : g(list) {}

  int op(int i) const { return g.op[i - 1]; }
  int n_in(int i) const { return g.in_off[i] - g.in_off[i - 1]; }
  int in(int i, int k) const { return g.in_node[g.in_off[i - 1] + k]; }
  std::vector<int> ins(int i) const {
    return std::vector<int>(g.in_node + g.in_off[i - 1], g.in_node + g.in_off[i]);
  }
  Shape shape(int i) const { return Shape(g.shape + g.shape_off[i - 1], g.shape + g.shape_off[i]); }
  int n_arg(int i) const { return g.arg_off[i] - g.arg_off[i - 1]; }
  double arg(int i, int k) const { return g.arg[g.arg_off[i - 1] + k]; }
  std::vector<int64_t> iargs(int i) const {
    std::vector<int64_t> a;
    for (int k = 0; k < n_arg(i); ++k) {          // an open slice end arrives as typemax(Int): clamp before the cast
      double v = arg(i, k);
      a.push_back(v >= 4.6e18 ? (int64_t)1 << 62 : v <= -4.6e18 ? -((int64_t)1 << 62) : (int64_t)v);
    }
    return a;
  }

  [[noreturn]] void fail(int i, const std::string& what) const {
    int o = op(i);
    no_match("node %d (%s%s): expected %s", i, o >= 0 && o <= LMB200_NODE_OTHER ? kOpNames[o] : "?",
             shape_text(shape(i)).c_str(), what.c_str());
  }
  std::vector<int> expect(int i, int code, const char* what = nullptr) const {
    if (op(i) != code) fail(i, what ? what : kOpNames[code]);
    return ins(i);
  }
  int expect1(int i, int code, const char* what = nullptr) const {
    auto v = expect(i, code, what);
    if (v.size() != 1) fail(i, what ? what : kOpNames[code]);
    return v[0];
  }
  void expect2(int i, int code, const char* what, int& a, int& b) const {
    auto v = expect(i, code, what);
    if (v.size() != 2) fail(i, what);
    a = v[0];
    b = v[1];
  }
  bool is_input(int i) const { return op(i) == LMB200_NODE_INPUT; }
  bool is_const(int i) const { return op(i) == LMB200_NODE_CONSTANT && n_arg(i) == 1; }
  double cval(int i) const { return arg(i, 0); }
  // Binary node with one Constant operand (either side) -> the other operand and the value.
  int with_const(int i, int code, const char* what, double& value) const {
    int a, b;
    expect2(i, code, what, a, b);
    if (is_const(b)) { value = cval(b); return a; }
    if (is_const(a)) { value = cval(a); return b; }
    fail(i, what);
  }
  int skip(int i, int code) const {
    while (op(i) == code && n_in(i) >= 1) i = in(i, 0);
    return i;
  }
  bool permute_is(int i, std::initializer_list<int64_t> dims) const {
    return op(i) == LMB200_NODE_PERMUTE && iargs(i) == std::vector<int64_t>(dims);
  }

  // MatMul(x, Permute[2,1](W)) with W a rank-2 input tensor and no bias (src/NN.jl:23-35).
  void linear(int i, int& x, int& w) const {
    int wt;
    expect2(i, LMB200_NODE_MATMUL, "a Linear's MatMul", x, wt);
    if (!permute_is(wt, {2, 1})) fail(wt, "Permute[2,1] of a weight");
    w = in(wt, 0);
    if (!(is_input(w) && shape(w).size() == 2)) fail(w, "a [out, in] weight input");
  }

  // x * expand(recip(sqrt(sum(x*x)*(1/n) + eps))) * expand(g)   (src/NN.jl:138-173 with mean_norm off,
  // src/HighLevelOps.jl:296-300)
  void rmsnorm(int i, int& x, int& gain, double& eps) const {
    int a, b;
    expect2(i, LMB200_NODE_MUL, "RMSNorm's scale by the gain", a, b);
    gain = skip(b, LMB200_NODE_EXPAND);
    if (!(is_input(gain) && shape(gain).size() == 1)) {
      std::swap(a, b);
      gain = skip(b, LMB200_NODE_EXPAND);
    }
    if (!(is_input(gain) && shape(gain).size() == 1)) fail(i, "RMSNorm's scale by a [hidden] gain");
    int inv;
    expect2(a, LMB200_NODE_MUL, "x * inv_rms", x, inv);
    int ex = expect1(inv, LMB200_NODE_EXPAND, "expand(inv_rms)");
    int sq = expect1(ex, LMB200_NODE_RECIP, "recip(sqrt(...))");
    int ms = expect1(sq, LMB200_NODE_SQRT, "sqrt(mean + eps)");
    int mean = with_const(ms, LMB200_NODE_ADD, "mean + eps", eps);
    double inv_n;
    int total = with_const(mean, LMB200_NODE_MUL, "sum * (1/n)", inv_n);
    Shape xs = shape(x);
    if (xs.empty()) fail(x, "a tensor to normalise");
    int64_t n = xs.back();
    if (std::fabs(inv_n * (double)n - 1.0) > 1e-5) fail(mean, "sum * (1/" + std::to_string(n) + ")");
    if (!(op(total) == LMB200_NODE_SUM_REDUCE && n_arg(total) == 1 && (int64_t)arg(total, 0) == (int64_t)xs.size()))
      fail(total, "sum over the last dim");
    int p, q;
    expect2(in(total, 0), LMB200_NODE_MUL, "x * x", p, q);
    if (!(p == q && p == x)) fail(in(total, 0), "x * x of the normalised tensor");
    if (shape(gain)[0] != n) fail(gain, "a gain of length " + std::to_string(n));
  }

  // a * (1 * recip(1 + exp2(a * -1 * (1/ln 2))))   (src/HighLevelOps.jl:153-160)
  int silu(int i) const {
    int a, s;
    expect2(i, LMB200_NODE_MUL, "silu(gate)", a, s);
    double one, one2, k, m1;
    int r = with_const(s, LMB200_NODE_MUL, "1 / (1 + exp2(..))", one);
    int den = expect1(r, LMB200_NODE_RECIP, "recip(1 + exp2(..))");
    int e = with_const(den, LMB200_NODE_ADD, "1 + exp2(..)", one2);
    int ar = expect1(e, LMB200_NODE_EXP2, "exp2(-a / ln 2)");
    int neg = with_const(ar, LMB200_NODE_MUL, "(-a) * (1/ln 2)", k);
    int src = with_const(neg, LMB200_NODE_MUL, "a * -1", m1);
    if (!(one == 1.0 && one2 == 1.0 && m1 == -1.0 && std::fabs(k - 1.0 / std::log(2.0)) < 1e-6 && src == a))
      fail(i, "silu(gate) with the reference's constants");
    return a;
  }

  // arange(n): cumsum(expand(1, n)) - 1, or expand(0, 1) for n == 1   (src/HighLevelOps.jl:336-345)
  int64_t arange(int i) const {
    if (op(i) == LMB200_NODE_EXPAND) {
      if (n_in(i) == 1 && is_const(in(i, 0)) && cval(in(i, 0)) == 0.0 && shape(i) == Shape{1}) return 1;
      fail(i, "arange(1)");
    }
    double m1;
    int c = with_const(i, LMB200_NODE_ADD, "cumsum(ones) - 1", m1);
    if (!(m1 == -1.0 && op(c) == LMB200_NODE_CUMSUM && n_in(c) == 1)) fail(i, "cumsum(ones) - 1");
    int ones = expect1(in(c, 0), LMB200_NODE_EXPAND, "expand(1, n)");
    if (!(is_const(ones) && cval(ones) == 1.0 && shape(c).size() == 1)) fail(c, "cumsum over expand(1, n)");
    return shape(c)[0];
  }

  // (lo, hi) of the last dimension of a Slice / Pad node's argument list
  bool last_pair_is(int i, int64_t lo, int64_t hi, bool others_zero) const {
    auto a = iargs(i);
    if (a.size() < 2 || a.size() % 2) return false;
    if (a[a.size() - 2] != lo || a[a.size() - 1] != hi) return false;
    if (others_zero)
      for (size_t k = 0; k + 2 < a.size(); ++k)
        if (a[k] != 0) return false;
    return true;
  }

  // apply_rotary_embeddings (src/NN.jl:253-303): the half-split rotation of pairs (j, j + D/2) that the
  // column-major reshape to [.., D/2, 2] produces.
  void rope(int i, int& src, double& base, int64_t& prev) const {
    Shape shp = shape(i);
    if (shp.size() != 4 || shp[3] % 2) fail(i, "RoPE output [batch, heads, seq, head_dim]");
    int64_t D = shp[3], half = D / 2;
    int cat = expect1(i, LMB200_NODE_RESHAPE, "reshape of the rotated pairs");
    int pa, pb;
    expect2(cat, LMB200_NODE_ADD, "concat of the two halves", pa, pb);
    int outs[2];
    const int parts[2] = {pa, pb};
    const int64_t want[2][2] = {{0, 1}, {1, 0}};
    for (int h = 0; h < 2; ++h) {
      int e = expect1(parts[h], LMB200_NODE_PAD, "pad of one half");
      if (!last_pair_is(parts[h], want[h][0], want[h][1], true)) fail(parts[h], "pad of one slot along the pair dim");
      outs[h] = expect1(e, LMB200_NODE_EXPAND, "expand(.., 5, 1)");
    }
    // x0' = x0 cos - x1 sin ; x1' = x0 sin + x1 cos
    int t0, t1, x0, cosn, x1, sinn, u0, u1;
    expect2(outs[0], LMB200_NODE_ADD, "x0*cos - x1*sin", t0, t1);
    expect2(t0, LMB200_NODE_MUL, "x0 * cos", x0, cosn);
    double neg;
    int m = with_const(t1, LMB200_NODE_MUL, "-(x1 * sin)", neg);
    expect2(m, LMB200_NODE_MUL, "x1 * sin", x1, sinn);
    expect2(outs[1], LMB200_NODE_ADD, "x0*sin + x1*cos", u0, u1);
    if (neg != -1.0 || op(u0) != LMB200_NODE_MUL || ins(u0) != std::vector<int>{x0, sinn} || op(u1) != LMB200_NODE_MUL ||
        ins(u1) != std::vector<int>{x1, cosn})
      fail(outs[1], "the rotation's second row over the same x0, x1, sin, cos");
    int ang = expect1(sinn, LMB200_NODE_SIN, "sin(angle)");
    int shifted = expect1(cosn, LMB200_NODE_SIN, "cos as sin(pi/2 - angle)");
    double hp, m1;
    int na = with_const(shifted, LMB200_NODE_ADD, "pi/2 - angle", hp);
    int a2 = with_const(na, LMB200_NODE_MUL, "angle * -1", m1);
    if (a2 != ang || m1 != -1.0 || std::fabs(hp - M_PI / 2) > 1e-6) fail(cosn, "sin(pi/2 - angle) of the same angle");
    int srcs[2];
    const int xs[2] = {x0, x1};
    for (int h = 0; h < 2; ++h) {
      int s = expect1(skip(xs[h], LMB200_NODE_CONTIGUOUS), LMB200_NODE_RESHAPE, "reshape of one pair element");
      if (!(op(s) == LMB200_NODE_SLICE && last_pair_is(s, h, h + 1, false))) fail(s, "slice of one element of the pair dim");
      int sp = in(s, 0);
      Shape wantshape = {shp[0], shp[1], shp[2], half, 2};
      if (!(op(sp) == LMB200_NODE_RESHAPE && shape(sp) == wantshape)) fail(sp, "reshape to [.., D/2, 2]");
      srcs[h] = in(sp, 0);
    }
    if (srcs[0] != srcs[1]) fail(i, "both pair elements from one tensor");
    int emb = skip(ang, LMB200_NODE_EXPAND);
    int pcol, frow;
    expect2(emb, LMB200_NODE_MATMUL, "positions x inverse frequencies", pcol, frow);
    double prevd;
    int pos = with_const(expect1(pcol, LMB200_NODE_EXPAND, "positions as a column"), LMB200_NODE_ADD, "arange(seq) + prev_seq", prevd);
    if (arange(pos) != shp[2] || prevd != std::floor(prevd) || prevd < 0) fail(pos, "arange(seq) + a whole prev_seq");
    int inv = expect1(expect1(frow, LMB200_NODE_EXPAND, "frequencies as a row"), LMB200_NODE_RECIP, "1 / base^(2j/D)");
    double lb, inv_d, two;
    int fr = with_const(expect1(inv, LMB200_NODE_EXP2, "exp2(log2(base) * 2j/D)"), LMB200_NODE_MUL, "freqs * log2(base)", lb);
    int f2 = with_const(fr, LMB200_NODE_MUL, "(2j) / D", inv_d);
    int ar = with_const(f2, LMB200_NODE_MUL, "2 * j", two);
    if (two != 2.0 || std::fabs(inv_d * (double)D - 1.0) > 1e-5 || arange(ar) != half) fail(fr, "arange(D/2) * 2 / D");
    // the graph holds log2(base) rounded to float32: snap back to the whole number it came from
    base = std::exp2(lb);
    if (base < std::exp2(40.0) && (double)log2f((float)std::round(base)) == lb) base = std::round(base);
    src = srcs[0];
    prev = (int64_t)prevd;
  }

  // expand(expand(triu(seq, 1) * -1e9))   (src/NN.jl:368-373, src/HighLevelOps.jl:347-361)
  void causal_mask(int i, int64_t seq) const {
    int m = skip(i, LMB200_NODE_EXPAND);
    double big, zero;
    int tri = with_const(m, LMB200_NODE_MUL, "triu * -1e9", big);
    int v, hh;
    expect2(tri, LMB200_NODE_LESSTHAN, "column index > row index", v, hh);
    int h = with_const(hh, LMB200_NODE_ADD, "row index - 0", zero);
    bool ok = big == -1e9 && zero == 0.0 && op(h) == LMB200_NODE_EXPAND && op(v) == LMB200_NODE_EXPAND && n_arg(h) == 2 &&
              n_arg(v) == 2 && (int64_t)arg(h, 0) == 1 && (int64_t)arg(v, 0) == 2;
    if (ok) ok = arange(in(h, 0)) == seq && arange(in(v, 0)) == seq && shape(tri) == Shape{seq, seq};
    if (!ok) fail(i, "the strict upper-triangular mask of size " + std::to_string(seq));
  }

  // exp2((a - expand(max a)) / ln 2) * recip(expand(sum ..)) over dim 4   (src/HighLevelOps.jl:318-327)
  int softmax_last(int i) const {
    int e, r;
    expect2(i, LMB200_NODE_MUL, "softmax's e / sum(e)", e, r);
    int s = expect1(expect1(r, LMB200_NODE_RECIP, "1 / sum(e)"), LMB200_NODE_EXPAND, "expand(sum(e))");
    if (!(op(s) == LMB200_NODE_SUM_REDUCE && n_arg(s) == 1 && (int64_t)arg(s, 0) == 4 && ins(s) == std::vector<int>{e}))
      fail(s, "sum(e) over the key dim");
    double k, m1;
    int d = with_const(expect1(e, LMB200_NODE_EXP2, "exp2(..)"), LMB200_NODE_MUL, "(a - max) * (1/ln 2)", k);
    int a, nm;
    expect2(d, LMB200_NODE_ADD, "a - max", a, nm);
    int mx = with_const(nm, LMB200_NODE_MUL, "max * -1", m1);
    int red = expect1(mx, LMB200_NODE_EXPAND, "expand(max)");
    if (!(std::fabs(k - 1.0 / std::log(2.0)) < 1e-6 && m1 == -1.0 && op(red) == LMB200_NODE_MAX_REDUCE && n_arg(red) == 1 &&
          (int64_t)arg(red, 0) == 4 && ins(red) == std::vector<int>{a}))
      fail(i, "a softmax over the key dim");
    return a;
  }

  // permute[1,3,2,4](reshape[B,S,heads,D](Linear(x)))
  void split_heads(int i, int& w, int64_t& heads, int64_t& D, int& x) const {
    if (!permute_is(i, {1, 3, 2, 4})) fail(i, "permute [1,3,2,4] of the head split");
    int rs = in(i, 0);
    int lin = expect1(rs, LMB200_NODE_RESHAPE, "reshape to [batch, seq, heads, head_dim]");
    linear(lin, x, w);
    Shape s = shape(rs);
    if (s.size() != 4) fail(rs, "reshape to [batch, seq, heads, head_dim]");
    heads = s[2];
    D = s[3];
  }

  // repeat_kv (src/NN.jl:305-317): reshape[B,H,S,D](expand(x, 3, groups)), or x itself when groups == 1
  int repeated(int i, int64_t H) const {
    Shape s = shape(i);
    if (s.size() == 4 && s[1] == H && op(i) == LMB200_NODE_RESHAPE && op(in(i, 0)) == LMB200_NODE_EXPAND) {
      int e = in(i, 0);
      Shape inner = shape(in(e, 0));
      if (!(n_arg(e) == 2 && (int64_t)arg(e, 0) == 3 && inner.size() >= 2 && (int64_t)arg(e, 1) * inner[1] == H))
        fail(e, "expand(kv, 3, heads / kv_heads)");
      return in(e, 0);
    }
    return i;
  }

  // SelfAttention's output projection and everything under it down to the tensor the q, k and v projections
  // read (src/NN.jl:320-387)
  int attention(int i, Block& p) const {
    int ctx;
    linear(i, ctx, p.o);
    Shape cs = shape(ctx);
    if (cs.size() != 3) fail(ctx, "attention output [batch, seq, hidden]");
    int64_t B = cs[0], S = cs[1], hidden = cs[2];
    int pv = expect1(ctx, LMB200_NODE_RESHAPE, "reshape to [batch, seq, hidden]");
    if (!permute_is(pv, {1, 3, 2, 4})) fail(pv, "permute [1,3,2,4] of the attention output");
    int probs, vals;
    expect2(in(pv, 0), LMB200_NODE_MATMUL, "probs x values", probs, vals);
    Shape ps = shape(probs);
    if (ps.size() != 4) fail(probs, "probabilities [batch, heads, seq, keys]");
    int64_t H = ps[1];
    int scores = softmax_last(probs);
    if (S > 1) {
      int sc, mask;
      expect2(scores, LMB200_NODE_ADD, "scores + causal mask", sc, mask);
      causal_mask(mask, S);
      scores = sc;
    }
    double scale;
    int qk = with_const(scores, LMB200_NODE_MUL, "q.k * 1/sqrt(head_dim)", scale);
    int q, kt;
    expect2(qk, LMB200_NODE_MATMUL, "queries x keys^T", q, kt);
    if (!permute_is(kt, {1, 2, 4, 3})) fail(kt, "permute [1,2,4,3] of the keys");
    int q_in, k_in;
    double base_q, base_k;
    int64_t prev_q, prev_k;
    rope(q, q_in, base_q, prev_q);
    rope(repeated(in(kt, 0), H), k_in, base_k, prev_k);
    int xq, xk, xv;
    int64_t Hq, D, KV, Dk, KVv, Dv;
    split_heads(q_in, p.q, Hq, D, xq);
    split_heads(k_in, p.k, KV, Dk, xk);
    split_heads(repeated(vals, H), p.v, KVv, Dv, xv);
    if (!(xq == xk && xk == xv)) fail(i, "q, k and v projections of one tensor");
    if (!(Hq == H && D == Dk && D == Dv && KV == KVv && KV > 0 && H % KV == 0 && H * D == hidden && base_q == base_k &&
          prev_q == prev_k && std::fabs(scale * std::sqrt((double)D) - 1.0) < 1e-5))
      fail(i, "consistent head counts, head_dim, RoPE base and 1/sqrt(head_dim) scale");
    p.H = H; p.KV = KV; p.D = D; p.base = base_q; p.prev = prev_q; p.B = B; p.S = S;
    return xq;
  }

  // ---- Whisper TextDecoder, one cached decode step (src/Whisper.jl:541-742) ------------------------------------
  int sc(int i) const { return skip(i, LMB200_NODE_CONTIGUOUS); }

  // Linear with an optional bias: MatMul(x, Permute[2,1](W)) [+ expand*(b)]   (src/NN.jl:22-35)
  void linear_bias(int i, int& x, int& w, int& b) const {
    b = 0;
    if (op(i) == LMB200_NODE_ADD && n_in(i) == 2) {
      int p = in(i, 0), q = in(i, 1);
      int bq = skip(q, LMB200_NODE_EXPAND), bp = skip(p, LMB200_NODE_EXPAND);
      if (op(p) == LMB200_NODE_MATMUL && is_input(bq) && shape(bq).size() == 1) { b = bq; i = p; }
      else if (op(q) == LMB200_NODE_MATMUL && is_input(bp) && shape(bp).size() == 1) { b = bp; i = q; }
      else fail(i, "a Linear's MatMul plus its [out] bias");
    }
    linear(i, x, w);
    if (b && shape(b)[0] != shape(w)[0]) fail(b, "a bias as long as the weight has rows");
  }

  // LayerNorm (src/NN.jl:138-173): std_norm(mean_norm(x)) * expand(w) + expand(b), over the last dim
  void layernorm(int i, int& x, int& gain, int& bias, double& eps) const {
    int a, bb;
    expect2(i, LMB200_NODE_ADD, "LayerNorm's + bias", a, bb);
    bias = skip(bb, LMB200_NODE_EXPAND);
    if (!(is_input(bias) && shape(bias).size() == 1)) {
      std::swap(a, bb);
      bias = skip(bb, LMB200_NODE_EXPAND);
    }
    if (!(is_input(bias) && shape(bias).size() == 1)) fail(i, "LayerNorm's + a [hidden] bias");
    int centred;
    rmsnorm(a, centred, gain, eps);                    // the scale part is the RMSNorm pattern over the centred tensor
    // mean_norm: x - expand(sum(x) * (1/n))  ==  x + (expand(..) * -1)
    int neg;
    expect2(centred, LMB200_NODE_ADD, "x - mean(x)", x, neg);
    double m1, inv_n;
    int ex = with_const(neg, LMB200_NODE_MUL, "mean * -1", m1);
    int mean = expect1(ex, LMB200_NODE_EXPAND, "expand(mean)");
    int total = with_const(mean, LMB200_NODE_MUL, "sum * (1/n)", inv_n);
    Shape xs = shape(x);
    if (xs.empty()) fail(x, "a tensor to normalise");
    if (!(m1 == -1.0 && std::fabs(inv_n * (double)xs.back() - 1.0) < 1e-5 && op(total) == LMB200_NODE_SUM_REDUCE &&
          n_arg(total) == 1 && (int64_t)arg(total, 0) == (int64_t)xs.size() && in(total, 0) == x))
      fail(centred, "x minus its mean over the last dim");
    if (shape(bias)[0] != xs.back()) fail(bias, "a bias of length " + std::to_string(xs.back()));
  }

  // 1 * recip(1 + exp2(z * -1 * (1/ln 2)))   (src/HighLevelOps.jl:153-155) -> z
  int sigmoid(int s) const {
    double one, one2, k, m1;
    int r = with_const(s, LMB200_NODE_MUL, "1 / (1 + exp2(..))", one);
    int den = expect1(r, LMB200_NODE_RECIP, "recip(1 + exp2(..))");
    int e = with_const(den, LMB200_NODE_ADD, "1 + exp2(..)", one2);
    int ar = expect1(e, LMB200_NODE_EXP2, "exp2(-z / ln 2)");
    int neg = with_const(ar, LMB200_NODE_MUL, "(-z) * (1/ln 2)", k);
    int z = with_const(neg, LMB200_NODE_MUL, "z * -1", m1);
    if (!(one == 1.0 && one2 == 1.0 && m1 == -1.0 && std::fabs(k - 1.0 / std::log(2.0)) < 1e-6))
      fail(s, "sigmoid with the reference's constants");
    return z;
  }

  // gelu (src/HighLevelOps.jl:162-168): a * 0.5 * (1 + tanh(0.7978845608 * a * (1 + 0.044715 * a * a))),
  // tanh(u) = sigmoid(2u) * 2 - 1 -> a
  int gelu(int i) const {
    int half_a, onep;
    expect2(i, LMB200_NODE_MUL, "gelu: (a * 0.5) * (1 + tanh(..))", half_a, onep);
    double c_half, one, m1, two, two2, c0, one2, c1;
    int a = with_const(half_a, LMB200_NODE_MUL, "a * 0.5", c_half);
    int th = with_const(onep, LMB200_NODE_ADD, "1 + tanh(..)", one);
    int sg2 = with_const(th, LMB200_NODE_ADD, "sigmoid(2u) * 2 - 1", m1);
    int sg = with_const(sg2, LMB200_NODE_MUL, "sigmoid(2u) * 2", two);
    int u2 = sigmoid(sg);
    int u = with_const(u2, LMB200_NODE_MUL, "u * 2", two2);
    int ca, poly;
    expect2(u, LMB200_NODE_MUL, "(0.79788 * a) * (1 + 0.044715 * a * a)", ca, poly);
    int a1 = with_const(ca, LMB200_NODE_MUL, "0.7978845608 * a", c0);
    int cub = with_const(poly, LMB200_NODE_ADD, "1 + 0.044715 * a * a", one2);
    int caa, a3;
    expect2(cub, LMB200_NODE_MUL, "(0.044715 * a) * a", caa, a3);
    int a2 = with_const(caa, LMB200_NODE_MUL, "0.044715 * a", c1);
    if (!(c_half == 0.5 && one == 1.0 && m1 == -1.0 && two == 2.0 && two2 == 2.0 && one2 == 1.0 &&
          std::fabs(c0 - 0.7978845608) < 1e-6 && std::fabs(c1 - 0.044715) < 1e-7 && a1 == a && a2 == a && a3 == a))
      fail(i, "gelu of one tensor with the reference's constants");
    return a;
  }

  // softmax over the last of four dims of MatMul(q, keys^T) -> the MatMul's operands
  void attn_probs(int probs, int& q, int& kt) const {
    int weights = softmax_last(probs);
    expect2(weights, LMB200_NODE_MATMUL, "queries x keys^T", q, kt);
  }

  // permute[1,3,2,4](reshape[B,1,H,D](Linear(x) [* scale])) -> the projection's parts
  void step_heads(int i, bool scaled, bool want_bias, int& x, int& w, int& b, int64_t& H, int64_t& D, double& scale) const {
    i = sc(i);
    if (!permute_is(i, {1, 3, 2, 4})) fail(i, "permute [1,3,2,4] of the head split");
    int rs = in(i, 0);
    int lin = expect1(rs, LMB200_NODE_RESHAPE, "reshape to [batch, 1, heads, head_dim]");
    Shape s = shape(rs);
    if (s.size() != 4 || s[1] != 1) fail(rs, "reshape to [batch, 1, heads, head_dim]");
    H = s[2];
    D = s[3];
    scale = 1.0;
    if (scaled) lin = with_const(lin, LMB200_NODE_MUL, "projection * head_dim^-0.25", scale);
    linear_bias(lin, x, w, b);
    if (want_bias != (b != 0)) fail(lin, want_bias ? "a projection with a bias" : "a projection without a bias");
  }

  // a node that is concat_along(a, b, 3) = pad(a, 3, 0, nb) + pad(b, 3, na, 0)   (src/HighLevelOps.jl:243-248)
  bool is_concat3(int i, int& a, int& b) const {
    if (!(op(i) == LMB200_NODE_ADD && n_in(i) == 2 && op(in(i, 0)) == LMB200_NODE_PAD && op(in(i, 1)) == LMB200_NODE_PAD)) return false;
    int pa = in(i, 0), pb = in(i, 1);
    a = in(pa, 0);
    b = in(pb, 0);
    Shape sa = shape(a), sb = shape(b);
    if (sa.size() != 4 || sb.size() != 4) return false;
    auto want = [&](int64_t l, int64_t r) { return std::vector<int64_t>{0, 0, 0, 0, l, r, 0, 0}; };
    return iargs(pa) == want(0, sb[2]) && iargs(pb) == want(sa[2], 0);
  }
  // Slice of an input [B, H, max_seq, D] along dim 3 only -> (input, start, stop)
  bool cache_slice(int i, int& past, int64_t& lo, int64_t& hi) const {
    if (op(i) != LMB200_NODE_SLICE || n_in(i) != 1) return false;
    past = in(i, 0);
    Shape ps = shape(past);
    auto a = iargs(i);
    if (!is_input(past) || ps.size() != 4 || a.size() != 8) return false;
    for (int d = 0; d < 4; ++d) {
      if (d == 2) continue;
      if (a[2 * d] != 0 || a[2 * d + 1] < ps[d]) return false;
    }
    lo = a[4];
    hi = std::min<int64_t>(a[5], ps[2]);
    return true;
  }
  // _kv_scatter (src/Whisper.jl:541-570): past[.., 0:s, :] ++ new_slot ++ past[.., s+1:, :] -> (past, new_slot, s)
  void kv_scatter(int i, int& past, int& slot, int64_t& step) const {
    std::vector<int> parts;
    int cur = i, a, b;
    while (is_concat3(cur, a, b)) {
      parts.insert(parts.begin(), b);
      cur = a;
    }
    parts.insert(parts.begin(), cur);
    if (parts.size() < 2 || parts.size() > 3) fail(i, "a cache with one slot replaced (slice ++ new ++ slice)");
    past = 0;
    slot = 0;
    int64_t at = 0, max_seq = shape(i).size() == 4 ? shape(i)[2] : 0;
    step = -1;
    for (int p : parts) {
      int src;
      int64_t lo, hi;
      if (cache_slice(p, src, lo, hi)) {
        if ((past && src != past) || lo != at || hi <= lo) fail(p, "consecutive slices of one past-cache input");
        past = src;
        at = hi;
      } else {
        Shape s = shape(p);
        if (slot || s.size() != 4 || s[2] != 1) fail(p, "one new [batch, heads, 1, head_dim] slot");
        slot = p;
        step = at;
        at += 1;
      }
    }
    if (!past || !slot || at != max_seq || shape(past)[2] != max_seq) fail(i, "a full-length cache built from one past input and one new slot");
  }
  // TransformerBlock (src/NN.jl:390-414): x + attn(norm(x)), then + mlp(norm(.)) -> the block's input
  int block(int i, Block& p) const {
    int h, ff;
    expect2(i, LMB200_NODE_ADD, "residual + mlp", h, ff);
    int act;
    linear(ff, act, p.down);
    int sg, up;
    expect2(act, LMB200_NODE_MUL, "silu(gate) * up", sg, up);
    int gate = silu(sg);
    int n2, n2b;
    linear(gate, n2, p.gate);
    linear(up, n2b, p.up);
    int h2;
    double eps2;
    rmsnorm(n2, h2, p.post, eps2);
    if (n2 != n2b || h2 != h) fail(ff, "gate and up projections of one normalised residual");
    int x, at;
    expect2(h, LMB200_NODE_ADD, "residual + attention", x, at);
    int n1 = attention(at, p);
    int x1;
    double eps1;
    rmsnorm(n1, x1, p.inp, eps1);
    if (x1 != x || eps1 != eps2) fail(at, "attention over the normalised block input, one epsilon per block");
    p.eps = eps1;
    return x;
  }
};

struct WhisperLayer {
  // input-tensor nodes by role
  int q_w = 0, q_b = 0, k_w = 0, v_w = 0, v_b = 0, o_w = 0, o_b = 0, n1_w = 0, n1_b = 0;
  int cq_w = 0, cq_b = 0, co_w = 0, co_b = 0, n2_w = 0, n2_b = 0, fc1_w = 0, fc1_b = 0, fc2_w = 0, fc2_b = 0, n3_w = 0, n3_b = 0;
  int cross_k = 0, cross_v = 0, self_k = 0, self_v = 0, new_k = 0, new_v = 0;
  int64_t H = 0, D = 0, step = 0, max_seq = 0, enc_seq = 0, B = 0;
  double eps = 0;
};

struct WhisperWalker : Walker {
  using Walker::Walker;

  void check_scale(int at, double scale, int64_t D) const {
    if (std::fabs(scale * scale * scale * scale * (double)D - 1.0) > 1e-4) fail(at, "the (hidden / heads)^-0.25 scale");
  }

  // whisper_self_attn_cached (src/Whisper.jl:584-625) from its out_proj -> the normalised input
  int self_attention(int at, WhisperLayer& L) const {
    int ctx;
    linear_bias(at, ctx, L.o_w, L.o_b);
    if (!L.o_b) fail(at, "out_proj with a bias");
    int pv = expect1(ctx, LMB200_NODE_RESHAPE, "reshape to [batch, 1, hidden]");
    if (!permute_is(pv, {1, 3, 2, 4})) fail(pv, "permute [1,3,2,4] of the attention output");
    int probs, v_ctx, q, kt;
    expect2(in(pv, 0), LMB200_NODE_MATMUL, "probs x values", probs, v_ctx);
    attn_probs(probs, q, kt);
    kt = sc(kt);
    if (!permute_is(kt, {1, 2, 4, 3})) fail(kt, "permute [1,2,4,3] of the cached keys");
    int k_ctx = in(kt, 0);
    // the context is new_cache[.., 0 : step + 1, :]
    auto context = [&](int c, int& cache) {
      if (op(c) != LMB200_NODE_SLICE) fail(c, "slice [0, step + 1) of the updated cache");
      auto a = iargs(c);
      cache = in(c, 0);
      if (a.size() != 8 || a[4] != 0) fail(c, "slice [0, step + 1) of the updated cache");
      return a[5];
    };
    int64_t kn = context(k_ctx, L.new_k), vn = context(v_ctx, L.new_v);
    int k_slot, v_slot;
    int64_t ks, vs;
    kv_scatter(L.new_k, L.self_k, k_slot, ks);
    kv_scatter(L.new_v, L.self_v, v_slot, vs);
    if (!(ks == vs && kn == ks + 1 && vn == vs + 1 && L.self_k != L.self_v)) fail(at, "keys and values written at one position and read up to it");
    L.step = ks;
    L.max_seq = shape(L.self_k)[2];
    int xq, xk, xv, nob;
    int64_t H2, D2, H3, D3;
    double sq, sk, sv;
    step_heads(q, true, true, xq, L.q_w, L.q_b, L.H, L.D, sq);
    step_heads(k_slot, true, false, xk, L.k_w, nob, H2, D2, sk);
    step_heads(v_slot, false, true, xv, L.v_w, L.v_b, H3, D3, sv);
    if (!(xq == xk && xk == xv && L.H == H2 && L.H == H3 && L.D == D2 && L.D == D3 && sq == sk)) fail(at, "q, k and v projections of one tensor with one head split");
    check_scale(q, sq, L.D);
    Shape ps = shape(L.self_k);
    if (!(ps[1] == L.H && ps[3] == L.D && shape(L.self_v) == ps)) fail(L.self_k, "past K and V of shape [batch, heads, max_seq, head_dim]");
    L.B = ps[0];
    return xq;
  }

  // whisper_cross_attn_cached (src/Whisper.jl:633-651)
  int cross_attention(int at, WhisperLayer& L) const {
    int ctx;
    linear_bias(at, ctx, L.co_w, L.co_b);
    if (!L.co_b) fail(at, "out_proj with a bias");
    int pv = expect1(ctx, LMB200_NODE_RESHAPE, "reshape to [batch, 1, hidden]");
    if (!permute_is(pv, {1, 3, 2, 4})) fail(pv, "permute [1,3,2,4] of the attention output");
    int probs, q, kt;
    expect2(in(pv, 0), LMB200_NODE_MATMUL, "probs x encoder values", probs, L.cross_v);
    attn_probs(probs, q, kt);
    kt = sc(kt);
    if (!permute_is(kt, {1, 2, 4, 3})) fail(kt, "permute [1,2,4,3] of the encoder keys");
    L.cross_k = in(kt, 0);
    Shape ks = shape(L.cross_k);
    if (!(is_input(L.cross_k) && is_input(L.cross_v) && ks.size() == 4 && shape(L.cross_v) == ks && L.cross_k != L.cross_v))
      fail(at, "encoder K and V inputs of one [batch, heads, enc_seq, head_dim] shape");
    int x;
    int64_t H, D;
    double s;
    step_heads(q, true, true, x, L.cq_w, L.cq_b, H, D, s);
    if (!(H == L.H && D == L.D && ks[0] == L.B && ks[1] == H && ks[3] == D)) fail(at, "the self attention's head split");
    check_scale(q, s, D);
    L.enc_seq = ks[2];
    return x;
  }

  // one decoder layer of build_decode_step! (src/Whisper.jl:712-729), from its output sum -> its input
  int layer(int i, WhisperLayer& L) const {
    int x2, ff, x1, cr, x0, at;
    expect2(i, LMB200_NODE_ADD, "residual + mlp", x2, ff);
    int act, h, n3, xa, xb, xc;
    linear_bias(ff, act, L.fc2_w, L.fc2_b);
    h = gelu(act);
    linear_bias(h, n3, L.fc1_w, L.fc1_b);
    if (!(L.fc1_b && L.fc2_b)) fail(ff, "fc1 and fc2 with biases");
    double e3, e2, e1;
    layernorm(n3, xa, L.n3_w, L.n3_b, e3);
    if (xa != x2) fail(ff, "the MLP over the normalised residual");
    expect2(x2, LMB200_NODE_ADD, "residual + cross attention", x1, cr);
    expect2(x1, LMB200_NODE_ADD, "residual + self attention", x0, at);
    int n1 = self_attention(at, L);
    layernorm(n1, xc, L.n1_w, L.n1_b, e1);
    int n2 = cross_attention(cr, L);
    layernorm(n2, xb, L.n2_w, L.n2_b, e2);
    if (xb != x1 || xc != x0 || e1 != e2 || e2 != e3) fail(i, "three pre-norm sub-layers over one residual stream, one epsilon");
    L.eps = e1;
    return x0;
  }
};

// ---- Whisper AudioEncoder (src/Whisper.jl:354-404) ---------------------------------------------------------------
struct EncoderLayer {
  int q_w = 0, q_b = 0, k_w = 0, v_w = 0, v_b = 0, o_w = 0, o_b = 0, n1_w = 0, n1_b = 0;
  int fc1_w = 0, fc1_b = 0, fc2_w = 0, fc2_b = 0, n2_w = 0, n2_b = 0;
  int64_t H = 0, D = 0, B = 0, S = 0;
  double eps = 0;
};

struct ConvStem {
  int w = 0, b = 0;
  int64_t c_in = 0, c_out = 0, kernel = 0, stride = 0, pad = 0, len_in = 0, len_out = 0, B = 0;
};

struct EncoderWalker : WhisperWalker {
  using WhisperWalker::WhisperWalker;

  // permute[perm](reshape[B, S, H, D](Linear(x) [* scale])) -> the projection's parts
  void seq_heads(int i, std::initializer_list<int64_t> perm, bool scaled, bool want_bias, int& x, int& w, int& b, int64_t& B,
                 int64_t& S, int64_t& H, int64_t& D, double& scale) const {
    i = sc(i);
    if (!permute_is(i, perm)) fail(i, "the permute of the head split");
    int rs = in(i, 0);
    int lin = expect1(rs, LMB200_NODE_RESHAPE, "reshape to [batch, seq, heads, head_dim]");
    Shape s = shape(rs);
    if (s.size() != 4) fail(rs, "reshape to [batch, seq, heads, head_dim]");
    B = s[0]; S = s[1]; H = s[2]; D = s[3];
    scale = 1.0;
    if (scaled) lin = with_const(lin, LMB200_NODE_MUL, "projection * head_dim^-0.25", scale);
    linear_bias(lin, x, w, b);
    if (want_bias != (b != 0)) fail(lin, want_bias ? "a projection with a bias" : "a projection without a bias");
  }

  // WhisperSelfAttention without a mask (src/Whisper.jl:253-276), from its out_proj -> the normalised input
  int enc_attention(int at, EncoderLayer& L) const {
    int ctx;
    linear_bias(at, ctx, L.o_w, L.o_b);
    if (!L.o_b) fail(at, "out_proj with a bias");
    int pv = expect1(ctx, LMB200_NODE_RESHAPE, "reshape to [batch, seq, hidden]");
    if (!permute_is(pv, {1, 3, 2, 4})) fail(pv, "permute [1,3,2,4] of the attention output");
    int probs, v, q, kt;
    expect2(in(pv, 0), LMB200_NODE_MATMUL, "probs x values", probs, v);
    attn_probs(probs, q, kt);
    int xq, xk, xv, nob;
    int64_t B2, S2, H2, D2, B3, S3, H3, D3;
    double sq, sk, sv;
    seq_heads(q, {1, 3, 2, 4}, true, true, xq, L.q_w, L.q_b, L.B, L.S, L.H, L.D, sq);
    seq_heads(kt, {1, 3, 4, 2}, true, false, xk, L.k_w, nob, B2, S2, H2, D2, sk);
    seq_heads(v, {1, 3, 2, 4}, false, true, xv, L.v_w, L.v_b, B3, S3, H3, D3, sv);
    if (!(xq == xk && xk == xv && L.H == H2 && L.H == H3 && L.D == D2 && L.D == D3 && L.S == S2 && L.S == S3 && L.B == B2 && L.B == B3 &&
          sq == sk))
      fail(at, "q, k and v projections of one tensor with one head split");
    check_scale(q, sq, L.D);
    return xq;
  }

  // EncoderTransformerBlock (src/Whisper.jl:343-352), from its output sum -> its input
  int enc_layer(int i, EncoderLayer& L) const {
    int x1, ff, x0, at;
    expect2(i, LMB200_NODE_ADD, "residual + mlp", x1, ff);
    int act, n2, xa, xb;
    linear_bias(ff, act, L.fc2_w, L.fc2_b);
    int h = gelu(act);
    linear_bias(h, n2, L.fc1_w, L.fc1_b);
    if (!(L.fc1_b && L.fc2_b)) fail(ff, "fc1 and fc2 with biases");
    double e1, e2;
    layernorm(n2, xa, L.n2_w, L.n2_b, e2);
    if (xa != x1) fail(ff, "the MLP over the normalised residual");
    expect2(x1, LMB200_NODE_ADD, "residual + self attention", x0, at);
    int n1 = enc_attention(at, L);
    layernorm(n1, xb, L.n1_w, L.n1_b, e1);
    if (xb != x0 || e1 != e2) fail(i, "two pre-norm sub-layers over one residual stream, one epsilon");
    L.eps = e1;
    return x0;
  }

  // NN.Conv1D (src/NN.jl:55-104): pad, Unfold, permute, column-major merge of (channel, tap), MatMul with the
  // [ch_out, ch_in * kernel] weight, permute back, + bias -> its input
  int conv1d(int i, ConvStem& c) const {
    int out, be;
    expect2(i, LMB200_NODE_ADD, "conv output + bias", out, be);
    c.b = skip(be, LMB200_NODE_EXPAND);
    if (!(is_input(c.b) && shape(c.b).size() == 1)) fail(i, "a [ch_out] bias expanded over batch and length");
    if (!permute_is(out, {1, 3, 2})) fail(out, "permute [1,3,2] back to [batch, ch_out, length]");
    int merged;
    linear(in(out, 0), merged, c.w);
    int perm = expect1(merged, LMB200_NODE_RESHAPE, "reshape to [batch, length, ch_in * kernel]");
    if (!permute_is(perm, {1, 3, 2, 4})) fail(perm, "permute [1,3,2,4] of the unfolded windows");
    int unf = in(perm, 0);
    auto ua = op(unf) == LMB200_NODE_UNFOLD ? iargs(unf) : std::vector<int64_t>();
    if (!(n_in(unf) == 1 && ua.size() == 3 && ua[0] >= 1 && ua[1] >= 1 && ua[2] == 1)) fail(unf, "Unfold over the last dim, dilation 1");
    c.kernel = ua[0];
    c.stride = ua[1];
    int src = in(unf, 0);
    c.pad = 0;
    if (op(src) == LMB200_NODE_PAD) {
      auto pa = iargs(src);
      if (!(pa.size() == 6 && pa[0] == 0 && pa[1] == 0 && pa[2] == 0 && pa[3] == 0 && pa[4] == pa[5] && pa[4] > 0))
        fail(src, "the same padding on both ends of the last dim");
      c.pad = pa[4];
      src = in(src, 0);
    }
    Shape xs = shape(src), us = shape(unf), ws = shape(c.w);
    if (xs.size() != 3 || us.size() != 4) fail(unf, "windows [batch, ch_in, length, kernel] of a [batch, ch_in, length] tensor");
    c.B = xs[0]; c.c_in = xs[1]; c.len_in = xs[2]; c.len_out = us[2];
    c.c_out = ws[0];
    if (!(ws == Shape{c.c_out, c.c_in * c.kernel} && shape(c.b)[0] == c.c_out && us == Shape{c.B, c.c_in, c.len_out, c.kernel} &&
          c.len_out == (c.len_in + 2 * c.pad - c.kernel) / c.stride + 1 && shape(merged) == Shape{c.B, c.len_out, c.c_in * c.kernel}))
      fail(i, "a Conv1D with a [ch_out, ch_in * kernel] weight and a [ch_out] bias");
    return src;
  }

  // sinusoids(channels, length) (src/Whisper.jl:208-231): concat(sin(t), cos(t), 2) with t = arange(length) x rates
  void sinusoid_table(int i, int64_t length, int64_t channels, int& rates) const {
    const int64_t half = channels / 2;
    int pa, pb;
    expect2(i, LMB200_NODE_ADD, "concat(sin(t), cos(t)) along dim 2", pa, pb);
    int s = expect1(pa, LMB200_NODE_PAD, "sin(t) padded to the full width");
    int c = expect1(pb, LMB200_NODE_PAD, "cos(t) padded to the full width");
    if (iargs(pa) != std::vector<int64_t>{0, 0, 0, half} || iargs(pb) != std::vector<int64_t>{0, 0, half, 0})
      fail(i, "two halves of " + std::to_string(half) + " columns each");
    int t = expect1(s, LMB200_NODE_SIN, "sin(t)");
    int shifted = expect1(c, LMB200_NODE_SIN, "cos as sin(pi/2 - t)");
    double hp, m1;
    int na = with_const(shifted, LMB200_NODE_ADD, "pi/2 - t", hp);
    int t2 = with_const(na, LMB200_NODE_MUL, "t * -1", m1);
    if (t2 != t || m1 != -1.0 || std::fabs(hp - M_PI / 2) > 1e-6) fail(c, "sin(pi/2 - t) of the same t");
    int ea, eb;
    expect2(t, LMB200_NODE_MUL, "positions x rates", ea, eb);
    int ar = expect1(ea, LMB200_NODE_EXPAND, "positions as a column");
    rates = expect1(eb, LMB200_NODE_EXPAND, "rates as a row");
    if (!(arange(ar) == length && is_input(rates) && shape(rates) == Shape{half} && shape(i) == Shape{length, channels}))
      fail(t, "arange(" + std::to_string(length) + ") x a [" + std::to_string(half) + "] input of rates");
  }
};

void validate_list(const lmb200_node_list* g);

struct EncoderMatch {
  lmb200_encoder_match info{};
  std::vector<std::pair<std::string, int>> weights;
};

// AudioEncoder(mel) (src/Whisper.jl:379-404) ending in its output node: layer_norm(block^L(permute(gelu(conv2(gelu(
// conv1(mel))))) + sinusoids)).
EncoderMatch match_whisper_encoder(const lmb200_node_list* g, int output_id) {
  validate_list(g);
  EncoderWalker w(*g);
  if (output_id < 1 || output_id > g->n_nodes) no_match("no node %d", output_id);
  int x, ln_w, ln_b;
  double eps;
  w.layernorm(output_id, x, ln_w, ln_b, eps);
  std::vector<EncoderLayer> layers;
  auto is_bottom = [&](int n) { return w.op(n) == LMB200_NODE_ADD && w.n_in(n) == 2 && w.permute_is(w.in(n, 0), {1, 3, 2}); };
  while (!is_bottom(x)) {
    if (w.op(x) != LMB200_NODE_ADD) w.fail(x, "an encoder layer's residual sum, or the conv stem + sinusoids");
    EncoderLayer L;
    x = w.enc_layer(x, L);
    layers.push_back(L);
  }
  if (layers.empty()) no_match("no encoder layer between the conv stem and the final norm");
  std::vector<EncoderLayer> ordered(layers.rbegin(), layers.rend());
  const int table = w.expect1(w.in(x, 1), LMB200_NODE_EXPAND, "the sinusoid table expanded over the batch");
  ConvStem c1, c2;
  const int g2 = w.gelu(w.in(w.in(x, 0), 0));
  const int g1 = w.gelu(w.conv1d(g2, c2));
  const int mel = w.conv1d(g1, c1);
  const EncoderLayer& f = ordered[0];
  const int64_t d = f.H * f.D, ffn = w.shape(f.fc1_w)[0];
  if (!w.is_input(mel)) w.fail(mel, "the mel input [batch, n_mels, frames]");
  if (!(c1.kernel == 3 && c1.stride == 1 && c1.pad == 1 && c2.kernel == 3 && c2.stride == 2 && c2.pad == 1 && c1.c_out == d &&
        c2.c_in == d && c2.c_out == d && c2.len_in == c1.len_out && c2.len_out == f.S && c1.B == f.B && c2.B == f.B))
    w.fail(x, "the stem conv1 (kernel 3, stride 1, padding 1) and conv2 (kernel 3, stride 2, padding 1) into width " + std::to_string(d));
  int rates;
  w.sinusoid_table(table, f.S, d, rates);
  for (size_t n = 0; n < ordered.size(); ++n) {
    const EncoderLayer& p = ordered[n];
    bool same = p.H == f.H && p.D == f.D && p.B == f.B && p.S == f.S && p.eps == eps;
    for (int EncoderLayer::* r : {&EncoderLayer::q_w, &EncoderLayer::k_w, &EncoderLayer::v_w, &EncoderLayer::o_w})
      same = same && w.shape(p.*r) == Shape{d, d};
    same = same && w.shape(p.fc1_w) == Shape{ffn, d} && w.shape(p.fc2_w) == Shape{d, ffn};
    if (!same) no_match("encoder layer %zu differs from layer 0 in its widths, head split, epsilon or sequence length", n);
  }
  if (w.shape(ln_w) != Shape{d}) w.fail(ln_w, "a final gain of length " + std::to_string(d));
  EncoderMatch m;
  m.weights = {{"model.encoder.conv1.weight", c1.w}, {"model.encoder.conv1.bias", c1.b}, {"model.encoder.conv2.weight", c2.w},
               {"model.encoder.conv2.bias", c2.b}, {"model.encoder.layer_norm.weight", ln_w}, {"model.encoder.layer_norm.bias", ln_b}};
  struct ERole { int EncoderLayer::* node; const char* name; };
  static const ERole roles[] = {
      {&EncoderLayer::q_w, "self_attn.q_proj.weight"}, {&EncoderLayer::q_b, "self_attn.q_proj.bias"},
      {&EncoderLayer::k_w, "self_attn.k_proj.weight"}, {&EncoderLayer::v_w, "self_attn.v_proj.weight"},
      {&EncoderLayer::v_b, "self_attn.v_proj.bias"}, {&EncoderLayer::o_w, "self_attn.out_proj.weight"},
      {&EncoderLayer::o_b, "self_attn.out_proj.bias"}, {&EncoderLayer::n1_w, "self_attn_layer_norm.weight"},
      {&EncoderLayer::n1_b, "self_attn_layer_norm.bias"}, {&EncoderLayer::fc1_w, "fc1.weight"}, {&EncoderLayer::fc1_b, "fc1.bias"},
      {&EncoderLayer::fc2_w, "fc2.weight"}, {&EncoderLayer::fc2_b, "fc2.bias"}, {&EncoderLayer::n2_w, "final_layer_norm.weight"},
      {&EncoderLayer::n2_b, "final_layer_norm.bias"}};
  for (size_t n = 0; n < ordered.size(); ++n)
    for (const ERole& r : roles)
      m.weights.push_back({"model.encoder.layers." + std::to_string(n) + "." + r.name, ordered[n].*(r.node)});
  std::set<int> distinct{mel, rates};
  for (auto& kv : m.weights) distinct.insert(kv.second);
  if (distinct.size() != m.weights.size() + 2) no_match("one input tensor plays two roles");
  m.info.d_model = (int32_t)d;
  m.info.heads = (int32_t)f.H;
  m.info.layers = (int32_t)ordered.size();
  m.info.ffn = (int32_t)ffn;
  m.info.n_mels = (int32_t)c1.c_in;
  m.info.batch = (int32_t)f.B;
  m.info.frames = (int32_t)c1.len_in;
  m.info.mel_node = mel;
  m.info.rates_node = rates;
  m.info.n_weights = (int32_t)m.weights.size();
  m.info.eps = (float)eps;
  return m;
}

struct Role {
  int Block::* node;
  const char* name;
};
const Role kRoles[] = {{&Block::q, "self_attn.q_proj"},  {&Block::k, "self_attn.k_proj"}, {&Block::v, "self_attn.v_proj"},
                       {&Block::o, "self_attn.o_proj"},  {&Block::gate, "mlp.gate_proj"}, {&Block::up, "mlp.up_proj"},
                       {&Block::down, "mlp.down_proj"},  {&Block::inp, "input_layernorm"},
                       {&Block::post, "post_attention_layernorm"}};

void validate_list(const lmb200_node_list* g) {
  if (!g || g->n_nodes <= 0 || !g->op || !g->in_off || !g->shape_off || !g->arg_off) no_match("empty or incomplete node list");
  for (int n = 1; n <= g->n_nodes; ++n) {
    if (g->in_off[n] < g->in_off[n - 1] || g->shape_off[n] < g->shape_off[n - 1] || g->arg_off[n] < g->arg_off[n - 1])
      no_match("node %d: offsets run backwards", n);
    if (g->op[n - 1] < 0 || g->op[n - 1] > LMB200_NODE_OTHER) no_match("node %d: unknown op code %d", n, g->op[n - 1]);
    for (int k = g->in_off[n - 1]; k < g->in_off[n]; ++k)
      if (g->in_node[k] < 1 || g->in_node[k] >= n) no_match("node %d: input %d is not an earlier node", n, g->in_node[k]);
  }
  // The movement ops carry their result shape twice, in their fields and in the shape recorded for the node
  // (src/Graph.jl:4-26 keeps both): a list in which the two disagree is not a traced graph.
  Walker w(*g);
  for (int n = 1; n <= g->n_nodes; ++n) {
    const int o = w.op(n);
    if (o != LMB200_NODE_PERMUTE && o != LMB200_NODE_EXPAND && o != LMB200_NODE_RESHAPE && o != LMB200_NODE_SLICE && o != LMB200_NODE_PAD) continue;
    if (w.n_in(n) != 1) no_match("node %d: a movement op takes one input", n);
    const Shape in = w.shape(w.in(n, 0)), out = w.shape(n);
    const std::vector<int64_t> a = w.iargs(n);
    Shape want;
    bool ok = true;
    if (o == LMB200_NODE_RESHAPE) {
      want = Shape(a.begin(), a.end());
    } else if (o == LMB200_NODE_PERMUTE) {
      ok = a.size() == in.size();
      for (size_t k = 0; ok && k < a.size(); ++k) {
        ok = a[k] >= 1 && a[k] <= (int64_t)in.size();
        if (ok) want.push_back(in[a[k] - 1]);
      }
    } else if (o == LMB200_NODE_EXPAND) {
      ok = a.size() == 2 && a[0] >= 1 && a[0] <= (int64_t)in.size() + 1;
      if (ok) {
        want = in;
        want.insert(want.begin() + (a[0] - 1), a[1]);
      }
    } else {
      ok = a.size() == 2 * in.size();
      for (size_t d = 0; ok && d < in.size(); ++d)
        want.push_back(o == LMB200_NODE_PAD ? in[d] + a[2 * d] + a[2 * d + 1]
                                            : std::min<int64_t>(a[2 * d + 1], in[d]) - std::max<int64_t>(a[2 * d], 0));
    }
    if (!ok || want != out) no_match("node %d (%s): its fields give %s from an input of %s, the node records %s", n, kOpNames[o],
                                     ok ? shape_text(want).c_str() : "no shape", shape_text(in).c_str(), shape_text(out).c_str());
  }
}

struct Match {
  lmb200_model_config cfg{};
  lmb200_decoder_match info{};
  std::vector<std::pair<std::string, int>> weights;
  std::vector<int> cache;        // Whisper: cross K, cross V, past self K, past self V, new self K, new self V; n_layers of each
};

Match match_decoder(const lmb200_node_list* g, int output_id) {
  validate_list(g);
  Walker w(*g);
  if (output_id < 1 || output_id > g->n_nodes) no_match("no node %d", output_id);
  int normed, w_head, x, g_final;
  double eps;
  w.linear(output_id, normed, w_head);
  w.rmsnorm(normed, x, g_final, eps);
  std::vector<Block> layers;
  while (w.op(x) != LMB200_NODE_GATHER) {
    if (w.op(x) != LMB200_NODE_ADD) w.fail(x, "a transformer block's residual sum, or the embedding gather");
    Block b;
    x = w.block(x, b);
    layers.push_back(b);
  }
  if (layers.empty()) no_match("no transformer block between the embedding and the final norm");
  std::vector<Block> ordered(layers.rbegin(), layers.rend());
  if (w.n_in(x) != 2) w.fail(x, "gather(embedding table input, token input)");
  int table = w.in(x, 0), tokens = w.in(x, 1);
  if (!(w.is_input(table) && w.shape(table).size() == 2 && w.is_input(tokens)))
    w.fail(x, "gather(embedding table input, token input)");
  const Block& f = ordered[0];
  for (size_t n = 0; n < ordered.size(); ++n) {
    const Block& p = ordered[n];
    bool same = p.H == f.H && p.KV == f.KV && p.D == f.D && p.base == f.base && p.prev == f.prev && p.B == f.B && p.S == f.S &&
                p.eps == eps;
    for (const Role& r : kRoles) same = same && w.shape(p.*(r.node)) == w.shape(f.*(r.node));
    if (!same) no_match("block %zu differs from block 0 in its head split, widths, epsilon or RoPE constants", n);
  }
  int64_t hidden = f.H * f.D, inter = w.shape(f.gate)[0];
  struct { int node; Shape want; const char* role; } checks[] = {
      {f.q, {hidden, hidden}, "q"},       {f.k, {f.KV * f.D, hidden}, "k"}, {f.v, {f.KV * f.D, hidden}, "v"},
      {f.o, {hidden, hidden}, "o"},       {f.gate, {inter, hidden}, "gate"}, {f.up, {inter, hidden}, "up"},
      {f.down, {hidden, inter}, "down"}};
  for (auto& c : checks)
    if (w.shape(c.node) != c.want) w.fail(c.node, std::string(c.role) + " weight of shape " + shape_text(c.want));
  int64_t vocab = w.shape(w_head)[0];
  if (w.shape(table) != Shape{vocab, hidden} || w.shape(w_head) != Shape{vocab, hidden} || w.shape(g_final) != Shape{hidden})
    w.fail(table, "[" + std::to_string(vocab) + ", " + std::to_string(hidden) + "] embedding table, lm_head and a final gain");
  if (w.shape(tokens) != Shape{f.B, f.S}) w.fail(tokens, "token ids of shape " + shape_text(Shape{f.B, f.S}));

  Match m;
  m.weights = {{"model.embed_tokens.weight", table}, {"model.norm.weight", g_final}, {"lm_head.weight", w_head}};
  for (size_t n = 0; n < ordered.size(); ++n)
    for (const Role& r : kRoles)
      m.weights.push_back({"model.layers." + std::to_string(n) + "." + r.name + ".weight", ordered[n].*(r.node)});
  std::set<int> distinct;
  for (auto& kv : m.weights) distinct.insert(kv.second);
  if (distinct.size() != m.weights.size()) no_match("one input tensor plays two weight roles");
  m.cfg.n_layers = (int32_t)ordered.size();
  m.cfg.hidden = (int32_t)hidden;
  m.cfg.n_heads = (int32_t)f.H;
  m.cfg.n_kv_heads = (int32_t)f.KV;
  m.cfg.head_dim = (int32_t)f.D;
  m.cfg.intermediate = (int32_t)inter;
  m.cfg.vocab = (int32_t)vocab;
  m.cfg.rms_eps = (float)eps;
  m.cfg.rope_base = (float)f.base;
  m.cfg.dtype = LMB200_F32;
  m.cfg.tp_size = 1;
  m.cfg.tp_rank = 0;
  m.cfg.arch = LMB200_ARCH_LLAMA;
  m.info.arch = LMB200_ARCH_LLAMA;
  m.info.batch = (int32_t)f.B;
  m.info.seq = (int32_t)f.S;
  m.info.prev_seq = (int32_t)f.prev;
  m.info.tokens_node = tokens;
  m.info.n_weights = (int32_t)m.weights.size();
  return m;
}

// build_decode_step! (src/Whisper.jl:687-742) ending in the logits node: the tied-embedding head over
// layer_norm(layer^L(embedding(token) + position slot)).
Match match_whisper_step(const lmb200_node_list* g, int output_id) {
  validate_list(g);
  WhisperWalker w(*g);
  if (output_id < 1 || output_id > g->n_nodes) no_match("no node %d", output_id);
  int first, wt;
  w.expect2(output_id, LMB200_NODE_MATMUL, "the head's MatMul", first, wt);
  if (!w.permute_is(wt, {2, 1})) w.fail(wt, "Permute[2,1] of the embedding table");
  int emb = w.in(wt, 0);
  first = w.sc(first);
  if (w.op(first) != LMB200_NODE_SLICE) w.fail(first, "slice of the first (only) position of the normalised output");
  int out = w.in(first, 0), x, ln_w, ln_b;
  double eps;
  w.layernorm(out, x, ln_w, ln_b, eps);
  std::vector<WhisperLayer> layers;
  auto is_bottom = [&](int n) {
    return w.op(n) == LMB200_NODE_ADD && w.n_in(n) == 2 && (w.op(w.in(n, 0)) == LMB200_NODE_GATHER || w.op(w.in(n, 1)) == LMB200_NODE_GATHER);
  };
  while (!is_bottom(x)) {
    if (w.op(x) != LMB200_NODE_ADD) w.fail(x, "a decoder layer's residual sum, or embedding + position");
    WhisperLayer L;
    x = w.layer(x, L);
    layers.push_back(L);
  }
  if (layers.empty()) no_match("no decoder layer between the embedding and the final norm");
  std::vector<WhisperLayer> ordered(layers.rbegin(), layers.rend());
  int ga = w.in(x, 0), pe = w.in(x, 1);
  if (w.op(ga) != LMB200_NODE_GATHER) std::swap(ga, pe);
  int table = w.in(ga, 0), tokens = w.in(ga, 1);
  const WhisperLayer& f = ordered[0];
  const int64_t hidden = f.H * f.D;
  if (!(table == emb && w.is_input(table) && w.is_input(tokens) && w.shape(table).size() == 2 && w.shape(table)[1] == hidden &&
        w.shape(tokens) == Shape{f.B, 1}))
    w.fail(ga, "gather(the head's embedding table, token ids [batch, 1])");
  // + expand(contiguous(slice(pos_embedding, 1, step, step + 1)), 1, batch)
  int slot = w.sc(w.expect1(pe, LMB200_NODE_EXPAND, "the position slot expanded over the batch"));
  if (w.op(slot) != LMB200_NODE_SLICE) w.fail(slot, "slice of one row of the position table");
  int pos = w.in(slot, 0);
  auto pr = w.iargs(slot);
  if (!(w.is_input(pos) && w.shape(pos).size() == 2 && w.shape(pos)[1] == hidden && pr.size() == 4 && pr[1] == pr[0] + 1 && pr[0] == f.step))
    w.fail(slot, "row `step` of a [max_positions, hidden] position table");
  int64_t ffn = w.shape(f.fc1_w)[0];
  for (size_t n = 0; n < ordered.size(); ++n) {
    const WhisperLayer& p = ordered[n];
    bool same = p.H == f.H && p.D == f.D && p.step == f.step && p.max_seq == f.max_seq && p.enc_seq == f.enc_seq && p.B == f.B &&
                p.eps == eps;
    for (int WhisperLayer::* r : {&WhisperLayer::q_w, &WhisperLayer::k_w, &WhisperLayer::v_w, &WhisperLayer::o_w, &WhisperLayer::cq_w,
                                 &WhisperLayer::co_w})
      same = same && w.shape(p.*r) == Shape{hidden, hidden};
    same = same && w.shape(p.fc1_w) == Shape{ffn, hidden} && w.shape(p.fc2_w) == Shape{hidden, ffn};
    if (!same) no_match("decoder layer %zu differs from layer 0 in its widths, head split, epsilon, position or cache shapes", n);
  }
  Match m;
  m.weights = {{"model.decoder.embed_tokens.weight", table}, {"model.decoder.embed_positions.weight", pos},
               {"model.decoder.layer_norm.weight", ln_w}, {"model.decoder.layer_norm.bias", ln_b}};
  struct WRole { int WhisperLayer::* node; const char* name; };
  static const WRole roles[] = {
      {&WhisperLayer::q_w, "self_attn.q_proj.weight"}, {&WhisperLayer::k_w, "self_attn.k_proj.weight"},
      {&WhisperLayer::v_w, "self_attn.v_proj.weight"}, {&WhisperLayer::q_b, "self_attn.q_proj.bias"},
      {&WhisperLayer::v_b, "self_attn.v_proj.bias"}, {&WhisperLayer::o_w, "self_attn.out_proj.weight"},
      {&WhisperLayer::o_b, "self_attn.out_proj.bias"}, {&WhisperLayer::n1_w, "self_attn_layer_norm.weight"},
      {&WhisperLayer::n1_b, "self_attn_layer_norm.bias"}, {&WhisperLayer::cq_w, "encoder_attn.q_proj.weight"},
      {&WhisperLayer::cq_b, "encoder_attn.q_proj.bias"}, {&WhisperLayer::co_w, "encoder_attn.out_proj.weight"},
      {&WhisperLayer::co_b, "encoder_attn.out_proj.bias"}, {&WhisperLayer::n2_w, "encoder_attn_layer_norm.weight"},
      {&WhisperLayer::n2_b, "encoder_attn_layer_norm.bias"}, {&WhisperLayer::fc1_w, "fc1.weight"},
      {&WhisperLayer::fc1_b, "fc1.bias"}, {&WhisperLayer::fc2_w, "fc2.weight"}, {&WhisperLayer::fc2_b, "fc2.bias"},
      {&WhisperLayer::n3_w, "final_layer_norm.weight"}, {&WhisperLayer::n3_b, "final_layer_norm.bias"}};
  for (size_t n = 0; n < ordered.size(); ++n)
    for (const WRole& r : roles)
      m.weights.push_back({"model.decoder.layers." + std::to_string(n) + "." + r.name, ordered[n].*(r.node)});
  std::set<int> distinct;
  for (auto& kv : m.weights) distinct.insert(kv.second);
  for (int WhisperLayer::*r : {&WhisperLayer::cross_k, &WhisperLayer::cross_v, &WhisperLayer::self_k, &WhisperLayer::self_v,
                               &WhisperLayer::new_k, &WhisperLayer::new_v})
    for (const WhisperLayer& p : ordered) {
      m.cache.push_back(p.*r);
      distinct.insert(p.*r);
    }
  if (distinct.size() != m.weights.size() + m.cache.size()) no_match("one input tensor plays two roles");
  m.cfg.n_layers = (int32_t)ordered.size();
  m.cfg.hidden = (int32_t)hidden;
  m.cfg.n_heads = m.cfg.n_kv_heads = (int32_t)f.H;
  m.cfg.head_dim = (int32_t)f.D;
  m.cfg.intermediate = (int32_t)ffn;
  m.cfg.vocab = (int32_t)w.shape(table)[0];
  m.cfg.rms_eps = (float)eps;
  m.cfg.rope_base = 10000.f;
  m.cfg.dtype = LMB200_F32;
  m.cfg.tp_size = 1;
  m.cfg.arch = LMB200_ARCH_WHISPER_DECODER;
  m.cfg.max_positions = (int32_t)w.shape(pos)[0];
  m.cfg.cross_len = (int32_t)f.enc_seq;
  m.info.arch = LMB200_ARCH_WHISPER_DECODER;
  m.info.batch = (int32_t)f.B;
  m.info.seq = 1;
  m.info.prev_seq = (int32_t)f.step;
  m.info.tokens_node = tokens;
  m.info.n_weights = (int32_t)m.weights.size();
  m.info.max_seq = (int32_t)f.max_seq;
  m.info.cross_len = (int32_t)f.enc_seq;
  return m;
}

// Which builder's graph ends here?  The Whisper step reads its head input through a slice of the first position.
Match match_any(const lmb200_node_list* g, int output_id) {
  validate_list(g);
  Walker w(*g);
  if (output_id >= 1 && output_id <= g->n_nodes && w.op(output_id) == LMB200_NODE_MATMUL && w.n_in(output_id) == 2 &&
      w.op(w.sc(w.in(output_id, 0))) == LMB200_NODE_SLICE)
    return match_whisper_step(g, output_id);
  return match_decoder(g, output_id);
}

int32_t report(const Match& m, lmb200_model_config* cfg, lmb200_decoder_match* info, int32_t* weight_nodes,
               int32_t weight_capacity, char* names_out, int64_t names_capacity) {
  if (cfg) *cfg = m.cfg;
  if (info) *info = m.info;
  if (weight_nodes)
    for (int32_t k = 0; k < weight_capacity && k < (int32_t)m.weights.size(); ++k) weight_nodes[k] = m.weights[k].second;
  if (names_out && names_capacity > 0) {
    std::string all;
    for (size_t k = 0; k < m.weights.size(); ++k) {
      const std::string add = (k ? "\n" : "") + m.weights[k].first;
      if ((int64_t)(all.size() + add.size()) >= names_capacity) break;
      all += add;
    }
    std::memcpy(names_out, all.c_str(), all.size() + 1);
  }
  return LMB200_OK;
}

}  // namespace

extern "C" int32_t lmb200_match_decoder(const lmb200_node_list* list, int32_t output_id, lmb200_model_config* cfg,
                                        lmb200_decoder_match* info, int32_t* weight_nodes, int32_t weight_capacity,
                                        char* names_out, int64_t names_capacity) {
  try {
    return report(match_decoder(list, output_id), cfg, info, weight_nodes, weight_capacity, names_out, names_capacity);
  } catch (const NoMatch& e) {
    return lmb::fail(LMB200_ENOMATCH, "%s", e.what.c_str());
  } catch (const std::exception& e) {
    return lmb::fail(LMB200_EINVAL, "node list: %s", e.what());
  }
}

extern "C" int32_t lmb200_match_whisper_step(const lmb200_node_list* list, int32_t logits_id, lmb200_model_config* cfg,
                                             lmb200_decoder_match* info, int32_t* weight_nodes, int32_t weight_capacity,
                                             char* names_out, int64_t names_capacity, int32_t* cache_nodes,
                                             int32_t cache_capacity) {
  try {
    Match m = match_whisper_step(list, logits_id);
    if (cache_nodes)
      for (int32_t k = 0; k < cache_capacity && k < (int32_t)m.cache.size(); ++k) cache_nodes[k] = m.cache[k];
    return report(m, cfg, info, weight_nodes, weight_capacity, names_out, names_capacity);
  } catch (const NoMatch& e) {
    return lmb::fail(LMB200_ENOMATCH, "%s", e.what.c_str());
  } catch (const std::exception& e) {
    return lmb::fail(LMB200_EINVAL, "node list: %s", e.what());
  }
}

extern "C" int32_t lmb200_match_whisper_encoder(const lmb200_node_list* list, int32_t output_id, lmb200_encoder_match* info,
                                                int32_t* weight_nodes, int32_t weight_capacity, char* names_out,
                                                int64_t names_capacity) {
  try {
    EncoderMatch m = match_whisper_encoder(list, output_id);
    Match names;
    names.weights = m.weights;
    if (info) *info = m.info;
    return report(names, nullptr, nullptr, weight_nodes, weight_capacity, names_out, names_capacity);
  } catch (const NoMatch& e) {
    return lmb::fail(LMB200_ENOMATCH, "%s", e.what.c_str());
  } catch (const std::exception& e) {
    return lmb::fail(LMB200_EINVAL, "node list: %s", e.what());
  }
}

extern "C" int32_t lmb200_compile_encoder_node_list(lmb200_ctx ctx, const lmb200_node_list* list, int32_t output_id,
                                                    const float* const* node_data, int32_t layout,
                                                    lmb200_whisper_encoder* encoder_out, lmb200_encoder_match* info) {
  LMB_REQUIRE(encoder_out && node_data, "lmb200_compile_encoder_node_list: null output or node_data");
  EncoderMatch m;
  try {
    m = match_whisper_encoder(list, output_id);
  } catch (const NoMatch& e) {
    return lmb::fail(LMB200_ENOMATCH, "%s", e.what.c_str());
  } catch (const std::exception& e) {
    return lmb::fail(LMB200_EINVAL, "node list: %s", e.what());
  }
  for (auto& kv : m.weights)
    if (!node_data[kv.second - 1]) return lmb::fail(LMB200_EINVAL, "%s (node %d) has no data", kv.first.c_str(), kv.second);
  // the fused encoder computes the sinusoid table itself, at the reference's rates, and normalises with eps 1e-5:
  // a graph with other constants is not the graph it stands for
  const float* rates = node_data[m.info.rates_node - 1];
  if (!rates) return lmb::fail(LMB200_EINVAL, "the sinusoid rates (node %d) have no data", m.info.rates_node);
  const int half = m.info.d_model / 2;
  const double inc = std::log(10000.0) / (half - 1);
  for (int i = 0; i < half; ++i) {
    const double want = std::exp(-inc * i);
    if (std::fabs((double)rates[i] - want) > 1e-6 * want + 1e-12)
      return lmb::fail(LMB200_ENOMATCH, "node %d: rate %d is %g, sinusoids() gives %g", m.info.rates_node, i, (double)rates[i], want);
  }
  if (std::fabs(m.info.eps - 1e-5f) > 1e-9f)
    return lmb::fail(LMB200_ENOMATCH, "LayerNorm epsilon %g: the fused encoder is built for 1e-5", (double)m.info.eps);
  lmb200_whisper_encoder enc = 0;
  int32_t rc = lmb200_whisper_encoder_create(ctx, m.info.d_model, m.info.heads, m.info.layers, m.info.ffn, m.info.n_mels, 0, &enc);
  if (rc != LMB200_OK) return rc;
  Walker w(*list);
  for (auto& kv : m.weights) {
    Shape s = w.shape(kv.second);
    rc = lmb200_whisper_encoder_set_weight(enc, kv.first.c_str(), node_data[kv.second - 1], (int32_t)s.size(), s.data(), layout);
    if (rc != LMB200_OK) { lmb200_whisper_encoder_destroy(enc); return rc; }
  }
  *encoder_out = enc;
  if (info) *info = m.info;
  return LMB200_OK;
}

extern "C" int32_t lmb200_compile_node_list(lmb200_ctx ctx, const lmb200_node_list* list, int32_t output_id,
                                            const float* const* node_data, int32_t layout, int32_t dtype, int32_t batch,
                                            int32_t max_ctx, lmb200_model* model_out, lmb200_session* session_out,
                                            lmb200_decoder_match* info) {
  LMB_REQUIRE(model_out && session_out && node_data, "lmb200_compile_node_list: null output or node_data");
  LMB_REQUIRE(dtype == LMB200_F32 || dtype == LMB200_BF16, "lmb200_compile_node_list: dtype must be float32 or bf16");
  Match m;
  try {
    m = match_any(list, output_id);
  } catch (const NoMatch& e) {
    return lmb::fail(LMB200_ENOMATCH, "%s", e.what.c_str());
  } catch (const std::exception& e) {
    return lmb::fail(LMB200_EINVAL, "node list: %s", e.what());
  }
  const bool whisper = m.info.arch == LMB200_ARCH_WHISPER_DECODER;
  if (!whisper && m.info.prev_seq != 0)
    return lmb::fail(LMB200_ENOMATCH, "the graph was traced with prev_seq = %d: a cached session starts at position 0",
                     m.info.prev_seq);
  for (auto& kv : m.weights)
    if (!node_data[kv.second - 1]) return lmb::fail(LMB200_EINVAL, "%s (node %d) has no data", kv.first.c_str(), kv.second);
  m.cfg.dtype = dtype;
  lmb200_model model = 0;
  int32_t rc = lmb200_model_create(ctx, &m.cfg, &model);
  if (rc != LMB200_OK) return rc;
  Walker w(*list);
  for (auto& kv : m.weights) {
    Shape s = w.shape(kv.second);
    rc = lmb200_model_set_weight(model, kv.first.c_str(), node_data[kv.second - 1], (int32_t)s.size(), s.data(), layout);
    if (rc != LMB200_OK) { lmb200_model_destroy(model); return rc; }
  }
  lmb200_session session = 0;
  rc = lmb200_session_create(model, batch > 0 ? batch : m.info.batch, whisper && max_ctx <= 0 ? m.info.max_seq : max_ctx, &session);
  if (rc != LMB200_OK) { lmb200_model_destroy(model); return rc; }
  if (whisper) {
    // the encoder K / V the step graph takes as inputs (decode_step! feeds them at every step, src/Whisper.jl:770-778)
    // are uploaded once, where the caller has them already
    const int L = m.cfg.n_layers;
    for (int l = 0; l < L; ++l) {
      const float* k = node_data[m.cache[l] - 1];
      const float* v = node_data[m.cache[L + l] - 1];
      if (!k && !v) continue;
      if (!k || !v || (batch > 0 && batch != m.info.batch))
        rc = lmb::fail(LMB200_EINVAL, "layer %d: cross K and V come as a pair, shaped for the graph's batch", l);
      else
        rc = lmb200_session_set_cross_kv(session, l, k, v, layout);
      if (rc != LMB200_OK) { lmb200_session_destroy(session); lmb200_model_destroy(model); return rc; }
    }
  }
  *model_out = model;
  *session_out = session;
  if (info) *info = m.info;
  return LMB200_OK;
}

"""Graph IR and graph-construction API: the Python stand-in for src/Ops.jl, src/Graph.jl and
src/HighLevelOps.jl, kept name for name (and 1-based axis for axis) so that model code written
against the reference reads the same here.  Pure graph building: no numerics."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, List, Tuple

import numpy as np

F32 = np.float32


# ---------------------------------------------------------------------------------------------
# Ops (src/Ops.jl:4-110)
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Op:
    pass


def _simple(name):
    return dataclass(frozen=True)(type(name, (Op,), {}))


Log2, Exp2, Sin, Sqrt, Cos, Recip, Contiguous, ReLU = map(_simple, "Log2 Exp2 Sin Sqrt Cos Recip Contiguous ReLU".split())
Add, Mul, Mod, Max, LessThan = map(_simple, "Add Mul Mod Max LessThan".split())
FusedMulAdd, FusedAddReLU, MatMul = map(_simple, "FusedMulAdd FusedAddReLU MatMul".split())


@dataclass(frozen=True)
class SumReduce(Op):
    dim: int


@dataclass(frozen=True)
class MaxReduce(Op):
    dim: int


@dataclass(frozen=True)
class Permute(Op):
    dims: Tuple[int, ...]


@dataclass(frozen=True)
class Expand(Op):
    dim: int
    size: int


@dataclass(frozen=True)
class Reshape(Op):
    shape: Tuple[int, ...]


@dataclass(frozen=True)
class Slice(Op):
    ranges: Tuple[Tuple[int, int], ...]


@dataclass(frozen=True)
class Pad(Op):
    padding: Tuple[Tuple[int, int], ...]


@dataclass(frozen=True)
class Unfold(Op):
    kernel_shape: Tuple[int, ...]
    stride_shape: Tuple[int, ...]
    dilation_shape: Tuple[int, ...]


@dataclass(frozen=True)
class Constant(Op):
    value: float


@dataclass(frozen=True)
class Function(Op):
    name: str


@dataclass(frozen=True)
class FlashAttentionOp(Op):
    scale: float
    causal: bool


ELEMENTWISE = (Log2, Exp2, Sin, Sqrt, Cos, Recip, ReLU, Add, Mul, Mod, Max, LessThan, FusedMulAdd, FusedAddReLU)

# ---------------------------------------------------------------------------------------------
# Graph (src/Graph.jl:4-81).  Node ids are 1-based insertion order = topological order.
# ---------------------------------------------------------------------------------------------
BIG = 1 << 62     # typemax(Int) stand-in for open slice ends


@dataclass
class Node:
    op: Op
    inputs: List[Tuple[int, int, Tuple[int, ...]]]      # (node id, output index, input shape)


@dataclass
class Graph:
    nodes: List[Node] = field(default_factory=list)
    shapes: List[Tuple[int, ...]] = field(default_factory=list)
    tensors: dict = field(default_factory=dict)           # (node id, output index) -> array


class GraphTensor:
    def __init__(self, id_, shape, graph):
        self.id, self.shape, self.graph_ref = id_, tuple(int(s) for s in shape), graph

    # operator overloads (src/HighLevelOps.jl:38-103)
    def __add__(self, o): return _binary(Add(), self, _lift(self, o))
    def __radd__(self, o): return self + o
    def __mul__(self, o): return _binary(Mul(), self, _lift(self, o))
    def __rmul__(self, o): return self * o
    def __neg__(self): return self * F32(-1.0)
    def __sub__(self, o): return self + (-o if isinstance(o, GraphTensor) else -F32(o))
    def __rsub__(self, o): return constant(self.graph_ref, o) - self
    def __truediv__(self, o):
        return self * reciprocal(o) if isinstance(o, GraphTensor) else self * (F32(1.0) / F32(o))
    def __rtruediv__(self, o): return constant(self.graph_ref, o) / self
    def __mod__(self, o): return _binary(Mod(), self, _lift(self, o))
    def __lt__(self, o): return _binary(LessThan(), self, _lift(self, o))
    def __gt__(self, o): return _binary(LessThan(), _lift(self, o), self)
    def __le__(self, o): return (self > o) * F32(-1.0) + F32(1.0)
    def __ge__(self, o): return (self < o) * F32(-1.0) + F32(1.0)
    def ne(self, o): return (self < o) + (self > o)
    def eq(self, o): return self.ne(o) * F32(-1.0) + F32(1.0)


def add_op(graph, op, inputs, output_shape):
    graph.nodes.append(Node(op, list(inputs)))
    graph.shapes.append(tuple(int(s) for s in output_shape))
    return GraphTensor(len(graph.nodes), output_shape, graph)


def tensor(graph, shape):
    if isinstance(shape, np.ndarray):
        shape = shape.shape
    return add_op(graph, Function("InputTensor"), [], shape)


def constant(graph, value):
    return add_op(graph, Constant(float(F32(value))), [], ())


def _lift(like, o):
    return o if isinstance(o, GraphTensor) else constant(like.graph_ref, o)


def broadcast_dims(d1, d2):      # src/HighLevelOps.jl:6-36: prepend 1s, then pairwise
    n = max(len(d1), len(d2))
    a = (1,) * (n - len(d1)) + tuple(d1)
    b = (1,) * (n - len(d2)) + tuple(d2)
    out = []
    for x, y in zip(a, b):
        if x == y or y == 1:
            out.append(x)
        elif x == 1:
            out.append(y)
        else:
            raise ValueError(f"Dimension mismatch in broadcasting: {x} vs {y}")
    return tuple(out)


def _inp(t):
    return (t.id, 0, t.shape)


def _binary(op, a, b):
    assert a.graph_ref is b.graph_ref, "Tensors must be from the same graph"
    return add_op(a.graph_ref, op, [_inp(a), _inp(b)], broadcast_dims(a.shape, b.shape))


def _unary(op, a):
    return add_op(a.graph_ref, op, [_inp(a)], a.shape)


# unary (src/HighLevelOps.jl:108-148)
def log2(a): return _unary(Log2(), a)
def exp2(a): return _unary(Exp2(), a)
def sin(a): return _unary(Sin(), a)
def cos(a): return sin(F32(math.pi / 2) - a)
def exp(a): return exp2(a * (F32(1.0) / F32(math.log(2.0))))
def sqrt(a): return _unary(Sqrt(), a)
def reciprocal(a): return _unary(Recip(), a)
def relu(a): return _unary(ReLU(), a)
def abs_(a): return relu(a) + relu(-a)


# activations (src/HighLevelOps.jl:153-168)
def sigmoid(a): return F32(1.0) / (F32(1.0) + exp2(-a * (F32(1.0) / F32(math.log(2.0)))))
def swish(a): return a * sigmoid(a)
silu = swish
def tanh(a): return sigmoid(a * F32(2.0)) * F32(2.0) - F32(1.0)
def gelu(a): return a * F32(0.5) * (F32(1.0) + tanh(F32(0.7978845608) * a * (F32(1.0) + F32(0.044715) * a * a)))


# movement (src/HighLevelOps.jl:173-248)
def contiguous(a):               # every op output is already contiguous (ShapeTracker is fresh)
    return a


def reshape(a, new_shape):
    new_shape = tuple(int(s) for s in new_shape)
    assert int(np.prod(new_shape)) == int(np.prod(a.shape)), f"Length mismatch in Reshape!: {new_shape} vs {a.shape}"
    return add_op(a.graph_ref, Reshape(new_shape), [_inp(a)], new_shape)


def permute(a, dims):
    dims = tuple(int(d) for d in dims)
    return add_op(a.graph_ref, Permute(dims), [_inp(a)], tuple(a.shape[d - 1] for d in dims))


def expand(a, dim, size):
    shp = list(a.shape)
    shp.insert(dim - 1, int(size))
    return add_op(a.graph_ref, Expand(int(dim), int(size)), [_inp(a)], shp)


def pad(a, padding):
    padding = tuple((int(l), int(r)) for l, r in padding)
    shp = [d + l + r for d, (l, r) in zip(a.shape, padding)]
    return add_op(a.graph_ref, Pad(padding), [_inp(a)], shp)


def pad_along(a, axis, left, right):
    p = [(0, 0)] * len(a.shape)
    p[axis - 1] = (left, right)
    return pad(a, p)


def slice_(a, ranges):
    ranges = tuple((max(0, int(s)), min(int(e), d)) for (s, e), d in zip(ranges, a.shape))
    shp = [e - s for s, e in ranges]
    return add_op(a.graph_ref, Slice(ranges), [_inp(a)], shp)


def slice_along(a, axis, start, stop):
    r = [(0, BIG)] * len(a.shape)
    r[axis - 1] = (start, stop)
    return slice_(a, r)


def concat_along(a, b, axis):    # pad both, then add
    return pad_along(a, axis, 0, b.shape[axis - 1]) + pad_along(b, axis, a.shape[axis - 1], 0)


def matmul(a, b):                # src/HighLevelOps.jl:252-264
    assert a.graph_ref is b.graph_ref and len(a.shape) >= 2 and len(b.shape) >= 2
    return add_op(a.graph_ref, MatMul(), [_inp(a), _inp(b)], a.shape[:-1] + (b.shape[-1],))


# reductions / normalisations / softmax (src/HighLevelOps.jl:269-327)
def _drop(shape, dim):
    s = list(shape)
    del s[dim - 1]
    return s


def sum_(a, dim): return add_op(a.graph_ref, SumReduce(int(dim)), [_inp(a)], _drop(a.shape, dim))
def max_reduce(a, dim): return add_op(a.graph_ref, MaxReduce(int(dim)), [_inp(a)], _drop(a.shape, dim))
def maximum(a, b):
    b = _lift(a, b)
    return (a < b) * b + (b <= a) * a
def mean(a, dim): return sum_(a, dim) * (F32(1.0) / F32(a.shape[dim - 1]))
def mean_norm(a, dim): return a - expand(mean(a, dim), dim, a.shape[dim - 1])


def std_norm(a, dim, epsilon=1e-5):
    inv_std = reciprocal(sqrt(mean(a * a, dim) + F32(epsilon)))
    return a * expand(inv_std, dim, a.shape[dim - 1])


def layer_norm(a, dim, epsilon=1e-5): return std_norm(mean_norm(a, dim), dim, epsilon)


def softmax(a, dim):
    n = a.shape[dim - 1]
    e = exp(a - expand(max_reduce(a, dim), dim, n))
    return e / expand(sum_(e, dim), dim, n)


# arange / triu / gather / flash attention (src/HighLevelOps.jl:332-388)
def cumsum_last_dim(a): return add_op(a.graph_ref, Function("CumSum"), [_inp(a)], a.shape)


def arange(graph, to):
    if to == 1:
        return expand(constant(graph, 0.0), 1, 1)
    return cumsum_last_dim(expand(constant(graph, 1.0), 1, to)) - F32(1.0)


def triu(graph, size, diagonal=0):
    h = expand(arange(graph, size), 1, size)
    v = expand(arange(graph, size), 2, size)
    return h - F32(diagonal - 1) > v


def gather(matrix, indexes):
    return add_op(matrix.graph_ref, Function("Gather"), [_inp(matrix), _inp(indexes)],
                  tuple(indexes.shape) + (matrix.shape[1],))


def unfold(a, kernel_shape, stride_shape, dilation_shape):      # src/HighLevelOps.jl:390-420
    spatial = len(kernel_shape)
    assert spatial == 1 and len(a.shape) > 1, "Unfold > 1D not implemented"
    s_i, k_i, d_i, st_i = a.shape[-1], kernel_shape[0], dilation_shape[0], stride_shape[0]
    o_i = (s_i - d_i * (k_i - 1) - 1) // st_i + 1
    return add_op(a.graph_ref, Unfold(tuple(kernel_shape), tuple(stride_shape), tuple(dilation_shape)), [_inp(a)],
                  tuple(a.shape[:-1]) + (o_i, k_i))


def flash_attention(q, k, v, scale=None, causal=False):
    if scale is None:
        scale = F32(1.0) / np.sqrt(F32(q.shape[-1]))
    return add_op(q.graph_ref, FlashAttentionOp(float(F32(scale)), bool(causal)), [_inp(q), _inp(k), _inp(v)], q.shape)

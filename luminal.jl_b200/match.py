"""A node list's text and array forms, and the host side of the library's structural matcher.

The reference has no plugin seam other than its graph: a backend sees `Graph.nodes` (src/Graph.jl:4-26), a
flat, topologically ordered list of primitive ops, with every NN layer already decomposed (src/NN.jl,
src/HighLevelOps.jl).  `export_graph` / `import_graph` give that list a JSON form (one record per node: op
name, op fields, inputs, output shape); `flatten_graph` gives it the array form of `lmb200_node_list`, which
is what a Julia shim passes through `ccall`.  The matcher itself is in the library (csrc/match.cu):
`lmb200_match_decoder` walks the list backwards from the logits node and recovers, by structure alone -- no
model object, no weight names -- what src/NN.jl:390-455 built: the layer count, the widths, the head split,
the RMSNorm epsilon, the RoPE base, and which input-tensor node plays which weight's role;
`lmb200_compile_node_list` hands that to the fused session.  `match_decoder` / `compile_b200` here are thin
callers of the two.  A graph that deviates anywhere (another activation, a bias, a different mask) raises
MatchError naming the node, and the caller falls back to compile(), which runs any graph one kernel per node."""
from __future__ import annotations

import ctypes as C
import json
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
# Array form of a node list (lmb200_node_list) and the library's matcher
# ---------------------------------------------------------------------------------------------
_NODE_CODES = {"Log2": 0, "Exp2": 1, "Sin": 2, "Sqrt": 3, "Cos": 4, "Recip": 5, "Contiguous": 6, "ReLU": 7, "Add": 8,
               "Mul": 9, "Mod": 10, "Max": 11, "LessThan": 12, "FusedMulAdd": 13, "FusedAddReLU": 14, "MatMul": 15,
               "SumReduce": 16, "MaxReduce": 17, "Permute": 18, "Expand": 19, "Reshape": 20, "Slice": 21, "Pad": 22,
               "Unfold": 23, "Constant": 24, "FlashAttentionOp": 28}
_FUNCTION_CODES = {"InputTensor": 25, "Gather": 26, "CumSum": 27}
_NODE_OTHER = 29


def _op_args(op) -> List[float]:
    if isinstance(op, (G.SumReduce, G.MaxReduce)):
        return [op.dim]
    if isinstance(op, G.Permute):
        return list(op.dims)
    if isinstance(op, G.Expand):
        return [op.dim, op.size]
    if isinstance(op, G.Reshape):
        return list(op.shape)
    if isinstance(op, G.Slice):
        return [v for r in op.ranges for v in r]
    if isinstance(op, G.Pad):
        return [v for r in op.padding for v in r]
    if isinstance(op, G.Unfold):
        return [*op.kernel_shape, *op.stride_shape, *op.dilation_shape]
    if isinstance(op, G.Constant):
        return [float(op.value)]
    if isinstance(op, G.FlashAttentionOp):
        return [float(op.scale), float(op.causal)]
    return []


class NodeList(C.Structure):
    """lmb200_node_list; `keep` holds the arrays the pointers refer to."""
    _fields_ = [("n_nodes", C.c_int32), ("reserved", C.c_int32), ("op", C.POINTER(C.c_int32)),
                ("in_off", C.POINTER(C.c_int32)), ("in_node", C.POINTER(C.c_int32)),
                ("shape_off", C.POINTER(C.c_int32)), ("shape", C.POINTER(C.c_int64)),
                ("arg_off", C.POINTER(C.c_int32)), ("arg", C.POINTER(C.c_double))]


class DecoderMatchInfo(C.Structure):
    """lmb200_decoder_match"""
    _fields_ = [(n, C.c_int32) for n in ("arch", "batch", "seq", "prev_seq", "tokens_node", "n_weights", "max_seq", "cross_len")]


def flatten_graph(graph) -> NodeList:
    ops, in_off, in_node, shape_off, shape, arg_off, arg = [], [0], [], [0], [], [0], []
    for node, shp in zip(graph.nodes, graph.shapes):
        op = node.op
        if isinstance(op, G.Function):
            ops.append(_FUNCTION_CODES.get(op.name, _NODE_OTHER))
        else:
            ops.append(_NODE_CODES.get(type(op).__name__, _NODE_OTHER))
        in_node.extend(int(i) for i, _, _ in node.inputs)
        in_off.append(len(in_node))
        shape.extend(int(s) for s in shp)
        shape_off.append(len(shape))
        arg.extend(float(a) for a in _op_args(op))
        arg_off.append(len(arg))
    arrays = [np.ascontiguousarray(a, dtype=t) for a, t in ((ops, np.int32), (in_off, np.int32), (in_node or [0], np.int32),
                                                             (shape_off, np.int32), (shape or [0], np.int64),
                                                             (arg_off, np.int32), (arg or [0.0], np.float64))]
    ptr = lambda a, t: a.ctypes.data_as(C.POINTER(t))
    nl = NodeList(len(ops), 0, ptr(arrays[0], C.c_int32), ptr(arrays[1], C.c_int32), ptr(arrays[2], C.c_int32),
                  ptr(arrays[3], C.c_int32), ptr(arrays[4], C.c_int64), ptr(arrays[5], C.c_int32), ptr(arrays[6], C.c_double))
    nl.keep = arrays
    return nl


@dataclass
class DecoderMatch:
    """What the matcher found.  `weights` maps the reference's registry names (src/NN.jl:180-225)
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


_ENOMATCH = -8


def _raise_match(err):
    if err.code == _ENOMATCH:
        raise MatchError(getattr(err, "message", str(err))) from None
    raise err


def match_decoder(graph, output_id: int) -> DecoderMatch:
    """Recognises Llama / Phi3 (src/NN.jl:417-507) ending in the logits node `output_id`:
    lm_head(norm(block^L(embedding(tokens)))) -- lmb200_match_decoder; needs no GPU.  Raises MatchError at the
    first node that does not fit."""
    from . import _lib
    from .session import ModelConfig
    nl = flatten_graph(graph)
    cfg, info = ModelConfig(), DecoderMatchInfo()
    cap = max(len(graph.nodes), 1)
    nodes = (C.c_int32 * cap)()
    names = C.create_string_buffer(64 * cap + 256)
    try:
        _lib.call("lmb200_match_decoder", C.byref(nl), int(output_id), C.byref(cfg), C.byref(info), nodes, cap, names, len(names))
    except _lib.LuminalB200Error as e:
        _raise_match(e)
    wnames = names.value.decode().split("\n")
    return DecoderMatch(n_layers=cfg.n_layers, hidden=cfg.hidden, n_heads=cfg.n_heads, n_kv_heads=cfg.n_kv_heads,
                        head_dim=cfg.head_dim, intermediate=cfg.intermediate, vocab=cfg.vocab, eps=float(cfg.rms_eps),
                        rope_base=float(cfg.rope_base), prev_seq=info.prev_seq, batch=info.batch, seq=info.seq,
                        tokens=info.tokens_node, weights={n: int(nodes[k]) for k, n in enumerate(wnames)})


@dataclass
class WhisperStepMatch:
    """What the matcher found in a build_decode_step graph (src/Whisper.jl:687-742).  `weights` maps the registry
    names of the model.decoder.* tensors the cached session needs to input node ids; the other lists are the ids of
    IncrementalDecodeGraph (src/Whisper.jl:662-672)."""
    n_layers: int
    d_model: int
    heads: int
    ffn: int
    vocab: int
    max_positions: int
    eps: float
    batch: int
    step_pos: int
    max_seq: int
    enc_seq: int
    tokens: int
    weights: Dict[str, int] = field(default_factory=dict)
    cross_k_ids: List[int] = field(default_factory=list)
    cross_v_ids: List[int] = field(default_factory=list)
    self_k_ids: List[int] = field(default_factory=list)
    self_v_ids: List[int] = field(default_factory=list)
    new_self_k_ids: List[int] = field(default_factory=list)
    new_self_v_ids: List[int] = field(default_factory=list)


def match_whisper_step(graph, logits_id: int) -> WhisperStepMatch:
    """Recognises the Whisper TextDecoder's incremental decode step ending in the logits node `logits_id` --
    lmb200_match_whisper_step; needs no GPU.  Raises MatchError at the first node that does not fit."""
    from . import _lib
    from .session import ModelConfig
    nl = flatten_graph(graph)
    cfg, info = ModelConfig(), DecoderMatchInfo()
    cap = max(len(graph.nodes), 1)
    nodes, cache = (C.c_int32 * cap)(), (C.c_int32 * cap)()
    names = C.create_string_buffer(64 * cap + 256)
    try:
        _lib.call("lmb200_match_whisper_step", C.byref(nl), int(logits_id), C.byref(cfg), C.byref(info), nodes, cap, names,
                  len(names), cache, cap)
    except _lib.LuminalB200Error as e:
        _raise_match(e)
    wnames = names.value.decode().split("\n")
    L = cfg.n_layers
    part = lambda k: [int(cache[k * L + l]) for l in range(L)]
    return WhisperStepMatch(n_layers=L, d_model=cfg.hidden, heads=cfg.n_heads, ffn=cfg.intermediate, vocab=cfg.vocab,
                            max_positions=cfg.max_positions, eps=float(cfg.rms_eps), batch=info.batch, step_pos=info.prev_seq,
                            max_seq=info.max_seq, enc_seq=info.cross_len, tokens=info.tokens_node,
                            weights={n: int(nodes[k]) for k, n in enumerate(wnames)}, cross_k_ids=part(0), cross_v_ids=part(1),
                            self_k_ids=part(2), self_v_ids=part(3), new_self_k_ids=part(4), new_self_v_ids=part(5))


class EncoderMatchInfo(C.Structure):
    """lmb200_encoder_match"""
    _fields_ = [(n, C.c_int32) for n in ("d_model", "heads", "layers", "ffn", "n_mels", "batch", "frames", "mel_node", "rates_node",
                                         "n_weights")] + [("eps", C.c_float)]


@dataclass
class WhisperEncoderMatch:
    """What the matcher found in an AudioEncoder graph (src/Whisper.jl:354-404).  `weights` maps the model.encoder.*
    registry names to input node ids; `mel` is the node the mel enters through, `rates` the input holding the
    sinusoid rates."""
    d_model: int
    heads: int
    layers: int
    ffn: int
    n_mels: int
    batch: int
    frames: int
    eps: float
    mel: int
    rates: int
    weights: Dict[str, int] = field(default_factory=dict)


def match_whisper_encoder(graph, output_id: int) -> WhisperEncoderMatch:
    """Recognises the Whisper AudioEncoder ending in the node `output_id` -- lmb200_match_whisper_encoder; needs no
    GPU.  Raises MatchError at the first node that does not fit."""
    from . import _lib
    nl = flatten_graph(graph)
    info = EncoderMatchInfo()
    cap = max(len(graph.nodes), 1)
    nodes = (C.c_int32 * cap)()
    names = C.create_string_buffer(64 * cap + 256)
    try:
        _lib.call("lmb200_match_whisper_encoder", C.byref(nl), int(output_id), C.byref(info), nodes, cap, names, len(names))
    except _lib.LuminalB200Error as e:
        _raise_match(e)
    wnames = names.value.decode().split("\n")
    return WhisperEncoderMatch(d_model=info.d_model, heads=info.heads, layers=info.layers, ffn=info.ffn, n_mels=info.n_mels,
                               batch=info.batch, frames=info.frames, eps=float(info.eps), mel=info.mel_node, rates=info.rates_node,
                               weights={n: int(nodes[k]) for k, n in enumerate(wnames)})


def compile_encoder_b200(graph, output_id, inputs=None, device=None):
    """compile() for an AudioEncoder graph (lmb200_compile_encoder_node_list): returns (whisper.FusedEncoder, match).
    The weights come from `inputs` or from graph.tensors, as for compile_b200.  The encoder then takes a mel of any
    batch and length (FusedEncoder.run), on the tensor cores, instead of one kernel per node of the graph."""
    from . import _lib
    from .device import DeviceArray, get_device
    from .whisper import FusedEncoder
    m = match_whisper_encoder(graph, output_id)
    dev = device or get_device()
    inputs = inputs or {}
    host, data = [], (C.c_void_p * len(graph.nodes))()
    for name, node_id in list(m.weights.items()) + [("the sinusoid rates", m.rates)]:
        a = inputs.get(node_id)
        if a is None:
            a = graph.tensors.get((node_id, 1))
        if a is None:
            raise KeyError(f"{name} (node {node_id}) has no data")
        a = np.ascontiguousarray(a.numpy() if isinstance(a, DeviceArray) else a, dtype=np.float32)
        if a.shape != tuple(graph.shapes[node_id - 1]):
            raise ValueError(f"node {node_id}: data of shape {a.shape}, node of shape {graph.shapes[node_id - 1]}")
        host.append(a)
        data[node_id - 1] = a.ctypes.data
    nl = flatten_graph(graph)
    handle, info = C.c_uint64(), EncoderMatchInfo()
    try:
        _lib.call("lmb200_compile_encoder_node_list", dev.handle, C.byref(nl), int(output_id), data, _lib.ROWMAJOR, C.byref(handle),
                  C.byref(info))
    except _lib.LuminalB200Error as e:
        _raise_match(e)
    return FusedEncoder.adopt(dev, handle.value, m.d_model), m


def compile_b200(graph, output_id, inputs=None, device=None, max_ctx=2048, dtype="f32", batch=None):
    """compile() for a graph one of the matchers recognises (lmb200_compile_node_list): returns (Session, match).
    The weights come from `inputs` (node id -> array, as execute() takes them) or from data pre-loaded into
    graph.tensors (src/Weights.jl:60-114 fills those).  The session keeps a KV cache, so the caller feeds it the
    tokens the graph was traced for (prefill) and then one token per step, instead of re-running a longer graph for
    every position as examples/llama.jl:39-99 does -- or, for a Whisper decode-step graph, instead of building and
    compiling one graph per position (src/Whisper.jl:679-801); encoder K/V inputs that have data are uploaded to the
    session's cross cache."""
    from . import _lib
    from .device import DeviceArray, get_device
    from .session import Model, Session, _dtype_code
    try:
        m = match_decoder(graph, output_id)
        if m.prev_seq != 0:
            raise MatchError("the graph was traced with prev_seq != 0: a cached session starts at position 0")
        whisper, needed = False, dict(m.weights)
    except MatchError as first:
        try:
            m = match_whisper_step(graph, output_id)
        except MatchError:
            raise first from None
        whisper, needed = True, dict(m.weights)
    dev = device or get_device()
    inputs = inputs or {}

    def data_of(node_id):
        a = inputs.get(node_id)
        if a is None:
            a = graph.tensors.get((node_id, 1))
        if a is None:
            return None
        a = np.ascontiguousarray(a.numpy() if isinstance(a, DeviceArray) else a, dtype=np.float32)
        if a.shape != tuple(graph.shapes[node_id - 1]):
            raise ValueError(f"node {node_id}: data of shape {a.shape}, node of shape {graph.shapes[node_id - 1]}")
        return a

    host, data = [], (C.c_void_p * len(graph.nodes))()
    for name, node_id in needed.items():
        a = data_of(node_id)
        if a is None:
            raise KeyError(f"{name} (node {node_id}) has no data")
        host.append(a)
        data[node_id - 1] = a.ctypes.data
    if whisper:
        for node_id in m.cross_k_ids + m.cross_v_ids:
            a = data_of(node_id)
            if a is not None:
                host.append(a)
                data[node_id - 1] = a.ctypes.data
    nl = flatten_graph(graph)
    model_h, session_h, info = C.c_uint64(), C.c_uint64(), DecoderMatchInfo()
    if whisper:
        max_ctx = m.max_seq
    try:
        _lib.call("lmb200_compile_node_list", dev.handle, C.byref(nl), int(output_id), data, _lib.ROWMAJOR,
                  _dtype_code(dtype), int(batch or 0), int(max_ctx), C.byref(model_h), C.byref(session_h), C.byref(info))
    except _lib.LuminalB200Error as e:
        _raise_match(e)
    if whisper:
        model = Model.adopt(dev, model_h.value, n_layers=m.n_layers, hidden=m.d_model, n_heads=m.heads, n_kv_heads=m.heads,
                            intermediate=m.ffn, vocab=m.vocab, eps=m.eps, rope_base=10000.0, dtype=dtype, arch=1,
                            max_positions=m.max_positions, cross_len=m.enc_seq)
    else:
        model = Model.adopt(dev, model_h.value, n_layers=m.n_layers, hidden=m.hidden, n_heads=m.n_heads,
                            n_kv_heads=m.n_kv_heads, intermediate=m.intermediate, vocab=m.vocab, eps=m.eps,
                            rope_base=m.rope_base, dtype=dtype)
    return Session.adopt(model, session_h.value, batch or m.batch, max_ctx), m


__all__ = ["MatchError", "DecoderMatch", "WhisperStepMatch", "NodeList", "export_graph", "import_graph", "flatten_graph",
           "match_decoder", "match_whisper_step", "compile_b200", "WhisperEncoderMatch", "match_whisper_encoder", "compile_encoder_b200"]

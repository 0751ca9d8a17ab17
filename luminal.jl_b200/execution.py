"""execute() and compile() on the B200 device: the Python stand-in for the interpreter of
src/Execution.jl:620-665 and for src/Compiler.jl:75-100, 181-364, dispatching every node to one
C entry point of libluminal_b200.so (what `execute_op!` methods on a B200 array type do through
ccall).  No node is computed on the host."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from . import graph as G
from .device import DeviceArray, get_device

_EW = {G.Add: "add", G.Mul: "mul", G.Mod: "mod", G.LessThan: "less_than", G.Max: "max", G.Log2: "log2",
       G.Exp2: "exp2", G.Sin: "sin", G.Cos: "cos", G.Sqrt: "sqrt", G.Recip: "recip", G.ReLU: "relu",
       G.Contiguous: "copy", G.FusedMulAdd: "fused_mul_add", G.FusedAddReLU: "fused_add_relu"}


def _p(a):
    return C.c_void_p(a.ptr)


def _ew(dev, name, out, ins):
    args = []
    for k in range(3):
        if k < len(ins):
            args += [_p(ins[k]), len(ins[k].shape), _lib.dims(ins[k].shape)]
        else:
            args += [None, 0, _lib.dims(())]
    _lib.call("lmb200_ew", dev.handle, _lib.OP[name], _p(out), len(out.shape), _lib.dims(out.shape), *args)


def execute_op(dev, op, out_shape, ins):
    """One node on the device; returns a new DeviceArray (the functional execute_op of
    src/Execution.jl:216-270)."""
    out = dev.empty(out_shape)
    run_op(dev, op, out, ins)
    return out


def run_op(dev, op, out, ins):
    """In-place form (execute_op!, src/Execution.jl:274-371, 565-618)."""
    t = type(op)
    h = dev.handle
    if t in _EW:
        _ew(dev, _EW[t], out, ins)
    elif t in (G.SumReduce, G.MaxReduce):
        a = ins[0]
        _lib.call("lmb200_reduce", h, _lib.REDUCE_SUM if t is G.SumReduce else _lib.REDUCE_MAX, _p(out), _p(a),
                  len(a.shape), _lib.dims(a.shape), op.dim - 1)
    elif t is G.MatMul:
        a, b = ins
        _lib.call("lmb200_matmul", h, _p(out), _p(a), len(a.shape), _lib.dims(a.shape), _p(b), len(b.shape),
                  _lib.dims(b.shape))
    elif t is G.Permute:
        a = ins[0]
        perm = (C.c_int32 * len(op.dims))(*[d - 1 for d in op.dims])
        _lib.call("lmb200_permute", h, _p(out), _p(a), len(a.shape), _lib.dims(a.shape), perm)
    elif t is G.Reshape:
        a = ins[0]
        _lib.call("lmb200_reshape_colmajor", h, _p(out), _p(a), len(a.shape), _lib.dims(a.shape), len(op.shape),
                  _lib.dims(op.shape))
    elif t is G.Expand:
        a = ins[0]
        _lib.call("lmb200_expand", h, _p(out), _p(a), len(a.shape), _lib.dims(a.shape), op.dim - 1, op.size)
    elif t is G.Slice:
        a = ins[0]
        starts = _lib.dims([s for s, _ in op.ranges])
        stops = _lib.dims([min(e, d) for (_, e), d in zip(op.ranges, a.shape)])
        _lib.call("lmb200_slice", h, _p(out), _p(a), len(a.shape), _lib.dims(a.shape), starts, stops)
    elif t is G.Pad:
        a = ins[0]
        _lib.call("lmb200_pad", h, _p(out), _p(a), len(a.shape), _lib.dims(a.shape),
                  _lib.dims([l for l, _ in op.padding]), _lib.dims([r for _, r in op.padding]))
    elif t is G.Unfold:
        a = ins[0]
        _lib.call("lmb200_unfold1d", h, _p(out), _p(a), int(np.prod(a.shape[:-1])), a.shape[-1], op.kernel_shape[0],
                  op.stride_shape[0], op.dilation_shape[0])
    elif t is G.FlashAttentionOp:
        q, k, v = ins
        B, H, S, D = q.shape
        _lib.call("lmb200_flash_attention", h, _p(out), _p(q), _p(k), _p(v), _lib.F32, B, H, S, D, op.scale,
                  int(op.causal))
    elif t is G.Function and op.name == "Gather":
        table, ids = ins
        _lib.call("lmb200_gather", h, _p(out), _p(table), table.shape[0], table.shape[1], _p(ids),
                  int(np.prod(ids.shape)))
    elif t is G.Function and op.name == "CumSum":
        a = ins[0]
        n = a.shape[-1]
        _lib.call("lmb200_cumsum_last", h, _p(out), _p(a), int(np.prod(a.shape)) // n, n)
    else:
        raise NotImplementedError(f"Function op with name {getattr(op, 'name', t.__name__)} not implemented.")


def execute(graph, output_ids, initial_inputs, device=None):
    """execute(graph, ids, inputs, device) of src/Execution.jl:620-670: inputs are host arrays keyed
    by node id, results come back as host arrays keyed by node id."""
    dev = device or get_device()
    single = isinstance(output_ids, int)
    ids = [output_ids] if single else list(output_ids)
    results = {k: (v if isinstance(v, DeviceArray) else dev.upload(np.asarray(v, dtype=np.float32)))
               for k, v in initial_inputs.items()}
    for (node_id, out_idx), data in graph.tensors.items():       # pre-loaded weights
        if node_id not in results and out_idx == 1:
            results[node_id] = data if isinstance(data, DeviceArray) else dev.upload(np.asarray(data, np.float32))
    for node_id, node in enumerate(graph.nodes, start=1):
        if node_id in results:
            continue
        op = node.op
        if isinstance(op, G.Constant):
            results[node_id] = dev.upload(np.asarray(op.value, dtype=np.float32))
        elif isinstance(op, G.Function) and op.name == "InputTensor":
            raise KeyError(f"input tensor node {node_id} has no data")
        else:
            ins = [results[i] for i, _, _ in node.inputs]
            results[node_id] = execute_op(dev, op, graph.shapes[node_id - 1], ins)
    out = {i: results[i].numpy() for i in ids}
    return out[output_ids] if single else out


from .compiler import CompiledGraph, compile  # noqa: E402,F401  (compile() with fusion lives in compiler.py)


__all__ = ["execute", "execute_op", "run_op", "compile", "CompiledGraph"]


def compile_fused(model, reg, inputs, device=None, batch=1, max_ctx=2048, dtype="f32", eps=1e-5):
    """The fused counterpart of compile() for a whole nn.Llama / nn.Phi3: instead of one kernel per
    primitive node, the model's registered weights (the same `reg` name -> tensor map and the same
    node-id -> array `inputs` that execute() takes) fill a device-resident model with a KV cache, and
    the returned Session runs prefill / decode_step / decode_n on it.  What the reference reaches by
    re-running the graph over the growing prefix (examples/llama.jl:39-99) becomes one cached step."""
    from .session import Model, Session
    dev = device or get_device()
    cfg = model.config
    m = Model(dev, n_layers=cfg["n_layers"], hidden=cfg["hidden"], n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"],
              intermediate=cfg["intermediate"], vocab=cfg["vocab"], eps=eps, rope_base=model.ROPE_BASE, dtype=dtype)
    for name, t in reg.items():
        data = inputs.get(t.id, model_graph_tensor(t))
        if data is None:
            raise KeyError(f"weight {name} (node {t.id}) has no data")
        m.set_weight(name, data.numpy() if isinstance(data, DeviceArray) else np.asarray(data, dtype=np.float32))
    missing = m.missing_weights()
    if missing:
        m.close()
        raise KeyError(f"the registry leaves {len(missing)} model tensors unset: {missing[:6]}")
    return Session(m, batch, max_ctx)


def model_graph_tensor(t):
    """Data pre-loaded into the graph for tensor t (graph.tensors, as load_weights! fills it), or None."""
    return t.graph_ref.tensors.get((t.id, 1))

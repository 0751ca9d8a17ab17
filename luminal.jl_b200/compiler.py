"""compile() with fusion: the Python stand-in for src/Compiler.jl:103-364.

The reference forms element-wise fusion groups -- an element-wise node (or constant) with exactly
one consumer that is itself element-wise disappears into that consumer (src/Compiler.jl:191-215,
build_fused_expr! :156-177) -- and runs each group's terminal node as one FusedElementwiseOp
(:323-357), everything else through execute_op!.  Here the same groups are formed by the same rule
and mapped to kernels of libluminal_b200.so:

  * a*b+c and max(a+b, 0)            -> the FusedMulAdd / FusedAddReLU opcodes of lmb200_ew
  * the SiLU-gate chain of NN.Mlp    -> lmb200_silu_gate
  * any other group                  -> lmb200_fused_ew, one kernel interpreting the group's
                                        postfix program per element
  * RMSNorm / LayerNorm sub-graphs (std_norm, mean_norm, gain, bias: src/NN.jl:138-173,
    src/HighLevelOps.jl:284-304), which span reductions and expands and therefore several of the
    reference's groups, are recognised as a whole -> lmb200_rmsnorm_scale / lmb200_layernorm

Values are those of the interpreter order (every operation rounded to float32, no contraction),
which is what parity is defined against; the reference's own CPU compile path may reorder terms
through SymbolicUtils (src/Compiler.jl:326).
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np

from . import _lib
from . import graph as G
from .device import get_device

# postfix program of lmb200_fused_ew: (opcode, argument) pairs
PUSH_IN, PUSH_CONST = 0, 1
_CODE = {G.Add: 2, G.Mul: 3, G.Mod: 4, G.LessThan: 5, G.Max: 6, G.Log2: 7, G.Exp2: 8, G.Sin: 9, G.Cos: 10,
         G.Sqrt: 11, G.Recip: 12, G.ReLU: 13, G.FusedMulAdd: 14, G.FusedAddReLU: 15}
MAX_INPUTS, MAX_INSTR, MAX_STACK = 8, 64, 16
_F32 = np.float32
_INV_LN2 = float(_F32(1.0) / _F32(math.log(2.0)))


def is_elementwise(op):
    """src/Compiler.jl:104-112 (a Constant counts as element-wise there, too)."""
    return isinstance(op, G.ELEMENTWISE) or isinstance(op, G.Constant)


def fusible_intermediates(graph):
    """Node ids that vanish into their consumer: element-wise, exactly one consuming edge, and that
    consumer element-wise (src/Compiler.jl:183-215)."""
    n = len(graph.nodes)
    edges = [0] * (n + 1)
    consumer = [0] * (n + 1)
    for nid, node in enumerate(graph.nodes, start=1):
        for i, _, _ in node.inputs:
            edges[i] += 1
            consumer[i] = nid
    out = set()
    for nid, node in enumerate(graph.nodes, start=1):
        if is_elementwise(node.op) and edges[nid] == 1 and is_elementwise(graph.nodes[consumer[nid] - 1].op):
            out.add(nid)
    return out


def group_program(graph, terminal, fusible):
    """Postfix program of the fusion group that ends in `terminal`, and its leaf inputs (node ids,
    each once).  Depth-first over the group's tree, operands in the node's input order."""
    inputs, code = [], []

    def emit(nid):
        node = graph.nodes[nid - 1]
        if nid != terminal and nid not in fusible:
            if nid not in inputs:
                inputs.append(nid)
            code.append((PUSH_IN, inputs.index(nid)))
            return
        if isinstance(node.op, G.Constant):
            code.append((PUSH_CONST, float(_F32(node.op.value))))
            return
        for i, _, _ in node.inputs:
            emit(i)
        code.append((_CODE[type(node.op)], 0))

    emit(terminal)
    return code, inputs


def _stack_depth(code):
    arity = {2: 2, 3: 2, 4: 2, 5: 2, 6: 2, 14: 3, 15: 2}
    d = top = 0
    for op, _ in code:
        d += 1 if op in (PUSH_IN, PUSH_CONST) else 1 - arity.get(op, 1)
        top = max(top, d)
    return top


# the chain silu(gate) * up as NN.Mlp builds it (src/NN.jl:246-249, src/HighLevelOps.jl:153-160):
# (gate * (1 * recip(exp2((gate * -1) * (1/ln2)) + 1))) * up   -- a Number on the left of + or * goes to the right
# (src/HighLevelOps.jl:46, 56), 1 / x is constant(1) * recip(x) (:63-65)
_SILU_GATE = [(PUSH_IN, 0), (PUSH_CONST, 1.0), (PUSH_IN, 0), (PUSH_CONST, -1.0), (3, 0), (PUSH_CONST, _INV_LN2), (3, 0),
              (8, 0), (PUSH_CONST, 1.0), (2, 0), (12, 0), (3, 0), (3, 0), (PUSH_IN, 1), (3, 0)]
_MUL_ADD = ([(PUSH_IN, 0), (PUSH_IN, 1), (3, 0), (PUSH_IN, 2), (2, 0)], (0, 1, 2))
_ADD_MUL = ([(PUSH_IN, 0), (PUSH_IN, 1), (PUSH_IN, 2), (3, 0), (2, 0)], (1, 2, 0))       # c + a*b
_ADD_RELU = [(PUSH_IN, 0), (PUSH_IN, 1), (2, 0), (13, 0)]


def _p(a):
    return C.c_void_p(a.ptr)


class _Matcher:
    """Structural access to the graph for the norm patterns."""

    def __init__(self, graph, edges):
        self.g, self.edges = graph, edges

    def op(self, nid):
        return self.g.nodes[nid - 1].op

    def ins(self, nid):
        return [i for i, _, _ in self.g.nodes[nid - 1].inputs]

    def shape(self, nid):
        return tuple(self.g.shapes[nid - 1])

    def is_(self, nid, cls):
        return isinstance(self.op(nid), cls)

    def const(self, nid):
        return float(self.op(nid).value) if self.is_(nid, G.Constant) else None

    def mul_by_const(self, nid):
        """nid == Mul(a, Constant) (either order) -> (a, value) or None"""
        if not self.is_(nid, G.Mul):
            return None
        a, b = self.ins(nid)
        if self.const(b) is not None:
            return a, self.const(b)
        if self.const(a) is not None:
            return b, self.const(a)
        return None

    def expanded_vector(self, nid, n):
        """nid == expand(...expand(w)) of a 1-D tensor of length n along leading axes (src/NN.jl:160-168) -> w or None"""
        chain = []
        while self.is_(nid, G.Expand) and self.op(nid).dim <= len(self.shape(nid)) - 1:
            chain.append(nid)
            nid = self.ins(nid)[0]
        return (nid, chain) if chain and self.shape(nid) == (n,) else None

    def std_norm(self, nid):
        """nid == x * expand(recip(sqrt(mean(x*x) + eps)), last) (std_norm, src/HighLevelOps.jl:299-304)
        -> (x, eps, interior node ids) or None"""
        if not self.is_(nid, G.Mul):
            return None
        x, ex = self.ins(nid)
        rank = len(self.shape(nid))
        n = self.shape(nid)[-1]
        if not (self.is_(ex, G.Expand) and self.op(ex).dim == rank and self.op(ex).size == n and self.shape(x) == self.shape(nid)):
            return None
        rc = self.ins(ex)[0]
        if not self.is_(rc, G.Recip):
            return None
        sq = self.ins(rc)[0]
        if not self.is_(sq, G.Sqrt):
            return None
        ad = self.ins(sq)[0]
        if not self.is_(ad, G.Add):
            return None
        mean, ce = self.ins(ad)
        eps = self.const(ce)
        mc = self.mul_by_const(mean)
        if eps is None or mc is None:
            return None
        sm, scale = mc
        if not (self.is_(sm, G.SumReduce) and self.op(sm).dim == rank and scale == float(_F32(1.0) / _F32(n))):
            return None
        sqr = self.ins(sm)[0]
        if not (self.is_(sqr, G.Mul) and self.ins(sqr) == [x, x]):
            return None
        interior = [ex, rc, sq, ad, ce, mean, sm, sqr] + [i for i in self.ins(mean) if self.const(i) is not None]
        return x, eps, interior

    def mean_norm(self, nid):
        """nid == x + expand(mean(x), last) * -1 (mean_norm, src/HighLevelOps.jl:292-297) -> (x, interior) or None"""
        if not self.is_(nid, G.Add):
            return None
        x, neg = self.ins(nid)
        mc = self.mul_by_const(neg)
        if mc is None or mc[1] != -1.0:
            return None
        ex = mc[0]
        rank, n = len(self.shape(nid)), self.shape(nid)[-1]
        if not (self.is_(ex, G.Expand) and self.op(ex).dim == rank and self.op(ex).size == n):
            return None
        mean = self.ins(ex)[0]
        mm = self.mul_by_const(mean)
        if mm is None or mm[1] != float(_F32(1.0) / _F32(n)):
            return None
        sm = mm[0]
        if not (self.is_(sm, G.SumReduce) and self.op(sm).dim == rank and self.ins(sm) == [x]):
            return None
        interior = [neg, ex, mean, sm] + [i for i in self.ins(neg) + self.ins(mean) if self.const(i) is not None]
        return x, interior

    def private(self, interior, allowed_outside):
        """every interior node feeds only nodes of the pattern (so that it need not be materialised)"""
        inside = set(interior) | set(allowed_outside)
        for nid, node in enumerate(self.g.nodes, start=1):
            if nid in inside:
                continue
            if any(i in interior for i, _, _ in node.inputs):
                return False
        return True


class CompiledGraph:
    """compile(graph): preallocated device buffers and a list of steps (src/Compiler.jl:75-100,
    181-364).  Calling it copies the inputs in and runs the steps; it returns the per-node device
    buffers indexed by node id, as the reference does.  Nodes that vanished into a fused step have no
    buffer (the reference leaves theirs at zero)."""

    def __init__(self, graph, device=None, fuse=True, capture=True, outputs=None):
        self.graph, self.dev = graph, device or get_device()
        self.results, self.steps = {}, []
        self.outputs = None if outputs is None else [int(i) for i in outputs]
        # execute_with_capture's cache (src/Compiler.jl:75-79, 97): after the first call "cuda_exec" holds the CUDA
        # graph of the steps, and every later call is one replay; capture=False runs the steps call by call
        self.cache, self.capture = {}, bool(capture)
        plan = plan_graph(graph, fuse)
        if self.outputs is None:
            for nid, what in plan:                   # buffers first: a step may read a constant planned after it
                self.results[nid] = self.dev.empty(graph.shapes[nid - 1])
        else:
            # only `outputs` are read after a call: the other step outputs share blocks by liveness (plan_buffers)
            from .device import DeviceArray
            missing = [i for i in self.outputs if i not in dict(plan)]
            if missing:
                raise KeyError(f"compile: output nodes {missing} have no buffer (they vanished into a fused step)")
            slot_of, capacity = plan_buffers(graph, plan, self.outputs)
            self.blocks = [self.dev.empty((n,)) for n in capacity]
            for nid, what in plan:
                if nid in slot_of:
                    self.results[nid] = DeviceArray(self.dev, self.blocks[slot_of[nid]].ptr, graph.shapes[nid - 1], owned=False)
                else:
                    self.results[nid] = self.dev.empty(graph.shapes[nid - 1])
        for nid, what in plan:
            buf = self.results[nid]
            if what[0] == "constant":
                _lib.call("lmb200_upload", self.dev.handle, C.c_void_p(buf.ptr), _lib.F32,
                          np.asarray([what[1]], np.float32).ctypes.data_as(C.c_void_p), 0, _lib.dims(()), 0)
            elif what[0] != "input":
                self.steps.append((what, buf))
        # data pre-loaded into the graph (load_weights!, src/Weights.jl:60-91; the sinusoid table of the Whisper
        # encoder) fills its input buffers once, here; the inputs of a call may still overwrite them
        from .device import DeviceArray
        for (node_id, out_idx), data in graph.tensors.items():
            if out_idx == 1 and node_id in self.results:
                a = data.numpy() if isinstance(data, DeviceArray) else np.ascontiguousarray(np.asarray(data, dtype=np.float32))
                buf = self.results[node_id]
                _lib.call("lmb200_upload", self.dev.handle, C.c_void_p(buf.ptr), _lib.F32, a.ctypes.data_as(C.c_void_p),
                          len(buf.shape), _lib.dims(buf.shape), 0)

    # -- execution -------------------------------------------------------------------------------
    def __call__(self, inputs, device=None):
        for node_id, data in inputs.items():
            buf = self.results[node_id]
            a = np.ascontiguousarray(np.asarray(data, dtype=np.float32))
            if a.size != buf.size:
                raise ValueError(f"Input size mismatch for node {node_id}: expected {buf.size}, got {a.size}")
            _lib.call("lmb200_upload", self.dev.handle, C.c_void_p(buf.ptr), _lib.F32, a.ctypes.data_as(C.c_void_p),
                      len(buf.shape), _lib.dims(buf.shape), 0)
        if self.capture:
            from .device import execute_with_capture
            execute_with_capture(self.dev, self.run_steps, self.cache)
        else:
            self.run_steps()
        return self.results

    def run_steps(self):
        """The steps, one library call each, on the device's stream."""
        from .execution import run_op
        h = self.dev.handle
        R = self.results
        for what, out in self.steps:
            kind = what[0]
            if kind == "op":
                run_op(self.dev, what[1], out, [R[i] for i in what[2]])
            elif kind == "fused":
                run_fused(self.dev, what[1], out, [R[i] for i in what[2]])
            elif kind == "silu_gate":
                _lib.call("lmb200_silu_gate", h, _p(out), _p(R[what[1]]), _p(R[what[2]]), out.size)
            elif kind == "rmsnorm":
                _, x, w, rows, n, eps = what
                _lib.call("lmb200_rmsnorm_scale", h, _p(out), _p(R[x]), _p(R[w]), rows, n, eps)
            elif kind == "layernorm":
                _, x, w, b, rows, n, eps = what
                _lib.call("lmb200_layernorm", h, _p(out), _p(R[x]), _p(R[w]), _p(R[b]) if b is not None else None, rows, n, eps)
        return self.results

    def kernel_count(self):
        """Kernels one call launches (the input uploads aside)."""
        return len(self.steps)

    def buffer_bytes(self):
        """Device memory behind the step outputs (inputs and constants aside)."""
        if self.outputs is not None:
            return 4 * sum(b.size for b in self.blocks)
        return 4 * sum(out.size for _, out in self.steps)

    def close(self):
        """Drops the recorded CUDA graph (the buffers go with their DeviceArrays)."""
        g = self.cache.pop("cuda_exec", None)
        if g is not None:
            self.dev.graph_destroy(g)

    def __del__(self):
        try:
            if getattr(self.dev, "handle", None):
                self.close()
        except Exception:
            pass


class _Planner:
    """Host-only planning of compile(): which nodes become which steps.  plan_graph() below is its entry."""

    def __init__(self, graph, fuse=True):
        self.plan = plan = []
        n = len(graph.nodes)
        edges = [0] * (n + 1)
        for node in graph.nodes:
            for i, _, _ in node.inputs:
                edges[i] += 1
        fusible = fusible_intermediates(graph) if fuse else set()
        absorbed = {}                 # terminal node id -> ("rmsnorm" | "layernorm", ...), for the norm patterns
        swallowed = set()             # interior nodes of a recognised norm: no step, no buffer
        if fuse:
            self._find_norms(graph, edges, absorbed, swallowed)
            fusible -= set(absorbed) | swallowed      # a recognised norm is a step of its own: a leaf for the groups around it
        for nid, node in enumerate(graph.nodes, start=1):
            op = node.op
            if nid in swallowed:
                continue
            if nid in absorbed:
                plan.append((nid, absorbed[nid]))
            elif isinstance(op, G.Constant):
                if nid not in fusible:
                    plan.append((nid, ("constant", float(op.value))))
            elif isinstance(op, G.Function) and op.name == "InputTensor":
                plan.append((nid, ("input",)))
            elif not is_elementwise(op):
                plan.append((nid, ("op", op, [i for i, _, _ in node.inputs])))
            elif nid not in fusible:
                code, leaves = group_program(graph, nid, fusible)
                if len(code) == 1 + len(node.inputs) or len(leaves) > MAX_INPUTS or len(code) > MAX_INSTR or _stack_depth(code) > MAX_STACK:
                    # a group of one node, or one too large for the interpreter kernel: node by node
                    for m in self._group_nodes(graph, nid, fusible):
                        mop = graph.nodes[m - 1].op
                        if isinstance(mop, G.Constant):
                            plan.append((m, ("constant", float(mop.value))))
                        else:
                            plan.append((m, ("op", mop, [i for i, _, _ in graph.nodes[m - 1].inputs])))
                else:
                    plan.append((nid, self._specialise(code, leaves)))
    # -- planning helpers ------------------------------------------------------------------------
    @staticmethod
    def _group_nodes(graph, terminal, fusible):
        order = []

        def walk(nid):
            if nid != terminal and nid not in fusible:
                return
            for i, _, _ in graph.nodes[nid - 1].inputs:
                walk(i)
            order.append(nid)
        walk(terminal)
        return order

    @staticmethod
    def _specialise(code, leaves):
        if code == _SILU_GATE:
            return ("silu_gate", leaves[0], leaves[1])
        for tmpl, order in (_MUL_ADD, _ADD_MUL):
            if code == tmpl:
                return ("op", G.FusedMulAdd(), [leaves[k] for k in order])
        if code == _ADD_RELU:
            return ("op", G.FusedAddReLU(), list(leaves))
        return ("fused", code, list(leaves))

    def _find_norms(self, graph, edges, absorbed, swallowed):
        m = _Matcher(graph, edges)
        for nid in range(len(graph.nodes), 0, -1):
            if nid in swallowed or nid in absorbed:
                continue
            found = self._match_norm(m, nid)
            if found is None:
                continue
            what, interior = found
            interior = [i for i in interior if i != nid]
            if any(i in swallowed or i in absorbed for i in interior) or not m.private(interior, [nid]):
                continue
            absorbed[nid] = what
            swallowed.update(interior)

    @staticmethod
    def _match_norm(m, nid):
        """(x [mean-centred]) * inv_std [* gain] [+ bias] ending at nid (NN.LayerNorm / RMSNorm, src/NN.jl:138-173)."""
        shape = m.shape(nid)
        if len(shape) < 1:
            return None
        n = shape[-1]
        interior, bias, gain, cur = [], None, None, nid
        if m.is_(cur, G.Add):                       # ... + expand(bias)
            a, b = m.ins(cur)
            ev = m.expanded_vector(b, n)
            if ev is not None and m.shape(a) == shape:
                bias, chain = ev
                interior += chain + [a]
                cur = a
        if m.is_(cur, G.Mul):                       # ... * expand(gain)
            a, b = m.ins(cur)
            ev = m.expanded_vector(b, n)
            if ev is not None and m.shape(a) == shape and m.std_norm(a) is not None:
                gain, chain = ev
                interior += chain + [a]
                cur = a
        sn = m.std_norm(cur)
        if sn is None or gain is None:
            return None
        x, eps, inner = sn
        interior += inner
        mn = m.mean_norm(x)
        if mn is not None:
            interior += [x] + mn[1]
            return ("layernorm", mn[0], gain, bias, int(np.prod(shape[:-1])), n, eps), interior
        if bias is not None:
            return None                             # RMS scale with a bias: not a layer the reference builds
        return ("rmsnorm", x, gain, int(np.prod(shape[:-1])), n, eps), interior


def plan_graph(graph, fuse=True):
    """[(node id, step)] in node order; step[0] is one of "input", "constant", "op", "fused", "silu_gate",
    "rmsnorm", "layernorm".  Needs no GPU."""
    return _Planner(graph, fuse).plan


def step_reads(what):
    """The node ids a planned step reads."""
    kind = what[0]
    if kind in ("op", "fused"):
        return list(what[2])
    if kind in ("silu_gate", "rmsnorm"):
        return [what[1], what[2]]
    if kind == "layernorm":
        return [i for i in what[1:4] if i is not None]
    return []


def plan_buffers(graph, plan, keep, slack=2.0):
    """Which step outputs may share device memory when only the nodes in `keep` are read after a call.  The reference
    gives every node a buffer of its own for the graph's lifetime (src/Compiler.jl:217-235); here a step's output
    takes over the block of a tensor whose last reader has run, if that block is large enough and at most `slack`
    times too large.  Inputs, constants and `keep` never share.  A step's output never takes a block one of its own
    inputs still occupies (the kernels are not in-place).  Returns ({node id: slot}, [slot capacity in floats]); needs
    no GPU."""
    keep = set(keep)
    steps = [(nid, what) for nid, what in plan if what[0] not in ("input", "constant")]
    produced = {nid for nid, _ in steps}
    last_use = {}
    for idx, (_, what) in enumerate(steps):
        for i in step_reads(what):
            last_use[i] = idx
    slot_of, capacity, free = {}, [], []
    for idx, (nid, what) in enumerate(steps):
        size = max(1, int(np.prod(graph.shapes[nid - 1])) if graph.shapes[nid - 1] else 1)
        fits = [s for s in free if size <= capacity[s] <= slack * size]
        if nid in keep or not fits:
            slot = len(capacity)
            capacity.append(size)
        else:
            slot = min(fits, key=lambda s: capacity[s])
            free.remove(slot)
        slot_of[nid] = slot
        released = {i for i in step_reads(what) if last_use.get(i) == idx and i in produced and i not in keep}
        if nid not in last_use and nid not in keep:
            released.add(nid)                      # nobody reads it: its block is free again at once
        for i in sorted(released):
            if slot_of[i] not in free:
                free.append(slot_of[i])
    return slot_of, capacity


def run_fused(dev, code, out, ins):
    """One fusion group through lmb200_fused_ew: inputs broadcast to the output's shape by the
    reference's rule (1-dims prepended, src/Execution.jl:207-214)."""
    n = len(ins)
    ptrs = (C.c_void_p * max(1, n))(*[a.ptr for a in ins])
    ranks = (C.c_int32 * max(1, n))(*[len(a.shape) for a in ins])
    flat = [d for a in ins for d in a.shape]
    dims = (C.c_int64 * max(1, len(flat)))(*flat)
    ops = (C.c_int32 * len(code))(*[op for op, _ in code])
    args = (C.c_float * len(code))(*[float(arg) for _, arg in code])
    _lib.call("lmb200_fused_ew", dev.handle, C.c_void_p(out.ptr), len(out.shape), _lib.dims(out.shape), n, ptrs, ranks, dims,
              len(code), ops, args)


def compile(graph, device=None, fuse=True, capture=True, outputs=None):     # noqa: A001  (the reference's name)
    """compile(graph) of src/Compiler.jl:181-364.  fuse: form the fusion groups; capture: replay a CUDA graph from the
    second call on; outputs: the node ids the caller reads after a call -- given them, the other intermediate tensors
    share device memory by liveness instead of holding one buffer each for the graph's lifetime."""
    return CompiledGraph(graph, device, fuse, capture, outputs)


__all__ = ["compile", "CompiledGraph", "plan_graph", "plan_buffers", "step_reads", "fusible_intermediates", "group_program", "is_elementwise", "run_fused"]

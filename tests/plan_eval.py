"""A NumPy evaluator of compile()'s plan (test helper): every step kind run with the oracle's primitives, so
the planner -- which nodes fuse, which patterns become which kernel, with which operands -- is checked
against node-by-node evaluation without a GPU."""
import numpy as np

import luminal_jl_b200 as L
import luminal_oracle as O

G = L.graph


def run_op(op, ins, out_shape):
    t=type(op)
    if t is G.Add: return O.add(*ins)
    if t is G.Mul: return O.mul(*ins)
    if t is G.Mod: return O.mod(*ins)
    if t is G.LessThan: return O.less_than(*ins)
    if t is G.Max: return np.maximum(*ins).astype(np.float32)
    if t is G.Log2: return O.log2(ins[0])
    if t is G.Exp2: return O.exp2(ins[0])
    if t is G.Sin: return O.sin(ins[0])
    if t is G.Sqrt: return O.sqrt(ins[0])
    if t is G.Recip: return O.recip(ins[0])
    if t is G.ReLU: return O.relu(ins[0])
    if t is G.FusedMulAdd: return O.fused_mul_add(*ins)
    if t is G.FusedAddReLU: return O.fused_add_relu(*ins)
    if t is G.SumReduce: return O.sum_reduce(ins[0], op.dim)
    if t is G.MaxReduce: return O.max_reduce(ins[0], op.dim)
    if t is G.MatMul: return O.matmul(*ins)
    if t is G.Permute: return O.permute(ins[0], op.dims)
    if t is G.Reshape: return O.reshape(ins[0], op.shape)
    if t is G.Expand: return O.expand(ins[0], op.dim, op.size)
    if t is G.Slice:
        a=ins[0]
        return a[tuple(slice(s, min(e,d)) for (s,e),d in zip(op.ranges,a.shape))]
    if t is G.Pad: return np.pad(ins[0], op.padding)
    if t is G.Unfold: return O.unfold1d(ins[0], op.kernel_shape[0], op.stride_shape[0], op.dilation_shape[0])
    if t is G.Function and op.name=="Gather": return O.gather(*ins)
    if t is G.Function and op.name=="CumSum": return O.cumsum_last(ins[0])
    raise NotImplementedError(op)
def eval_graph(g, inputs, want):
    """Node-by-node evaluation of a graph with the oracle's primitives: the CPU counterpart of execute()."""
    vals = {}
    for n, (node, shp) in enumerate(zip(g.nodes, g.shapes), start=1):
        op = node.op
        if isinstance(op, G.Function) and op.name == "InputTensor":
            if n in inputs:
                vals[n] = np.asarray(inputs[n], np.float32)
            elif (n, 1) in g.tensors:
                vals[n] = np.asarray(g.tensors[(n, 1)], np.float32)
        elif isinstance(op, G.Constant):
            vals[n] = np.float32(op.value)
        else:
            vals[n] = run_op(op, [vals[i] for i, _, _ in node.inputs], shp)
    return [vals[i] for i in want]


def eval_step(graph, nid, w, R):
    """The value of one planned step from the values R of the nodes it reads."""
    k=w[0]
    if k=='op': return run_op(w[1],[R[i] for i in w[2]],graph.shapes[nid-1])
    if k=='fused':
        st=[]
        for op,arg in w[1]:
            if op==0: st.append(R[w[2][int(arg)]])
            elif op==1: st.append(np.float32(arg))
            else:
                cls={v:k2 for k2,v in L.compiler._CODE.items()}[op]
                ar=3 if cls is G.FusedMulAdd else (2 if cls in (G.Add,G.Mul,G.Mod,G.LessThan,G.Max,G.FusedAddReLU) else 1)
                args=st[-ar:]; del st[-ar:]
                st.append(run_op(cls(),args,None))
        return np.broadcast_to(st[0],graph.shapes[nid-1]).astype(np.float32)
    if k=='silu_gate': return O.mul(O.swish(R[w[1]]),R[w[2]])
    if k=='rmsnorm': return O.rms_norm(R[w[1]],R[w[2]],w[5])
    if k=='layernorm': return O.layer_norm(R[w[1]],R[w[2]],R[w[3]] if w[3] is not None else None,w[6])
    raise NotImplementedError(k)


def _leaves(graph, plan, inputs):
    R={}
    for nid,w in plan:
        k=w[0]
        if k=='input':
            R[nid]=np.asarray(inputs[nid] if nid in inputs else graph.tensors[(nid,1)],np.float32)
        elif k=='constant': R[nid]=np.float32(w[1])
    return R


def eval_plan(graph, plan, inputs):
    R=_leaves(graph, plan, inputs)
    for nid,w in plan:
        if w[0] not in ('input','constant'): R[nid]=eval_step(graph, nid, w, R)
    return R


def eval_plan_shared(graph, plan, inputs, keep):
    """The plan run with the block sharing plan_buffers() decides: every step output is written into its block, and a
    step reads its operands out of the blocks as they are at that moment -- so a block handed on too early shows as a
    wrong value.  Returns ({node: value} for `keep`, the slot map, the capacities)."""
    slot_of, capacity = L.compiler.plan_buffers(graph, plan, keep)
    blocks=[np.full(n, np.nan, np.float32) for n in capacity]
    leaves=_leaves(graph, plan, inputs)
    shape_of=lambda nid: tuple(graph.shapes[nid-1])

    class View(dict):
        def __missing__(self, nid):
            if nid in leaves: return leaves[nid]
            n=int(np.prod(shape_of(nid))) if shape_of(nid) else 1
            return blocks[slot_of[nid]][:n].reshape(shape_of(nid))
    R=View()
    for nid,w in plan:
        if w[0] in ('input','constant'): continue
        val=np.ascontiguousarray(eval_step(graph, nid, w, R), np.float32)
        blocks[slot_of[nid]][:val.size]=val.reshape(-1)
    return {nid: R[nid].copy() for nid in keep}, slot_of, capacity

"""compile() with fusion: the groups the reference forms (src/Compiler.jl:183-215) and what they map
to, checked on the host (the plan) and on the GPU (values).  The two graphs of the reference's own
fusion test, tests/test_fusion.jl:7-56, must compile to ONE step each."""
import collections

import numpy as np
import pytest

import luminal_oracle as O
import whisper_oracle as W


def _steps(plan):
    return [w for _, w in plan if w[0] not in ("input", "constant")]


def test_reference_fusion_cases_compile_to_one_step(lib_built):
    L = lib_built
    G = L.graph
    g = L.Graph()
    a, b, c = (L.tensor(g, [3, 3]) for _ in range(3))
    d = (a + b) * c                                     # tests/test_fusion.jl:8-20
    steps = _steps(L.compiler.plan_graph(g))
    assert len(steps) == 1 and steps[0][0] == "fused" and steps[0][2] == [a.id, b.id, c.id]
    g2 = L.Graph()
    x, w, bias = (L.tensor(g2, [2, 2]) for _ in range(3))
    out = G.relu((x * w) + bias)                        # tests/test_fusion.jl:33-46
    steps = _steps(L.compiler.plan_graph(g2))
    assert len(steps) == 1 and steps[0][0] == "fused"
    assert len(_steps(L.compiler.plan_graph(g2, fuse=False))) == 3
    assert d.id and out.id


def test_named_fusions_map_to_their_kernels(lib_built):
    L = lib_built
    G = L.graph
    g = L.Graph()
    a, b, c = (L.tensor(g, [4]) for _ in range(3))
    _ = a * b + c
    s = _steps(L.compiler.plan_graph(g))
    assert len(s) == 1 and s[0][0] == "op" and isinstance(s[0][1], G.FusedMulAdd) and s[0][2] == [a.id, b.id, c.id]
    g = L.Graph()
    a, b = L.tensor(g, [4]), L.tensor(g, [4])
    _ = G.relu(a + b)
    s = _steps(L.compiler.plan_graph(g))
    assert len(s) == 1 and isinstance(s[0][1], G.FusedAddReLU)
    g = L.Graph()
    gate, up = L.tensor(g, [2, 8]), L.tensor(g, [2, 8])
    _ = G.silu(gate) * up                                # NN.Mlp, src/NN.jl:246-249
    s = _steps(L.compiler.plan_graph(g))
    assert s == [("silu_gate", gate.id, up.id)]
    g = L.Graph()
    x = L.tensor(g, [2, 3, 16])
    y = L.nn.RMSNorm(16, g)(x)
    s = _steps(L.compiler.plan_graph(g))
    assert len(s) == 1 and s[0][0] == "rmsnorm" and s[0][1] == x.id and s[0][3:5] == (6, 16) and abs(s[0][5] - 1e-5) < 1e-9 and y.id
    g = L.Graph()
    x = L.tensor(g, [5, 16])
    y = L.nn.LayerNorm(16, g)(x)
    s = _steps(L.compiler.plan_graph(g))
    assert len(s) == 1 and s[0][0] == "layernorm" and s[0][1] == x.id and s[0][4:6] == (5, 16) and abs(s[0][6] - 1e-5) < 1e-9 and y.id


def test_a_value_used_twice_is_not_fused_away(lib_built):
    """Only single-consumer element-wise nodes vanish (src/Compiler.jl:196-213): t feeds two nodes, so it is a step of
    its own and a leaf of both consumers."""
    L = lib_built
    g = L.Graph()
    a, b = L.tensor(g, [4]), L.tensor(g, [4])
    t = a + b
    _ = (t * a) + (t * b)
    plan = dict(L.compiler.plan_graph(g))
    assert plan[t.id][0] == "op"
    assert t.id not in L.compiler.fusible_intermediates(g)


def test_llama_graph_step_count(lib_built):
    L = lib_built
    g, reg = L.Graph(), {}
    m = L.nn.Llama(g, reg, vocab_size=64, hidden=32, n_layers=2, n_heads=4, n_kv_heads=2, intermediate=48)
    m(L.tensor(g, [2, 5]), 0)
    fused, plain = _steps(L.compiler.plan_graph(g)), _steps(L.compiler.plan_graph(g, fuse=False))
    kinds = collections.Counter(s[0] for s in fused)
    assert kinds["rmsnorm"] == 5 and kinds["silu_gate"] == 2          # 2 per block + the final norm; one MLP per block
    assert len(fused) < 0.65 * len(plain)


@pytest.mark.gpu
def test_fused_groups_equal_node_by_node(lib_built, device):
    """The interpreter kernel rounds every operation on its own: bit-identical to the unfused compile."""
    L = lib_built
    G = L.graph
    rng = np.random.default_rng(0)
    g = L.Graph()
    a, b, c = L.tensor(g, [4, 1, 6]), L.tensor(g, [5, 6]), L.tensor(g, [6])
    t = G.exp2(a * b + c) * G.sin(b) + G.sqrt(G.relu(a) + np.float32(0.5))
    out = G.maximum(t, c) % np.float32(3.0) + (a < b) * G.reciprocal(c * c + np.float32(1.0))
    vals = {a.id: rng.standard_normal((4, 1, 6)).astype(np.float32), b.id: rng.standard_normal((5, 6)).astype(np.float32),
            c.id: rng.standard_normal(6).astype(np.float32)}
    f, p = L.compile(g, device), L.compile(g, device, fuse=False)
    assert f.kernel_count() < p.kernel_count()
    got, want = f(vals)[out.id].numpy(), p(vals)[out.id].numpy()
    assert got.shape == (4, 5, 6) and np.array_equal(got, want)
    # the reference's two cases, values as tests/test_fusion.jl:26-29, 48-55 checks them
    g1 = L.Graph()
    x, w, bias = (L.tensor(g1, [2, 2]) for _ in range(3))
    o1 = G.relu((x * w) + bias)
    xv, wv, bv = (rng.random((2, 2)).astype(np.float32) for _ in range(3))
    bv -= np.float32(0.5)
    c1 = L.compile(g1, device)
    assert c1.kernel_count() == 1
    assert np.allclose(c1({x.id: xv, w.id: wv, bias.id: bv})[o1.id].numpy(), np.maximum(xv * wv + bv, 0.0))


@pytest.mark.gpu
def test_compiled_llama_graph_matches_oracle(lib_built, device):
    L = lib_built
    cfg = dict(O.CONFIGS["tiny_gqa128"], n_layers=1, hidden=256, n_heads=2, n_kv_heads=1, intermediate=192, vocab=96)
    w = O.synth_llama_weights(cfg, seed=5)
    g, reg = L.Graph(), {}
    m = L.nn.Llama(g, reg, vocab_size=cfg["vocab"], hidden=cfg["hidden"], n_layers=1, n_heads=2, n_kv_heads=1,
                   intermediate=cfg["intermediate"])
    tok_t = L.tensor(g, [2, 4])
    out = m(tok_t, 0)
    tokens = O.synth_tokens(5, 9, (2, 4), cfg["vocab"])
    inputs = {t.id: w[name] for name, t in reg.items()}
    inputs[tok_t.id] = tokens.astype(np.float32)
    ref = O.llama_forward(tokens, w, cfg)
    cg = L.compile(g, device)
    got = cg(inputs)[out.id].numpy()
    assert np.abs(got - ref).max() <= 1e-3
    plain = L.compile(g, device, fuse=False)
    assert cg.kernel_count() < 0.65 * plain.kernel_count()
    assert np.abs(plain(inputs)[out.id].numpy() - ref).max() <= 1e-3


@pytest.mark.gpu
def test_compiled_whisper_encoder_matches_oracle(lib_built, device):
    """A graph that is not a Llama: the Whisper AudioEncoder through compile() -- LayerNorms become one kernel each,
    the GELU chains one fused kernel -- against the oracle's encoder."""
    L = lib_built
    cfg = W.CONFIGS["whisper_test"]
    w = W.synth_weights(cfg, seed=13)
    mel = O.synth_normal(13, 5, (2, cfg["n_mels"], 60), 1.0)
    g, reg = L.Graph(), {}
    enc = L.whisper.AudioEncoder(g, reg, d_model=cfg["d_model"], heads=cfg["heads"], layers=cfg["enc_layers"], ffn=cfg["ffn"],
                                 n_mels=cfg["n_mels"])
    mel_t = L.tensor(g, mel.shape)
    out = enc(mel_t)
    inputs = {t.id: w[name] for name, t in reg.items()}
    inputs[mel_t.id] = mel
    cg, plain = L.compile(g, device), L.compile(g, device, fuse=False)
    kinds = collections.Counter(s[0][0] for s in cg.steps)
    assert kinds["layernorm"] == 2 * cfg["enc_layers"] + 1
    assert cg.kernel_count() < 0.7 * plain.kernel_count()
    ref = W.encoder(mel, w, cfg)
    got = cg(inputs)[out.id].numpy()
    assert got.shape == ref.shape and np.abs(got - ref).max() <= 1e-3


def test_plans_evaluate_to_the_same_values_on_the_host(lib_built):
    """Fused and unfused plans of the Whisper encoder graph and of a Llama graph, evaluated with the oracle's
    primitives on the CPU: the fused plan must give the unfused plan's values and the oracle model's."""
    from plan_eval import eval_plan
    L = lib_built
    cfg = W.CONFIGS["whisper_test"]
    w = W.synth_weights(cfg, seed=13)
    mel = O.synth_normal(13, 5, (2, cfg["n_mels"], 40), 1.0)
    g, reg = L.Graph(), {}
    enc = L.whisper.AudioEncoder(g, reg, d_model=cfg["d_model"], heads=cfg["heads"], layers=cfg["enc_layers"], ffn=cfg["ffn"],
                                 n_mels=cfg["n_mels"])
    mel_t = L.tensor(g, mel.shape)
    out = enc(mel_t)
    inputs = {t.id: w[name] for name, t in reg.items()}
    inputs[mel_t.id] = mel
    ref = W.encoder(mel, w, cfg)
    for fuse in (False, True):
        got = eval_plan(g, L.compiler.plan_graph(g, fuse), inputs)[out.id]
        assert np.abs(got - ref).max() <= 1e-5, fuse
    lcfg = dict(O.CONFIGS["tiny_gqa128"], n_layers=1, hidden=64, n_heads=2, n_kv_heads=1, intermediate=48, vocab=40)
    lw = O.synth_llama_weights(lcfg, seed=5)
    g, reg = L.Graph(), {}
    m = L.nn.Llama(g, reg, vocab_size=40, hidden=64, n_layers=1, n_heads=2, n_kv_heads=1, intermediate=48)
    tok_t = L.tensor(g, [2, 3])
    out = m(tok_t, 0)
    tokens = O.synth_tokens(5, 9, (2, 3), 40)
    inputs = {t.id: lw[name] for name, t in reg.items()}
    inputs[tok_t.id] = tokens.astype(np.float32)
    ref = O.llama_forward(tokens, lw, lcfg)
    for fuse in (False, True):
        got = eval_plan(g, L.compiler.plan_graph(g, fuse), inputs)[out.id]
        assert np.abs(got - ref).max() <= 1e-5, fuse


def test_execute_with_capture_host_logic():
    """execute_with_capture's bookkeeping (src/Device.jl:106-121) against a stand-in device: the first call runs f()
    and records it, later calls only replay; a recording that fails leaves f() running call by call."""
    from luminal_jl_b200 import _lib
    from luminal_jl_b200.device import execute_with_capture

    class FakeDevice:
        def __init__(self, fail=False):
            self.fail, self.recorded, self.replays = fail, 0, 0

        def capture(self, f):
            if self.fail:
                raise _lib.LuminalB200Error(-5, "upload: not between capture_begin and capture_end")
            f()
            self.recorded += 1
            return 7

        def graph_launch(self, graph):
            assert graph == 7
            self.replays += 1

    runs = []
    dev, cache = FakeDevice(), {}
    for _ in range(4):
        execute_with_capture(dev, lambda: runs.append(1), cache)
    assert cache["cuda_exec"] == 7 and dev.recorded == 1 and dev.replays == 3
    assert len(runs) == 2                         # once for real, once while recording
    runs.clear()
    dev, cache = FakeDevice(fail=True), {}
    for _ in range(3):
        execute_with_capture(dev, lambda: runs.append(1), cache)
    assert cache["cuda_exec"] is None and "capture_begin" in cache["cuda_exec_error"]
    assert len(runs) == 3 and dev.replays == 0


def test_buffer_sharing_plan_keeps_every_value_alive(lib_built):
    """plan_buffers(): with the blocks shared as planned, the kept outputs of a 2-layer Llama graph, of the Whisper
    encoder graph and of a graph with two outputs equal the unshared evaluation; the shared plan needs a
    fraction of the memory; no step's output shares a block with one of its own operands."""
    from luminal_jl_b200 import nn, whisper as WG
    from plan_eval import eval_plan, eval_plan_shared
    L = lib_built
    G = L.graph
    cases = []
    g, reg = G.Graph(), {}
    model = nn.Llama(g, reg, vocab_size=50, hidden=32, n_layers=2, n_heads=4, n_kv_heads=2, intermediate=48)
    tok = G.tensor(g, [2, 5])
    out = model(tok, 0)
    inputs = {t.id: O.synth_normal(3, t.id, t.shape, 0.3) for t in reg.values()}
    inputs[tok.id] = O.synth_tokens(3, 999, (2, 5), 50).astype(np.float32)
    cases.append((g, inputs, [out.id]))
    g, reg = G.Graph(), {}
    enc = WG.AudioEncoder(g, reg, d_model=32, heads=2, layers=2, ffn=48, n_mels=8)
    mel = G.tensor(g, [2, 8, 21])
    out = enc(mel)
    inputs = {t.id: O.synth_normal(4, t.id, t.shape, 0.3) for t in reg.values()}
    inputs[mel.id] = O.synth_normal(4, 999, (2, 8, 21), 1.0)
    cases.append((g, inputs, [out.id]))
    g = G.Graph()
    a, b = G.tensor(g, [4, 6]), G.tensor(g, [4, 6])
    c = G.relu(a * b + a)
    d = G.sum_(c * c, 2)
    e = G.exp2(c) + G.expand(d, 2, 6)
    cases.append((g, {a.id: O.synth_normal(5, 1, (4, 6), 1.0), b.id: O.synth_normal(5, 2, (4, 6), 1.0)}, [d.id, e.id]))
    for g, inputs, keep in cases:
        for fuse in (True, False):
            plan = L.compiler.plan_graph(g, fuse)
            want = eval_plan(g, plan, inputs)
            got, slot_of, capacity = eval_plan_shared(g, plan, inputs, keep)
            for nid in keep:
                # (not bit for bit: NumPy's matmul takes another path for the blocks' contiguous views)
                assert np.allclose(got[nid], want[nid], rtol=1e-4, atol=1e-5), (nid, fuse)
            for nid, what in plan:
                if nid in slot_of:
                    assert all(slot_of.get(i) != slot_of[nid] for i in L.compiler.step_reads(what)), nid
            assert len({slot_of[n] for n in keep}) == len(keep)
            own = sum(int(np.prod(g.shapes[n - 1])) if g.shapes[n - 1] else 1 for n in slot_of)
            if len(slot_of) > 20:
                assert sum(capacity) < 0.35 * own, (sum(capacity), own)


@pytest.mark.gpu
def test_compile_with_outputs_shares_buffers(lib_built, device):
    """compile(graph, outputs=[...]): the intermediate tensors share blocks by liveness; the kept outputs equal those
    of the graph compiled with one buffer per node, on the first (step by step) call and on the replays."""
    from luminal_jl_b200 import nn
    L = lib_built
    G = L.graph
    g, reg = G.Graph(), {}
    model = nn.Llama(g, reg, vocab_size=200, hidden=64, n_layers=2, n_heads=4, n_kv_heads=2, intermediate=96)
    tok = G.tensor(g, [2, 16])
    out = model(tok, 0)
    inputs = {t.id: O.synth_normal(3, t.id, t.shape, 0.3) for t in reg.values()}
    own, shared = L.compile(g, device), L.compile(g, device, outputs=[out.id])
    assert shared.buffer_bytes() < 0.35 * own.buffer_bytes()
    for seed in range(3):
        inputs[tok.id] = O.synth_tokens(seed, 999, (2, 16), 200).astype(np.float32)
        assert np.array_equal(shared(inputs)[out.id].numpy(), own(inputs)[out.id].numpy())
    assert shared.cache.get("cuda_exec") is not None
    own.close(); shared.close()
    with pytest.raises(KeyError):
        interior = next(n for n in range(len(g.nodes), 0, -1) if n not in dict(L.compiler.plan_graph(g)))
        L.compile(g, device, outputs=[interior])


def test_buffer_sharing_on_random_graphs(lib_built):
    """plan_buffers() on seeded random graphs (element-wise chains, reductions, expands, permutes, matmuls, values read
    many steps after they were made, several kept outputs): the shared run equals the unshared one and no step's output
    shares a block with an operand."""
    from plan_eval import eval_plan, eval_plan_shared
    L = lib_built
    G = L.graph
    rng = np.random.default_rng(77)
    for trial in range(40):
        g = G.Graph()
        n = int(rng.choice([3, 4, 6]))
        pool = [G.tensor(g, [n, n]) for _ in range(int(rng.integers(1, 4)))]
        inputs = {t.id: rng.standard_normal((n, n)).astype(np.float32) for t in pool}
        for _ in range(int(rng.integers(5, 40))):
            a = pool[int(rng.integers(len(pool)))] if rng.random() < 0.4 else pool[-1 - int(rng.integers(min(3, len(pool))))]
            b = pool[int(rng.integers(len(pool)))]
            kind = int(rng.integers(8))
            if kind == 0:
                t = a + b
            elif kind == 1:
                t = a * b * np.float32(0.5)
            elif kind == 2:
                t = G.relu(a) + np.float32(0.25)
            elif kind == 3:
                t = G.sin(a)
            elif kind == 4:
                t = G.expand(G.sum_(a, 2), 2, n) * np.float32(1.0 / n)
            elif kind == 5:
                t = G.permute(a, [2, 1])
            elif kind == 6:
                t = G.matmul(a, b) * np.float32(1.0 / n)
            else:
                t = G.expand(G.max_reduce(a, 1), 1, n)
            pool.append(t)
        made = [t.id for t in pool if t.id not in inputs]
        # the fusion groups change which nodes are materialised, never a value
        fused, plain = eval_plan(g, L.compiler.plan_graph(g, True), inputs), eval_plan(g, L.compiler.plan_graph(g, False), inputs)
        assert set(fused) <= set(plain) and set(made) <= set(plain)
        for nid in fused:
            assert np.array_equal(np.asarray(fused[nid]), np.asarray(plain[nid]), equal_nan=True), (trial, nid)
        for fuse in (True, False):
            plan = L.compiler.plan_graph(g, fuse)
            planned = {nid for nid, what in plan if what[0] not in ("input", "constant")}
            candidates = [i for i in made if i in planned]
            keep = sorted(set(int(i) for i in rng.choice(candidates, size=min(len(candidates), int(rng.integers(1, 4))), replace=False)))
            want = eval_plan(g, plan, inputs)
            got, slot_of, capacity = eval_plan_shared(g, plan, inputs, keep)
            for nid in keep:
                assert np.allclose(got[nid], want[nid], rtol=1e-4, atol=1e-5, equal_nan=True), (trial, fuse, nid)
            for nid, what in plan:
                if nid in slot_of:
                    assert all(slot_of.get(i) != slot_of[nid] for i in L.compiler.step_reads(what)), (trial, nid)
            assert len({slot_of[i] for i in keep}) == len(keep)

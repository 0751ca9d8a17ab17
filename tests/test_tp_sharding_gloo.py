"""Tensor-parallel sharding on CPU: two gloo ranks each build their shard of a GQA model from the
library's own index maps (lmb200_shard_map, host arithmetic), run one prompt + decode steps with
NumPy in the library's internal layouts, all-reduce the row-parallel partial sums, and must
reproduce the unsharded oracle.  This pins the head / MLP-column partition, the q = kv + KV*g and
f = h + H*d conventions under sharding, and the two all-reduces per layer, without a GPU."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _rank_main(rank, world, port, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import torch
    import torch.distributed as dist
    import luminal_jl_b200 as L
    import luminal_oracle as O

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    cfg = O.CONFIGS["tiny_gqa128"]
    w = O.synth_llama_weights(cfg, seed=21)
    H, KV, hid = cfg["n_heads"], cfg["n_kv_heads"], cfg["hidden"]
    D, G = hid // H, H // KV
    B, P, steps = 2, 5, 3

    def shard(matrix, names):
        rows, cols, rmap, cmap = L.shard_layout(cfg, matrix, world, rank)
        W = np.zeros((rows, cols), np.float32)
        for i, (slot, lrow) in enumerate(rmap):
            if slot >= 0:
                W[i] = w[names[slot]][lrow, cmap]
        return W, rmap, cmap

    def allreduce(a):
        t = torch.from_numpy(np.ascontiguousarray(a))
        dist.all_reduce(t)
        return t.numpy()

    inv = O.rope_inv_freqs(D, cfg["rope_base"])
    kcache = [dict() for _ in range(cfg["n_layers"])]       # (b, kv head) -> list of k / v rows
    logits_all = []

    def step(tokens, pos):
        x = w["model.embed_tokens.weight"][tokens]                              # [B, hid], replicated
        for l in range(cfg["n_layers"]):
            n = O.layer_names(l)
            Wqkv, rmap, _ = shard("qkv", [n["q"], n["k"], n["v"]])
            xn = O.rms_norm(x, w[n["attn_norm"]], cfg["eps"])
            y = xn @ Wqkv.T                                                     # internal rows
            qh, kh, vh = {}, {}, {}
            for i, (slot, f) in enumerate(rmap):
                if slot == 0:
                    qh[(f % H, f // H)] = y[:, i]
                elif slot == 1:
                    kh[(f % KV, f // KV)] = y[:, i]
                elif slot == 2:
                    vh[(f % KV, f // KV)] = y[:, i]
            heads = sorted({h for h, _ in qh})
            kvs = sorted({h for h, _ in kh})
            assert len(heads) == H // world and len(kvs) == KV // world
            assert all((h % KV) in kvs for h in heads)                         # q heads travel with their kv head

            def rope(vecs, h):
                v = np.stack([vecs[(h, d)] for d in range(D)], axis=1)          # [B, D]
                return O.apply_rotary_embeddings(v[:, None, None, :], pos, cfg["rope_base"])[:, 0, 0, :]

            for kvh in kvs:
                k = rope(kh, kvh)
                v = np.stack([vh[(kvh, d)] for d in range(D)], axis=1)
                for b in range(B):
                    kcache[l].setdefault((b, kvh), ([], []))
                    kcache[l][(b, kvh)][0].append(k[b])
                    kcache[l][(b, kvh)][1].append(v[b])
            attn = {}
            for h in heads:
                qv = rope(qh, h)
                for b in range(B):
                    K = np.stack(kcache[l][(b, h % KV)][0]); V = np.stack(kcache[l][(b, h % KV)][1])
                    s = (K @ qv[b]) / np.sqrt(np.float32(D))
                    p = np.exp(s - s.max()); p /= p.sum()
                    attn[(b, h)] = p @ V
            Wo, _, cmap_o = shard("o", [n["o"]])
            a_int = np.zeros((B, len(cmap_o)), np.float32)
            for k_i, f in enumerate(cmap_o):
                for b in range(B):
                    a_int[b, k_i] = attn[(b, f % H)][f // H]
            x = x + allreduce(a_int @ Wo.T)                                     # all-reduce #1
            Wgu, rmap_gu, _ = shard("gate_up", [n["gate"], n["up"]])
            xn = O.rms_norm(x, w[n["ffn_norm"]], cfg["eps"])
            y = xn @ Wgu.T
            Wd, _, cmap_d = shard("down", [n["down"]])
            gate = {lr: y[:, i] for i, (s_, lr) in enumerate(rmap_gu) if s_ == 0}
            up = {lr: y[:, i] for i, (s_, lr) in enumerate(rmap_gu) if s_ == 1}
            act = np.stack([O.mul(O.silu(gate[c]), up[c]) for c in cmap_d], axis=1)
            x = x + allreduce(act @ Wd.T)                                       # all-reduce #2
        x = O.rms_norm(x, w["model.norm.weight"], cfg["eps"])
        return x @ w["lm_head.weight"].T

    prompt = O.synth_tokens(21, 1000, (B, P), cfg["vocab"])
    for i in range(P):
        logits = step(prompt[:, i], i)
    toks = []
    for s_ in range(steps):
        nxt = logits.argmax(-1)
        toks.append(nxt)
        logits_all.append(logits)
        logits = step(nxt, P + s_)
    if rank == 0:
        ref_tok, ref_log = O.CachedLlama(w, cfg, B, 16).greedy(prompt, steps)
        q.put((np.array_equal(np.stack(toks, 1), ref_tok), float(np.abs(np.stack(logits_all, 1) - ref_log).max())))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharded_decode_matches_oracle(lib_built):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    same_tokens, err = q.get(timeout=600)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert same_tokens
    assert err <= 1e-4


def test_shard_config_errors(lib_built):
    import luminal_jl_b200 as L
    import luminal_oracle as O
    cfg = O.CONFIGS["tiny_gqa128"]
    with pytest.raises(L.LuminalB200Error, match="does not divide"):
        L.shard_layout(cfg, "qkv", 4, 0)            # 2 kv heads cannot be split over 4 ranks
    with pytest.raises(L.LuminalB200Error, match="tp rank"):
        L.shard_layout(cfg, "qkv", 2, 2)

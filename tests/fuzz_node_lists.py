"""Corrupted node lists against the three structural matchers (run as a child process by tests/test_match.py, so that a
crash of the host code shows as an exit code): one op code, input edge, op field, recorded shape, offset or the output
id of a valid Llama / Whisper-step / Whisper-encoder list is changed at random; every call must come back with a
status -- accepted or refused -- and never fault.  Prints the counts."""
import ctypes as C
import sys

import numpy as np

import luminal_jl_b200  # noqa: F401  (loads the library)
from luminal_jl_b200 import _lib, graph as G, match as M, nn, whisper as WG
from luminal_jl_b200.session import ModelConfig


def graphs():
    g, reg = G.Graph(), {}
    model = nn.Llama(g, reg, vocab_size=64, hidden=32, n_layers=2, n_heads=4, n_kv_heads=2, intermediate=48)
    yield g, model(G.tensor(g, [2, 3]), 0).id
    g, reg = G.Graph(), {}
    td = WG.TextDecoder(g, reg, d_model=32, heads=2, layers=2, ffn=48, vocab=50, max_positions=12)
    yield g, WG.build_decode_step(td, g, 7, 3, batch=2).logits_id
    g, reg = G.Graph(), {}
    enc = WG.AudioEncoder(g, reg, d_model=32, heads=2, layers=2, ffn=48, n_mels=8)
    yield g, enc(G.tensor(g, [2, 8, 21])).id


def main(seed, trials):
    rng = np.random.default_rng(seed)
    accepted = refused = 0
    for g, out_id in graphs():
        for _ in range(trials):
            nl = M.flatten_graph(g)
            ops, in_off, in_node, shape_off, shape, arg_off, arg = nl.keep
            n, oid = len(ops), out_id
            kind = int(rng.integers(6))
            if kind == 0:
                ops[rng.integers(n)] = rng.integers(0, 30)
            elif kind == 1:
                k = int(rng.integers(len(in_node)))
                node = int(np.searchsorted(in_off, k, side="right"))
                in_node[k] = rng.integers(1, max(2, node))
            elif kind == 2:
                arg[rng.integers(len(arg))] = rng.choice([0, 1, 2, 3, -1, 1e9, 1e19, 0.5, 7])
            elif kind == 3:
                shape[rng.integers(len(shape))] = rng.choice([0, 1, 2, 3, 5, 64])
            elif kind == 4:                       # one node loses its last field or input: the offsets after it shift
                node = int(rng.integers(1, n + 1))
                off = arg_off if rng.integers(2) else in_off
                if off[node] > off[node - 1]:
                    off[node:] -= 1
            else:
                oid = int(rng.integers(-1, n + 3))
            cfg, info, einfo = ModelConfig(), M.DecoderMatchInfo(), M.EncoderMatchInfo()
            nodes, cache = (C.c_int32 * n)(), (C.c_int32 * n)()
            names = C.create_string_buffer(64 * n + 256)
            calls = (("lmb200_match_decoder", (C.byref(cfg), C.byref(info), nodes, n, names, len(names))),
                     ("lmb200_match_whisper_step", (C.byref(cfg), C.byref(info), nodes, n, names, len(names), cache, n)),
                     ("lmb200_match_whisper_encoder", (C.byref(einfo), nodes, n, names, len(names))))
            for name, rest in calls:
                try:
                    _lib.call(name, C.byref(nl), oid, *rest)
                    accepted += 1
                except _lib.LuminalB200Error:
                    refused += 1
    print(f"accepted {accepted} refused {refused}")


if __name__ == "__main__":
    main(int(sys.argv[1]), int(sys.argv[2]))

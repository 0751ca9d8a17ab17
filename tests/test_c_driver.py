"""The C ABI used from plain C: tests/cabi_driver.c is compiled with gcc as strict C99 against
include/luminal_b200.h and linked to the shared library.  Without a GPU it must fail loudly at
lmb200_init; on a B200 its greedy tokens must equal the CPU oracle's."""
import json
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def driver(lib_built, tmp_path_factory):
    from importlib import import_module
    lib = import_module("luminal_jl_b200._build").LIB
    exe = str(tmp_path_factory.mktemp("cabi") / "cabi_driver")
    cmd = ["gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-O1", os.path.join(ROOT, "tests", "cabi_driver.c"),
           "-I", os.path.join(ROOT, "include"), "-L", os.path.dirname(lib), "-lluminal_b200",
           "-Wl,-rpath," + os.path.dirname(lib), "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def test_header_is_plain_c_and_driver_fails_loudly_without_a_gpu(driver):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the GPU test runs the driver")
    r = subprocess.run([driver, "0", "1", "4", "2", "1234"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 2 and "lmb200_init" in r.stderr and r.stdout == ""
    assert subprocess.run([driver], capture_output=True).returncode == 64


@pytest.mark.gpu
@pytest.mark.parametrize("batch,prompt,steps", [(1, 32, 24), (3, 9, 12)])
def test_c_driver_tokens_match_the_oracle(driver, batch, prompt, steps):
    import luminal_oracle as O
    r = subprocess.run([driver, "0", str(batch), str(prompt), str(steps), "1234"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    got = json.loads(r.stdout)
    cfg = O.CONFIGS["small_llama"]
    w = O.synth_llama_weights(cfg, seed=1234)
    toks = np.array([[(7 * i + 3 + 11 * b) % cfg["vocab"] for i in range(prompt)] for b in range(batch)], dtype=np.int64)
    ref_tok, _ = O.CachedLlama(w, cfg, batch, prompt + steps + 1).greedy(toks, steps + 1)
    ref_tok = np.asarray(ref_tok)                     # [batch, steps + 1]: the prompt's prediction, then one per step
    assert got["position"] == prompt + steps
    assert got["first"] == ref_tok[:, 0].tolist()
    assert np.array_equal(np.array(got["tokens"]).reshape(steps, batch).T, ref_tok[:, 1:])


@pytest.mark.gpu
def test_c_driver_bf16_runs(driver):
    r = subprocess.run([driver, "1", "2", "16", "8", "7"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    got = json.loads(r.stdout)
    assert got["position"] == 24 and len(got["tokens"]) == 16 and all(0 <= t < 1024 for t in got["tokens"])


def test_matchers_from_plain_c(lib_built, tmp_path):
    """tests/cabi_match.c (strict C99, no GPU): node lists of the three kinds written to a file, read back into
    lmb200_node_list by the C program and matched there; what it prints equals what the ctypes caller gets."""
    from importlib import import_module
    import luminal_jl_b200 as L
    from luminal_jl_b200 import graph as G, match as M, nn, whisper as WG
    lib = import_module("luminal_jl_b200._build").LIB
    exe = str(tmp_path / "cabi_match")
    cmd = ["gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-O1", os.path.join(ROOT, "tests", "cabi_match.c"),
           "-I", os.path.join(ROOT, "include"), "-L", os.path.dirname(lib), "-lluminal_b200",
           "-Wl,-rpath," + os.path.dirname(lib), "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr

    def dump(g, path):
        nl = M.flatten_graph(g)
        ops, in_off, in_node, shape_off, shape, arg_off, arg = nl.keep
        n_in, n_shape, n_arg = int(in_off[-1]), int(shape_off[-1]), int(arg_off[-1])
        with open(path, "wb") as f:
            f.write(np.array([len(ops), n_in, n_shape, n_arg], np.int32).tobytes())
            for a, count in ((ops, len(ops)), (in_off, len(ops) + 1), (in_node, n_in), (shape_off, len(ops) + 1), (shape, n_shape),
                             (arg_off, len(ops) + 1), (arg, n_arg)):
                f.write(a[:count].tobytes())

    def run(path, kind, out_id):
        return subprocess.run([exe, path, kind, str(out_id)], capture_output=True, text=True, timeout=60)

    g, reg = G.Graph(), {}
    model = nn.Llama(g, reg, vocab_size=64, hidden=32, n_layers=2, n_heads=4, n_kv_heads=2, intermediate=48)
    tok = G.tensor(g, [2, 3])
    out = model(tok, 0)
    path = str(tmp_path / "llama.bin")
    dump(g, path)
    r = run(path, "decoder", out.id)
    assert r.returncode == 0, r.stderr
    got, m = json.loads(r.stdout), M.match_decoder(g, out.id)
    assert (got["n_layers"], got["hidden"], got["n_heads"], got["n_kv_heads"], got["intermediate"], got["vocab"]) == (2, 32, 4, 2, 48, 64)
    assert (got["batch"], got["seq"], got["prev_seq"], got["tokens"]) == (2, 3, 0, tok.id)
    assert got["nodes"] == list(m.weights.values()) and got["first_name"] == next(iter(m.weights))
    assert run(path, "step", out.id).returncode == 3 and run(path, "encoder", out.id).returncode == 3      # LMB200_ENOMATCH
    r = run(path, "decoder", out.id - 1)
    assert r.returncode == 3 and "node" in r.stderr

    g, reg = G.Graph(), {}
    td = WG.TextDecoder(g, reg, d_model=32, heads=2, layers=2, ffn=48, vocab=50, max_positions=12)
    idg = WG.build_decode_step(td, g, 7, 3, batch=2)
    path = str(tmp_path / "step.bin")
    dump(g, path)
    r = run(path, "step", idg.logits_id)
    assert r.returncode == 0, r.stderr
    got, m = json.loads(r.stdout), M.match_whisper_step(g, idg.logits_id)
    assert (got["arch"], got["n_layers"], got["hidden"], got["n_heads"], got["vocab"], got["prev_seq"]) == (1, 2, 32, 2, 50, 3)
    assert got["nodes"] == list(m.weights.values())

    g, reg = G.Graph(), {}
    enc = WG.AudioEncoder(g, reg, d_model=32, heads=2, layers=2, ffn=48, n_mels=8)
    mel = G.tensor(g, [2, 8, 21])
    out = enc(mel)
    path = str(tmp_path / "enc.bin")
    dump(g, path)
    r = run(path, "encoder", out.id)
    assert r.returncode == 0, r.stderr
    got, m = json.loads(r.stdout), M.match_whisper_encoder(g, out.id)
    assert (got["d_model"], got["heads"], got["layers"], got["ffn"], got["n_mels"], got["batch"], got["frames"], got["mel"]) == (
        32, 2, 2, 48, 8, 2, 21, mel.id)
    assert got["nodes"] == list(m.weights.values()) and got["first_name"] == "model.encoder.conv1.weight"

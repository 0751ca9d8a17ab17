"""Safetensors ingest (the reference's load_weights!, src/Weights.jl:60-114): the file format on the
CPU, and on the GPU a model filled from a file against the same model filled from arrays."""
import json
import struct

import numpy as np
import pytest

import luminal_oracle as O


def test_safetensors_roundtrip_f32_and_bf16(tmp_path, lib_built):
    W = lib_built.weights
    rng = np.random.default_rng(0)
    tensors = {"a.weight": rng.standard_normal((5, 7), dtype=np.float32), "b": rng.standard_normal((3,), dtype=np.float32),
               "scalar": np.float32(2.5).reshape(())}
    W.write_safetensors(tmp_path / "m.safetensors", tensors)
    back = W.read_safetensors(tmp_path / "m.safetensors")
    assert set(back) == set(tensors)
    for k in tensors:
        assert back[k].shape == tensors[k].shape and np.array_equal(back[k], tensors[k])
    W.write_safetensors(tmp_path / "h.safetensors", tensors, dtype="BF16")
    back = W.read_safetensors(tmp_path / "h.safetensors")
    for k in tensors:
        assert np.array_equal(back[k], O.bf16_round(tensors[k]))


def test_safetensors_header_layout_and_errors(tmp_path, lib_built):
    W = lib_built.weights
    # the layout the reference's own test writes: 8-byte length, JSON, raw row-major data
    data = np.arange(6, dtype="<f4").reshape(2, 3)
    header = json.dumps({"__metadata__": {"format": "pt"},
                         "w": {"dtype": "F32", "shape": [2, 3], "data_offsets": [0, 24]}}).encode()
    path = tmp_path / "raw.safetensors"
    path.write_bytes(struct.pack("<Q", len(header)) + header + data.tobytes())
    got = W.read_safetensors(path)
    assert list(got) == ["w"] and np.array_equal(got["w"], data)
    bad = json.dumps({"w": {"dtype": "F32", "shape": [2, 3], "data_offsets": [0, 20]}}).encode()
    path.write_bytes(struct.pack("<Q", len(bad)) + bad + data.tobytes())
    with pytest.raises(ValueError):
        W.read_safetensors(path)
    with pytest.raises(FileNotFoundError):
        W.load_safetensors(None, str(tmp_path / "missing"))


@pytest.mark.gpu
def test_model_from_safetensors_shards_matches_arrays(tmp_path, lib_built, device):
    L = lib_built
    cfg = O.CONFIGS["small_llama"]
    w = O.synth_llama_weights(cfg, seed=3)
    names = sorted(w)
    L.weights.write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {k: w[k] for k in names[: len(names) // 2]})
    L.weights.write_safetensors(tmp_path / "model-00002-of-00002.safetensors",
                                dict({k: w[k] for k in names[len(names) // 2:]}, **{"rotary.inv_freq": np.ones(4, np.float32)}))
    kw = dict(n_layers=cfg["n_layers"], hidden=cfg["hidden"], n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"],
              intermediate=cfg["intermediate"], vocab=cfg["vocab"], eps=cfg["eps"], rope_base=cfg["rope_base"], dtype="f32")
    a, b = L.Model(device, **kw), L.Model(device, **kw)
    a.set_weights(w)
    loaded, skipped = L.weights.load_safetensors(b, str(tmp_path))
    assert sorted(loaded) == names and skipped == ["rotary.inv_freq"]
    prompt = O.synth_tokens(3, 1, (2, 9), cfg["vocab"]).astype(np.int32)
    sa, sb = L.Session(a, 2, 32), L.Session(b, 2, 32)
    assert np.array_equal(sa.prefill(prompt), sb.prefill(prompt))
    for s in (sa, sb):
        s.close()
    a.close(); b.close()


class _FakeModel:
    """Host-only stand-in for Model: knows two tensors, refuses a wrong shape like the library does."""
    def __init__(self, L):
        self.L, self.shapes, self.got = L, {"a.weight": (4, 8), "b.weight": (8,)}, {}

    def set_weight(self, name, array):
        if name not in self.shapes:
            raise self.L.LuminalB200Error(-7, f"set_weight: unknown tensor '{name}'")
        if tuple(array.shape) != self.shapes[name]:
            raise self.L.LuminalB200Error(-1, f"set_weight: '{name}' has shape {array.shape}")
        self.got[name] = array

    def missing_weights(self):
        return [n for n in self.shapes if n not in self.got]


def test_loader_skips_unknown_names_only_and_reports_missing(tmp_path, lib_built):
    """Only 'the model has no such tensor' is a skip; a wrong shape is an error, and model tensors
    that no file provided are warned about (load_weights!, src/Weights.jl:86-91)."""
    L = lib_built
    W = L.weights
    good = tmp_path / "good.safetensors"
    W.write_safetensors(good, {"a.weight": np.ones((4, 8), np.float32), "extra": np.ones(3, np.float32)})
    m = _FakeModel(L)
    with pytest.warns(UserWarning, match="b.weight"):
        loaded, skipped = W.load_safetensors(m, str(good))
    assert loaded == ["a.weight"] and skipped == ["extra"]
    bad = tmp_path / "bad.safetensors"
    W.write_safetensors(bad, {"a.weight": np.ones((4, 4), np.float32)})
    with pytest.raises(L.LuminalB200Error, match="shape"):
        W.load_safetensors(_FakeModel(L), str(bad))


@pytest.mark.gpu
def test_wrong_shaped_tensor_is_refused(lib_built, device):
    """A checkpoint of another width under a known name must not be read past its end."""
    L = lib_built
    cfg = O.CONFIGS["small_llama"]
    m = L.Model(device, n_layers=cfg["n_layers"], hidden=cfg["hidden"], n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"],
                intermediate=cfg["intermediate"], vocab=cfg["vocab"], eps=cfg["eps"], rope_base=cfg["rope_base"], dtype="f32")
    hid = cfg["hidden"]
    with pytest.raises(L.LuminalB200Error, match=r"expects \[256, 256\]") as e:
        m.set_weight("model.layers.0.self_attn.q_proj.weight", np.zeros((hid // 2, hid), np.float32))
    assert e.value.code == -1
    with pytest.raises(L.LuminalB200Error, match="expects") as e:
        m.set_weight("model.norm.weight", np.zeros(hid + 1, np.float32))
    assert e.value.code == -1
    with pytest.raises(L.LuminalB200Error) as e:
        m.set_weight("model.layers.0.no_such.weight", np.zeros(4, np.float32))
    assert e.value.code == -7
    n_expected = 3 + 9 * cfg["n_layers"]
    assert len(m.missing_weights()) == n_expected
    m.set_weight("model.norm.weight", np.ones(hid, np.float32))
    assert len(m.missing_weights()) == n_expected - 1 and "model.norm.weight" not in m.missing_weights()
    m.init_random(1, 0.02)
    assert m.missing_weights() == []
    m.close()


# ----------------------------------------------------------------------------------------------------------------
# tests/test_weight_loading.jl restated: the registry, the names the Whisper builders register, load_weights!
# ----------------------------------------------------------------------------------------------------------------
TINY = dict(d_model=384, heads=6, layers=4, ffn=1536)


def test_weight_registry_basic(lib_built):                   # tests/test_weight_loading.jl:5-15
    L = lib_built
    g, reg = L.Graph(), L.weights.WeightRegistry()
    t = L.tensor(g, [4, 4])
    assert L.weights.register_weight(reg, "layer.weight", t) is t
    assert len(reg.mapping) == 1 and reg.mapping["layer.weight"] == t.id


def test_whisper_registries(lib_built):                      # tests/test_weight_loading.jl:17-71
    L = lib_built
    WG = L.whisper
    g, reg = L.Graph(), L.weights.WeightRegistry()
    WG.AudioEncoder(g, reg, n_mels=80, reference_names=True, **TINY)
    keys = list(reg.mapping)
    for part in ("conv1.weight", "conv2.weight", "layer_norm.weight", "layers.0", "layers.0.attn.q_proj.weight", "layers.0.mlp.fc1.weight"):
        assert any(part in k for k in keys), part
    n_enc = len(keys)
    WG.TextDecoder(g, reg, vocab=51864, max_positions=448, **TINY)
    keys = list(reg.mapping)
    for part in ("embed_tokens.weight", "embed_positions.weight", "layers.0.self_attn.q_proj.weight", "layers.0.encoder_attn.q_proj.weight",
                 "layer_norm.weight"):
        assert any(part in k for k in keys), part
    enc_keys = [k for k in keys if k.startswith("model.encoder")]
    dec_keys = [k for k in keys if k.startswith("model.decoder")]
    assert len(enc_keys) == n_enc > 0 and len(dec_keys) > 0 and len(keys) > 50
    # the same encoder under the checkpoint's spelling: one canonical name per reference name, and nothing else differs
    g2, reg2 = L.Graph(), {}
    WG.AudioEncoder(g2, reg2, n_mels=80, **TINY)
    assert sorted(WG.canonical_name(k) for k in enc_keys) == sorted(reg2)
    assert WG.canonical_name("model.decoder.layers.0.self_attn.q_proj.weight") == "model.decoder.layers.0.self_attn.q_proj.weight"


def test_load_weights_into_the_graph(tmp_path, lib_built):   # tests/test_weight_loading.jl:73-115
    L = lib_built
    g, reg = L.Graph(), L.weights.WeightRegistry()
    lin = L.nn.Linear(4, 8, g, bias=False)
    L.weights.register_weight(reg, "test.weight", lin.weight)
    dummy = np.arange(1, 33, dtype=np.float32).reshape(8, 4)       # row-major [8, 4], as the file stores it
    path = str(tmp_path / "dummy.safetensors")
    L.weights.write_safetensors(path, {"test.weight": dummy, "not.registered": np.zeros(3, np.float32)})
    assert L.weights.load_weights(g, reg, path) == []
    loaded = g.tensors[(lin.weight.id, 1)]                          # @test haskey(g.tensors, (l.weight.id, 1))
    assert loaded.size == 32 and np.array_equal(loaded, dummy)
    # from a dict, from a directory of shards, a missing key (warned about), a wrong shape (refused)
    g2, reg2 = L.Graph(), {}
    a, b = L.tensor(g2, [2, 3]), L.tensor(g2, [5])
    reg2["a"], reg2["b"] = a, b
    with pytest.warns(UserWarning, match="Missing weights: 1 of 2"):
        assert L.weights.load_weights(g2, reg2, {"a": np.ones((2, 3))}) == ["b"]
    shard_dir = tmp_path / "shards"
    shard_dir.mkdir()
    L.weights.write_safetensors(str(shard_dir / "model-00001.safetensors"), {"a": np.full((2, 3), 2.0, np.float32)})
    L.weights.write_safetensors(str(shard_dir / "model-00002.safetensors"), {"b": np.arange(5, dtype=np.float32)}, dtype="BF16")
    assert L.weights.load_weights(g2, reg2, str(shard_dir)) == []
    assert np.array_equal(g2.tensors[(a.id, 1)], np.full((2, 3), 2.0, np.float32)) and np.array_equal(g2.tensors[(b.id, 1)], np.arange(5))
    with pytest.raises(ValueError, match="shape"):
        L.weights.load_weights(g2, reg2, {"a": np.ones((3, 2))})
    with pytest.raises(FileNotFoundError):
        L.weights.load_weights(g2, reg2, str(tmp_path / "nothing"))


@pytest.mark.gpu
def test_fused_encoder_takes_the_reference_spelling(lib_built, device):
    """The tensor-core encoder fed under the names the reference's encoder blocks register (attn.*, attn_layer_norm.*,
    mlp.fc1.*, mlp.fc2.*) gives the output it gives under the checkpoint's names; so does the compiled graph whose
    weights load_weights placed by those names."""
    import luminal_oracle as O
    import whisper_oracle as W
    L = lib_built
    WG, M = L.whisper, L.match
    cfg = W.CONFIGS["whisper_test"]
    w = W.synth_weights(cfg, seed=31)
    kw = dict(d_model=cfg["d_model"], heads=cfg["heads"], ffn=cfg["ffn"], n_mels=cfg["n_mels"])
    g, reg = L.Graph(), L.weights.WeightRegistry()
    enc = WG.AudioEncoder(g, reg, layers=cfg["enc_layers"], reference_names=True, **kw)
    mel = L.tensor(g, [2, cfg["n_mels"], 40])
    out = enc(mel)
    by_reference_name = {name: w[WG.canonical_name(name)] for name in reg}
    assert any(".attn." in n for n in by_reference_name) and not any("self_attn" in n for n in by_reference_name)
    x = O.synth_normal(31, 5, (2, cfg["n_mels"], 40), 1.0)
    a = WG.FusedEncoder(device, enc_layers=cfg["enc_layers"], dec_layers=0, **kw)
    b = WG.FusedEncoder(device, enc_layers=cfg["enc_layers"], dec_layers=0, **kw)
    assert len(a.set_weights(by_reference_name)) == len(by_reference_name)
    b.set_weights({k: v for k, v in w.items() if k.startswith("model.encoder.")})
    want = b.run(x)
    assert np.array_equal(a.run(x), want)
    assert L.weights.load_weights(g, reg, by_reference_name) == []
    c, m = M.compile_encoder_b200(g, out.id, device=device)
    assert np.array_equal(c.run(x), want)
    a.close(); b.close(); c.close()


def test_phi3_weight_loading(lib_built):                     # tests/test_phi3_loading.jl
    L = lib_built
    g, reg = L.Graph(), L.weights.WeightRegistry()
    L.nn.Phi3(g, reg, vocab_size=100, hidden=64, n_layers=1, n_heads=4, n_kv_heads=1, intermediate=128)
    for key in ("model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.weight", "model.layers.0.mlp.gate_proj.weight",
                "model.norm.weight", "lm_head.weight"):
        assert key in reg.mapping
    tensors = {key: O.synth_normal(9, node_id, g.shapes[node_id - 1], 1.0) for key, node_id in reg.mapping.items()}
    assert L.weights.load_weights(g, reg, tensors) == []
    for key, node_id in reg.mapping.items():
        data = g.tensors[(node_id, 1)]
        assert data.shape == tuple(g.shapes[node_id - 1]) and not np.isnan(data).any()
    # with a forward pass traced, the graph carries everything the node-list compiler asks for: the matcher's weight
    # roles are the registry
    g2, reg2 = L.Graph(), L.weights.WeightRegistry()
    model = L.nn.Phi3(g2, reg2, vocab_size=100, hidden=64, n_layers=1, n_heads=4, n_kv_heads=1, intermediate=128)
    out = model(L.tensor(g2, [1, 4]), 0)
    L.weights.load_weights(g2, reg2, tensors)
    m = L.match_decoder(g2, out.id)
    assert m.weights == dict(reg2.mapping) and all((node_id, 1) in g2.tensors for node_id in m.weights.values())
    assert m.rope_base == 10000.0


def test_conv_weight_from_a_checkpoint(lib_built):
    """A checkpoint stores a Conv1D weight as [ch_out, ch_in, kernel]; NN.Conv1D multiplies by [ch_out, ch_in * kernel]
    with column c + ch_in * k.  The converted matrix in the oracle's Conv1D gives the plain convolution."""
    import whisper_oracle as W
    L = lib_built
    rng = np.random.default_rng(3)
    ch_out, ch_in, kernel, length = 5, 4, 3, 11
    w3 = rng.standard_normal((ch_out, ch_in, kernel)).astype(np.float32)
    bias = rng.standard_normal(ch_out).astype(np.float32)
    x = rng.standard_normal((2, ch_in, length)).astype(np.float32)
    for stride in (1, 2):
        got = W.conv1d(x, L.whisper.conv_weight_from_checkpoint(w3), bias, kernel, stride, 1)
        xp = np.pad(x, ((0, 0), (0, 0), (1, 1)))
        n_out = (length + 2 - kernel) // stride + 1
        want = np.stack([np.einsum("bck,ock->bo", xp[:, :, o * stride:o * stride + kernel], w3) for o in range(n_out)], axis=2) + bias[None, :, None]
        assert got.shape == want.shape and np.allclose(got, want, atol=1e-5)
    w2 = L.whisper.conv_weight_from_checkpoint(w3)
    assert L.whisper.conv_weight_from_checkpoint(w2) is not None and np.array_equal(L.whisper.conv_weight_from_checkpoint(w2), w2)
    # load_weights places a checkpoint-shaped conv weight into the 2-D node
    g, reg = L.Graph(), L.weights.WeightRegistry()
    conv = L.whisper.Conv1D(ch_in, ch_out, kernel, g, reg, "model.encoder.conv1", stride=1, padding=1)
    assert L.weights.load_weights(g, reg, {"model.encoder.conv1.weight": w3, "model.encoder.conv1.bias": bias}) == []
    assert np.array_equal(g.tensors[(conv.weight.id, 1)], w2)


def test_fused_encoder_set_weights_host_logic(lib_built):
    """FusedEncoder.set_weights against a stand-in library: names outside the encoder are left out, a checkpoint-shaped
    conv weight goes down as the 2-D matrix, a name the encoder does not have (LMB200_ENOTFOUND) is skipped, any other
    failure is raised."""
    import ctypes as C
    L = lib_built
    _lib = L._lib

    class FakeLib:
        LuminalB200Error = _lib.LuminalB200Error
        dims = staticmethod(_lib.dims)

        def __init__(self):
            self.seen = {}

        def call(self, fn, handle, name, ptr, ndim, dims, layout):
            n = name.decode()
            if "decoder" in n:
                raise _lib.LuminalB200Error(-7, "unknown tensor")
            if "bad" in n:
                raise _lib.LuminalB200Error(-1, "shape")
            self.seen[n] = [dims[i] for i in range(ndim)]

    enc = L.whisper.FusedEncoder.__new__(L.whisper.FusedEncoder)
    enc._lib, enc._C, enc.handle = FakeLib(), C, None
    used = enc.set_weights({"model.encoder.conv1.bias": np.zeros(3), "model.encoder.conv1.weight": np.zeros((5, 4, 3)),
                            "model.encoder.layers.0.attn.q_proj.weight": np.zeros((4, 4), np.float64),
                            "model.decoder.layers.0.encoder_attn.k_proj.weight": np.zeros((2, 2)), "lm_head.weight": np.zeros(2)})
    assert used == ["model.encoder.conv1.bias", "model.encoder.conv1.weight", "model.encoder.layers.0.attn.q_proj.weight"]
    assert enc._lib.seen["model.encoder.conv1.weight"] == [5, 12]
    with pytest.raises(_lib.LuminalB200Error):
        enc.set_weights({"model.encoder.bad": np.zeros(3)})

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

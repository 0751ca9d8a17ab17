"""Safetensors ingest for the fused session: the stand-in for load_weights! (src/Weights.jl:60-114),
which fills the graph's weight nodes from a `.safetensors` file or a directory of shards by registry
name.  Here the tensors go straight to the model's device shards through set_weight (the same
HuggingFace names the registry uses, src/NN.jl:180-225); tensors the model does not know are skipped,
as the reference skips tensors that are not registered.

File format: 8-byte little-endian header length, a JSON header {name: {dtype, shape, data_offsets}},
then the raw row-major tensors (the layout tests/test_weight_loading.jl:82-104 of the reference writes)."""
from __future__ import annotations

import json
import os
import struct

import numpy as np

from ._lib import LuminalB200Error

_DTYPES = {"F32": (np.float32, 4), "F16": (np.float16, 2), "BF16": (np.uint16, 2), "F64": (np.float64, 8)}


def _to_f32(raw, dtype):
    if dtype == "BF16":
        return (raw.astype(np.uint32) << np.uint32(16)).view(np.float32)
    return raw.astype(np.float32)


def read_safetensors(path):
    """name -> float32 array of every tensor in one file (F32, F16, BF16 or F64 on disk)."""
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen).decode("utf-8"))
        base = 8 + hlen
        out = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            if info["dtype"] not in _DTYPES:
                raise ValueError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
            np_dt, esz = _DTYPES[info["dtype"]]
            lo, hi = info["data_offsets"]
            shape = tuple(int(s) for s in info["shape"])
            count = int(np.prod(shape)) if shape else 1
            if hi - lo != count * esz:
                raise ValueError(f"{path}: tensor {name}: {hi - lo} bytes for shape {shape}")
            f.seek(base + lo)
            raw = np.frombuffer(f.read(hi - lo), dtype=np.dtype(np_dt).newbyteorder("<"))
            out[name] = _to_f32(raw, info["dtype"]).reshape(shape)
        return out


def write_safetensors(path, tensors, dtype="F32"):
    """Writes float arrays as F32 or BF16 (round to nearest even); used by the tests and for export."""
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        shape = list(np.shape(a))
        a = np.ascontiguousarray(np.asarray(a, dtype=np.float32)).reshape(-1)
        if dtype == "BF16":
            u = a.view(np.uint32).astype(np.uint64)
            blob = (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype("<u2").tobytes()
        else:
            blob = a.astype("<f4").tobytes()
        header[name] = {"dtype": dtype, "shape": shape, "data_offsets": [off, off + len(blob)]}
        off += len(blob)
        blobs.append(blob)
    hj = json.dumps(header).encode("utf-8")
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def _files(path):
    if os.path.isdir(path):
        return sorted(os.path.join(path, n) for n in os.listdir(path) if n.endswith(".safetensors"))
    return [path] if os.path.exists(path) else []


ENOTFOUND = -7          # LMB200_ENOTFOUND: the model has no tensor of that name


def load_safetensors(model, path, warn_missing=True):
    """Sets every tensor of the file (or of the shards in the directory) that the model knows.
    Returns (loaded names, skipped names).  Only names the model does not have are skipped; a tensor
    of the wrong shape, a CUDA error or any other failure is raised.  Model tensors that no file
    provided are reported with a warning, as load_weights! does for missing keys
    (src/Weights.jl:86-91); `model.missing_weights()` returns them."""
    files = _files(path)
    if not files:
        raise FileNotFoundError(f"No safetensors files found at: {path}")
    loaded, skipped = [], []
    for file in files:
        for name, a in read_safetensors(file).items():
            try:
                model.set_weight(name, a)
                loaded.append(name)
            except LuminalB200Error as e:
                if e.code != ENOTFOUND:
                    raise
                skipped.append(name)
    if warn_missing and hasattr(model, "missing_weights"):
        missing = model.missing_weights()
        if missing:
            import warnings
            warnings.warn(f"{len(missing)} model tensors were not found in {path}: " + ", ".join(missing[:8]) +
                          (" ..." if len(missing) > 8 else ""), stacklevel=2)
    return loaded, skipped


class WeightRegistry(dict):
    """WeightRegistry of src/Weights.jl:28-42: registry name -> graph node id.  The graph builders of this package
    take any dict and store the GraphTensor itself; this class stores ids, as the reference's `mapping` does, and
    accepts either when written to."""

    def __setitem__(self, name, t):
        super().__setitem__(str(name), int(getattr(t, "id", t)))

    @property
    def mapping(self):
        return self


def register_weight(reg, name, t):            # register_weight!, src/Weights.jl:38-42
    reg[name] = t
    return t


def load_weights(graph, reg, source, device=None):
    """load_weights!(graph, reg, path | tensors) of src/Weights.jl:60-114: every tensor of the `.safetensors` file, of
    the shards of a directory, or of a dict of arrays whose name is registered goes, as float32, into
    graph.tensors[(node id, 1)] -- where execute(), compile() and the node-list compilers look for weights; other
    tensors are ignored.  With a device the arrays are uploaded (to_device), otherwise they stay on the host and are
    uploaded by whoever runs the graph.  Registered names no source provided are warned about and returned."""
    ids = {name: int(getattr(t, "id", t)) for name, t in reg.items()}
    if isinstance(source, dict):
        sources = [source]
    else:
        files = _files(source)
        if not files:
            raise FileNotFoundError(f"No safetensors files found at: {source}")
        sources = (read_safetensors(f) for f in files)
    for tensors in sources:
        for name, node_id in ids.items():
            if name in tensors:
                a = np.ascontiguousarray(np.asarray(tensors[name], dtype=np.float32))
                want = tuple(graph.shapes[node_id - 1])
                if a.ndim == 3 and len(want) == 2 and a.shape[0] == want[0] and a.shape[1] * a.shape[2] == want[1]:
                    from .whisper import conv_weight_from_checkpoint      # a checkpoint's [out, in, kernel] Conv1D weight
                    a = conv_weight_from_checkpoint(a)
                if a.shape != want:
                    raise ValueError(f"{name}: tensor of shape {a.shape}, node {node_id} of shape {want}")
                graph.tensors[(node_id, 1)] = device.upload(a) if device is not None else a
    missing = [name for name, node_id in ids.items() if (node_id, 1) not in graph.tensors]
    if missing:
        import warnings
        warnings.warn(f"Missing weights: {len(missing)} of {len(ids)} registered tensors: " + ", ".join(sorted(missing)[:8]) +
                      (" ..." if len(missing) > 8 else ""), stacklevel=2)
    return missing


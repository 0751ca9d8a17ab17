"""The B200 device: the counterpart of the reference's device structs and of
to_device / from_device (src/Device.jl:9-16, 82-105) for `libluminal_b200.so`."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import BF16, COLMAJOR, F32, ROWMAJOR, LuminalB200Error


class DeviceArray:
    """A row-major tensor in B200 HBM (what a CuArray is to the reference)."""

    def __init__(self, device, ptr, shape, dtype=F32, owned=True):
        self.device, self.ptr, self.shape, self.dtype, self._owned = device, ptr, tuple(int(s) for s in shape), dtype, owned

    @property
    def size(self):
        return int(np.prod(self.shape)) if self.shape else 1

    def numpy(self, layout=ROWMAJOR):
        """from_device: float32 NumPy array of the logical shape."""
        out = np.empty(self.shape, dtype=np.float32, order="F" if layout == COLMAJOR else "C")
        _lib.call("lmb200_download", self.device.handle, out.ctypes.data_as(C.c_void_p), C.c_void_p(self.ptr),
                  self.dtype, len(self.shape), _lib.dims(self.shape), layout)
        return out

    def free(self):
        if self._owned and self.ptr:
            ptr, self.ptr = self.ptr, 0
            if getattr(self.device, "recording", False):
                self.device.deferred_free.append(ptr)          # a free waits for the stream: not while calls are recorded
            else:
                _lib.call("lmb200_free", self.device.handle, C.c_void_p(ptr))

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class B200Device:
    """One context on one GPU.  Fails loudly when there is no sm_100 GPU or no built library."""

    def __init__(self, ordinal=0, stream=None):
        h = C.c_uint64(0)
        _lib.call("lmb200_init", int(ordinal), C.byref(h))
        self.handle = h
        self.ordinal = int(ordinal)
        self.recording, self.deferred_free = False, []     # see capture()
        if stream is not None:
            self.set_stream(stream)

    def set_stream(self, cuda_stream_ptr):
        _lib.call("lmb200_set_stream", self.handle, C.c_void_p(int(cuda_stream_ptr or 0)))

    def sync(self):
        _lib.call("lmb200_sync", self.handle)

    def launch_count(self):
        n = C.c_int64(0)
        _lib.call("lmb200_launch_count", self.handle, C.byref(n))
        return n.value

    def alloc(self, nbytes):
        p = C.c_void_p(0)
        _lib.call("lmb200_alloc", self.handle, int(nbytes), C.byref(p))
        return p.value

    def empty(self, shape, dtype=F32):
        n = int(np.prod(shape)) if len(shape) else 1
        return DeviceArray(self, self.alloc(n * (2 if dtype == BF16 else 4)), shape, dtype)

    def upload(self, array, dtype=F32, layout=ROWMAJOR):
        """to_device: `array` holds the logical tensor; with layout=COLMAJOR its memory image is
        Julia's (column-major) and the library re-lays it out."""
        a = np.asarray(array, dtype=np.float32)
        host = np.asfortranarray(a) if layout == COLMAJOR else np.ascontiguousarray(a)
        out = self.empty(a.shape, dtype)
        _lib.call("lmb200_upload", self.handle, C.c_void_p(out.ptr), dtype, host.ctypes.data_as(C.c_void_p),
                  a.ndim, _lib.dims(a.shape), layout)
        return out

    # CUDA-graph capture of op-level calls
    def capture(self, f):
        """Records the op-level calls f() makes into a CUDA graph (nothing runs) and returns its handle."""
        _lib.call("lmb200_capture_begin", self.handle)
        self.recording = True
        h = C.c_uint64(0)
        try:
            try:
                f()
            except BaseException:
                try:
                    _lib.call("lmb200_capture_end", self.handle, C.byref(h))
                except _lib.LuminalB200Error:
                    pass
                else:
                    _lib.call("lmb200_graph_destroy", self.handle, h)
                raise
            _lib.call("lmb200_capture_end", self.handle, C.byref(h))
        finally:
            self.recording = False
            while self.deferred_free:                              # arrays collected while the calls were recorded
                _lib.call("lmb200_free", self.handle, C.c_void_p(self.deferred_free.pop()))
        return h

    def graph_launch(self, graph):
        _lib.call("lmb200_graph_launch", self.handle, graph)

    def graph_destroy(self, graph):
        _lib.call("lmb200_graph_destroy", self.handle, graph)

    # tensor-parallel communicator (one rank per process)
    @staticmethod
    def comm_unique_id():
        buf = (C.c_uint8 * 128)()
        _lib.call("lmb200_comm_unique_id", buf)
        return bytes(buf)

    def comm_init(self, n_ranks, rank, unique_id):
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        _lib.call("lmb200_comm_init", self.handle, int(n_ranks), int(rank), buf)

    def comm_destroy(self):
        _lib.call("lmb200_comm_destroy", self.handle)

    def comm_resync(self):
        """Collective, after a tensor-parallel call failed with LMB200_ETIMEOUT: brings the ranks back in step."""
        _lib.call("lmb200_comm_resync", self.handle)

    def close(self):
        if self.handle:
            _lib.call("lmb200_shutdown", self.handle)
            self.handle = C.c_uint64(0)


def device_count():
    n = C.c_int32(0)
    _lib.call("lmb200_device_count", C.byref(n))
    return n.value


_default = None


def get_device():
    """get_device() of src/Device.jl:27-74 for this backend: the B200 or an error, never a CPU
    fallback."""
    global _default
    if _default is None:
        _default = B200Device(0)
    return _default


def to_device(data, device):
    if isinstance(data, dict):
        return {k: to_device(v, device) for k, v in data.items()}
    if isinstance(data, DeviceArray):
        return data
    return device.upload(np.asarray(data, dtype=np.float32))


def from_device(data):
    return data.numpy() if isinstance(data, DeviceArray) else data


def execute_with_capture(device, f, cache):
    """execute_with_capture(device, f, cache) of src/Device.jl:106-121: runs f() on the device; "if supported, it
    captures the execution into a graph stored in cache and replays it on subsequent calls".  The first call runs f()
    as it is (kernels that size a scratch buffer on first use do so here) and then records it; every later call is one
    replay of cache["cuda_exec"].  If f() makes a call that cannot be recorded, cache["cuda_exec"] is None, the reason
    is kept in cache["cuda_exec_error"], and f() keeps running call by call."""
    graph = cache.get("cuda_exec")
    if graph is not None:
        device.graph_launch(graph)
        return
    f()
    if "cuda_exec" not in cache:
        try:
            cache["cuda_exec"] = device.capture(f)
        except _lib.LuminalB200Error as e:
            cache["cuda_exec"], cache["cuda_exec_error"] = None, str(e)


__all__ = ["B200Device", "DeviceArray", "get_device", "to_device", "from_device", "execute_with_capture", "device_count",
           "LuminalB200Error", "F32", "BF16", "ROWMAJOR", "COLMAJOR"]

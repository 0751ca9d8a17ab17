"""ctypes binding of libluminal_b200.so: one Python function per entry point of
include/luminal_b200.h, raising `LuminalB200Error` with the library's message on a non-zero
status.  There is no fallback: if the library is missing or a call fails, the caller sees it."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libluminal_b200.so")

F32, BF16, I32 = 0, 1, 2
ROWMAJOR, COLMAJOR = 0, 1

OP = dict(add=0, mul=1, mod=2, less_than=3, max=4, log2=8, exp2=9, sin=10, cos=11, sqrt=12,
          recip=13, relu=14, copy=15, fused_mul_add=16, fused_add_relu=17)
REDUCE_SUM, REDUCE_MAX = 0, 1


class LuminalB200Error(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"libluminal_b200 error {code}: {message}")
        self.code = code
        self.message = message


class ModelConfig(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("hidden", C.c_int32), ("n_heads", C.c_int32),
                ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("intermediate", C.c_int32),
                ("vocab", C.c_int32), ("rms_eps", C.c_float), ("rope_base", C.c_float),
                ("dtype", C.c_int32), ("tp_size", C.c_int32), ("tp_rank", C.c_int32),
                ("arch", C.c_int32), ("max_positions", C.c_int32), ("cross_len", C.c_int32),
                ("reserved", C.c_int32)]


_i32, _i64, _u64, _f32, _vp = C.c_int32, C.c_int64, C.c_uint64, C.c_float, C.c_void_p
_pi64 = C.POINTER(C.c_int64)
_pi32 = C.POINTER(C.c_int32)
_pf32 = C.POINTER(C.c_float)

# name -> argtypes (every function returns int32 except last_error)
SIGNATURES = {
    "lmb200_version": [],
    "lmb200_device_count": [_pi32],
    "lmb200_init": [_i32, C.POINTER(_u64)],
    "lmb200_shutdown": [_u64],
    "lmb200_set_stream": [_u64, _vp],
    "lmb200_sync": [_u64],
    "lmb200_launch_count": [_u64, _pi64],
    "lmb200_capture_begin": [_u64],
    "lmb200_capture_end": [_u64, C.POINTER(_u64)],
    "lmb200_graph_launch": [_u64, _u64],
    "lmb200_graph_destroy": [_u64, _u64],
    "lmb200_comm_unique_id": [C.POINTER(C.c_uint8)],
    "lmb200_comm_init": [_u64, _i32, _i32, C.POINTER(C.c_uint8)],
    "lmb200_comm_destroy": [_u64],
    "lmb200_comm_resync": [_u64],
    "lmb200_allreduce_sum_f32": [_u64, _vp, _i64],
    "lmb200_alloc": [_u64, _i64, C.POINTER(_vp)],
    "lmb200_free": [_u64, _vp],
    "lmb200_upload": [_u64, _vp, _i32, _vp, _i32, _pi64, _i32],
    "lmb200_download": [_u64, _vp, _vp, _i32, _i32, _pi64, _i32],
    "lmb200_ew": [_u64, _i32, _vp, _i32, _pi64, _vp, _i32, _pi64, _vp, _i32, _pi64, _vp, _i32, _pi64],
    "lmb200_fused_ew": [_u64, _vp, _i32, _pi64, _i32, C.POINTER(_vp), _pi32, _pi64, _i32, _pi32, _pf32],
    "lmb200_reduce": [_u64, _i32, _vp, _vp, _i32, _pi64, _i32],
    "lmb200_matmul": [_u64, _vp, _vp, _i32, _pi64, _vp, _i32, _pi64],
    "lmb200_permute": [_u64, _vp, _vp, _i32, _pi64, _pi32],
    "lmb200_reshape_colmajor": [_u64, _vp, _vp, _i32, _pi64, _i32, _pi64],
    "lmb200_expand": [_u64, _vp, _vp, _i32, _pi64, _i32, _i64],
    "lmb200_slice": [_u64, _vp, _vp, _i32, _pi64, _pi64, _pi64],
    "lmb200_pad": [_u64, _vp, _vp, _i32, _pi64, _pi64, _pi64],
    "lmb200_gather": [_u64, _vp, _vp, _i64, _i64, _vp, _i64],
    "lmb200_cumsum_last": [_u64, _vp, _vp, _i64, _i64],
    "lmb200_unfold1d": [_u64, _vp, _vp, _i64, _i64, _i64, _i64, _i64],
    "lmb200_flash_attention": [_u64, _vp, _vp, _vp, _vp, _i32, _i64, _i64, _i64, _i64, _f32, _i32],
    "lmb200_rmsnorm_scale": [_u64, _vp, _vp, _vp, _i64, _i64, _f32],
    "lmb200_layernorm": [_u64, _vp, _vp, _vp, _vp, _i64, _i64, _f32],
    "lmb200_silu_gate": [_u64, _vp, _vp, _vp, _i64],
    "lmb200_rope": [_u64, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _f32],
    "lmb200_argmax": [_u64, _vp, _vp, _i64, _i64],
    "lmb200_linear_gemv": [_u64, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp],
    "lmb200_prefill_gemm": [_u64, _i32, _i32, _i32, _vp, _vp, _vp],
    "lmb200_whisper_encoder_create": [_u64, _i32, _i32, _i32, _i32, _i32, _i32, C.POINTER(_u64)],
    "lmb200_whisper_encoder_destroy": [_u64],
    "lmb200_whisper_encoder_set_weight": [_u64, C.c_char_p, _vp, _i32, _pi64, _i32],
    "lmb200_whisper_canonical_name": [C.c_char_p, C.c_char_p, _i64],
    "lmb200_whisper_encoder_run": [_u64, _vp, _i32, _i32, _vp],
    "lmb200_whisper_encoder_cross_kv": [_u64, _u64],
    "lmb200_model_create": [_u64, C.POINTER(ModelConfig), C.POINTER(_u64)],
    "lmb200_shard_extent": [C.POINTER(ModelConfig), _i32, _pi32, _pi32],
    "lmb200_shard_map": [C.POINTER(ModelConfig), _i32, _i32, _i32, _pi32, _pi32, _pi32],
    "lmb200_model_destroy": [_u64],
    "lmb200_model_set_weight": [_u64, C.c_char_p, _vp, _i32, _pi64, _i32],
    "lmb200_model_missing_weights": [_u64, C.c_char_p, _i64, _pi32],
    "lmb200_model_init_random": [_u64, _u64, _f32],
    "lmb200_model_weight_bytes": [_u64, _pi64],
    "lmb200_session_create": [_u64, _i32, _i32, C.POINTER(_u64)],
    "lmb200_session_destroy": [_u64],
    "lmb200_session_reset": [_u64],
    "lmb200_session_position": [_u64, _pi32],
    "lmb200_session_set_position": [_u64, _i32],
    "lmb200_session_set_positions": [_u64, _pi32],
    "lmb200_session_positions": [_u64, _pi32],
    "lmb200_prefill_ragged": [_u64, _vp, _vp, _i32, _vp],
    "lmb200_session_fill_kv_random": [_u64, _i32, _u64],
    "lmb200_session_set_capture": [_u64, _i32],
    "lmb200_session_read_layer_output": [_u64, _i32, _vp],
    "lmb200_session_set_cross_kv": [_u64, _i32, _vp, _vp, _i32],
    "lmb200_prefill": [_u64, _vp, _i32, _vp],
    "lmb200_decode_step": [_u64, _vp, _vp, _vp],
    "lmb200_decode_n": [_u64, _vp, _i32, _vp],
    "lmb200_decode_until": [_u64, _vp, _i32, _i32, _vp, _pi32],
    "lmb200_decode_n_device": [_u64, _vp, _i32, _vp],
    "lmb200_session_step_bytes": [_u64, _i32, _pi64],
    "lmb200_match_decoder": [_vp, _i32, _vp, _vp, _pi32, _i32, C.c_char_p, _i64],
    "lmb200_match_whisper_step": [_vp, _i32, _vp, _vp, _pi32, _i32, C.c_char_p, _i64, _pi32, _i32],
    "lmb200_match_whisper_encoder": [_vp, _i32, _vp, _pi32, _i32, C.c_char_p, _i64],
    "lmb200_compile_encoder_node_list": [_u64, _vp, _i32, _vp, _i32, C.POINTER(_u64), _vp],
    "lmb200_compile_node_list": [_u64, _vp, _i32, _vp, _i32, _i32, _i32, _i32, C.POINTER(_u64), C.POINTER(_u64), _vp],
    "lmb200_decode_attention_splitkv": [_u64, _i32, _vp, _vp, _i32],
    "lmb200_session_kv_layer": [_u64, _i32, C.POINTER(_vp), _pi64, _pi64],
    "lmb200_decode_attention_noalloc": [_u64, _i32, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _i32, _i32, _i32],
}

_lib = None


def load():
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LuminalB200Error(-1, f"{LIB_PATH} is missing: run `python __graft_entry__.py` "
                                   "(or luminal.jl_b200/_build.py) to build it with nvcc")
    lib = C.CDLL(LIB_PATH)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = C.c_int32
    lib.lmb200_last_error.argtypes = []
    lib.lmb200_last_error.restype = C.c_char_p
    _lib = lib
    return lib


def check(status):
    if status != 0:
        raise LuminalB200Error(status, load().lmb200_last_error().decode("utf-8", "replace"))


def call(name, *args):
    check(getattr(load(), name)(*args))


def dims(shape):
    return (C.c_int64 * max(1, len(shape)))(*shape)

"""luminal.jl_b200 -- host side of the B200 backend for Luminal.jl's transformer decode path.

Everything numeric runs in libluminal_b200.so (hand-written sm_100a CUDA behind a C ABI, see
include/luminal_b200.h).  This package is the Python stand-in for the Julia shim: the same
device / execute / NN vocabulary as the reference, bound with ctypes instead of ccall.  There
is no CPU fallback: without the built library or without a B200 every entry point raises."""
from . import _lib
from ._lib import BF16, COLMAJOR, F32, ROWMAJOR, LuminalB200Error
from .device import B200Device, DeviceArray, device_count, execute_with_capture, from_device, get_device, to_device
from . import graph, match, nn, weights, whisper
from .match import MatchError, compile_b200, compile_encoder_b200, export_graph, import_graph, match_decoder, match_whisper_encoder, match_whisper_step
from .execution import CompiledGraph, compile, compile_fused, execute
from .graph import Graph, GraphTensor, constant, tensor
from .session import Model, Session, WhisperDecoderModel, decode_attention_noalloc, greedy_generate, linear_gemv, prefill_gemm, shard_layout

__all__ = ["Graph", "GraphTensor", "tensor", "constant", "execute", "compile", "compile_fused", "compile_b200", "compile_encoder_b200", "match_decoder", "match_whisper_step", "match_whisper_encoder", "export_graph", "import_graph", "MatchError", "CompiledGraph", "graph", "match", "nn", "weights", "whisper",
           "B200Device", "DeviceArray", "Model", "Session", "WhisperDecoderModel", "greedy_generate", "decode_attention_noalloc", "shard_layout", "linear_gemv", "prefill_gemm", "get_device", "to_device", "execute_with_capture",
           "from_device", "device_count", "LuminalB200Error", "F32", "BF16", "ROWMAJOR", "COLMAJOR"]

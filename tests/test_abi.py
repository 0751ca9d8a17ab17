"""The C-ABI library loads and exports exactly what include/luminal_b200.h declares; the host
mirror binds every symbol; without a GPU the entry points fail with an error, never a fallback."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "luminal_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lmb200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = header_symbols()
    assert "lmb200_decode_step" in syms and "lmb200_flash_attention" in syms and len(syms) >= 45


def test_library_exports_every_declared_symbol(lib_built):
    lib = ctypes.CDLL(os.path.join(ROOT, "luminal.jl_b200", "libluminal_b200.so"))
    missing = [s for s in header_symbols() if not hasattr(lib, s)]
    assert not missing, f"declared but not exported: {missing}"


def test_host_mirror_binds_every_symbol(lib_built):
    from importlib import import_module
    _lib = import_module("luminal_jl_b200._lib")
    bound = set(_lib.SIGNATURES) | {"lmb200_last_error"}
    assert set(header_symbols()) == bound
    assert _lib.load().lmb200_version() >= 100


def test_every_declaration_cites_the_reference_or_says_why_not():
    """Each entry point's comment names the reference code it replaces (file:line) or states that
    the reference has no counterpart."""
    text = open(os.path.join(ROOT, "include", "luminal_b200.h")).read()
    assert len(re.findall(r"src/[A-Za-z]+\.jl:\d+", text)) >= 40
    assert "no counterpart in the reference" in text


def test_no_gpu_means_error_not_fallback(lib_built):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = lib_built
    with pytest.raises(L.LuminalB200Error):
        L.B200Device(0)
    with pytest.raises(L.LuminalB200Error):
        L.device_count()


def test_bad_handles_are_rejected(lib_built):
    from importlib import import_module
    _lib = import_module("luminal_jl_b200._lib")
    lib = _lib.load()
    assert lib.lmb200_sync(ctypes.c_uint64(0)) != 0
    assert b"invalid context" in lib.lmb200_last_error()
    assert lib.lmb200_session_destroy(ctypes.c_uint64(0)) != 0
    assert lib.lmb200_model_destroy(ctypes.c_uint64(0)) != 0

"""The C-ABI library loads and exports exactly what include/sana_b200.h declares; argument
validation returns negative statuses before anything touches a GPU."""
import ctypes as C
import os
import re

import pytest

from sana_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    src = open(os.path.join(ROOT, "include", "sana_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(sana_[a-z0-9_]+)\s*\(", src)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(_lib.SIGNATURES)


def test_every_declared_symbol_is_exported(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert lib.sana_abi_version() == 1


def test_invalid_arguments_are_rejected_on_the_host(lib):
    assert lib.sana_ln_modulate(None, None, None, None, 1, 1, 64, 0, 1, 1e-6, _lib.SANA_BF16, None) == -1
    assert b"null" in lib.sana_last_error()
    assert lib.sana_la_state(None, None, 64, None, None, 0, 1, 16, 2, _lib.SANA_BF16, None) == -1
    assert lib.sana_la_apply(None, 64, None, None, 64, 1, 16, 2, 1e-8, _lib.SANA_BF16, None) == -1
    assert lib.sana_dwconv_glu(None, None, None, None, None, None, 4, 4, 4, 0, 8, _lib.SANA_BF16, None) == -1
    assert lib.sana_gemm(None, 8, None, 8, None, 8, 8, 8, 8, None, _lib.SANA_BF16, None) == -1
    assert lib.sana_gemm_simt(None, 8, None, 8, None, 8, 8, 8, 8, None, _lib.SANA_F32, None) == -1
    # fake but non-null, aligned pointers: shape/stride checks fire before any launch
    p = C.c_void_p(0x1000)
    assert lib.sana_la_state(p, p, 60, p, p, 1 << 30, 1, 16, 2, _lib.SANA_BF16, None) == -1  # ld < H*32
    assert lib.sana_dwconv_glu(p, None, None, p, None, p, 4, 4, 4, 0, 12, _lib.SANA_BF16, None) == -1  # hid % 8
    assert lib.sana_dwconv_glu(p, None, None, p, None, p, 4, 4, 4, 2, 8, _lib.SANA_BF16, None) == -1  # halo needed
    assert b"halo_top" in lib.sana_last_error()
    assert lib.sana_gemm(p, 4, p, 8, p, 8, 8, 8, 8, None, _lib.SANA_BF16, None) == -1  # lda < K
    ep = _lib.GemmEpilogue()
    ep.act = 7
    assert lib.sana_gemm(p, 8, p, 8, p, 8, 8, 8, 8, C.byref(ep), _lib.SANA_BF16, None) == -1
    assert lib.sana_la_state_workspace_bytes(0, 16, 2) == 0
    assert lib.sana_la_state_workspace_bytes(1, 1024, 36) >= 36 * 33 * 32 * 4


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libsana_b200.so")
    with pytest.raises(_lib.SanaLibraryError, match="no CPU or PyTorch fallback"):
        _lib.load()

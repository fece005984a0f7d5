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


def test_invalid_arguments_of_the_newer_entry_points(lib):
    p = C.c_void_p(0x1000)
    assert lib.sana_ln_modulate_rows(p, p, p, p, 1, 4, 64, 2, 0, 2, 1, 0, 0, 1e-6, _lib.SANA_BF16, None) == -1  # table row 2 of 2
    assert b"table row" in lib.sana_last_error()
    assert lib.sana_ln_modulate_rows(p, p, p, p, 1, 4, 64, 2, 0, 1, 1, 0, 1, 1e-6, _lib.SANA_BF16, None) == -1  # row 1 of t [B,1,C]
    assert lib.sana_ln_modulate_rows(p, p, p, p, 1, 4, 60, 2, 0, 1, 1, 0, 0, 1e-6, _lib.SANA_BF16, None) == -1  # C % 8
    assert lib.sana_rope(p, 32, p, p, 1, 4, 64, 32, _lib.SANA_BF16, None) == -1  # ld < C
    assert lib.sana_rope(p, 64, p, p, 1, 4, 64, 24, _lib.SANA_BF16, None) == -1  # C not whole heads
    assert lib.sana_rope(None, 64, p, p, 1, 4, 64, 32, _lib.SANA_BF16, None) == -1
    assert lib.sana_patchify(p, p, 8, 1, 4, 6, 6, 4, _lib.SANA_BF16, None) == -1  # H % p
    assert lib.sana_patchify(p, p, 8, 1, 4, 8, 8, 2, _lib.SANA_BF16, None) == -1  # row stride < Cin*p*p
    assert lib.sana_unpatchify(p, 8, p, 1, 4, 2, 2, 2, _lib.SANA_BF16, None) == -1  # row stride < p*p*Cout
    assert lib.sana_timestep_embedding(p, p, 2, 1, 10000.0, _lib.SANA_F32, None) == -1  # dim < 2
    assert lib.sana_timestep_embedding(p, p, 2, 256, 1.0, _lib.SANA_F32, None) == -1  # max_period
    assert lib.sana_silu(p, p, 0, _lib.SANA_BF16, None) == -1
    assert lib.sana_silu(p, p, 8, 7, None) != 0  # unknown dtype
    assert lib.sana_halo_exchange_buffer_bytes(0) == 0
    assert lib.sana_halo_exchange_buffer_bytes(1792000) == 1024 + 2 * 1792000
    assert lib.sana_halo_exchange(p, p, 100, p, p, p, 1, None) == -1  # row not a multiple of 16 bytes
    assert lib.sana_halo_exchange(None, p, 160, p, p, None, 1, None) == -1  # upper neighbour without a first row
    assert lib.sana_halo_exchange(p, p, 160, None, None, None, 1, None) == -1
    status = C.c_int(7)
    assert lib.sana_dwconv_glu_take_device_status(None) == -1
    ep = _lib.GemmEpilogue()
    ep.act = 3  # GELU (tanh) is a valid activation code ...
    ep.gate_table = 0x1000  # ... but a gate table needs gate_t
    assert lib.sana_gemm(p, 8, p, 8, p, 8, 8, 8, 8, C.byref(ep), _lib.SANA_BF16, None) == -1
    assert b"gate_t" in lib.sana_last_error()


def test_invalid_arguments_of_the_rotated_linear_attention(lib):
    p = C.c_void_p(0x1000)
    bf = _lib.SANA_BF16
    assert lib.sana_la_rope_state_workspace_bytes(1, 64, 2, 40) == 0  # head dimension not a multiple of 16
    assert lib.sana_la_rope_state_workspace_bytes(1, 64, 2, 144) == 0  # wider than 128
    assert lib.sana_la_rope_state_workspace_bytes(0, 64, 2, 112) == 0
    assert lib.sana_la_rope_state_workspace_bytes(1, 4096, 20, 112) >= 20 * 113 * 112 * 4
    assert lib.sana_la_rope_state(None, p, 224, p, p, p, p, 1 << 30, 1, 64, 2, 112, bf, None) == -1
    assert b"null" in lib.sana_last_error()
    assert lib.sana_la_rope_state(p, p, 224, p, p, p, p, 1 << 30, 1, 64, 2, 40, bf, None) == -1
    assert b"head dimension" in lib.sana_last_error()
    assert lib.sana_la_rope_state(p, p, 200, p, p, p, p, 1 << 30, 1, 64, 2, 112, bf, None) == -1  # ld < H*D
    assert lib.sana_la_rope_state(p, p, 224, p, p, p, p, 16, 1, 64, 2, 112, bf, None) == -1  # workspace too small
    assert b"workspace" in lib.sana_last_error()
    assert lib.sana_la_rope_state(p, p, 224, p, p, p, p, 1 << 30, 1, 64, 2, 112, 9, None) == -1  # dtype
    assert lib.sana_la_rope_apply(p, 224, p, p, p, None, 224, 1, 64, 2, 112, 1e-8, bf, None) == -1
    assert lib.sana_la_rope_apply(p, 224, p, p, p, p, 100, 1, 64, 2, 112, 1e-8, bf, None) == -1  # ldo < H*D
    assert lib.sana_la_rope_apply(p, 224, p, p, p, p, 224, 1, 64, 2, 24, 1e-8, bf, None) == -1
    assert lib.sana_la_rope_apply(p, 224, C.c_void_p(0x1004), p, p, p, 224, 1, 64, 2, 112, 1e-8, bf, None) == -1  # alignment
    assert lib.sana_la_rope_take_device_status(None) == -1


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libsana_b200.so")
    with pytest.raises(_lib.SanaLibraryError, match="no CPU or PyTorch fallback"):
        _lib.load()

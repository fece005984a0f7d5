"""ctypes binding of libsana_b200.so (the C ABI declared in include/sana_b200.h).

There is no fallback: if the shared library is missing or a call returns a non-zero status
a ``SanaLibraryError`` is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

PKG = os.path.dirname(os.path.abspath(__file__))
# SANA_B200_LIBRARY names another build of the same library (e.g. one compiled with tuning counters)
LIB_PATH = os.environ.get("SANA_B200_LIBRARY") or os.path.join(PKG, "lib", "libsana_b200.so")

SANA_F32 = 0
SANA_BF16 = 1


class SanaLibraryError(RuntimeError):
    pass


class GemmEpilogue(C.Structure):
    """Mirror of ``struct sana_gemm_epilogue``."""

    _fields_ = [
        ("bias", C.c_void_p),
        ("act", C.c_int32),
        ("gate_row", C.c_int32),
        ("relu_cols", C.c_int64),
        ("gate_table", C.c_void_p),
        ("gate_t", C.c_void_p),
        ("rows_per_batch", C.c_int64),
        ("residual", C.c_void_p),
        ("ldr", C.c_int64),
    ]


_i64, _i32, _f32, _vp = C.c_int64, C.c_int, C.c_float, C.c_void_p

# name -> (restype, argtypes); must list every symbol include/sana_b200.h declares
SIGNATURES = {
    "sana_abi_version": (_i32, []),
    "sana_last_error": (C.c_char_p, []),
    "sana_ln_modulate": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _f32, _i32, _vp]),
    "sana_ln_modulate_rows": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _f32, _i32,
                                     _vp]),
    "sana_rmsnorm": (_i32, [_vp, _i64, _vp, _vp, _i64, _i64, _i64, _f32, _i32, _vp]),
    "sana_rope": (_i32, [_vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp]),
    "sana_la_state_workspace_bytes": (_i64, [_i64, _i64, _i64]),
    "sana_la_state": (_i32, [_vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _vp]),
    "sana_la_state_noalloc": (_i32, [_vp, _vp, _i64, _vp, _i64, _i64, _i64, _i32, _vp]),
    "sana_la_state_sp_buffer_bytes": (_i64, [_i64, _i64]),
    "sana_la_state_sp": (_i32, [_vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _i32, C.POINTER(C.c_void_p), _i32, _i32,
                                C.c_uint32, _vp]),
    "sana_halo_exchange_buffer_bytes": (_i64, [_i64]),
    "sana_halo_exchange": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, C.c_uint32, _vp]),
    "sana_exchange_set_wait_limit_ns": (_i32, [_i64]),
    "sana_la_apply": (_i32, [_vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _f32, _i32, _vp]),
    "sana_la_rope_state_workspace_bytes": (_i64, [_i64, _i64, _i64, _i64]),
    "sana_la_rope_state": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "sana_la_rope_state_sp_buffer_bytes": (_i64, [_i64, _i64, _i64]),
    "sana_la_rope_state_sp": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32,
                                     C.POINTER(C.c_void_p), _i32, _i32, C.c_uint32, _vp]),
    "sana_la_rope_state_add": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "sana_add_f32": (_i32, [_vp, _vp, _vp, _i64, _vp]),
    "sana_la_rope_apply": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _f32, _i32, _vp]),
    "sana_cross_attention": (_i32, [_vp, _i64, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "sana_cross_attention_set_variant": (_i32, [_i32]),
    "sana_cross_attention_take_device_status": (_i32, [C.POINTER(C.c_int)]),
    "sana_dwconv_glu": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "sana_gemm": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, C.POINTER(GemmEpilogue), _i32, _vp]),
    "sana_gemm_simt": (_i32, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _i64, C.POINTER(GemmEpilogue), _i32, _vp]),
    "sana_gemm_take_device_status": (_i32, [C.POINTER(C.c_int)]),
    "sana_la_rope_take_device_status": (_i32, [C.POINTER(C.c_int)]),
    "sana_dwconv_glu_take_device_status": (_i32, [C.POINTER(C.c_int)]),
    "sana_gemm_set_variant": (_i32, [_i32]),
    "sana_nvfp4_sf_bytes": (_i64, [_i64, _i64]),
    "sana_nvfp4_quantize": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _vp]),
    "sana_gemm_nvfp4": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, C.POINTER(GemmEpilogue), _vp]),
    "sana_gemm_nvfp4_take_device_status": (_i32, [C.POINTER(C.c_int)]),
    "sana_nvfp4_scale_roll": (_i32, [_vp, _i64, _f32, _vp]),
    "sana_nvfp4_quantize_scaled": (_i32, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _vp]),
    "sana_ln_modulate_fp4": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _f32, _vp]),
    "sana_la_apply_fp4": (_i32, [_vp, _i64, _vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _vp]),
    "sana_dwconv_glu_amax": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp]),
    "sana_patchify": (_i32, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "sana_unpatchify": (_i32, [_vp, _i64, _vp, _i64, _i64, _i64, _i64, _i64, _i32, _vp]),
    "sana_timestep_embedding": (_i32, [_vp, _vp, _i64, _i64, _f32, _i32, _vp]),
    "sana_silu": (_i32, [_vp, _vp, _i64, _i32, _vp]),
}

_lock = threading.Lock()
_lib = None


def load() -> C.CDLL:
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise SanaLibraryError(
                    f"{LIB_PATH} not found: build it with `python -m sana_b200.build` (needs nvcc). "
                    "There is no CPU or PyTorch fallback for these operators.")
            lib = C.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().sana_last_error().decode("utf-8", "replace")
        raise SanaLibraryError(f"{what} failed with status {status}: {msg}")

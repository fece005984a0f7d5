"""The C-ABI kernels as torch custom operators (namespace ``sana_b200``), with fake (meta)
implementations so that tracing / ``torch.compile`` / fake-tensor propagation see shapes and
dtypes without touching the GPU.

    torch.ops.sana_b200.gemm(a, w, bias, act, relu_cols, gate_table, gate_t, gate_row, rows_per_batch, residual)
    torch.ops.sana_b200.ln_modulate(x, table, t, shift_row, scale_row, eps)
    torch.ops.sana_b200.la_state(k, v, B, N, H)
    torch.ops.sana_b200.la_apply(q, state, B, N, H, eps)
    torch.ops.sana_b200.dwconv_glu(u, weight, bias, W, H, row0, halo_top, halo_bot)
    torch.ops.sana_b200.rmsnorm_(x, weight, eps)          # in place
    torch.ops.sana_b200.rope_(x, cos, sin, B, N, head_dim)  # in place
    torch.ops.sana_b200.cross_attention(q, k, v, mask, B, N, L, heads, head_dim)
    torch.ops.sana_b200.la_rope_state(k, v, cos, sin, B, N, H, D, prior)
    torch.ops.sana_b200.la_rope_apply(q, cos, sin, state, B, N, H, D, eps)
    torch.ops.sana_b200.add_f32(a, b)
    torch.ops.sana_b200.ln_modulate_rows(x, table, t, table_shift_row, table_scale_row, t_shift_row, t_scale_row, eps)
    torch.ops.sana_b200.patchify(x, p) / unpatchify(tok, B, Cout, Hp, Wp, p)
    torch.ops.sana_b200.timestep_embedding(t, dim, dtype, max_period) / silu(x)
    torch.ops.sana_b200.nvfp4_quantize(x) -> (codes, scale_tiles, scales)
    torch.ops.sana_b200.gemm_nvfp4(a_codes, a_sf, a_scales, w_codes, w_sf, w_scales, bias, act, relu_cols,
                                   gate_table, gate_t, gate_row, rows_per_batch, residual)

They are thin: each forwards to :mod:`sana_b200.ops`, which passes raw device pointers and the
current stream to libsana_b200.so.  The modules call :mod:`sana_b200.ops` directly (same
kernels, without the dispatcher's per-call overhead).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops

_lib_ns = "sana_b200"
# the ctypes-level functions, captured before any routing replaces the names in `ops`
_D = {n: getattr(ops, n) for n in ("gemm", "ln_modulate", "ln_modulate_rows", "la_state", "la_apply", "dwconv_glu", "rmsnorm_",
                                   "rope_", "cross_attention", "la_rope_state", "la_rope_apply", "add_f32", "patchify",
                                   "unpatchify", "timestep_embedding", "silu", "nvfp4_quantize", "gemm_nvfp4")}


@torch.library.custom_op(f"{_lib_ns}::gemm", mutates_args=())
def gemm(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], act: int, relu_cols: int,
         gate_table: Optional[torch.Tensor], gate_t: Optional[torch.Tensor], gate_row: int, rows_per_batch: int,
         residual: Optional[torch.Tensor]) -> torch.Tensor:
    gate = (gate_table, gate_t, gate_row, rows_per_batch) if gate_table is not None else None
    return _D["gemm"](a, w, bias=bias, act=act, relu_cols=relu_cols, gate=gate, residual=residual)


@gemm.register_fake
def _(a, w, bias, act, relu_cols, gate_table, gate_t, gate_row, rows_per_batch, residual):
    return a.new_empty(a.shape[0], w.shape[0])


@torch.library.custom_op(f"{_lib_ns}::ln_modulate", mutates_args=())
def ln_modulate(x: torch.Tensor, table: torch.Tensor, t: torch.Tensor, shift_row: int, scale_row: int,
                eps: float) -> torch.Tensor:
    return _D["ln_modulate"](x, table, t, shift_row, scale_row, eps)


@ln_modulate.register_fake
def _(x, table, t, shift_row, scale_row, eps):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@torch.library.custom_op(f"{_lib_ns}::la_state", mutates_args=())
def la_state(k: torch.Tensor, v: torch.Tensor, B: int, N: int, H: int) -> torch.Tensor:
    return _D["la_state"](k, v, B, N, H)


@la_state.register_fake
def _(k, v, B, N, H):
    return k.new_empty(B, H, ops.STATE_ROWS, ops.HEAD_DIM, dtype=torch.float32)


@torch.library.custom_op(f"{_lib_ns}::la_apply", mutates_args=())
def la_apply(q: torch.Tensor, state: torch.Tensor, B: int, N: int, H: int, eps: float) -> torch.Tensor:
    return _D["la_apply"](q, state, B, N, H, eps)


@la_apply.register_fake
def _(q, state, B, N, H, eps):
    return q.new_empty(B * N, H * ops.HEAD_DIM)


@torch.library.custom_op(f"{_lib_ns}::dwconv_glu", mutates_args=())
def dwconv_glu(u: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], W: int, H: int, row0: int,
               halo_top: Optional[torch.Tensor], halo_bot: Optional[torch.Tensor]) -> torch.Tensor:
    return _D["dwconv_glu"](u, weight, bias, W, H, row0=row0, halo_top=halo_top, halo_bot=halo_bot)


@dwconv_glu.register_fake
def _(u, weight, bias, W, H, row0, halo_top, halo_bot):
    return u.new_empty(u.shape[0], u.shape[1] // 2)


@torch.library.custom_op(f"{_lib_ns}::rmsnorm_", mutates_args=("x",))
def rmsnorm_(x: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    _D["rmsnorm_"](x, weight, eps)


@rmsnorm_.register_fake
def _(x, weight, eps):
    return None


@torch.library.custom_op(f"{_lib_ns}::rope_", mutates_args=("x",))
def rope_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, B: int, N: int, head_dim: int) -> None:
    _D["rope_"](x, cos, sin, B, N, head_dim)


@rope_.register_fake
def _(x, cos, sin, B, N, head_dim):
    return None


@torch.library.custom_op(f"{_lib_ns}::cross_attention", mutates_args=())
def cross_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: Optional[torch.Tensor], B: int, N: int,
                    L: int, heads: int, head_dim: int) -> torch.Tensor:
    return _D["cross_attention"](q, k, v, mask, B, N, L, heads, head_dim)


@cross_attention.register_fake
def _(q, k, v, mask, B, N, L, heads, head_dim):
    return q.new_empty(B * N, heads * head_dim)


@torch.library.custom_op(f"{_lib_ns}::la_rope_state", mutates_args=())
def la_rope_state(k: torch.Tensor, v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, B: int, N: int, H: int,
                  D: int, prior: Optional[torch.Tensor]) -> torch.Tensor:
    return _D["la_rope_state"](k, v, cos, sin, B, N, H, D, prior=prior)


@la_rope_state.register_fake
def _(k, v, cos, sin, B, N, H, D, prior):
    return k.new_empty(B, H, D + 1, D, dtype=torch.float32)


@torch.library.custom_op(f"{_lib_ns}::la_rope_apply", mutates_args=())
def la_rope_apply(q: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, state: torch.Tensor, B: int, N: int, H: int,
                  D: int, eps: float) -> torch.Tensor:
    return _D["la_rope_apply"](q, cos, sin, state, B, N, H, D, eps)


@la_rope_apply.register_fake
def _(q, cos, sin, state, B, N, H, D, eps):
    return q.new_empty(B * N, H * D)


@torch.library.custom_op(f"{_lib_ns}::add_f32", mutates_args=())
def add_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return _D["add_f32"](a, b)


@add_f32.register_fake
def _(a, b):
    return torch.empty_like(a)


@torch.library.custom_op(f"{_lib_ns}::ln_modulate_rows", mutates_args=())
def ln_modulate_rows(x: torch.Tensor, table: torch.Tensor, t: torch.Tensor, table_shift_row: int, table_scale_row: int,
                     t_shift_row: int, t_scale_row: int, eps: float) -> torch.Tensor:
    return _D["ln_modulate_rows"](x, table, t, table_shift_row, table_scale_row, t_shift_row, t_scale_row, eps)


@ln_modulate_rows.register_fake
def _(x, table, t, table_shift_row, table_scale_row, t_shift_row, t_scale_row, eps):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@torch.library.custom_op(f"{_lib_ns}::patchify", mutates_args=())
def patchify(x: torch.Tensor, p: int) -> torch.Tensor:
    return _D["patchify"](x, p)


@patchify.register_fake
def _(x, p):
    B, Cin, H, W = x.shape
    return x.new_empty(B * (H // p) * (W // p), Cin * p * p)


@torch.library.custom_op(f"{_lib_ns}::unpatchify", mutates_args=())
def unpatchify(tok: torch.Tensor, B: int, Cout: int, Hp: int, Wp: int, p: int) -> torch.Tensor:
    return _D["unpatchify"](tok, B, Cout, Hp, Wp, p)


@unpatchify.register_fake
def _(tok, B, Cout, Hp, Wp, p):
    return tok.new_empty(B, Cout, Hp * p, Wp * p)


@torch.library.custom_op(f"{_lib_ns}::timestep_embedding", mutates_args=())
def timestep_embedding(t: torch.Tensor, dim: int, dtype: torch.dtype, max_period: float) -> torch.Tensor:
    return _D["timestep_embedding"](t, dim, dtype, max_period)


@timestep_embedding.register_fake
def _(t, dim, dtype, max_period):
    return t.new_empty(t.numel(), dim, dtype=dtype)


@torch.library.custom_op(f"{_lib_ns}::silu", mutates_args=())
def silu(x: torch.Tensor) -> torch.Tensor:
    return _D["silu"](x)


@silu.register_fake
def _(x):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


def _sf_bytes(rows: int, K: int) -> int:
    """Bytes of the E4M3 scale tiles of a [rows, K] NVFP4 matrix: 512-byte tiles of 128 rows x 4 blocks of 16."""
    return ((rows + 127) // 128) * ((K // 16 + 3) // 4) * 512


@torch.library.custom_op(f"{_lib_ns}::nvfp4_quantize", mutates_args=())
def nvfp4_quantize(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    t = _D["nvfp4_quantize"](x)
    return t.q, t.sf, t.scales


@nvfp4_quantize.register_fake
def _(x):
    rows, K = x.shape
    return (x.new_empty(rows, K // 2, dtype=torch.uint8), x.new_empty(_sf_bytes(rows, K), dtype=torch.uint8),
            x.new_empty(4, dtype=torch.float32))


@torch.library.custom_op(f"{_lib_ns}::gemm_nvfp4", mutates_args=())
def gemm_nvfp4(a_codes: torch.Tensor, a_sf: torch.Tensor, a_scales: torch.Tensor, w_codes: torch.Tensor,
               w_sf: torch.Tensor, w_scales: torch.Tensor, bias: Optional[torch.Tensor], act: int, relu_cols: int,
               gate_table: Optional[torch.Tensor], gate_t: Optional[torch.Tensor], gate_row: int, rows_per_batch: int,
               residual: Optional[torch.Tensor]) -> torch.Tensor:
    a = ops.NvFp4Tensor(a_codes, a_sf, a_scales, a_codes.shape[0], 2 * a_codes.shape[1])
    w = ops.NvFp4Tensor(w_codes, w_sf, w_scales, w_codes.shape[0], 2 * w_codes.shape[1])
    gate = (gate_table, gate_t, gate_row, rows_per_batch) if gate_table is not None else None
    return _D["gemm_nvfp4"](a, w, bias=bias, act=act, relu_cols=relu_cols, gate=gate, residual=residual)


@gemm_nvfp4.register_fake
def _(a_codes, a_sf, a_scales, w_codes, w_sf, w_scales, bias, act, relu_cols, gate_table, gate_t, gate_row,
      rows_per_batch, residual):
    return a_codes.new_empty(a_codes.shape[0], w_codes.shape[0], dtype=torch.bfloat16)


# ---- optional: the modules through the dispatcher ---------------------------------------------------------
# The modules call `sana_b200.ops` directly (no dispatcher overhead per launch).  For tracing, export or fake-tensor
# shape propagation of a whole module, route_modules(True) replaces those names in `ops` by wrappers that go
# through torch.ops.sana_b200 whenever the call uses only what the operator schemas carry (no preallocated output,
# no NVFP4 side outputs); anything else keeps the direct path.

def _r_gemm(a, w, bias=None, act=ops.ACT_NONE, relu_cols=0, gate=None, residual=None, out=None):
    if out is not None:
        return _D["gemm"](a, w, bias=bias, act=act, relu_cols=relu_cols, gate=gate, residual=residual, out=out)
    gt, tt, gr, rpb = gate if gate is not None else (None, None, 0, 1)
    return torch.ops.sana_b200.gemm(a, w, bias, act, relu_cols, gt, tt, gr, rpb, residual)


def _r_ln_modulate(x, table, t, shift_row, scale_row, eps=1e-6):
    return torch.ops.sana_b200.ln_modulate(x, table, t, shift_row, scale_row, eps)


def _r_la_apply(q, state, B, N, H, eps, out=None):
    if out is not None:
        return _D["la_apply"](q, state, B, N, H, eps, out=out)
    return torch.ops.sana_b200.la_apply(q, state, B, N, H, eps)


def _r_dwconv_glu(u, weight, bias, W, H, row0=0, halo_top=None, halo_bot=None, amax_out=None):
    if amax_out is not None:
        return _D["dwconv_glu"](u, weight, bias, W, H, row0=row0, halo_top=halo_top, halo_bot=halo_bot, amax_out=amax_out)
    return torch.ops.sana_b200.dwconv_glu(u, weight, bias, W, H, row0, halo_top, halo_bot)


def _r_rmsnorm_(x, weight, eps):
    torch.ops.sana_b200.rmsnorm_(x, weight, eps)
    return x


def _r_rope_(x, cos, sin, B, N, head_dim=ops.HEAD_DIM):
    torch.ops.sana_b200.rope_(x, cos, sin, B, N, head_dim)
    return x


def _r_la_rope_state(k, v, cos, sin, B, N, H, D, prior=None):
    return torch.ops.sana_b200.la_rope_state(k, v, cos, sin, B, N, H, D, prior)


def _r_la_rope_apply(q, cos, sin, state, B, N, H, D, eps, out=None):
    if out is not None:
        return _D["la_rope_apply"](q, cos, sin, state, B, N, H, D, eps, out=out)
    return torch.ops.sana_b200.la_rope_apply(q, cos, sin, state, B, N, H, D, eps)


def _r_ln_modulate_rows(x, table, t, table_shift_row, table_scale_row, t_shift_row, t_scale_row, eps=1e-6):
    return torch.ops.sana_b200.ln_modulate_rows(x, table, t, table_shift_row, table_scale_row, t_shift_row, t_scale_row, eps)


def _r_timestep_embedding(t, dim, dtype, max_period=10000.0):
    return torch.ops.sana_b200.timestep_embedding(t, dim, dtype, float(max_period))


_ROUTED = {"gemm": _r_gemm, "ln_modulate": _r_ln_modulate, "la_state": torch.ops.sana_b200.la_state, "la_apply": _r_la_apply,
           "dwconv_glu": _r_dwconv_glu, "rmsnorm_": _r_rmsnorm_, "rope_": _r_rope_,
           "cross_attention": torch.ops.sana_b200.cross_attention, "la_rope_state": _r_la_rope_state,
           "la_rope_apply": _r_la_rope_apply, "add_f32": torch.ops.sana_b200.add_f32, "ln_modulate_rows": _r_ln_modulate_rows,
           "patchify": torch.ops.sana_b200.patchify, "unpatchify": torch.ops.sana_b200.unpatchify,
           "timestep_embedding": _r_timestep_embedding, "silu": torch.ops.sana_b200.silu}


def route_modules(enabled: bool = True) -> None:
    """Send the modules' kernel calls through torch.ops.sana_b200 (True) or straight to the C ABI (False, the default)."""
    for name, fn in _ROUTED.items():
        setattr(ops, name, fn if enabled else _D[name])

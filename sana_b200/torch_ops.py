"""The C-ABI kernels as torch custom operators (namespace ``sana_b200``), with fake (meta)
implementations so that tracing / ``torch.compile`` / fake-tensor propagation see shapes and
dtypes without touching the GPU.

    torch.ops.sana_b200.gemm(a, w, bias, act, relu_cols, gate_table, gate_t, gate_row, rows_per_batch, residual)
    torch.ops.sana_b200.ln_modulate(x, table, t, shift_row, scale_row, eps)
    torch.ops.sana_b200.la_state(k, v, B, N, H)
    torch.ops.sana_b200.la_apply(q, state, B, N, H, eps)
    torch.ops.sana_b200.dwconv_glu(u, weight, bias, W, H, row0, halo_top, halo_bot)
    torch.ops.sana_b200.rmsnorm_(x, weight, eps)          # in place

They are thin: each forwards to :mod:`sana_b200.ops`, which passes raw device pointers and the
current stream to libsana_b200.so.  The modules call :mod:`sana_b200.ops` directly (same
kernels, without the dispatcher's per-call overhead).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops

_lib_ns = "sana_b200"


@torch.library.custom_op(f"{_lib_ns}::gemm", mutates_args=())
def gemm(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], act: int, relu_cols: int,
         gate_table: Optional[torch.Tensor], gate_t: Optional[torch.Tensor], gate_row: int, rows_per_batch: int,
         residual: Optional[torch.Tensor]) -> torch.Tensor:
    gate = (gate_table, gate_t, gate_row, rows_per_batch) if gate_table is not None else None
    return ops.gemm(a, w, bias=bias, act=act, relu_cols=relu_cols, gate=gate, residual=residual)


@gemm.register_fake
def _(a, w, bias, act, relu_cols, gate_table, gate_t, gate_row, rows_per_batch, residual):
    return a.new_empty(a.shape[0], w.shape[0])


@torch.library.custom_op(f"{_lib_ns}::ln_modulate", mutates_args=())
def ln_modulate(x: torch.Tensor, table: torch.Tensor, t: torch.Tensor, shift_row: int, scale_row: int,
                eps: float) -> torch.Tensor:
    return ops.ln_modulate(x, table, t, shift_row, scale_row, eps)


@ln_modulate.register_fake
def _(x, table, t, shift_row, scale_row, eps):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@torch.library.custom_op(f"{_lib_ns}::la_state", mutates_args=())
def la_state(k: torch.Tensor, v: torch.Tensor, B: int, N: int, H: int) -> torch.Tensor:
    return ops.la_state(k, v, B, N, H)


@la_state.register_fake
def _(k, v, B, N, H):
    return k.new_empty(B, H, ops.STATE_ROWS, ops.HEAD_DIM, dtype=torch.float32)


@torch.library.custom_op(f"{_lib_ns}::la_apply", mutates_args=())
def la_apply(q: torch.Tensor, state: torch.Tensor, B: int, N: int, H: int, eps: float) -> torch.Tensor:
    return ops.la_apply(q, state, B, N, H, eps)


@la_apply.register_fake
def _(q, state, B, N, H, eps):
    return q.new_empty(B * N, H * ops.HEAD_DIM)


@torch.library.custom_op(f"{_lib_ns}::dwconv_glu", mutates_args=())
def dwconv_glu(u: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], W: int, H: int, row0: int,
               halo_top: Optional[torch.Tensor], halo_bot: Optional[torch.Tensor]) -> torch.Tensor:
    return ops.dwconv_glu(u, weight, bias, W, H, row0=row0, halo_top=halo_top, halo_bot=halo_bot)


@dwconv_glu.register_fake
def _(u, weight, bias, W, H, row0, halo_top, halo_bot):
    return u.new_empty(u.shape[0], u.shape[1] // 2)


@torch.library.custom_op(f"{_lib_ns}::rmsnorm_", mutates_args=("x",))
def rmsnorm_(x: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    ops.rmsnorm_(x, weight, eps)


@rmsnorm_.register_fake
def _(x, weight, eps):
    return None

"""Tensor-level wrappers of the C ABI: validate torch tensors, allocate outputs with torch,
pass raw device pointers and the current CUDA stream to libsana_b200.so.

PyTorch is used here only for device memory and streams; all arithmetic happens in the
library's CUDA kernels.  Nothing here falls back to torch math.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import SANA_BF16, SANA_F32, GemmEpilogue, SanaLibraryError

HEAD_DIM = 32
STATE_ROWS = HEAD_DIM + 1

ACT_NONE, ACT_SILU, ACT_RELU_COLS, ACT_GELU_TANH = 0, 1, 2, 3


class _Counters:
    """Kernel launches issued through this module (the benchmark reports them) and, when
    ``gemm_timing`` is on, CUDA-event pairs around every tensor-core GEMM launch."""

    def __init__(self):
        self.launches = 0
        self.gemm_timing = False
        self.gemm_events = []  # (start, end, flops, label)
        self.gemm_bytes = []   # operand + result bytes of each timed launch, every element once

    def reset(self):
        self.launches = 0
        self.gemm_events = []
        self.gemm_bytes = []


counters = _Counters()


def _dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return SANA_BF16
    if dt == torch.float32:
        return SANA_F32
    raise SanaLibraryError(f"unsupported dtype {dt}: the kernels exist for bfloat16 and float32 only")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _need_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise SanaLibraryError("sana_b200 operators run on CUDA tensors only (no CPU path)")


def _rows2d(t: torch.Tensor, what: str) -> Tuple[int, int, int]:
    """(rows, cols, row stride) of a 2-D tensor whose last dimension is contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise SanaLibraryError(f"{what}: expected a 2-D tensor with contiguous rows, got shape {tuple(t.shape)} "
                               f"strides {t.stride()}")
    return t.shape[0], t.shape[1], t.stride(0)


def ln_modulate(x: torch.Tensor, table: torch.Tensor, t: torch.Tensor, shift_row: int, scale_row: int,
                eps: float = 1e-6) -> torch.Tensor:
    """z = LayerNorm(x) * (1 + scale) + shift with scale/shift = table[row] + t[b, row].

    x [B, N, C]; table [6, C]; t [B, 6*C]."""
    _need_cuda(x, table, t)
    B, N, Cc = x.shape
    x = x.contiguous()
    table = table.contiguous()
    t = t.reshape(B, 6 * Cc).contiguous()
    if table.shape != (6, Cc) or table.dtype != x.dtype or t.dtype != x.dtype:
        raise SanaLibraryError("ln_modulate: table must be [6, C] and t [B, 6C] in x's dtype")
    z = torch.empty_like(x)
    lib = _lib.load()
    _lib.check(lib.sana_ln_modulate(x.data_ptr(), table.data_ptr(), t.data_ptr(), z.data_ptr(), B, N, Cc,
                                    shift_row, scale_row, eps, _dtype_code(x.dtype), _stream()), "sana_ln_modulate")
    counters.launches += 1
    return z


def ln_modulate_rows(x: torch.Tensor, table: torch.Tensor, t: torch.Tensor, table_shift_row: int, table_scale_row: int,
                     t_shift_row: int, t_scale_row: int, eps: float = 1e-6) -> torch.Tensor:
    """Like :func:`ln_modulate` with table [R, C] and t [B, Rt, C] and the rows named separately
    (the final layer: table [2, C], t [B, 1, C], rows (0, 1) of the table and row 0 of t twice)."""
    _need_cuda(x, table, t)
    B, N, Cc = x.shape
    x = x.contiguous()
    table = table.contiguous()
    t = t.reshape(B, -1, Cc).contiguous()
    if table.dim() != 2 or table.shape[1] != Cc or table.dtype != x.dtype or t.dtype != x.dtype:
        raise SanaLibraryError("ln_modulate_rows: table must be [R, C] and t [B, Rt, C] in x's dtype")
    z = torch.empty_like(x)
    lib = _lib.load()
    _lib.check(lib.sana_ln_modulate_rows(x.data_ptr(), table.data_ptr(), t.data_ptr(), z.data_ptr(), B, N, Cc,
                                         table.shape[0], table_shift_row, table_scale_row, t.shape[1], t_shift_row,
                                         t_scale_row, eps, _dtype_code(x.dtype), _stream()), "sana_ln_modulate_rows")
    counters.launches += 1
    return z


def patchify(x: torch.Tensor, p: int) -> torch.Tensor:
    """Latent [B, Cin, H, W] -> patch rows [B*(H/p)*(W/p), Cin*p*p] (the unfold of a stride-p,
    kernel-p convolution; column order matches the conv weight viewed as [embed, Cin*p*p])."""
    _need_cuda(x)
    B, Cin, H, W = x.shape
    x = x.contiguous()
    out = torch.empty(B * (H // p) * (W // p), Cin * p * p, dtype=x.dtype, device=x.device)
    _lib.check(_lib.load().sana_patchify(x.data_ptr(), out.data_ptr(), out.stride(0), B, Cin, H, W, p,
                                         _dtype_code(x.dtype), _stream()), "sana_patchify")
    counters.launches += 1
    return out


def unpatchify(tok: torch.Tensor, B: int, Cout: int, Hp: int, Wp: int, p: int) -> torch.Tensor:
    """Token rows [B*Hp*Wp, p*p*Cout] -> images [B, Cout, Hp*p, Wp*p]."""
    _need_cuda(tok)
    rows, cols, ld = _rows2d(tok, "unpatchify tokens")
    if rows != B * Hp * Wp or cols != p * p * Cout:
        raise SanaLibraryError(f"unpatchify: expected [{B * Hp * Wp}, {p * p * Cout}] token rows, got {tuple(tok.shape)}")
    out = torch.empty(B, Cout, Hp * p, Wp * p, dtype=tok.dtype, device=tok.device)
    _lib.check(_lib.load().sana_unpatchify(tok.data_ptr(), ld, out.data_ptr(), B, Cout, Hp, Wp, p,
                                           _dtype_code(tok.dtype), _stream()), "sana_unpatchify")
    counters.launches += 1
    return out


def timestep_embedding(t: torch.Tensor, dim: int, dtype: torch.dtype, max_period: float = 10000.0) -> torch.Tensor:
    """Sinusoidal features [B, dim] (cos half, then sin half) of fp32 timesteps t [B]."""
    _need_cuda(t)
    t = t.reshape(-1).to(torch.float32).contiguous()
    out = torch.empty(t.numel(), dim, dtype=dtype, device=t.device)
    _lib.check(_lib.load().sana_timestep_embedding(t.data_ptr(), out.data_ptr(), t.numel(), dim, max_period,
                                                   _dtype_code(dtype), _stream()), "sana_timestep_embedding")
    counters.launches += 1
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    _need_cuda(x)
    x = x.contiguous()
    out = torch.empty_like(x)
    _lib.check(_lib.load().sana_silu(x.data_ptr(), out.data_ptr(), x.numel(), _dtype_code(x.dtype), _stream()),
               "sana_silu")
    counters.launches += 1
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Out-of-place RMSNorm with weight over the last dimension of a 2-D tensor."""
    _need_cuda(x, weight)
    rows, Cc, ld = _rows2d(x, "rmsnorm x")
    if weight.numel() != Cc or weight.dtype != x.dtype:
        raise SanaLibraryError("rmsnorm: weight must be [C] in x's dtype")
    out = torch.empty(rows, Cc, dtype=x.dtype, device=x.device)
    _lib.check(_lib.load().sana_rmsnorm(x.data_ptr(), ld, weight.contiguous().data_ptr(), out.data_ptr(), Cc, rows, Cc,
                                        eps, _dtype_code(x.dtype), _stream()), "sana_rmsnorm")
    counters.launches += 1
    return out


def rmsnorm_(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """In-place RMSNorm with weight over the last dimension of a 2-D view (rows may be strided,
    e.g. the q or k column block of a qkv projection).  Returns ``x``."""
    _need_cuda(x, weight)
    rows, Cc, ld = _rows2d(x, "rmsnorm x")
    if weight.numel() != Cc or weight.dtype != x.dtype:
        raise SanaLibraryError("rmsnorm: weight must be [C] in x's dtype")
    weight = weight.contiguous()
    lib = _lib.load()
    _lib.check(lib.sana_rmsnorm(x.data_ptr(), ld, weight.data_ptr(), x.data_ptr(), ld, rows, Cc, eps,
                                _dtype_code(x.dtype), _stream()), "sana_rmsnorm")
    counters.launches += 1
    return x


def rope_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, B: int, N: int, head_dim: int = HEAD_DIM) -> torch.Tensor:
    """In-place rotary embedding of a [B*N, C] view (q or k block of a qkv projection) with
    per-position tables cos, sin [N, head_dim] (any float dtype; used in fp32).  Returns ``x``."""
    _need_cuda(x, cos, sin)
    rows, Cc, ld = _rows2d(x, "rope x")
    if rows != B * N or tuple(cos.shape) != (N, head_dim) or tuple(sin.shape) != (N, head_dim):
        raise SanaLibraryError(f"rope: expected x [{B * N}, C] and tables [{N}, {head_dim}]")
    cf, sf = cos.to(torch.float32).contiguous(), sin.to(torch.float32).contiguous()
    _lib.check(_lib.load().sana_rope(x.data_ptr(), ld, cf.data_ptr(), sf.data_ptr(), B, N, Cc, head_dim,
                                     _dtype_code(x.dtype), _stream()), "sana_rope")
    counters.launches += 1
    return x


def la_state(k: torch.Tensor, v: torch.Tensor, B: int, N: int, H: int) -> torch.Tensor:
    """state[b,h,i,j] = sum_n [v;1][b,n,h,i] * relu(k[b,n,h,j]); k, v are [B*N, H*32] views
    (e.g. column slices of the qkv projection).  Returns fp32 [B, H, 33, 32]."""
    _need_cuda(k, v)
    rk, ck, ldk = _rows2d(k, "la_state k")
    rv, cv, ldv = _rows2d(v, "la_state v")
    if rk != B * N or rv != B * N or ck != H * HEAD_DIM or cv != H * HEAD_DIM or ldk != ldv or k.dtype != v.dtype:
        raise SanaLibraryError("la_state: k and v must be [B*N, H*32] with the same row stride and dtype")
    lib = _lib.load()
    ws_bytes = lib.sana_la_state_workspace_bytes(B, N, H)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=k.device)
    state = torch.empty(B, H, STATE_ROWS, HEAD_DIM, dtype=torch.float32, device=k.device)
    _lib.check(lib.sana_la_state(k.data_ptr(), v.data_ptr(), ldk, state.data_ptr(), ws.data_ptr(), ws.numel(), B, N, H,
                                 _dtype_code(k.dtype), _stream()), "sana_la_state")
    counters.launches += 2  # partial states + fixed-order reduction
    return state


def la_state_sp_buffer_bytes(B: int, H: int) -> int:
    return _lib.load().sana_la_state_sp_buffer_bytes(B, H)


def la_state_sp(k: torch.Tensor, v: torch.Tensor, B: int, N: int, H: int, peer_ptrs, rank: int, world: int,
                step: int) -> torch.Tensor:
    """Like :func:`la_state` for this rank's tokens, with the all-reduce over the ranks fused
    into the reduction kernel (peer-memory loads, no NCCL).  ``peer_ptrs[r]`` is the device
    address of rank r's exchange buffer as mapped in this process; ``step`` counts 1, 2, ..."""
    _need_cuda(k, v)
    rk, ck, ldk = _rows2d(k, "la_state_sp k")
    rv, cv, ldv = _rows2d(v, "la_state_sp v")
    if rk != B * N or rv != B * N or ck != H * HEAD_DIM or cv != H * HEAD_DIM or ldk != ldv or k.dtype != v.dtype:
        raise SanaLibraryError("la_state_sp: k and v must be [B*N, H*32] with the same row stride and dtype")
    lib = _lib.load()
    ws_bytes = lib.sana_la_state_workspace_bytes(B, N, H)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=k.device)
    state = torch.empty(B, H, STATE_ROWS, HEAD_DIM, dtype=torch.float32, device=k.device)
    arr = (C.c_void_p * world)(*[C.c_void_p(int(p)) for p in peer_ptrs])
    _lib.check(lib.sana_la_state_sp(k.data_ptr(), v.data_ptr(), ldk, state.data_ptr(), ws.data_ptr(), ws.numel(), B, N, H,
                                    _dtype_code(k.dtype), arr, rank, world, step, _stream()), "sana_la_state_sp")
    counters.launches += 2
    return state


def halo_exchange_buffer_bytes(row_bytes: int) -> int:
    return _lib.load().sana_halo_exchange_buffer_bytes(row_bytes)


def halo_exchange(first_row: Optional[torch.Tensor], last_row: Optional[torch.Tensor], row_bytes: int, mine: int,
                  upper: Optional[int], lower: Optional[int], step: int) -> None:
    """Pushes this rank's boundary rows into the neighbours' halo slots over peer memory and
    waits for theirs (see sana_halo_exchange).  ``mine`` / ``upper`` / ``lower`` are device
    addresses of the exchange buffers (None where there is no neighbour in the same frame)."""
    _need_cuda(first_row, last_row)
    for r in (first_row, last_row):
        if r is not None and (not r.is_contiguous() or r.numel() * r.element_size() != row_bytes):
            raise SanaLibraryError("halo_exchange: rows must be contiguous and row_bytes long")
    _lib.check(_lib.load().sana_halo_exchange(first_row.data_ptr() if first_row is not None else None,
                                              last_row.data_ptr() if last_row is not None else None, row_bytes, mine,
                                              upper, lower, step, _stream()), "sana_halo_exchange")
    counters.launches += 1


def set_exchange_wait_limit(seconds: float) -> None:
    """Limit of the waits for a peer GPU inside the fused exchange kernels (0 = the default, 2 s)."""
    _lib.check(_lib.load().sana_exchange_set_wait_limit_ns(int(seconds * 1e9)), "sana_exchange_set_wait_limit_ns")


def la_apply(q: torch.Tensor, state: torch.Tensor, B: int, N: int, H: int, eps: float,
             out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """o[b,n,h,:] = state[b,h,:32] relu(q) / (state[b,h,32] . relu(q) + eps); q [B*N, H*32] view."""
    _need_cuda(q, state)
    rq, cq, ldq = _rows2d(q, "la_apply q")
    if rq != B * N or cq != H * HEAD_DIM:
        raise SanaLibraryError("la_apply: q must be [B*N, H*32]")
    if state.shape != (B, H, STATE_ROWS, HEAD_DIM) or state.dtype != torch.float32 or not state.is_contiguous():
        raise SanaLibraryError("la_apply: state must be contiguous fp32 [B, H, 33, 32]")
    if out is None:
        out = torch.empty(B * N, H * HEAD_DIM, dtype=q.dtype, device=q.device)
    ro, co, ldo = _rows2d(out, "la_apply out")
    if ro != B * N or co != H * HEAD_DIM or out.dtype != q.dtype:
        raise SanaLibraryError("la_apply: bad output tensor")
    lib = _lib.load()
    _lib.check(lib.sana_la_apply(q.data_ptr(), ldq, state.data_ptr(), out.data_ptr(), ldo, B, N, H, eps,
                                 _dtype_code(q.dtype), _stream()), "sana_la_apply")
    counters.launches += 1
    return out


def _rope_tables(cos: torch.Tensor, sin: torch.Tensor, N: int, D: int, what: str) -> None:
    for tb in (cos, sin):
        if tb.shape != (N, D // 2) or tb.dtype != torch.float32 or not tb.is_contiguous():
            raise SanaLibraryError(f"{what}: cos / sin tables must be contiguous fp32 [N, head_dim / 2]")


def add_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a + b for contiguous fp32 tensors of one shape (two attention states)."""
    _need_cuda(a, b)
    if a.dtype != torch.float32 or b.dtype != torch.float32 or a.shape != b.shape or not (a.is_contiguous() and b.is_contiguous()):
        raise SanaLibraryError("add_f32: two contiguous fp32 tensors of one shape")
    out = torch.empty_like(a)
    _lib.check(_lib.load().sana_add_f32(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _stream()), "sana_add_f32")
    counters.launches += 1
    return out


def la_rope_state(k: torch.Tensor, v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, B: int, N: int, H: int,
                  D: int, prior: Optional[torch.Tensor] = None) -> torch.Tensor:
    """State of the ReLU-then-rotate linear attention (see sana_la_rope_state): k, v [B*N, H*D]
    views, cos / sin fp32 [N, D/2].  Returns fp32 [B, H, D+1, D]; row D is the unrotated key sum.
    ``prior``: a state of the same shape carried over from earlier tokens, added in."""
    _need_cuda(k, v, cos, sin)
    rk, ck, ldk = _rows2d(k, "la_rope_state k")
    rv, cv, ldv = _rows2d(v, "la_rope_state v")
    if rk != B * N or rv != B * N or ck != H * D or cv != H * D or ldk != ldv or k.dtype != v.dtype:
        raise SanaLibraryError("la_rope_state: k and v must be [B*N, H*D] with the same row stride and dtype")
    _rope_tables(cos, sin, N, D, "la_rope_state")
    lib = _lib.load()
    ws_bytes = lib.sana_la_rope_state_workspace_bytes(B, N, H, D)
    if ws_bytes <= 0:
        raise SanaLibraryError(f"la_rope_state: head dimension {D} is not a multiple of 16 in [16, 128]")
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=k.device)
    state = torch.empty(B, H, D + 1, D, dtype=torch.float32, device=k.device)
    if prior is not None:
        if prior.shape != state.shape or prior.dtype != torch.float32 or not prior.is_contiguous() or not prior.is_cuda:
            raise SanaLibraryError("la_rope_state: prior must be a contiguous fp32 CUDA tensor [B, H, D+1, D]")
        _lib.check(lib.sana_la_rope_state_add(k.data_ptr(), v.data_ptr(), ldk, cos.data_ptr(), sin.data_ptr(), prior.data_ptr(),
                                              state.data_ptr(), ws.data_ptr(), ws.numel(), B, N, H, D, _dtype_code(k.dtype),
                                              _stream()), "sana_la_rope_state_add")
        counters.launches += 2
        return state
    _lib.check(lib.sana_la_rope_state(k.data_ptr(), v.data_ptr(), ldk, cos.data_ptr(), sin.data_ptr(), state.data_ptr(),
                                      ws.data_ptr(), ws.numel(), B, N, H, D, _dtype_code(k.dtype), _stream()),
               "sana_la_rope_state")
    counters.launches += 2  # partial states + fixed-order reduction
    return state


def la_rope_state_sp_buffer_bytes(B: int, H: int, D: int) -> int:
    return _lib.load().sana_la_rope_state_sp_buffer_bytes(B, H, D)


def la_rope_state_sp(k: torch.Tensor, v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, B: int, N: int, H: int,
                     D: int, peer_ptrs, rank: int, world: int, step: int) -> torch.Tensor:
    """Like :func:`la_rope_state` for this rank's tokens (``cos`` / ``sin`` hold their rows), with the all-reduce
    over the ranks fused into the reduction kernel (peer-memory loads, no NCCL); arguments as in
    :func:`la_state_sp`."""
    _need_cuda(k, v, cos, sin)
    rk, ck, ldk = _rows2d(k, "la_rope_state_sp k")
    rv, cv, ldv = _rows2d(v, "la_rope_state_sp v")
    if rk != B * N or rv != B * N or ck != H * D or cv != H * D or ldk != ldv or k.dtype != v.dtype:
        raise SanaLibraryError("la_rope_state_sp: k and v must be [B*N, H*D] with the same row stride and dtype")
    _rope_tables(cos, sin, N, D, "la_rope_state_sp")
    lib = _lib.load()
    ws_bytes = lib.sana_la_rope_state_workspace_bytes(B, N, H, D)
    if ws_bytes <= 0:
        raise SanaLibraryError(f"la_rope_state_sp: head dimension {D} is not a multiple of 16 in [16, 128]")
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=k.device)
    state = torch.empty(B, H, D + 1, D, dtype=torch.float32, device=k.device)
    arr = (C.c_void_p * world)(*[C.c_void_p(int(p)) for p in peer_ptrs])
    _lib.check(lib.sana_la_rope_state_sp(k.data_ptr(), v.data_ptr(), ldk, cos.data_ptr(), sin.data_ptr(), state.data_ptr(),
                                         ws.data_ptr(), ws.numel(), B, N, H, D, _dtype_code(k.dtype), arr, rank, world, step,
                                         _stream()), "sana_la_rope_state_sp")
    counters.launches += 2
    return state


def la_rope_apply(q: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, state: torch.Tensor, B: int, N: int, H: int,
                  D: int, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """o = state[:D] rot(relu(q)) / (state[D] . relu(q) + eps), token-major; q [B*N, H*D] view."""
    _need_cuda(q, cos, sin, state)
    rq, cq, ldq = _rows2d(q, "la_rope_apply q")
    if rq != B * N or cq != H * D:
        raise SanaLibraryError("la_rope_apply: q must be [B*N, H*D]")
    _rope_tables(cos, sin, N, D, "la_rope_apply")
    if state.shape != (B, H, D + 1, D) or state.dtype != torch.float32 or not state.is_contiguous():
        raise SanaLibraryError("la_rope_apply: state must be contiguous fp32 [B, H, D+1, D]")
    if out is None:
        out = torch.empty(B * N, H * D, dtype=q.dtype, device=q.device)
    ro, co, ldo = _rows2d(out, "la_rope_apply out")
    if ro != B * N or co != H * D or out.dtype != q.dtype:
        raise SanaLibraryError("la_rope_apply: bad output tensor")
    _lib.check(_lib.load().sana_la_rope_apply(q.data_ptr(), ldq, cos.data_ptr(), sin.data_ptr(), state.data_ptr(),
                                              out.data_ptr(), ldo, B, N, H, D, eps, _dtype_code(q.dtype), _stream()),
               "sana_la_rope_apply")
    counters.launches += 1
    return out


def cross_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: Optional[torch.Tensor], B: int, N: int,
                    L: int, heads: int, head_dim: int) -> torch.Tensor:
    """softmax(q k^T / sqrt(head_dim) + (1 - mask) * -10000) v, token-major.  q [B*N, heads*head_dim];
    k, v [B*L, heads*head_dim] views with one row stride; mask [B, L] of 0/1 or None."""
    _need_cuda(q, k, v, mask)
    rq, cq, ldq = _rows2d(q, "cross_attention q")
    rk, ck, ldk = _rows2d(k, "cross_attention k")
    rv, cv, ldv = _rows2d(v, "cross_attention v")
    Cc = heads * head_dim
    if rq != B * N or rk != B * L or rv != B * L or cq != Cc or ck != Cc or cv != Cc or ldk != ldv:
        raise SanaLibraryError("cross_attention: q must be [B*N, C], k and v [B*L, C] with one row stride")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise SanaLibraryError("cross_attention: q, k, v must share a dtype")
    if mask is not None:
        if mask.shape != (B, L):
            raise SanaLibraryError("cross_attention: mask must be [B, L]")
        mask = mask.to(q.dtype).contiguous()
    out = torch.empty(B * N, Cc, dtype=q.dtype, device=q.device)
    lib = _lib.load()
    _lib.check(lib.sana_cross_attention(q.data_ptr(), ldq, k.data_ptr(), v.data_ptr(), ldk,
                                        mask.data_ptr() if mask is not None else None, out.data_ptr(), Cc, B, N, L, heads,
                                        head_dim, _dtype_code(q.dtype), _stream()), "sana_cross_attention")
    counters.launches += 1
    return out


def set_cross_attention_variant(variant: int) -> None:
    """0 = choose per problem, 1 = warp-level kernel, 2 = tcgen05 kernel (bf16 sana_cross_attention)."""
    _lib.check(_lib.load().sana_cross_attention_set_variant(variant), "sana_cross_attention_set_variant")


def take_cross_attention_device_status() -> int:
    """Code recorded by a timed-out wait inside the tcgen05 cross-attention kernel (0 = none).  Synchronises."""
    v = C.c_int(0)
    _lib.check(_lib.load().sana_cross_attention_take_device_status(C.byref(v)), "sana_cross_attention_take_device_status")
    return int(v.value)


def dwconv_glu(u: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], W: int, H: int, row0: int = 0,
               halo_top: Optional[torch.Tensor] = None, halo_bot: Optional[torch.Tensor] = None,
               amax_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """3x3 depthwise conv + bias + SiLU-GLU.  u [rows*W, 2*hid] (channels last, image rows
    stacked; frames are H rows tall, global row = row0 + local row); weight [2*hid, 1, 3, 3]
    or [2*hid, 3, 3]; halos [W, 2*hid].  Returns [rows*W, hid]."""
    _need_cuda(u, weight, bias, halo_top, halo_bot)
    if u.dim() != 2 or not u.is_contiguous():
        raise SanaLibraryError("dwconv_glu: u must be a contiguous [rows*W, 2*hid] tensor")
    T, C2 = u.shape
    if T % W != 0 or C2 % 2 != 0:
        raise SanaLibraryError("dwconv_glu: u rows must be a multiple of W and channels even")
    rows, hid = T // W, C2 // 2
    weight = weight.reshape(C2, 9).contiguous()
    if weight.dtype != u.dtype or (bias is not None and (bias.dtype != u.dtype or bias.numel() != C2)):
        raise SanaLibraryError("dwconv_glu: weight/bias dtype or size mismatch")
    for hname, h in (("halo_top", halo_top), ("halo_bot", halo_bot)):
        if h is not None and (h.shape != (W, C2) or h.dtype != u.dtype or not h.is_contiguous()):
            raise SanaLibraryError(f"dwconv_glu: {hname} must be contiguous [W, 2*hid] in u's dtype")
    out = torch.empty(T, hid, dtype=u.dtype, device=u.device)
    lib = _lib.load()
    if amax_out is not None:  # bf16: also raise the device float amax_out[0] to max |out|
        if u.dtype != torch.bfloat16 or amax_out.dtype != torch.float32:
            raise SanaLibraryError("dwconv_glu: amax_out needs a bf16 input and an fp32 accumulator")
        _lib.check(lib.sana_dwconv_glu_amax(u.data_ptr(), halo_top.data_ptr() if halo_top is not None else None,
                                            halo_bot.data_ptr() if halo_bot is not None else None, weight.data_ptr(),
                                            bias.contiguous().data_ptr() if bias is not None else None, out.data_ptr(), rows, W,
                                            H, row0, hid, amax_out.data_ptr(), _stream()), "sana_dwconv_glu_amax")
        counters.launches += 1
        return out
    _lib.check(lib.sana_dwconv_glu(u.data_ptr(), halo_top.data_ptr() if halo_top is not None else None,
                                   halo_bot.data_ptr() if halo_bot is not None else None, weight.data_ptr(),
                                   bias.contiguous().data_ptr() if bias is not None else None, out.data_ptr(), rows, W, H,
                                   row0, hid, _dtype_code(u.dtype), _stream()), "sana_dwconv_glu")
    counters.launches += 1
    return out


def take_dwconv_glu_device_status() -> int:
    """Code recorded by a timed-out wait inside the bf16 depthwise kernel (0 = none).  Synchronises."""
    v = C.c_int(0)
    lib = _lib.load()
    _lib.check(lib.sana_dwconv_glu_take_device_status(C.byref(v)), "sana_dwconv_glu_take_device_status")
    return int(v.value)


def take_la_rope_device_status() -> int:
    """Code recorded by a timed-out wait inside the bf16 la_rope_state kernel (0 = none).  Synchronises."""
    v = C.c_int(0)
    _lib.check(_lib.load().sana_la_rope_take_device_status(C.byref(v)), "sana_la_rope_take_device_status")
    return int(v.value)


def _epi_tag(bias, act, gate, residual) -> str:
    return (" +bias" if bias is not None else "") + (" +silu" if act == ACT_SILU else " +gelu" if act == ACT_GELU_TANH else "") + \
        (" *gate" if gate is not None else "") + (" +res" if residual is not None else "")


def _epilogue(M: int, Nn: int, dtype, bias, act, relu_cols, gate, residual):
    """Fills a GemmEpilogue; returns it with the tensors that must stay alive during the call."""
    ep = GemmEpilogue()
    keep = []
    if bias is not None:
        if bias.numel() != Nn or bias.dtype != dtype:
            raise SanaLibraryError("gemm: bias must be [N] in the output dtype")
        bias = bias.contiguous()
        keep.append(bias)
        ep.bias = bias.data_ptr()
    ep.act = act
    ep.relu_cols = relu_cols
    ep.rows_per_batch = 1
    if gate is not None:
        table, t, row, rows_per_batch = gate
        if table.shape != (6, Nn) or t.numel() % (6 * Nn) != 0 or table.dtype != dtype or t.dtype != dtype:
            raise SanaLibraryError("gemm: gate table must be [6, N] and t [B, 6N] in the output dtype")
        if (M + rows_per_batch - 1) // rows_per_batch > t.numel() // (6 * Nn):
            raise SanaLibraryError("gemm: gate t has fewer batch rows than M / rows_per_batch")
        table, t = table.contiguous(), t.contiguous()
        keep += [table, t]
        ep.gate_table, ep.gate_t, ep.gate_row, ep.rows_per_batch = table.data_ptr(), t.data_ptr(), row, rows_per_batch
    if residual is not None:
        Mr, Nr, ldr = _rows2d(residual, "gemm residual")
        if Mr != M or Nr != Nn or residual.dtype != dtype:
            raise SanaLibraryError("gemm: residual must be [M, N] in the output dtype")
        ep.residual, ep.ldr = residual.data_ptr(), ldr
    return ep, keep


def _gemm(fn_name: str, a: torch.Tensor, w: torch.Tensor, bias, act, relu_cols, gate, residual, out):
    _need_cuda(a, w, bias, residual, out)
    M, K, lda = _rows2d(a, "gemm A")
    Nn, Kw, ldw = _rows2d(w, "gemm W")
    if Kw != K or w.dtype != a.dtype:
        raise SanaLibraryError(f"gemm: A is [{M},{K}] but W is [{Nn},{Kw}] ({a.dtype} vs {w.dtype})")
    if out is None:
        out = torch.empty(M, Nn, dtype=a.dtype, device=a.device)
    Mo, No, ldo = _rows2d(out, "gemm out")
    if Mo != M or No != Nn or out.dtype != a.dtype:
        raise SanaLibraryError("gemm: bad output tensor")
    ep, keep = _epilogue(M, Nn, a.dtype, bias, act, relu_cols, gate, residual)
    lib = _lib.load()
    timed = counters.gemm_timing and fn_name == "sana_gemm" and a.dtype == torch.bfloat16
    if timed:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    _lib.check(getattr(lib, fn_name)(a.data_ptr(), lda, w.data_ptr(), ldw, out.data_ptr(), ldo, M, Nn, K, C.byref(ep),
                                     _dtype_code(a.dtype), _stream()), fn_name)
    if timed:
        e1.record()
        counters.gemm_events.append((e0, e1, 2.0 * M * Nn * K, f"bf16 {M}x{Nn}x{K}" + _epi_tag(bias, act, gate, residual)))
        counters.gemm_bytes.append(2.0 * (M * K + Nn * K + M * Nn * (2 if residual is not None else 1)))
    counters.launches += 1
    return out


def gemm(a, w, bias=None, act: int = ACT_NONE, relu_cols: int = 0, gate=None, residual=None, out=None) -> torch.Tensor:
    """out = epilogue(a @ w.T); a [M, K], w [N, K] (nn.Linear layout).

    epilogue: +bias, activation (ACT_SILU, or ACT_RELU_COLS on the first ``relu_cols``
    columns), * gate, + residual.  ``gate`` = (scale_shift_table [6, N], t [B, 6N], row,
    rows_per_batch).  bf16 runs the tcgen05 tensor-core kernel, fp32 the SIMT kernel."""
    return _gemm("sana_gemm", a, w, bias, act, relu_cols, gate, residual, out)


def gemm_simt(a, w, bias=None, act: int = ACT_NONE, relu_cols: int = 0, gate=None, residual=None, out=None):
    """Same contract as :func:`gemm`, always the SIMT kernel (device-side cross-check)."""
    return _gemm("sana_gemm_simt", a, w, bias, act, relu_cols, gate, residual, out)


def set_gemm_variant(variant: int) -> None:
    """0 = choose per problem, 1 = single-CTA tcgen05 kernel, 2 = CTA-pair (cta_group::2) kernel."""
    _lib.check(_lib.load().sana_gemm_set_variant(variant), "sana_gemm_set_variant")


def take_gemm_device_status() -> int:
    """Code recorded by a timed-out wait inside the tensor-core GEMM (0 = none).  Synchronises."""
    v = C.c_int(0)
    lib = _lib.load()
    _lib.check(lib.sana_gemm_take_device_status(C.byref(v)), "sana_gemm_take_device_status")
    return v.value


class NvFp4Tensor:
    """A [rows, K] matrix quantised to NVFP4: ``q`` packed E2M1 codes [rows, K/2] (uint8),
    ``sf`` E4M3 block scales in the tensor core's 512-byte tiles, ``scales`` = device floats
    (amax, tensor_scale)."""

    __slots__ = ("q", "sf", "scales", "rows", "K")

    def __init__(self, q, sf, scales, rows, K):
        self.q, self.sf, self.scales, self.rows, self.K = q, sf, scales, rows, K

    def dequantize(self) -> torch.Tensor:
        """fp32 [rows, K] reconstruction (torch math; for tests and diagnostics only)."""
        lut = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
                           device=self.q.device)
        codes = torch.stack([self.q & 15, self.q >> 4], dim=-1).reshape(self.rows, self.K).long()
        vals = lut[codes]
        ktiles4 = self.sf.numel() // 512 // ((self.rows + 127) // 128)
        r = torch.arange(self.rows, device=self.q.device)[:, None]
        kb = torch.arange(self.K // 16, device=self.q.device)[None, :]
        off = ((r // 128) * ktiles4 + kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kb % 4
        bs = self.sf.view(torch.float8_e4m3fn).float()[off]
        return (vals.reshape(self.rows, self.K // 16, 16) * (bs * self.scales[1])[..., None]).reshape(self.rows, self.K)


def nvfp4_quantize(x: torch.Tensor) -> NvFp4Tensor:
    """Quantises a bf16 [rows, K] matrix (contiguous rows) along K; K must be a multiple of 32."""
    _need_cuda(x)
    rows, K, ld = _rows2d(x, "nvfp4_quantize x")
    if x.dtype != torch.bfloat16 or K % 32 != 0:
        raise SanaLibraryError("nvfp4_quantize: needs a bf16 matrix with K a multiple of 32")
    lib = _lib.load()
    q = torch.empty(rows, K // 2, dtype=torch.uint8, device=x.device)
    sf = torch.empty(lib.sana_nvfp4_sf_bytes(rows, K), dtype=torch.uint8, device=x.device)
    scales = torch.empty(4, dtype=torch.float32, device=x.device)
    _lib.check(lib.sana_nvfp4_quantize(x.data_ptr(), ld, q.data_ptr(), sf.data_ptr(), scales.data_ptr(), rows, K,
                                       _stream()), "sana_nvfp4_quantize")
    counters.launches += 2
    return NvFp4Tensor(q, sf, scales, rows, K)


class Fp4Buffers:
    """Reusable output buffers of the kernels that emit NVFP4 directly: codes [rows, K/2], scale tiles
    (zero-filled once: the kernels never write the bytes of padding rows and tiles) and the four-float
    scale record {amax in use, tensor scale in use, amax seen since the last roll, unused}."""

    def __init__(self, rows: int, K: int, device, record: Optional[torch.Tensor] = None):
        lib = _lib.load()
        self.rows, self.K = rows, K
        self.q = torch.empty(rows, K // 2, dtype=torch.uint8, device=device)
        self.sf = torch.zeros(lib.sana_nvfp4_sf_bytes(rows, K), dtype=torch.uint8, device=device)
        self.record = record if record is not None else torch.zeros(4, dtype=torch.float32, device=device)

    def tensor(self) -> NvFp4Tensor:
        return NvFp4Tensor(self.q, self.sf, self.record, self.rows, self.K)


def nvfp4_scale_roll(records: torch.Tensor, margin: float = 1.0) -> None:
    """records [n, 4] fp32: adopts each record's "amax seen" (x margin) as its amax / tensor scale in use."""
    _need_cuda(records)
    if records.dtype != torch.float32 or not records.is_contiguous() or records.shape[-1] != 4:
        raise SanaLibraryError("nvfp4_scale_roll: records must be contiguous fp32 [n, 4]")
    _lib.check(_lib.load().sana_nvfp4_scale_roll(records.data_ptr(), records.numel() // 4, margin, _stream()),
               "sana_nvfp4_scale_roll")
    counters.launches += 1


def nvfp4_quantize_scaled(x: torch.Tensor, buf: Fp4Buffers) -> NvFp4Tensor:
    """Quantises bf16 x [rows, K] with the amax in buf.record[0] (nothing is measured)."""
    _need_cuda(x)
    rows, K, ld = _rows2d(x, "nvfp4_quantize_scaled x")
    if x.dtype != torch.bfloat16 or (rows, K) != (buf.rows, buf.K):
        raise SanaLibraryError("nvfp4_quantize_scaled: x must be bf16 of the buffers' shape")
    _lib.check(_lib.load().sana_nvfp4_quantize_scaled(x.data_ptr(), ld, buf.q.data_ptr(), buf.sf.data_ptr(), buf.record.data_ptr(),
                                                      rows, K, _stream()), "sana_nvfp4_quantize_scaled")
    counters.launches += 1
    return buf.tensor()


def ln_modulate_fp4(x: torch.Tensor, table: torch.Tensor, t: torch.Tensor, shift_row: int, scale_row: int, buf: Fp4Buffers,
                    eps: float = 1e-6, keep_bf16: bool = False):
    """:func:`ln_modulate` (bf16) whose output is written as NVFP4 into ``buf`` with the tensor scale of
    buf.record; the largest magnitude produced is accumulated into the record.  Returns the NvFp4Tensor
    (and the bf16 tensor too with ``keep_bf16``)."""
    _need_cuda(x, table, t)
    B, N, Cc = x.shape
    x = x.contiguous()
    table = table.contiguous()
    t = t.reshape(B, 6 * Cc).contiguous()
    if x.dtype != torch.bfloat16 or table.shape != (6, Cc) or table.dtype != x.dtype or t.dtype != x.dtype:
        raise SanaLibraryError("ln_modulate_fp4: bf16 x with table [6, C] and t [B, 6C] in the same dtype")
    if (buf.rows, buf.K) != (B * N, Cc):
        raise SanaLibraryError("ln_modulate_fp4: buffers sized for another shape")
    z = torch.empty_like(x) if keep_bf16 else None
    rec = buf.record
    _lib.check(_lib.load().sana_ln_modulate_fp4(x.data_ptr(), table.data_ptr(), t.data_ptr(), z.data_ptr() if keep_bf16 else None,
                                                buf.q.data_ptr(), buf.sf.data_ptr(), rec.data_ptr(), rec.data_ptr() + 8, B, N, Cc,
                                                shift_row, scale_row, eps, _stream()), "sana_ln_modulate_fp4")
    counters.launches += 1
    return (buf.tensor(), z) if keep_bf16 else buf.tensor()


def la_apply_fp4(q: torch.Tensor, state: torch.Tensor, B: int, N: int, H: int, eps: float, buf: Fp4Buffers,
                 keep_bf16: bool = False):
    """:func:`la_apply` (bf16) whose output is written as NVFP4 into ``buf`` (see :func:`ln_modulate_fp4`)."""
    _need_cuda(q, state)
    rq, cq, ldq = _rows2d(q, "la_apply_fp4 q")
    if rq != B * N or cq != H * HEAD_DIM or q.dtype != torch.bfloat16:
        raise SanaLibraryError("la_apply_fp4: q must be bf16 [B*N, H*32]")
    if state.shape != (B, H, STATE_ROWS, HEAD_DIM) or state.dtype != torch.float32 or not state.is_contiguous():
        raise SanaLibraryError("la_apply_fp4: state must be contiguous fp32 [B, H, 33, 32]")
    if (buf.rows, buf.K) != (B * N, H * HEAD_DIM):
        raise SanaLibraryError("la_apply_fp4: buffers sized for another shape")
    out = torch.empty(B * N, H * HEAD_DIM, dtype=q.dtype, device=q.device) if keep_bf16 else None
    rec = buf.record
    _lib.check(_lib.load().sana_la_apply_fp4(q.data_ptr(), ldq, state.data_ptr(), out.data_ptr() if keep_bf16 else None,
                                             H * HEAD_DIM, buf.q.data_ptr(), buf.sf.data_ptr(), rec.data_ptr(), rec.data_ptr() + 8,
                                             B, N, H, eps, _stream()), "sana_la_apply_fp4")
    counters.launches += 1
    return (buf.tensor(), out) if keep_bf16 else buf.tensor()


def gemm_nvfp4(a: NvFp4Tensor, w: NvFp4Tensor, bias=None, act: int = ACT_NONE, relu_cols: int = 0, gate=None,
               residual=None, out=None) -> torch.Tensor:
    """out [M, N] bf16 = epilogue(dequant(a) @ dequant(w).T) on the block-scaled FP4 tensor cores."""
    if a.K != w.K:
        raise SanaLibraryError(f"gemm_nvfp4: K mismatch ({a.K} vs {w.K})")
    M, Nn, K = a.rows, w.rows, a.K
    if out is None:
        out = torch.empty(M, Nn, dtype=torch.bfloat16, device=a.q.device)
    Mo, No, ldo = _rows2d(out, "gemm_nvfp4 out")
    if Mo != M or No != Nn or out.dtype != torch.bfloat16:
        raise SanaLibraryError("gemm_nvfp4: bad output tensor")
    _need_cuda(bias, residual, out)
    ep, keep = _epilogue(M, Nn, torch.bfloat16, bias, act, relu_cols, gate, residual)
    lib = _lib.load()
    timed = counters.gemm_timing
    if timed:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    _lib.check(lib.sana_gemm_nvfp4(a.q.data_ptr(), a.sf.data_ptr(), a.scales.data_ptr(), w.q.data_ptr(), w.sf.data_ptr(),
                                   w.scales.data_ptr(), out.data_ptr(), ldo, M, Nn, K, C.byref(ep), _stream()),
               "sana_gemm_nvfp4")
    if timed:
        e1.record()
        counters.gemm_events.append((e0, e1, 2.0 * M * Nn * K, f"nvfp4 {M}x{Nn}x{K}" + _epi_tag(bias, act, gate, residual)))
        counters.gemm_bytes.append(0.5625 * (M * K + Nn * K) + 2.0 * M * Nn * (2 if residual is not None else 1))
    counters.launches += 1
    return out


def take_gemm_nvfp4_device_status() -> int:
    v = C.c_int(0)
    lib = _lib.load()
    _lib.check(lib.sana_gemm_nvfp4_take_device_status(C.byref(v)), "sana_gemm_nvfp4_take_device_status")
    return v.value

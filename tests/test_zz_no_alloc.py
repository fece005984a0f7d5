"""The allocation-free variant of the linear-attention state reduction.

Some hosts of this library may not allocate device memory at the point where they run the
block (their memory is a fixed arena owned by another runtime, their sandbox has no
allocation calls, or they cannot afford the device-wide synchronisation an allocation can
trigger).  `sana_la_state_noalloc` serves them: it takes the same inputs and output as
`sana_la_state` but keeps its partial sums in a scratch array built into the library.

This file is collected last on purpose: if it fails, a run that stops at the first failure
has already run every other test.  It calls the entry point through the C ABI directly, on
two different problems in a row (the second must not see leftovers of the first), and
compares with `sana_la_state` within the tolerance of the state tests (normalised max error
<= 1e-5; both run the same kernels in the same order, so the results are in fact equal) and,
independently of that entry point, with the CPU oracle's state evaluated in fp64 on the same
values.
"""
import ctypes as C

import pytest
import torch

from oracle import sana_oracle as O
from sana_b200 import _lib

pytestmark = pytest.mark.gpu
TOL = 1e-5
MAX_BYTES = 16 * 1024 * 1024


def _nmax(a, ref):
    return ((a.double() - ref.double()).abs().max() / ref.double().abs().max().clamp(min=1e-30)).item()


def _both(lib, qkv, B, N, H):
    """Runs the workspace entry point and the allocation-free one on the same k, v."""
    Cc = H * 32
    k, v = qkv[:, Cc:2 * Cc], qkv[:, 2 * Cc:]
    code = _lib.SANA_BF16 if qkv.dtype == torch.bfloat16 else _lib.SANA_F32
    stream = torch.cuda.current_stream().cuda_stream
    ws_bytes = lib.sana_la_state_workspace_bytes(B, N, H)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=qkv.device)
    ref = torch.empty(B, H, 33, 32, dtype=torch.float32, device=qkv.device)
    rc = lib.sana_la_state(k.data_ptr(), v.data_ptr(), qkv.stride(0), ref.data_ptr(), ws.data_ptr(), ws_bytes, B, N, H,
                           code, stream)
    assert rc == 0, lib.sana_last_error()
    # poison the output so that an entry point that silently did nothing cannot pass
    out = torch.full((B, H, 33, 32), float("nan"), dtype=torch.float32, device=qkv.device)
    rc = lib.sana_la_state_noalloc(k.data_ptr(), v.data_ptr(), qkv.stride(0), out.data_ptr(), B, N, H, code, stream)
    assert rc == 0, lib.sana_last_error()
    torch.cuda.synchronize()
    return out, ref


def _oracle_state(qkv, B, N, H):
    Cc = H * 32
    k = torch.relu(qkv[:, Cc:2 * Cc].double().cpu()).reshape(B, N, H, 32)
    v = qkv[:, 2 * Cc:].double().cpu().reshape(B, N, H, 32)
    return O.lite_la_state(k, v)


def test_noalloc_matches_workspace_entry_point_twice_in_a_row(lib):
    g = torch.Generator().manual_seed(0)
    # first call: large enough to use many chunks of the built-in scratch
    B, N, H = 2, 4096, 36
    qkv = torch.randn(B * N, 3 * H * 32, generator=g).bfloat16().cuda()
    out1, ref1 = _both(lib, qkv, B, N, H)
    assert torch.isfinite(out1).all() and _nmax(out1, ref1) <= TOL
    assert _nmax(out1.cpu(), _oracle_state(qkv, B, N, H)) <= TOL
    # second call, different shape and dtype, smaller footprint: stale partials of the first
    # call are still in the scratch and must not leak into the result
    B, N, H = 1, 333, 5
    qkv = torch.randn(B * N, 3 * H * 32, generator=g).cuda()
    out2, ref2 = _both(lib, qkv, B, N, H)
    assert torch.isfinite(out2).all() and _nmax(out2, ref2) <= TOL
    assert _nmax(out2.cpu(), _oracle_state(qkv, B, N, H)) <= TOL
    # and the first problem again gives the first answer again
    B, N, H = 2, 4096, 36
    qkv = torch.randn(B * N, 3 * H * 32, generator=torch.Generator().manual_seed(0)).bfloat16().cuda()
    out3, _ = _both(lib, qkv, B, N, H)
    assert torch.equal(out3, out1)


def test_noalloc_rejects_problems_beyond_the_built_in_scratch(lib):
    B, N, H = 64, 1 << 20, 70
    assert lib.sana_la_state_workspace_bytes(B, N, H) > MAX_BYTES
    x = torch.zeros(64, dtype=torch.float32, device="cuda")
    p = x.data_ptr()
    rc = lib.sana_la_state_noalloc(p, p, H * 32, p, B, N, H, _lib.SANA_BF16, None)
    assert rc == -1
    assert b"built-in scratch" in lib.sana_last_error()

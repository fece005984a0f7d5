"""The tcgen05 cross-attention kernel (bf16, 17..304 keys) against the fp64 softmax attention on the
same bf16 values, and against the warp-level kernel it replaces as the default.

Tolerance 8e-3 (normalised max error), as for the warp-level kernel: the probabilities enter the
second product rounded to bf16 (2^-9 per term) and the output is rounded once."""
import pytest
import torch
import torch.nn.functional as F

from sana_b200 import ops

from conftest import nmax_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 8e-3


def _ref(q, kv, mask, B, N, L, h, hd):
    C = h * hd
    qh = q.double().reshape(B, N, h, hd).transpose(1, 2)
    kh = kv[:, :C].double().reshape(B, L, h, hd).transpose(1, 2)
    vh = kv[:, C:].double().reshape(B, L, h, hd).transpose(1, 2)
    am = ((1 - mask.double()) * -10000.0)[:, None, None] if mask is not None else None
    return F.scaled_dot_product_attention(qh, kh, vh, attn_mask=am).transpose(1, 2).reshape(B * N, C)


def _inputs(B, N, L, h, hd, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    C = h * hd
    q = (torch.randn(B * N, C, generator=g) * scale).bfloat16()
    kv = torch.randn(B * L, 2 * C, generator=g).bfloat16()
    return q, kv


@pytest.fixture()
def tensor_core_kernel():
    ops.set_cross_attention_variant(2)
    yield
    ops.set_cross_attention_variant(0)


@pytest.mark.parametrize("B,N,L,h,hd,masked", [
    (1, 300, 300, 2, 112, False),   # the 1.6B shape: 160 + 144 keys, two 64-channel blocks
    (2, 200, 77, 3, 72, True),      # the 0.6B head: 72 channels (not a multiple of 16), ragged keys and queries
    (1, 129, 17, 1, 16, False),     # smallest covered: 16 + 16 keys of which 17 real, one block
    (2, 1024, 304, 2, 128, True),   # widest: 304 keys x 128 channels
    (1, 256, 160, 4, 64, True),
    (3, 64, 33, 2, 96, False),
    (1, 2048, 300, 20, 112, True),  # more (sample, head) pairs than a CTA sees tiles of: K / V reloads
])
def test_against_fp64_softmax_attention(tensor_core_kernel, B, N, L, h, hd, masked):
    q, kv = _inputs(B, N, L, h, hd, seed=N + L)
    C = h * hd
    mask = None
    if masked:
        mask = torch.ones(B, L)
        for b in range(B):
            mask[b, max(1, L - 5 - 9 * b):] = 0
    ref = _ref(q, kv, mask, B, N, L, h, hd)
    d = kv.to(DEV)
    out = ops.cross_attention(q.to(DEV), d[:, :C], d[:, C:], mask.to(DEV) if masked else None, B, N, L, h, hd)
    assert ops.take_cross_attention_device_status() == 0
    assert out.shape == (B * N, C) and torch.isfinite(out.float()).all()
    assert nmax_err(out, ref) < TOL
    # the kernel it replaces gives the same answer within the same budget
    ops.set_cross_attention_variant(1)
    old = ops.cross_attention(q.to(DEV), d[:, :C], d[:, C:], mask.to(DEV) if masked else None, B, N, L, h, hd)
    assert nmax_err(out, old) < 2 * TOL


def test_late_maximum_takes_the_rescale_path(tensor_core_kernel):
    """Rows whose largest score sits in the second key chunk, far (> 2^8) above everything in the
    first: the kernel must rescale what the first chunk accumulated.  Other rows of the same warp
    keep their shift; a fully masked first chunk (scores near -10000) is the extreme case."""
    B, N, L, h, hd = 1, 256, 300, 2, 112
    C = h * hd
    q, kv = _inputs(B, N, L, h, hd, seed=5)
    kv = kv.float()
    kv[200:230, :C] *= 6.0  # keys 200..229 (second chunk: keys >= 160) dominate for most queries
    kv = kv.bfloat16()
    ref = _ref(q, kv, None, B, N, L, h, hd)
    d = kv.to(DEV)
    out = ops.cross_attention(q.to(DEV), d[:, :C], d[:, C:], None, B, N, L, h, hd)
    assert ops.take_cross_attention_device_status() == 0
    assert nmax_err(out, ref) < TOL
    mask = torch.ones(B, L)
    mask[:, :170] = 0  # every key of the first chunk masked
    ref = _ref(q, kv, mask, B, N, L, h, hd)
    out = ops.cross_attention(q.to(DEV), d[:, :C], d[:, C:], mask.to(DEV), B, N, L, h, hd)
    assert torch.isfinite(out.float()).all() and nmax_err(out, ref) < TOL
    mask[:] = 0  # every key masked: the -10000 cancels, plain softmax
    ref = _ref(q, kv, mask, B, N, L, h, hd)
    out = ops.cross_attention(q.to(DEV), d[:, :C], d[:, C:], mask.to(DEV), B, N, L, h, hd)
    assert nmax_err(out, ref) < TOL
    assert ops.take_cross_attention_device_status() == 0


def test_strided_views_and_uncovered_shapes(tensor_core_kernel):
    """q, k, v and the output may be column slices of wider projections (row strides larger than
    C); shapes outside the tensor-core kernel's range are refused when it is forced."""
    B, N, L, h, hd = 2, 192, 120, 2, 64
    C = h * hd
    g = torch.Generator().manual_seed(9)
    wide_q = torch.randn(B * N, 3 * C, generator=g).bfloat16()
    kv = torch.randn(B * L, 2 * C, generator=g).bfloat16()
    ref = _ref(wide_q[:, C:2 * C], kv, None, B, N, L, h, hd)
    dq, dkv = wide_q.to(DEV), kv.to(DEV)
    out = ops.cross_attention(dq[:, C:2 * C], dkv[:, :C], dkv[:, C:], None, B, N, L, h, hd)
    assert nmax_err(out, ref) < TOL
    with pytest.raises(Exception):
        ops.cross_attention(dq[:B * N, :C], dkv[:B * 8, :C], dkv[:B * 8, C:], None, B, N, 8, h, hd)  # 8 keys
    assert ops.take_cross_attention_device_status() == 0

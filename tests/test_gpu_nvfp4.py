"""NVFP4 path on a B200: the quantiser against the oracle's fake-quantiser (bit for bit) and
the block-scaled tcgen05 GEMM against fp64 math on the dequantised operands (the only
differences are fp32 accumulation order and one bf16 rounding of the output: <= 5e-3
normalised max error); block level: cosine >= 0.995 against the oracle block run on the
dequantised tensors."""
import pytest
import torch
import torch.nn.functional as F

from oracle import sana_oracle as O
from sana_b200 import ops

from conftest import cosine, nmax_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 5e-3


def _r(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


@pytest.mark.parametrize("rows,K", [(1, 32), (128, 64), (200, 96), (333, 2240), (77, 5600), (1024, 256)])
def test_quantiser_matches_oracle_bit_for_bit(rows, K):
    x = _r(rows, K, seed=rows + K, scale=1.7).bfloat16()
    x[0, :16] = 0  # an all-zero block
    if rows > 2:
        x[2, 5] = 40.0  # an outlier that sets the tensor scale
    t = ops.nvfp4_quantize(x.to(DEV))
    vals, bs, ts = O.nvfp4_quantize(x.float())
    ref = O.nvfp4_dequantize(vals, bs, ts)
    got = t.dequantize().cpu()
    assert abs(t.scales[1].item() - ts) == 0.0
    assert abs(t.scales[0].item() - x.float().abs().max().item()) == 0.0
    assert torch.equal(got, ref)
    # codes lie on the E2M1 grid and the quantisation error is bounded by half a step of the block
    assert (got - x.float()).abs().max() <= 0.51 * x.float().abs().max()


GEMM_SHAPES = [(128, 128, 256), (128, 128, 64), (200, 136, 96), (1, 8, 32), (513, 520, 736), (1024, 2240, 2240),
               (300, 2240, 5600), (4096, 6720, 2240)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_nvfp4_plain(M, N, K):
    a, w = _r(M, K, seed=M).bfloat16().to(DEV), _r(N, K, seed=N + 1, scale=0.05).bfloat16().to(DEV)
    qa, qw = ops.nvfp4_quantize(a), ops.nvfp4_quantize(w)
    out = ops.gemm_nvfp4(qa, qw)
    torch.cuda.synchronize()
    assert ops.take_gemm_nvfp4_device_status() == 0
    ref = qa.dequantize().double() @ qw.dequantize().double().t()
    assert out.dtype == torch.bfloat16 and out.shape == (M, N)
    assert nmax_err(out, ref) < TOL
    # and the quantised product tracks the unquantised one (coarse sanity, not a tolerance claim)
    full = a.double() @ w.double().t()
    if K >= 64:
        assert cosine(out, full) > 0.98


@pytest.mark.parametrize("variant", ["bias", "bias_silu", "relu_cols", "gate_res", "bias_gate_res"])
def test_gemm_nvfp4_epilogues(variant):
    B, rpb, N, K = 3, 50, 192, 160
    M = B * rpb - 7
    dt = torch.bfloat16
    a, w = _r(M, K, seed=1).to(dt).to(DEV), _r(N, K, seed=2, scale=0.1).to(dt).to(DEV)
    bias = _r(N, seed=3).to(dt) if "bias" in variant else None
    act = ops.ACT_SILU if "silu" in variant else (ops.ACT_RELU_COLS if variant == "relu_cols" else 0)
    relu_cols = 128 if variant == "relu_cols" else 0
    gate = (_r(6, N, seed=4).to(dt), _r(B, 6 * N, seed=5).to(dt), 5, rpb) if "gate" in variant else None
    res = _r(M, N, seed=6).to(dt) if "res" in variant else None
    qa, qw = ops.nvfp4_quantize(a), ops.nvfp4_quantize(w)
    v = qa.dequantize().double().cpu() @ qw.dequantize().double().cpu().t()
    if bias is not None:
        v = v + bias.double()
    if act == ops.ACT_SILU:
        v = F.silu(v)
    elif act == ops.ACT_RELU_COLS:
        v[:, :relu_cols] = torch.relu(v[:, :relu_cols])
    if gate is not None:
        g = gate[0].double()[gate[2]][None] + gate[1].double().reshape(-1, 6, N)[:, gate[2]]
        v = v * g.repeat_interleave(rpb, dim=0)[:M]
    if res is not None:
        v = v + res.double()
    dgate = (gate[0].to(DEV), gate[1].to(DEV), gate[2], gate[3]) if gate else None
    out = ops.gemm_nvfp4(qa, qw, bias=bias.to(DEV) if bias is not None else None, act=act, relu_cols=relu_cols,
                         gate=dgate, residual=res.to(DEV) if res is not None else None)
    assert nmax_err(out, v) < TOL
    assert ops.take_gemm_nvfp4_device_status() == 0

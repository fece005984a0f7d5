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


@pytest.fixture(params=[1, 2], ids=["single_cta", "cta_pair"])
def kernel_variant(request):
    """Both tensor-core kernels behind sana_gemm_nvfp4: 128 x 128 tiles on one CTA, 256 x 128 on a CTA pair."""
    ops.set_gemm_variant(request.param)
    yield request.param
    ops.set_gemm_variant(0)


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_nvfp4_plain(kernel_variant, M, N, K):
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
def test_gemm_nvfp4_epilogues(kernel_variant, variant):
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


def _fp4_block_case(C, heads, B, HW, L, seed):
    import sana_b200
    from sana_b200 import synthetic

    dt = torch.bfloat16
    shp = synthetic.BlockShape("fp4", C, heads, B, HW, text_len=L)
    params = synthetic.make_block_params(C, shp.ffn_hidden, seed=seed)
    x, y, t = synthetic.make_block_inputs(shp, seed=seed)
    blk = sana_b200.SanaMSBlock(C, heads, mlp_ratio=2.5, attn_type="linear", ffn_type="glumbconv").eval()
    blk.load_state_dict(params, strict=True)
    blk = blk.to(DEV, dt)
    blk.set_nvfp4(True)
    r = lambda v: v.to(dt).float()
    p32 = {k: r(v) for k, v in params.items()}
    ref, a_ref, f_ref = O.sana_ms_block_forward(r(x), r(y), r(t), p32, heads, HW, return_branches=True,
                                               quant_fn=O.nvfp4_fake_quant)
    out = blk(x.to(DEV, dt), y.to(DEV, dt), t.to(DEV, dt), None, HW)
    # the two branches on the oracle's modulated input
    mod = (p32["scale_shift_table"][None] + r(t).reshape(B, 6, -1)).chunk(6, dim=1)
    z1 = O.t2i_modulate(O.layer_norm(r(x)), mod[0], mod[1]).to(dt)
    a = blk.attn(z1.to(DEV), HW=HW)
    f = blk.mlp(z1.to(DEV), HW=HW)
    a_ref1 = O.lite_la_forward(z1.float(), O.sub(p32, "attn"), heads=C // 32, eps=1e-8, quant_fn=O.nvfp4_fake_quant)
    f_ref1 = O.glumbconv_forward(z1.float(), O.sub(p32, "mlp"), HW, quant_fn=O.nvfp4_fake_quant)
    # and the distance of the FP4 block from the unquantised golden block, for the record
    gold = O.sana_ms_block_forward(r(x), r(y), r(t), p32, heads, HW)
    return dict(block=cosine(out, ref), attn=cosine(a, a_ref1), mlp=cosine(f, f_ref1),
                block_err=nmax_err(out, ref), vs_unquantised=cosine(out, gold))


@pytest.mark.parametrize("C,heads,B,HW,L", [(256, 4, 2, (12, 16), 20), (2240, 20, 1, (32, 32), 300)])
def test_nvfp4_block_cosine(C, heads, B, HW, L):
    """Block with NVFP4 projections against the oracle block run on the dequantised tensors:
    cosine >= 0.995 on the LiteLA output, the GLUMBConv output and the block output."""
    res = _fp4_block_case(C, heads, B, HW, L, seed=3)
    print(res)
    assert res["attn"] >= 0.995 and res["mlp"] >= 0.995 and res["block"] >= 0.995, res
    assert ops.take_gemm_nvfp4_device_status() == 0 and ops.take_gemm_device_status() == 0


def test_nvfp4_block_cosine_at_the_benchmark_shape():
    """The FP4 configuration at its stated size - hidden 2240, batch 8, 64 x 64 = 4096 tokens per sample
    (32 768 token rows: the CTA-pair kernels) - against the CPU oracle block run on the dequantised
    tensors: cosine >= 0.995 on the block output and on both branches."""
    res = _fp4_block_case(2240, 20, 8, (64, 64), 300, seed=5)
    print(res)
    assert res["attn"] >= 0.995 and res["mlp"] >= 0.995 and res["block"] >= 0.995, res
    assert ops.take_gemm_nvfp4_device_status() == 0 and ops.take_gemm_device_status() == 0


def _same_fp4(a, b):
    return torch.equal(a.q, b.q) and torch.equal(a.sf, b.sf)


@pytest.mark.parametrize("B,N,C", [(2, 130, 256), (1, 1000, 2240), (3, 64, 96)])
def test_ln_modulate_writes_the_same_fp4_as_the_two_step_path(B, N, C):
    """The LayerNorm-modulate kernel that emits NVFP4 directly against ln_modulate (bf16) followed by the
    stand-alone quantiser: with the same tensor maximum the codes and block scales are equal bit for bit,
    the bf16 copy it can keep is the plain kernel's output, and it reports the maximum it produced."""
    dt = torch.bfloat16
    x = _r(B, N, C, seed=C).to(dt).to(DEV)
    table = _r(6, C, seed=1, scale=0.3).to(dt).to(DEV)
    t = _r(B, 6 * C, seed=2, scale=0.3).to(dt).to(DEV)
    z = ops.ln_modulate(x, table, t, 3, 4)
    ref = ops.nvfp4_quantize(z.reshape(B * N, C))
    buf = ops.Fp4Buffers(B * N, C, DEV)
    buf.record[:2] = ref.scales[:2]
    got, z2 = ops.ln_modulate_fp4(x, table, t, 3, 4, buf, keep_bf16=True)
    assert torch.equal(z2, z) and _same_fp4(got, ref)
    assert buf.record[2].item() == ref.scales[0].item()  # the maximum it saw is the measured one
    got = ops.ln_modulate_fp4(x, table, t, 3, 4, buf)  # without the bf16 copy
    assert _same_fp4(got, ref)
    # against the oracle's quantiser given the same maximum
    vals, bs, ts = O.nvfp4_quantize(z.reshape(B * N, C).float().cpu(), amax=ref.scales[0].item())
    assert torch.equal(got.dequantize().cpu(), O.nvfp4_dequantize(vals, bs, ts))
    # a smaller maximum than the data's: values saturate exactly as in the oracle
    buf.record[0] = ref.scales[0] * 0.5
    buf.record[1] = ref.scales[1] * 0.5
    got = ops.ln_modulate_fp4(x, table, t, 3, 4, buf)
    vals, bs, ts = O.nvfp4_quantize(z.reshape(B * N, C).float().cpu(), amax=ref.scales[0].item() * 0.5)
    assert torch.equal(got.dequantize().cpu(), O.nvfp4_dequantize(vals, bs, ts))


@pytest.mark.parametrize("B,N,H", [(2, 200, 8), (1, 1024, 70), (1, 77, 3)])
def test_la_apply_writes_the_same_fp4_as_the_two_step_path(B, N, H):
    C = H * 32
    g = torch.Generator().manual_seed(H)
    qkv = torch.randn(B * N, 3 * C, generator=g).bfloat16().to(DEV)
    state = ops.la_state(qkv[:, C:2 * C], qkv[:, 2 * C:], B, N, H)
    o = ops.la_apply(qkv[:, :C], state, B, N, H, 1e-8)
    if C % 32 != 0:
        pytest.skip("K must be a multiple of 32")
    ref = ops.nvfp4_quantize(o)
    buf = ops.Fp4Buffers(B * N, C, DEV)
    buf.record[:2] = ref.scales[:2]
    got, o2 = ops.la_apply_fp4(qkv[:, :C], state, B, N, H, 1e-8, buf, keep_bf16=True)
    assert torch.equal(o2, o) and _same_fp4(got, ref)
    assert buf.record[2].item() == ref.scales[0].item()
    assert _same_fp4(ops.la_apply_fp4(qkv[:, :C], state, B, N, H, 1e-8, buf), ref)


def test_dwconv_reports_its_maximum_and_scaled_quantiser_matches():
    hid, W, H = 160, 12, 9
    u = _r(2 * H * W, 2 * hid, seed=4).bfloat16().to(DEV)
    w = _r(2 * hid, 1, 3, 3, seed=5, scale=0.3).bfloat16().to(DEV)
    b = _r(2 * hid, seed=6, scale=0.2).bfloat16().to(DEV)
    ref = ops.dwconv_glu(u, w, b, W, H)
    buf = ops.Fp4Buffers(2 * H * W, hid, DEV)
    out = ops.dwconv_glu(u, w, b, W, H, amax_out=buf.record[2:3])
    assert torch.equal(out, ref) and buf.record[2].item() == ref.float().abs().max().item()
    ops.nvfp4_scale_roll(buf.record.view(1, 4))
    assert buf.record[0].item() == ref.float().abs().max().item() and buf.record[2].item() == 0.0
    measured = ops.nvfp4_quantize(ref)
    assert buf.record[1].item() == measured.scales[1].item()
    assert _same_fp4(ops.nvfp4_quantize_scaled(ref, buf), measured)


@pytest.mark.parametrize("C,heads,B,HW,L", [(256, 4, 2, (12, 16), 20), (2240, 20, 2, (32, 32), 300)])
def test_delayed_scaling_block(C, heads, B, HW, L):
    """Block with the activations quantised where they are produced.  The first forward measures; a second
    forward on the same input uses exactly the measured maxima and therefore reproduces the measuring path
    bit for bit; a forward on other data runs on the previous forward's maxima (times a margin) and stays
    within the cosine bar against the oracle block on dequantised tensors."""
    import sana_b200
    from sana_b200 import synthetic

    dt = torch.bfloat16
    shp = synthetic.BlockShape("fp4", C, heads, B, HW, text_len=L)
    params = synthetic.make_block_params(C, shp.ffn_hidden, seed=11)
    x, y, t = synthetic.make_block_inputs(shp, seed=11)
    blk = sana_b200.SanaMSBlock(C, heads, mlp_ratio=2.5, attn_type="linear", ffn_type="glumbconv").eval()
    blk.load_state_dict(params, strict=True)
    blk = blk.to(DEV, dt)
    xd, yd, td = x.to(DEV, dt), y.to(DEV, dt), t.to(DEV, dt)
    blk.set_nvfp4(True)
    measured = blk(xd, yd, td, None, HW)
    blk.set_nvfp4(True, delayed_scaling=True, margin=1.0)
    first = blk(xd, yd, td, None, HW)   # calibrating forward = the measuring path
    second = blk(xd, yd, td, None, HW)  # producers emit FP4 with the maxima just measured
    assert torch.equal(first, measured) and torch.equal(second, measured)
    before = ops.counters.launches
    blk(xd, yd, td, None, HW)
    fused_launches = ops.counters.launches - before
    blk.set_nvfp4(True)
    before = ops.counters.launches
    blk(xd, yd, td, None, HW)
    assert fused_launches < ops.counters.launches - before  # fewer kernels than the measuring path
    # other data, scales delayed by one forward (margin 1.25 as a serving loop would use)
    blk.set_nvfp4(True, delayed_scaling=True, margin=1.25)
    blk(xd, yd, td, None, HW)
    x2 = (x * 0.9 + 0.05 * torch.randn(x.shape, generator=torch.Generator().manual_seed(1)))
    out = blk(x2.to(DEV, dt), yd, td, None, HW)
    r = lambda v: v.to(dt).float()
    ref = O.sana_ms_block_forward(r(x2), r(y), r(t), {k: r(v) for k, v in params.items()}, heads, HW,
                                  quant_fn=O.nvfp4_fake_quant)
    assert cosine(out, ref) >= 0.995
    assert ops.take_gemm_nvfp4_device_status() == 0


def test_weight_pack_round_trip(tmp_path):
    """Pack the FP4 projection weights of a block, store, load into a fresh block whose bf16
    weights were wiped: the loaded block reproduces the packing block's FP4 output bit for bit
    (so it runs from the packed codes, not from re-quantised weights)."""
    import sana_b200
    from sana_b200 import synthetic

    C, heads, grid = 256, 4, (8, 8)
    shp = synthetic.BlockShape("p", C, heads, 2, grid, text_len=12)
    params = synthetic.make_block_params(C, shp.ffn_hidden, seed=7, std=0.05)
    x, y, t = synthetic.make_block_inputs(shp, seed=7, std=0.05, text_dim=64)
    mk = lambda: sana_b200.SanaMSBlock(C, heads, mlp_ratio=2.5, attn_type="linear", ffn_type="glumbconv").eval()
    a = mk()
    a.load_state_dict(params, strict=True)
    a = a.to(DEV, torch.bfloat16)
    pack = sana_b200.pack_nvfp4_weights(a)
    assert len(pack) == 4 * 4 and all(v.device.type == "cpu" for v in pack.values())
    path = tmp_path / "block.nvfp4.pt"
    torch.save(pack, path)
    a.set_nvfp4(True)
    xd, yd, td = x.to(DEV, torch.bfloat16), y.to(DEV, torch.bfloat16), t.to(DEV, torch.bfloat16)
    ref = a(xd, yd, td, None, grid)
    b = mk()
    b.load_state_dict(params, strict=True)
    b = b.to(DEV, torch.bfloat16)
    assert sana_b200.load_nvfp4_weights(b, torch.load(path)) == 4
    for w in (b.attn.qkv.weight, b.attn.proj.weight, b.mlp.inverted_conv.conv.weight, b.mlp.point_conv.conv.weight):
        w.data.zero_()  # the bf16 copies are not consulted any more
    assert torch.equal(b(xd, yd, td, None, grid), ref)
    with pytest.raises(ValueError):
        sana_b200.load_nvfp4_weights(sana_b200.SanaMSBlock(2 * C, heads, mlp_ratio=2.5, attn_type="linear",
                                                           ffn_type="glumbconv"), pack)

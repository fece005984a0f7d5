"""Kernel-level parity on a B200: every C-ABI entry point against the CPU oracle on the same
seeded inputs.  Tolerances (normalised max error, max|a-ref|/max|ref|): fp32 <= 1e-5; bf16
kernels are compared with the oracle evaluated in fp64 on the bf16-rounded inputs, where
the only differences are the fp32 accumulation order and one bf16 rounding of the output
(<= 2^-8 relative = 3.9e-3; the block-level budget is 2e-2)."""
import pytest
import torch
import torch.nn.functional as F

from oracle import sana_oracle as O
from sana_b200 import ops

from conftest import nmax_err

pytestmark = pytest.mark.gpu

BF16_OUT = 5e-3  # one bf16 rounding of the output plus accumulation-order noise
DEV = "cuda"


def _r(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


# ------------------------------------------------------------------ LN + modulate
@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, BF16_OUT)])
@pytest.mark.parametrize("B,N,C", [(2, 37, 64), (1, 130, 1152), (3, 9, 2240), (1, 5, 4096)])
def test_ln_modulate(dt, tol, B, N, C):
    x, table, t = _r(B, N, C, seed=1, scale=2.0) + 0.3, _r(6, C, seed=2, scale=0.1), _r(B, 6 * C, seed=3, scale=0.5)
    xd, td, tt = x.to(dt), table.to(dt), t.to(dt)
    for (sh, sc) in ((0, 1), (3, 4)):
        z = ops.ln_modulate(xd.to(DEV), td.to(DEV), tt.to(DEV), sh, sc)
        m = (td.double()[None] + tt.double().reshape(B, 6, C))
        ref = O.t2i_modulate(O.layer_norm(xd.double()), m[:, sh:sh + 1], m[:, sc:sc + 1])
        assert z.dtype == dt and nmax_err(z, ref) < tol


# ------------------------------------------------------------------ RMSNorm (qk norm)
@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, BF16_OUT)])
@pytest.mark.parametrize("rows,C", [(37, 64), (300, 1152), (130, 2240)])
def test_rmsnorm_in_place_on_a_column_block(dt, tol, rows, C):
    big = (_r(rows, 3 * C, seed=rows, scale=1.5) + 0.2).to(dt)
    w = (1.0 + 0.2 * _r(C, seed=1)).to(dt)
    ref = O.rms_norm(big[:, C:2 * C].double(), w.double(), 1e-5)
    d = big.to(DEV)
    ops.rmsnorm_(d[:, C:2 * C], w.to(DEV), 1e-5)
    assert nmax_err(d[:, C:2 * C], ref) < tol
    assert torch.equal(d[:, :C].cpu(), big[:, :C]) and torch.equal(d[:, 2 * C:].cpu(), big[:, 2 * C:])


# ------------------------------------------------------------------ linear attention core
def _la_ref(q, k, v, eps):
    """fp64 oracle on token-major [B, N, h, 32] tensors."""
    st = O.lite_la_state(torch.relu(k.double()), v.double())
    return st, O.lite_la_apply(torch.relu(q.double()), st, eps)


@pytest.mark.parametrize("dt,tol_state,tol_out", [(torch.float32, 1e-5, 1e-5), (torch.bfloat16, 1e-5, BF16_OUT)])
@pytest.mark.parametrize("B,N,H", [(1, 16, 1), (2, 100, 3), (1, 1024, 36), (1, 33, 9), (2, 777, 10), (1, 4096, 70)])
def test_la_state_apply(dt, tol_state, tol_out, B, N, H):
    C = H * 32
    qkv = _r(B * N, 3 * C, seed=N + H).to(dt)
    q, k, v = (qkv[:, i * C:(i + 1) * C].reshape(B, N, H, 32) for i in range(3))
    st_ref, o_ref = _la_ref(q, k, v, 1e-8)
    d = qkv.to(DEV)
    state = ops.la_state(d[:, C:2 * C], d[:, 2 * C:], B, N, H)
    assert state.shape == (B, H, 33, 32) and state.dtype == torch.float32
    assert nmax_err(state, st_ref) < tol_state
    out = ops.la_apply(d[:, :C], state, B, N, H, 1e-8)
    assert out.dtype == dt and nmax_err(out.reshape(B, N, H, 32), o_ref) < tol_out
    # bit-reproducible (fixed reduction order)
    state2 = ops.la_state(d[:, C:2 * C], d[:, 2 * C:], B, N, H)
    assert torch.equal(state, state2)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_la_all_negative_query_gives_zero(dt):
    B, N, H = 1, 48, 2
    qkv = _r(B * N, 3 * 64, seed=5).to(dt)
    qkv[7, :64] = -qkv[7, :64].abs() - 0.1
    d = qkv.to(DEV)
    state = ops.la_state(d[:, 64:128], d[:, 128:], B, N, H)
    out = ops.la_apply(d[:, :64], state, B, N, H, 1e-8)
    assert torch.all(out[7] == 0) and torch.isfinite(out).all()


def test_la_state_is_additive_over_token_shards():
    """The sequence-parallel identity: states of disjoint token ranges add up."""
    B, N, H = 1, 1000, 4
    qkv = _r(N, 3 * 128, seed=9).bfloat16().to(DEV)
    full = ops.la_state(qkv[:, 128:256], qkv[:, 256:], B, N, H)
    parts = sum(ops.la_state(qkv[a:b, 128:256], qkv[a:b, 256:], B, b - a, H) for a, b in ((0, 336), (336, 672), (672, 1000)))
    assert nmax_err(parts, full) < 1e-6


def test_la_state_sp_with_one_rank_equals_la_state():
    """The fused reduction + exchange kernel degenerates to the plain reduction for world = 1
    (several steps in a row on the same exchange buffer: both slot parities)."""
    B, N, H = 2, 600, 5
    buf = torch.zeros(ops.la_state_sp_buffer_bytes(B, H), dtype=torch.uint8, device=DEV)
    for step in (1, 2, 3):
        qkv = _r(B * N, 3 * H * 32, seed=step).bfloat16().to(DEV)
        k, v = qkv[:, H * 32:2 * H * 32], qkv[:, 2 * H * 32:]
        got = ops.la_state_sp(k, v, B, N, H, [buf.data_ptr()], 0, 1, step)
        assert torch.equal(got, ops.la_state(k, v, B, N, H))
    assert buf[320:324].view(torch.int32).item() == 0


# ------------------------------------------------------------------ cross-attention softmax core
@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, 8e-3)])
@pytest.mark.parametrize("B,N,L,h,hd,masked", [(2, 30, 9, 4, 16, True), (1, 200, 300, 2, 72, False), (2, 130, 300, 3, 112, True),
                                               (1, 64, 65, 2, 64, True), (1, 1024, 300, 20, 112, False), (3, 77, 1, 1, 128, False)])
def test_cross_attention_core(dt, tol, B, N, L, h, hd, masked):
    """bf16 tolerance: P is rounded to bf16 before the second product (2^-9 per term) plus one
    rounding of the output."""
    C = h * hd
    q = _r(B * N, C, seed=N).to(dt)
    kv = _r(B * L, 2 * C, seed=L + 1).to(dt)
    mask = None
    if masked:
        mask = torch.ones(B, L)
        for b in range(B):
            mask[b, max(1, L - 1 - 2 * b):] = 0
    qh = q.double().reshape(B, N, h, hd).transpose(1, 2)
    kh = kv[:, :C].double().reshape(B, L, h, hd).transpose(1, 2)
    vh = kv[:, C:].double().reshape(B, L, h, hd).transpose(1, 2)
    am = ((1 - mask.double()) * -10000.0)[:, None, None] if masked else None
    ref = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=am).transpose(1, 2).reshape(B * N, C)
    d = kv.to(DEV)
    out = ops.cross_attention(q.to(DEV), d[:, :C], d[:, C:], mask.to(DEV) if masked else None, B, N, L, h, hd)
    assert out.dtype == dt and out.shape == (B * N, C)
    assert nmax_err(out, ref) < tol


# ------------------------------------------------------------------ depthwise conv + GLU
def _dw_ref(u, w, b, frames, H, W):
    """fp64 oracle: per-frame conv2d + chunk + SiLU-GLU, channels-last in/out."""
    C2 = u.shape[-1]
    x = u.double().reshape(frames, H, W, C2).permute(0, 3, 1, 2)
    y = F.conv2d(x, w.double().reshape(C2, 1, 3, 3), None if b is None else b.double(), padding=1, groups=C2)
    a, g = torch.chunk(y, 2, dim=1)
    return (a * F.silu(g)).permute(0, 2, 3, 1).reshape(frames * H * W, C2 // 2)


@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, BF16_OUT)])
@pytest.mark.parametrize("frames,H,W,hid,bias", [(1, 6, 5, 8, True), (2, 4, 7, 160, True), (3, 5, 8, 72, False),
                                                  (1, 32, 32, 2880, True), (4, 9, 33, 200, True), (1, 70, 17, 64, True),
                                                  (1, 4, 2, 16, True), (1, 1, 1, 8, True), (1, 2, 9, 24, False)])
def test_dwconv_glu(dt, tol, frames, H, W, hid, bias):
    C2 = 2 * hid
    u = _r(frames * H * W, C2, seed=hid + W).to(dt)
    w = _r(C2, 1, 3, 3, seed=1, scale=0.3).to(dt)
    b = _r(C2, seed=2, scale=0.2).to(dt) if bias else None
    ref = _dw_ref(u, w, b, frames, H, W)
    out = ops.dwconv_glu(u.to(DEV), w.to(DEV), b.to(DEV) if bias else None, W, H)
    assert out.dtype == dt and out.shape == (frames * H * W, hid)
    assert nmax_err(out, ref) < tol
    assert ops.take_dwconv_glu_device_status() == 0


@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, BF16_OUT)])
def test_dwconv_glu_row_shards_with_halo(dt, tol):
    """Row-range calls with neighbour halos reproduce the full-grid result (frames 3 x 5 rows;
    the cuts at rows 4, 5 (a frame boundary), 9 and 13 cover every halo combination)."""
    frames, H, W, hid = 3, 5, 8, 40
    C2 = 2 * hid
    u = _r(frames * H * W, C2, seed=4).to(dt)
    w = _r(C2, 1, 3, 3, seed=5, scale=0.3).to(dt)
    b = _r(C2, seed=6, scale=0.2).to(dt)
    ref = _dw_ref(u, w, b, frames, H, W)
    ud, wd, bd = u.to(DEV), w.to(DEV), b.to(DEV)
    rows = ud.reshape(frames * H, W, C2)
    cuts = [0, 4, 5, 9, 13, 15]
    outs = []
    for r0, r1 in zip(cuts, cuts[1:]):
        top = rows[r0 - 1].contiguous() if r0 % H != 0 else None
        bot = rows[r1].contiguous() if r1 % H != 0 else None
        outs.append(ops.dwconv_glu(rows[r0:r1].reshape(-1, C2).contiguous(), wd, bd, W, H, row0=r0, halo_top=top,
                                   halo_bot=bot))
    assert nmax_err(torch.cat(outs), ref) < tol
    assert ops.take_dwconv_glu_device_status() == 0
    # CPU oracle of the same sharded computation agrees with the full-grid oracle
    o = O.depthwise_glu_rows(u.double().reshape(frames * H, W, C2)[4:9], u.double().reshape(frames * H, W, C2)[3],
                             u.double().reshape(frames * H, W, C2)[9], w.double(), b.double(), 4, H)
    assert nmax_err(o.reshape(-1, hid), ref[4 * W:9 * W]) < 1e-12


# ------------------------------------------------------------------ projections
def _gemm_ref(a, w, bias, act, relu_cols, gate, residual):
    v = a.double() @ w.double().t()
    if bias is not None:
        v = v + bias.double()
    if act == ops.ACT_SILU:
        v = F.silu(v)
    elif act == ops.ACT_RELU_COLS:
        v[:, :relu_cols] = torch.relu(v[:, :relu_cols])
    if gate is not None:
        table, t, row, rpb = gate
        N = w.shape[0]
        g = table.double()[row][None] + t.double().reshape(-1, 6, N)[:, row]  # [B, N]
        v = v * g.repeat_interleave(rpb, dim=0)[: v.shape[0]]
    if residual is not None:
        v = v + residual.double()
    return v


GEMM_SHAPES = [(128, 128, 64), (200, 136, 72), (1, 8, 8), (300, 448, 2240), (1024, 1152, 1152), (77, 3456, 1152),
               (4096, 2240, 5600), (513, 520, 200)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_bf16_tensor_core_plain(M, N, K):
    a, w = _r(M, K, seed=M).bfloat16(), _r(N, K, seed=N + 1, scale=0.05).bfloat16()
    ref = _gemm_ref(a, w, None, 0, 0, None, None)
    out = ops.gemm(a.to(DEV), w.to(DEV))
    torch.cuda.synchronize()
    assert ops.take_gemm_device_status() == 0
    assert nmax_err(out, ref) < BF16_OUT
    simt = ops.gemm_simt(a.to(DEV), w.to(DEV))
    assert nmax_err(simt, ref) < BF16_OUT


@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, BF16_OUT)])
@pytest.mark.parametrize("variant", ["bias", "bias_silu", "relu_cols", "gate_res", "bias_gate_res", "res"])
def test_gemm_epilogues(dt, tol, variant):
    B, rpb, N, K = 3, 50, 192, 136
    M = B * rpb - 7  # last batch element is ragged
    a, w = _r(M, K, seed=1).to(dt), _r(N, K, seed=2, scale=0.1).to(dt)
    bias = _r(N, seed=3).to(dt) if "bias" in variant else None
    act = ops.ACT_SILU if "silu" in variant else (ops.ACT_RELU_COLS if variant == "relu_cols" else 0)
    relu_cols = 128 if variant == "relu_cols" else 0
    gate = (_r(6, N, seed=4).to(dt), _r(B, 6 * N, seed=5).to(dt), 2, rpb) if "gate" in variant else None
    res = _r(M, N, seed=6).to(dt) if "res" in variant else None
    ref = _gemm_ref(a, w, bias, act, relu_cols, gate, res)
    dgate = (gate[0].to(DEV), gate[1].to(DEV), gate[2], gate[3]) if gate else None
    out = ops.gemm(a.to(DEV), w.to(DEV), bias=bias.to(DEV) if bias is not None else None, act=act, relu_cols=relu_cols,
                   gate=dgate, residual=res.to(DEV) if res is not None else None)
    assert out.dtype == dt and nmax_err(out, ref) < tol
    if dt == torch.bfloat16:
        assert ops.take_gemm_device_status() == 0


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("M,N,K", [(256, 224, 64), (300, 448, 2240), (1, 8, 8), (513, 520, 200), (4096, 2240, 5600),
                                   (2050, 6720, 2240)])
def test_gemm_bf16_both_tensor_core_kernels(variant, M, N, K):
    """Single-CTA (1) and CTA-pair / cta_group::2 (2) kernels, forced, with the full epilogue."""
    B, rpb = 3, (M + 2) // 3
    a, w = _r(M, K, seed=M).bfloat16(), _r(N, K, seed=N + 1, scale=0.05).bfloat16()
    bias = _r(N, seed=3).bfloat16()
    gate = (_r(6, N, seed=4).bfloat16(), _r(B, 6 * N, seed=5).bfloat16(), 2, rpb)
    res = _r(M, N, seed=6).bfloat16()
    ref_plain = _gemm_ref(a, w, None, 0, 0, None, None)
    ref_full = _gemm_ref(a, w, bias, 0, 0, gate, res)
    ref_silu = _gemm_ref(a, w, bias, ops.ACT_SILU, 0, None, None)
    ops.set_gemm_variant(variant)
    try:
        ad, wd = a.to(DEV), w.to(DEV)
        out_plain = ops.gemm(ad, wd)
        out_full = ops.gemm(ad, wd, bias=bias.to(DEV), gate=(gate[0].to(DEV), gate[1].to(DEV), 2, rpb), residual=res.to(DEV))
        out_silu = ops.gemm(ad, wd, bias=bias.to(DEV), act=ops.ACT_SILU)
        torch.cuda.synchronize()
    finally:
        ops.set_gemm_variant(0)
    assert ops.take_gemm_device_status() == 0
    assert nmax_err(out_plain, ref_plain) < BF16_OUT
    assert nmax_err(out_full, ref_full) < BF16_OUT
    assert nmax_err(out_silu, ref_silu) < BF16_OUT


def test_gemm_strided_operands():
    """A and the output may be column slices of wider tensors (qkv slices, residual views)."""
    M, N, K = 160, 64, 96
    big = _r(M, 3 * K, seed=1).bfloat16().to(DEV)
    w = _r(N, K, seed=2, scale=0.1).bfloat16().to(DEV)
    a = big[:, K:2 * K]
    outbuf = torch.zeros(M, 2 * N, dtype=torch.bfloat16, device=DEV)
    ops.gemm(a, w, out=outbuf[:, N:])
    ref = _gemm_ref(a.cpu(), w.cpu(), None, 0, 0, None, None)
    assert nmax_err(outbuf[:, N:], ref) < BF16_OUT and torch.all(outbuf[:, :N] == 0)


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("M,N,K", [(2050, 328, 200), (77, 72, 64), (2307, 2240, 136), (9450, 2240, 136), (9450, 2208, 72)])
def test_gemm_staged_epilogue_edges(variant, M, N, K):
    """The bulk-tensor epilogue on ragged tiles: rows and columns that end inside a 32 x 64 box,
    the output a column slice of a wider buffer (its neighbours must stay untouched), the
    residual read in place from the output location, bias + gate on top.  The 9 450-row cases are one eighth of a 75 600-token
    grid (37 row tiles of the CTA-pair kernel, the last one 234 rows); N = 2208 ends in a 160-column tile."""
    rpb = 500
    B = (M + rpb - 1) // rpb
    a = _r(M, K, seed=M).bfloat16().to(DEV)
    w = _r(N, K, seed=N, scale=0.1).bfloat16().to(DEV)
    bias = _r(N, seed=3, scale=0.2).bfloat16().to(DEV)
    table = _r(6, N, seed=4, scale=0.3).bfloat16().to(DEV)
    t = _r(B, 6 * N, seed=5, scale=0.3).bfloat16().to(DEV)
    buf = _r(M, N + 128, seed=6).bfloat16().to(DEV)
    before = buf.clone()
    view = buf[:, 64:64 + N]
    ref = _gemm_ref(a.cpu(), w.cpu(), bias.cpu(), 0, 0, (table.cpu(), t.cpu(), 2, rpb), before[:, 64:64 + N].cpu())
    ops.set_gemm_variant(variant)
    try:
        ops.gemm(a, w, bias=bias, gate=(table, t, 2, rpb), residual=view, out=view)
    finally:
        ops.set_gemm_variant(0)
    assert nmax_err(view, ref) < BF16_OUT
    assert torch.equal(buf[:, :64], before[:, :64]) and torch.equal(buf[:, 64 + N:], before[:, 64 + N:])
    assert ops.take_gemm_device_status() == 0


def test_gemm_full_size_sampled_rows():
    """The 1.6B-width QKV projection at 16 384 tokens, checked on rows sampled from every
    128-row tile position against the CPU oracle."""
    M, N, K = 16384, 6720, 2240
    g = torch.Generator(device=DEV).manual_seed(0)
    a = torch.randn(M, K, generator=g, device=DEV).bfloat16()
    w = (torch.randn(N, K, generator=g, device=DEV) * 0.02).bfloat16()
    out = ops.gemm(a, w)
    torch.cuda.synchronize()
    assert ops.take_gemm_device_status() == 0
    rows = torch.arange(0, M, 129)[:100]
    ref = a[rows].cpu().double() @ w.cpu().double().t()
    assert nmax_err(out[rows], ref) < BF16_OUT


def test_dwconv_glu_long_segments_sampled_channels():
    """Full 1.6B width on four 128-row frames: the launch uses 256-row segments (two frames per
    warp, so frame edges fall inside a segment); checked on a sample of channels against the
    fp64 oracle evaluated on those channels only."""
    frames, H, W, hid = 4, 128, 128, 5600
    C2 = 2 * hid
    g = torch.Generator(device=DEV).manual_seed(11)
    u = (torch.randn(frames * H * W, C2, generator=g, device=DEV) * 0.7).bfloat16()
    w = (torch.randn(C2, 1, 3, 3, generator=g, device=DEV) * 0.3).bfloat16()
    b = (torch.randn(C2, generator=g, device=DEV) * 0.2).bfloat16()
    out = ops.dwconv_glu(u, w, b, W, H)
    assert ops.take_dwconv_glu_device_status() == 0
    pick = torch.tensor([0, 1, 63, 64, 65, 2047, 2048, 5535, 5567, 5568, 5598, 5599], device=DEV)
    both = torch.cat([pick, pick + hid])
    ref = _dw_ref(u[:, both].cpu(), w[both].cpu(), b[both].cpu(), frames, H, W)
    assert nmax_err(out[:, pick], ref) < BF16_OUT

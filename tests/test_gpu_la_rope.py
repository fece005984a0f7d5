"""ReLU-then-rotate linear attention (upstream's LiteLAReLURope) on a B200 against the CPU oracle.

Tolerances (normalised max error): fp32 <= 1e-5.  bf16: the rotated k is rounded to bf16 before
the first product (as upstream's `type_as`), so the state differs from the fp64 oracle on the
bf16 inputs by 2^-9 per term with random sign (<= 3e-3 after the sum); the output adds the bf16
rounding of the state, of the rotated q and of the result (<= 1e-2; the block budget is 2e-2)."""
import pytest
import torch

from oracle import sana_oracle as O
import sana_b200
from sana_b200 import ops

from conftest import nmax_err

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _r(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


def _tables(N, D, seed):
    """Unit complex numbers with arbitrary angles, as fp64 complex [1, 1, N, D/2] and fp32 tables."""
    ang = _r(N, D // 2, seed=seed, scale=3.0).double()
    return torch.polar(torch.ones_like(ang), ang)[None, None], ang.cos().float(), ang.sin().float()


def _rot(a, fr):
    """a [B, N, h, d] real fp64, fr complex [1, 1, N, d/2] -> rotated pairs, [B, N, h, d]."""
    f = fr[0, 0][None, :, None, :]
    return torch.view_as_real(torch.view_as_complex(a.unflatten(-1, (-1, 2)).contiguous()) * f).flatten(-2)


def _reference(qkv, B, N, H, D, fr, eps):
    q, k, v = (qkv[:, i * H * D:(i + 1) * H * D].double().reshape(B, N, H, D) for i in range(3))
    q, k = q.relu(), k.relu()
    state = O.lite_la_rope_state(k, _rot(k, fr), v)
    return state, O.lite_la_rope_apply(q, _rot(q, fr), state, eps)


@pytest.mark.parametrize("dt,tol_state,tol_out", [(torch.float32, 1e-5, 1e-5), (torch.bfloat16, 3e-3, 1e-2)])
@pytest.mark.parametrize("B,N,H,D", [(1, 16, 1, 16), (2, 100, 3, 48), (1, 1, 2, 32), (1, 63, 2, 112), (2, 65, 1, 128),
                                     (1, 1000, 5, 112), (2, 777, 2, 64), (1, 4096, 20, 112), (1, 300, 3, 80),
                                     (1, 129, 2, 96)])
def test_la_rope_state_apply(dt, tol_state, tol_out, B, N, H, D):
    C = H * D
    qkv = (_r(B * N, 3 * C, seed=N + H + D) + 0.1).to(dt)
    fr, cos, sin = _tables(N, D, seed=D)
    st_ref, o_ref = _reference(qkv, B, N, H, D, fr, 1e-8)
    d, cos, sin = qkv.to(DEV), cos.to(DEV), sin.to(DEV)
    state = ops.la_rope_state(d[:, C:2 * C], d[:, 2 * C:], cos, sin, B, N, H, D)
    assert state.shape == (B, H, D + 1, D) and state.dtype == torch.float32
    assert nmax_err(state[:, :, :D], st_ref[:, :, :D]) < tol_state
    assert nmax_err(state[:, :, D], st_ref[:, :, D]) < 1e-5  # the key sum is fp32 in both dtypes
    out = ops.la_rope_apply(d[:, :C], cos, sin, state, B, N, H, D, 1e-8)
    assert out.dtype == dt and torch.isfinite(out).all()
    assert nmax_err(out.reshape(B, N, H, D), o_ref) < tol_out
    # bit-reproducible (fixed reduction order)
    assert torch.equal(state, ops.la_rope_state(d[:, C:2 * C], d[:, 2 * C:], cos, sin, B, N, H, D))
    assert ops.take_la_rope_device_status() == 0  # no bounded wait timed out


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_la_rope_identity_rotation_matches_plain_sums(dt):
    """cos = 1, sin = 0: the state is sum v k^T and the output the plain ReLU linear attention."""
    B, N, H, D = 1, 200, 2, 48
    C = H * D
    qkv = _r(B * N, 3 * C, seed=3).to(dt)
    cos, sin = torch.ones(N, D // 2, device=DEV), torch.zeros(N, D // 2, device=DEV)
    d = qkv.to(DEV)
    state = ops.la_rope_state(d[:, C:2 * C], d[:, 2 * C:], cos, sin, B, N, H, D)
    q, k, v = (qkv[:, i * C:(i + 1) * C].double().reshape(B, N, H, D) for i in range(3))
    vk = torch.einsum("bnhi,bnhj->bhij", v, k.relu())
    assert nmax_err(state[:, :, :D], vk) < 1e-5  # exact bf16 products, fp32 sums
    out = ops.la_rope_apply(d[:, :C], cos, sin, state, B, N, H, D, 1e-8)
    ref = torch.einsum("bhij,bnhj->bnhi", vk, q.relu()) / (torch.einsum("bhj,bnhj->bnh", k.relu().sum(1), q.relu())[..., None] + 1e-8)
    assert nmax_err(out.reshape(B, N, H, D), ref) < (1e-5 if dt == torch.float32 else 8e-3)


def test_la_rope_all_negative_query_gives_zero():
    B, N, H, D = 1, 70, 2, 48
    C = H * D
    qkv = _r(B * N, 3 * C, seed=5).bfloat16()
    qkv[7, :C] = -qkv[7, :C].abs() - 0.1
    _, cos, sin = _tables(N, D, seed=1)
    d, cos, sin = qkv.to(DEV), cos.to(DEV), sin.to(DEV)
    state = ops.la_rope_state(d[:, C:2 * C], d[:, 2 * C:], cos, sin, B, N, H, D)
    out = ops.la_rope_apply(d[:, :C], cos, sin, state, B, N, H, D, 1e-8)
    assert torch.all(out[7] == 0) and torch.isfinite(out).all()


def test_la_rope_state_is_additive_over_token_shards():
    B, N, H, D = 1, 1000, 2, 112
    C = H * D
    qkv = _r(N, 3 * C, seed=9).bfloat16().to(DEV)
    _, cos, sin = _tables(N, D, seed=2)
    cos, sin = cos.to(DEV), sin.to(DEV)
    full = ops.la_rope_state(qkv[:, C:2 * C], qkv[:, 2 * C:], cos, sin, B, N, H, D)
    parts = sum(ops.la_rope_state(qkv[a:b, C:2 * C], qkv[a:b, 2 * C:], cos[a:b].contiguous(), sin[a:b].contiguous(), B,
                                  b - a, H, D) for a, b in ((0, 336), (336, 672), (672, 1000)))
    assert nmax_err(parts, full) < 1e-6


def test_la_rope_rejects_bad_shapes():
    d = torch.zeros(32, 3 * 40, device=DEV, dtype=torch.bfloat16)
    t = torch.zeros(32, 20, device=DEV)
    with pytest.raises(sana_b200.SanaLibraryError):
        ops.la_rope_state(d[:, 40:80], d[:, 80:], t, t, 1, 32, 1, 40)  # head dimension not a multiple of 16
    d = torch.zeros(32, 3 * 48, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(sana_b200.SanaLibraryError):
        ops.la_rope_state(d[:, 48:96], d[:, 96:], t, t, 1, 32, 1, 48)  # tables of the wrong width


# ------------------------------------------------------------------ the module against upstream's outputs
@pytest.mark.parametrize("norm", ["", "_qknorm"])
@pytest.mark.parametrize("tag,dt,tol", [("f32", torch.float32, 1e-5), ("bf16", torch.bfloat16, 2e-2)])
def test_module_matches_upstream_fixture(golden, tag, dt, tol, norm):
    g = golden("litela_relu_rope")
    C, heads = g["C"], g["heads"]
    m = sana_b200.LiteLAReLURope(C, C, heads=heads, eps=1e-8, qk_norm=bool(norm))
    m.load_state_dict({**g["params"], **(g["norm_params"] if norm else {})}, strict=True)
    m = m.to(DEV, dt).eval()
    with torch.no_grad():
        out = m(g["x"].to(DEV, dt), rotary_emb=g["freqs"])
    ref64 = O.lite_la_relu_rope_forward(g["x"].double(), {k: v.double() for k, v in
                                                          {**g["params"], **(g["norm_params"] if norm else {})}.items()},
                                        heads, g["freqs"], eps=1e-8)
    assert out.dtype == dt
    assert nmax_err(out, g[f"out{norm}_f32"]) < tol and nmax_err(out, ref64) < tol
    if dt == torch.bfloat16:  # no further from the fp64 result than upstream's own bf16 run, up to rounding noise
        assert nmax_err(out, ref64) < 2 * nmax_err(g[f"out{norm}_bf16"], ref64) + 4e-3


@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_module_video_head_width(dt, tol):
    """Heads of 112 channels (upstream's 2B video model) on a 3 x 8 x 13 token grid."""
    C, heads, fhw, B = 224, 2, (3, 8, 13), 2
    N = fhw[0] * fhw[1] * fhw[2]
    p = {"qkv.weight": _r(3 * C, C, seed=1, scale=0.06), "proj.weight": _r(C, C, seed=2, scale=0.06),
         "proj.bias": _r(C, seed=3, scale=0.05)}
    x = _r(B, N, C, seed=4, scale=0.8)
    freqs = sana_b200.wan_rotary_freqs(C // heads, fhw)
    m = sana_b200.LiteLAReLURope(C, C, heads=heads, eps=1e-8)
    m.load_state_dict(p, strict=True)
    m = m.to(DEV, dt).eval()
    pd = {k: v.to(dt).double() for k, v in p.items()}
    ref = O.lite_la_relu_rope_forward(x.to(dt).double(), pd, heads, freqs, eps=1e-8)
    with torch.no_grad():
        out = m(x.to(DEV, dt), rotary_emb=freqs.to(DEV))
        again = m(x.to(DEV, dt), rotary_emb=(freqs[0, 0].real.float(), freqs[0, 0].imag.float()))
    assert nmax_err(out, ref) < tol and torch.equal(out, again)


# ------------------------------------------------------------------ the video block against upstream's outputs
def _video_params(g):
    from sana_b200 import synthetic
    p = synthetic.make_block_params(g["C"], g["hid"], g["param_seed"], std=g["param_std"])
    p["mlp.t_conv.weight"] = g["t_conv"]
    return p


@pytest.mark.parametrize("tname", ["t", "t_frames"])
@pytest.mark.parametrize("tag,dt,tol", [("f32", torch.float32, 1e-5), ("bf16", torch.bfloat16, 2e-2)])
def test_video_block_matches_upstream_fixture(golden, tag, dt, tol, tname):
    """SanaVideoMSBlock: LiteLAReLURope + cross-attention + GLUMBConvTemp, one modulation per sample
    (t [B, 6C]) and one per frame (t [B, 1, F, 6C])."""
    g = golden("video_block")
    C = g["C"]
    blk = sana_b200.SanaVideoMSBlock(C, g["heads"], mlp_ratio=g["hid"] / C, attn_type="LiteLAReLURope",
                                     ffn_type="GLUMBConvTemp", linear_head_dim=g["linear_head_dim"])
    blk.load_state_dict(_video_params(g), strict=True)
    blk = blk.to(DEV, dt).eval()
    with torch.no_grad():
        out = blk(g["x"].to(DEV, dt), g["y"].to(DEV, dt), g[tname].to(DEV, dt), mask=g["mask"].to(DEV), THW=g["THW"],
                  rotary_emb=g["freqs"])
    key = "out_" if tname == "t" else "out_frames_"
    assert out.dtype == dt and nmax_err(out, g[key + "f32"]) < tol
    if dt == torch.bfloat16:  # no further from upstream's fp32 result than upstream's own bf16 run, up to rounding noise
        assert nmax_err(out, g[key + "f32"]) < 2 * nmax_err(g[key + "bf16"], g[key + "f32"]) + 4e-3


def test_video_block_with_spatial_ffn_and_plain_linear_attention():
    """The other covered options: GLUMBConv per frame, and LiteLA (no rotation) as the self-attention."""
    from sana_b200 import synthetic
    C, hid, THW, B, L = 64, 160, (2, 4, 6), 2, 5
    N = THW[0] * THW[1] * THW[2]
    p = synthetic.make_block_params(C, hid, 21, std=0.06)
    x, y, t = _r(B, N, C, seed=1, scale=0.7), _r(B, L, C, seed=2, scale=0.7), _r(B, 6 * C, seed=3, scale=0.3)
    blk = sana_b200.SanaVideoMSBlock(C, 2, mlp_ratio=hid / C, attn_type="linear", ffn_type="glumbconv", linear_head_dim=32)
    blk.load_state_dict(p, strict=True)
    blk = blk.to(DEV).eval()
    ref = O.sana_ms_block_forward(x, y, t, p, 2, THW)
    with torch.no_grad():
        out = blk(x.to(DEV), y.to(DEV), t.to(DEV), THW=THW)
    assert nmax_err(out, ref) < 1e-5
    fr = sana_b200.wan_rotary_freqs(16, THW)
    blk2 = sana_b200.SanaVideoMSBlock(C, 2, mlp_ratio=hid / C, attn_type="LiteLAReLURope", ffn_type="glumbconv",
                                      linear_head_dim=16)
    blk2.load_state_dict(p, strict=True)
    blk2 = blk2.to(DEV).eval()
    ref2 = O.sana_video_block_forward(x, y, t, p, 2, THW, fr, linear_head_dim=16)
    with torch.no_grad():
        out2 = blk2(x.to(DEV), y.to(DEV), t.to(DEV), THW=THW, rotary_emb=fr)
    assert nmax_err(out2, ref2) < 1e-5


def test_rotated_attention_on_sequence_shards_emulated_on_one_gpu():
    """A (frames x rows) grid cut into contiguous row ranges: per-shard states with the shard's slice of
    the rotation tables add up to the full state, and the per-shard outputs concatenate to the full
    output.  The module on a one-rank shard equals the unsharded module."""
    from sana_b200 import sharding
    frames, H, W, heads, D = 3, 6, 8, 2, 48
    C, N = heads * D, 3 * 6 * 8
    qkv = _r(N, 3 * C, seed=7).bfloat16().to(DEV)
    freqs = sana_b200.wan_rotary_freqs(D, (frames, H, W))
    cos, sin = freqs[0, 0].real.float().to(DEV).contiguous(), freqs[0, 0].imag.float().to(DEV).contiguous()
    full_state = ops.la_rope_state(qkv[:, C:2 * C], qkv[:, 2 * C:], cos, sin, 1, N, heads, D)
    full_out = ops.la_rope_apply(qkv[:, :C], cos, sin, full_state, 1, N, heads, D, 1e-8)
    for world in (2, 4):
        shards = [sharding.SequenceShard(frames, H, W, r, world) for r in range(world)]
        parts = []
        for s in shards:
            a, b = s.token_range
            parts.append(ops.la_rope_state(qkv[a:b, C:2 * C], qkv[a:b, 2 * C:], cos[a:b].contiguous(), sin[a:b].contiguous(),
                                           1, b - a, heads, D))
        total = torch.stack(parts).sum(0)
        assert nmax_err(total, full_state) < 1e-6
        outs = [ops.la_rope_apply(qkv[s.token_range[0]:s.token_range[1], :C], cos[s.token_range[0]:s.token_range[1]].contiguous(),
                                  sin[s.token_range[0]:s.token_range[1]].contiguous(), total, 1, s.tokens, heads, D, 1e-8)
                for s in shards]
        assert nmax_err(torch.cat(outs), full_out) < 1e-2
    m = sana_b200.LiteLAReLURope(C, C, heads=heads, eps=1e-8).to(DEV, torch.bfloat16).eval()
    x = _r(1, N, C, seed=8).bfloat16().to(DEV)
    with torch.no_grad():
        ref = m(x, rotary_emb=freqs)
        m.seq_shard = sharding.SequenceShard(frames, H, W, 0, 1)
        got = m(x, rotary_emb=freqs)
    assert torch.equal(ref, got)


def test_la_rope_state_sp_with_one_rank_equals_la_rope_state():
    """The reduction fused with the peer-memory exchange degenerates to the plain reduction for world = 1 (three
    steps on the same buffer: both slot parities).  20 heads of 112 channels: more state elements than one
    resident wave of threads, so the kernel's threads stride over them."""
    B, N, H, D = 2, 700, 20, 112
    buf = torch.zeros(ops.la_rope_state_sp_buffer_bytes(B, H, D), dtype=torch.uint8, device=DEV)
    cos, sin = (t.to(DEV) for t in _tables(N, D, seed=4)[1:])
    for step in (1, 2, 3):
        g = torch.Generator().manual_seed(step)
        kv = torch.randn(B * N, 2 * H * D, generator=g).bfloat16().to(DEV)
        k, v = kv[:, :H * D], kv[:, H * D:]
        got = ops.la_rope_state_sp(k, v, cos, sin, B, N, H, D, [buf.data_ptr()], 0, 1, step)
        assert torch.equal(got, ops.la_rope_state(k, v, cos, sin, B, N, H, D))
    assert buf[320:324].view(torch.int32).item() == 0
    assert ops.la_rope_state_sp_buffer_bytes(B, H, 40) == 0  # heads of 40 channels: not a multiple of 16

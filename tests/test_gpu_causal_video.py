"""The autoregressive variants of the Sana-Video block parts on a B200, against the outputs of the unmodified
upstream modules (tests/golden/causal_video.pt): ChunkCausalAttention, and CachedCausalAttention /
CachedGLUMBConvTemp called chunk after chunk with the cache list handed on.  fp32 <= 1e-5; bf16 <= 2e-2 and no
further from upstream's fp32 result than twice upstream's own bf16 run plus 4e-3 (normalised max error)."""
import pytest
import torch

import sana_b200
from oracle import sana_oracle as O
from sana_b200 import ops

from conftest import nmax_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
CASES = [("f32", torch.float32, 1e-5), ("bf16", torch.bfloat16, 2e-2)]


def _close(out, g, key, dt, tol):
    err = nmax_err(out, g[key + "_f32"])
    assert err < tol, (key, err)
    if dt == torch.bfloat16:
        assert err < 2 * nmax_err(g[key + "_bf16"], g[key + "_f32"]) + 4e-3, (key, err)


@pytest.mark.parametrize("tag,dt,tol", CASES)
def test_chunk_causal_attention(golden, tag, dt, tol):
    g = golden("causal_video")
    C, heads, fhw = g["C"], g["heads"], g["fhw"]
    m = sana_b200.ChunkCausalAttention(C, C, heads=heads, eps=1e-8).eval()
    m.load_state_dict(g["params"], strict=True)
    m = m.to(DEV, dt)
    x = g["x"].to(DEV, dt)
    with torch.no_grad():
        out = m(x, HW=fhw, rotary_emb=g["freqs"], chunk_index=list(g["chunk_index"]))
        whole = m(x, HW=fhw, rotary_emb=g["freqs"])  # one chunk: the plain rotated attention
    _close(out, g, "chunk", dt, tol)
    p = {k: v.to(dt).double() for k, v in g["params"].items()}
    ref = O.lite_la_relu_rope_forward(g["x"].to(dt).double(), p, heads, g["freqs"], eps=1e-8)
    assert nmax_err(whole, ref) < tol
    assert nmax_err(out, whole) > 1e-3  # the cut really changes what the early frames see
    assert ops.take_la_rope_device_status() == 0


@pytest.mark.parametrize("tag,dt,tol", CASES)
def test_chunk_temporal_ffn(golden, tag, dt, tol):
    """ChunkGLUMBConvTemp: the next-frame tap stops at the chunk cuts, the previous-frame tap crosses them."""
    g = golden("causal_video")
    C, fhw, hid = g["C"], g["fhw"], g["hid"]
    ffn = sana_b200.ChunkGLUMBConvTemp(in_features=C, hidden_features=hid, use_bias=(True, True, False),
                                       norm=(None, None, None), act=("silu", "silu", None)).eval()
    ffn.load_state_dict(g["mlp_params"], strict=True)
    ffn = ffn.to(DEV, dt)
    x = g["x"].to(DEV, dt)
    with torch.no_grad():
        out = ffn(x, HW=fhw, chunk_index=list(g["chunk_index"]))
        whole = ffn(x, HW=fhw)
    _close(out, g, "chunk_ffn", dt, tol)
    mp = {k: v.to(dt).double() for k, v in g["mlp_params"].items()}
    assert nmax_err(whole, O.glumbconv_temp_forward(g["x"].to(dt).double(), mp, fhw)) < tol
    assert nmax_err(out, whole) > 1e-3


@pytest.mark.parametrize("per_frame", [False, True])
def test_chunk_causal_video_block_equals_the_parts(golden, per_frame):
    """SanaVideoMSBlock with upstream's names for the chunk-causal pair ("chunkcausal" + "ChunkGLUMBConvTemp"), fp32:
    the fused block (gates in the projection epilogues) against the oracle's parts put together as upstream's
    forward / forward_frame_aware do."""
    from sana_b200 import synthetic
    g = golden("causal_video")
    C, heads, fhw, hid = g["C"], g["heads"], g["fhw"], g["hid"]
    F_, hw = fhw[0], fhw[1] * fhw[2]
    B, N, L = 2, F_ * hw, 6
    p = synthetic.make_block_params(C, hid, 31, std=0.06)
    gen = torch.Generator().manual_seed(32)
    p["mlp.t_conv.weight"] = torch.randn(C, C, 3, 1, generator=gen) * 0.05
    x, y = g["x"], torch.randn(B, L, C, generator=gen) * 0.7
    t = torch.randn(B, 1, F_, 6 * C, generator=gen) * 0.3 if per_frame else torch.randn(B, 6 * C, generator=gen) * 0.3
    ci = list(g["chunk_index"])
    blk = sana_b200.SanaVideoMSBlock(C, heads, mlp_ratio=hid / C, attn_type="chunkcausal", ffn_type="ChunkGLUMBConvTemp",
                                     linear_head_dim=C // heads)
    blk.load_state_dict(p, strict=True)
    blk = blk.to(DEV).eval()
    with torch.no_grad():
        out = blk(x.to(DEV), y.to(DEV), t.to(DEV), THW=fhw, rotary_emb=g["freqs"], chunk_index=ci)
    # the oracle's parts, composed
    tt = t.reshape(B, F_, 6, C) if per_frame else t.reshape(B, 1, 6, C)
    mod = (p["scale_shift_table"][None, None] + tt).chunk(6, dim=-2)  # each [B, F or 1, 1, C]
    rows = lambda v: v.reshape(B, -1, hw if per_frame else N, C)
    z = O.t2i_modulate(rows(O.layer_norm(x)), mod[0], mod[1]).reshape(B, N, C)
    a = O.chunk_causal_forward(z, O.sub(p, "attn"), heads, g["freqs"], fhw, ci, eps=O.BLOCK_LA_EPS)
    x1 = x + (mod[2] * rows(a)).reshape(B, N, C)
    x1 = x1 + O.cross_attention_forward(x1, y, O.sub(p, "cross_attn"), heads)
    z = O.t2i_modulate(rows(O.layer_norm(x1)), mod[3], mod[4]).reshape(B, N, C)
    ref = x1 + (mod[5] * rows(O.chunk_glumbconv_temp_forward(z, O.sub(p, "mlp"), fhw, ci))).reshape(B, N, C)
    assert nmax_err(out, ref) < 1e-5


@pytest.mark.parametrize("tag,dt,tol", CASES)
def test_cached_attention_and_temporal_ffn_chunk_after_chunk(golden, tag, dt, tol):
    g = golden("causal_video")
    C, heads, fhw, hid = g["C"], g["heads"], g["fhw"], g["hid"]
    hw = fhw[1] * fhw[2]
    N = fhw[0] * hw
    att = sana_b200.CachedCausalAttention(C, C, heads=heads, eps=1e-8).eval()
    att.load_state_dict(g["params"], strict=True)
    ffn = sana_b200.CachedGLUMBConvTemp(in_features=C, hidden_features=hid, use_bias=(True, True, False),
                                        norm=(None, None, None), act=("silu", "silu", None)).eval()
    ffn.load_state_dict(g["mlp_params"], strict=True)
    att, ffn = att.to(DEV, dt), ffn.to(DEV, dt)
    fr = g["freqs"].reshape(1, 1, N, -1)
    cache = [None, None, None]
    with torch.no_grad():
        for i in range(2):
            xs = g["x"][:, i * 2 * hw:(i + 1) * 2 * hw].to(DEV, dt)
            o, cache = att(xs, HW=(2, fhw[1], fhw[2]), rotary_emb=fr[:, :, i * 2 * hw:(i + 1) * 2 * hw], save_kv_cache=True,
                           kv_cache=cache)
            _close(o, g, f"cached_attn{i}", dt, tol)
            o, cache = ffn(xs, HW=(2, fhw[1], fhw[2]), save_kv_cache=True, kv_cache=cache)
            _close(o, g, f"cached_ffn{i}", dt, tol)
    # the cache holds upstream's shapes
    d = C // heads
    assert cache[0].shape == (2, heads, d, d) and cache[1].shape == (2, heads, 1, d) and cache[2].shape == (2, C, 1, hw)
    # without a cache list a call returns the tensor only and equals the first chunk's result
    with torch.no_grad():
        xs = g["x"][:, :2 * hw].to(DEV, dt)
        o = att(xs, HW=(2, fhw[1], fhw[2]), rotary_emb=fr[:, :, :2 * hw])
    assert torch.is_tensor(o)
    _close(o, g, "cached_attn0", dt, tol)


def test_cached_video_block_equals_the_parts():
    """SanaVideoMSBlock with the cached attention and temporal FFN, two chunks in a row: the fused block (gate and
    residual in the projection epilogues) against the oracle assembled from the pinned parts."""
    from sana_b200 import synthetic

    C, heads, D, hid, L, B = 96, 2, 48, 240, 5, 2
    T, H, W = 2, 3, 5
    hw, N = H * W, 2 * H * W
    p = synthetic.make_block_params(C, hid, 31, std=0.06)
    g = torch.Generator().manual_seed(31)
    p["mlp.t_conv.weight"] = torch.randn(C, C, 3, 1, generator=g) * 0.05
    xs = [torch.randn(B, N, C, generator=g) * 0.7 for _ in range(2)]
    y = torch.randn(B, L, C, generator=g) * 0.7
    t = torch.randn(B, 6 * C, generator=g) * 0.3
    freqs = sana_b200.wan_rotary_freqs(D, (2 * T, H, W)).reshape(1, 1, 2 * N, -1)
    blk = sana_b200.SanaVideoMSBlock(C, heads, mlp_ratio=hid / C, attn_type="CachedCausalAttention",
                                     ffn_type="CachedGLUMBConvTemp", linear_head_dim=D).eval()
    blk.load_state_dict(p, strict=True)
    blk = blk.to(DEV)
    cache, ocache = [None, None, None], [None, None, None]
    mod = (p["scale_shift_table"][None] + t.reshape(B, 6, -1)).chunk(6, dim=1)
    for i in range(2):
        fr = freqs[:, :, i * N:(i + 1) * N]
        with torch.no_grad():
            out, cache = blk(xs[i].to(DEV), y.to(DEV), t.to(DEV), THW=(T, H, W), rotary_emb=fr, kv_cache=cache, save_kv_cache=True)
        x = xs[i]
        a, ocache = O.cached_causal_forward(O.t2i_modulate(O.layer_norm(x), mod[0], mod[1]), O.sub(p, "attn"), heads, fr, ocache,
                                            True, eps=O.BLOCK_LA_EPS)
        x = x + mod[2] * a
        x = x + O.cross_attention_forward(x, y, O.sub(p, "cross_attn"), heads)
        f, ocache = O.cached_glumbconv_temp_forward(O.t2i_modulate(O.layer_norm(x), mod[3], mod[4]), O.sub(p, "mlp"), (T, H, W),
                                                    ocache, True)
        ref = x + mod[5] * f
        assert nmax_err(out, ref) < 1e-5, i

"""The kernels are also registered as torch custom operators (namespace sana_b200) with fake
implementations: shapes propagate without a GPU; on a GPU they give the direct path's result."""
import pytest
import torch

import sana_b200.torch_ops  # noqa: F401  (registers the operators)
from sana_b200 import ops


def test_operators_are_registered_with_fake_implementations():
    from torch._subclasses.fake_tensor import FakeTensorMode

    for name in ("gemm", "ln_modulate", "la_state", "la_apply", "dwconv_glu", "rmsnorm_", "rope_", "cross_attention",
                 "la_rope_state", "la_rope_apply", "add_f32", "ln_modulate_rows", "patchify", "unpatchify",
                 "timestep_embedding", "silu", "nvfp4_quantize", "gemm_nvfp4"):
        assert hasattr(torch.ops.sana_b200, name), name
    with FakeTensorMode():
        a = torch.empty(100, 64, dtype=torch.bfloat16)
        w = torch.empty(192, 64, dtype=torch.bfloat16)
        qkv = torch.ops.sana_b200.gemm(a, w, None, 0, 0, None, None, 0, 1, None)
        assert qkv.shape == (100, 192) and qkv.dtype == torch.bfloat16
        st = torch.ops.sana_b200.la_state(qkv[:, 64:128], qkv[:, 128:], 1, 100, 2)
        assert st.shape == (1, 2, 33, 32) and st.dtype == torch.float32
        o = torch.ops.sana_b200.la_apply(qkv[:, :64], st, 1, 100, 2, 1e-8)
        assert o.shape == (100, 64)
        u = torch.empty(20 * 5, 320, dtype=torch.bfloat16)
        g = torch.ops.sana_b200.dwconv_glu(u, torch.empty(320, 1, 3, 3, dtype=torch.bfloat16), None, 5, 20, 0, None, None)
        assert g.shape == (100, 160)
        z = torch.ops.sana_b200.ln_modulate(torch.empty(2, 50, 64, dtype=torch.bfloat16), torch.empty(6, 64, dtype=torch.bfloat16),
                                            torch.empty(2, 384, dtype=torch.bfloat16), 0, 1, 1e-6)
        assert z.shape == (2, 50, 64)


@pytest.mark.gpu
def test_custom_ops_match_the_direct_path():
    g = torch.Generator().manual_seed(0)
    a = torch.randn(160, 96, generator=g).bfloat16().cuda()
    w = (torch.randn(192, 96, generator=g) * 0.1).bfloat16().cuda()
    b = torch.randn(192, generator=g).bfloat16().cuda()
    r = torch.randn(160, 192, generator=g).bfloat16().cuda()
    via_op = torch.ops.sana_b200.gemm(a, w, b, ops.ACT_SILU, 0, None, None, 0, 1, r)
    direct = ops.gemm(a, w, bias=b, act=ops.ACT_SILU, residual=r)
    assert torch.equal(via_op, direct)
    st = torch.ops.sana_b200.la_state(via_op[:, 64:128], via_op[:, 128:], 1, 160, 2)
    assert torch.equal(st, ops.la_state(direct[:, 64:128], direct[:, 128:], 1, 160, 2))
    x = via_op[:, :64]
    ref = x.clone()
    wt = torch.ones(64, dtype=torch.bfloat16, device="cuda")
    torch.ops.sana_b200.rmsnorm_(x, wt, 1e-6)
    assert torch.equal(x, ops.rmsnorm_(ref, wt, 1e-6))


def test_remaining_operators_propagate_shapes_without_a_gpu():
    from torch._subclasses.fake_tensor import FakeTensorMode

    bf = torch.bfloat16
    with FakeTensorMode():
        q = torch.empty(2 * 50, 224, dtype=bf)
        kv = torch.empty(2 * 9, 448, dtype=bf)
        o = torch.ops.sana_b200.cross_attention(q, kv[:, :224], kv[:, 224:], torch.empty(2, 9), 2, 50, 9, 2, 112)
        assert o.shape == (100, 224) and o.dtype == bf
        cos = torch.empty(50, 56)
        st = torch.ops.sana_b200.la_rope_state(q, q, cos, cos, 2, 50, 2, 112, None)
        assert st.shape == (2, 2, 113, 112) and st.dtype == torch.float32
        st2 = torch.ops.sana_b200.la_rope_state(q, q, cos, cos, 2, 50, 2, 112, st)
        assert torch.ops.sana_b200.add_f32(st, st2).shape == st.shape
        assert torch.ops.sana_b200.la_rope_apply(q, cos, cos, st, 2, 50, 2, 112, 1e-8).shape == (100, 224)
        assert torch.ops.sana_b200.rope_(q, torch.empty(50, 32), torch.empty(50, 32), 2, 50, 32) is None
        z = torch.ops.sana_b200.ln_modulate_rows(torch.empty(2, 50, 64, dtype=bf), torch.empty(2, 64, dtype=bf),
                                                 torch.empty(2, 1, 64, dtype=bf), 0, 1, 0, 0, 1e-6)
        assert z.shape == (2, 50, 64)
        pt = torch.ops.sana_b200.patchify(torch.empty(2, 32, 16, 8, dtype=bf), 2)
        assert pt.shape == (2 * 8 * 4, 128)
        assert torch.ops.sana_b200.unpatchify(pt, 2, 32, 8, 4, 2).shape == (2, 32, 16, 8)
        te = torch.ops.sana_b200.timestep_embedding(torch.empty(3), 256, bf, 10000.0)
        assert te.shape == (3, 256) and te.dtype == bf
        assert torch.ops.sana_b200.silu(te).shape == (3, 256)
        a = torch.empty(300, 64, dtype=bf)
        qa = torch.ops.sana_b200.nvfp4_quantize(a)
        assert qa[0].shape == (300, 32) and qa[1].numel() == 3 * 1 * 512 and qa[2].shape == (4,)
        qw = torch.ops.sana_b200.nvfp4_quantize(torch.empty(96, 64, dtype=bf))
        out = torch.ops.sana_b200.gemm_nvfp4(*qa, *qw, None, 0, 0, None, None, 0, 1, None)
        assert out.shape == (300, 96) and out.dtype == bf


@pytest.mark.gpu
def test_remaining_custom_ops_match_the_direct_path():
    g = torch.Generator().manual_seed(1)
    bf = torch.bfloat16
    B, N, L, h, hd = 2, 130, 20, 2, 112
    q = torch.randn(B * N, h * hd, generator=g).to(bf).cuda()
    kv = torch.randn(B * L, 2 * h * hd, generator=g).to(bf).cuda()
    mask = (torch.rand(B, L, generator=g) > 0.2).float().cuda()
    assert torch.equal(torch.ops.sana_b200.cross_attention(q, kv[:, :h * hd], kv[:, h * hd:], mask, B, N, L, h, hd),
                       ops.cross_attention(q, kv[:, :h * hd], kv[:, h * hd:], mask, B, N, L, h, hd))
    ang = torch.randn(N, hd // 2, generator=g).cuda()
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    st = torch.ops.sana_b200.la_rope_state(q, q, cos, sin, B, N, h, hd, None)
    assert torch.equal(st, ops.la_rope_state(q, q, cos, sin, B, N, h, hd))
    assert torch.equal(torch.ops.sana_b200.la_rope_state(q, q, cos, sin, B, N, h, hd, st),
                       ops.la_rope_state(q, q, cos, sin, B, N, h, hd, prior=st))
    assert torch.equal(torch.ops.sana_b200.la_rope_apply(q, cos, sin, st, B, N, h, hd, 1e-8),
                       ops.la_rope_apply(q, cos, sin, st, B, N, h, hd, 1e-8))
    assert torch.equal(torch.ops.sana_b200.add_f32(st, st), st + st)
    lat = torch.randn(2, 32, 16, 8, generator=g).to(bf).cuda()
    pt = torch.ops.sana_b200.patchify(lat, 2)
    assert torch.equal(pt, ops.patchify(lat, 2))
    assert torch.equal(torch.ops.sana_b200.unpatchify(pt, 2, 32, 8, 4, 2), ops.unpatchify(pt, 2, 32, 8, 4, 2))
    a = torch.randn(300, 64, generator=g).to(bf).cuda()
    w = (torch.randn(96, 64, generator=g) * 0.1).to(bf).cuda()
    qa, qw = torch.ops.sana_b200.nvfp4_quantize(a), torch.ops.sana_b200.nvfp4_quantize(w)
    da, dw = ops.nvfp4_quantize(a), ops.nvfp4_quantize(w)
    assert torch.equal(qa[0], da.q) and torch.equal(qa[1], da.sf) and torch.equal(qa[2][:2], da.scales[:2])
    assert torch.equal(torch.ops.sana_b200.gemm_nvfp4(*qa, *qw, None, 0, 0, None, None, 0, 1, None), ops.gemm_nvfp4(da, dw))


def test_a_whole_block_propagates_shapes_through_the_dispatcher_without_a_gpu():
    """route_modules(True): the modules' kernel calls go through torch.ops.sana_b200, so fake tensors on a CUDA device
    that does not exist flow through SanaMSBlock.forward - what tracing and export need."""
    from torch._subclasses.fake_tensor import FakeTensorMode

    import sana_b200
    import sana_b200.torch_ops as T

    old = torch.get_default_dtype()
    T.route_modules(True)
    try:
        torch.set_default_dtype(torch.bfloat16)
        with FakeTensorMode(), torch.device("cuda"):
            blk = sana_b200.SanaMSBlock(64, 2, mlp_ratio=2.5, attn_type="linear", ffn_type="glumbconv", qk_norm=True)
            out = blk(torch.empty(2, 24, 64), torch.empty(2, 5, 64), torch.empty(2, 384), torch.empty(2, 5), (4, 6))
            assert out.shape == (2, 24, 64) and out.dtype == torch.bfloat16 and out.device.type == "cuda"
            stack = sana_b200.BlockStack(64, 2, depth=2)
            assert stack(torch.empty(1, 24, 64), torch.empty(1, 5, 64), torch.empty(1, 384), None, (4, 6)).shape == (1, 24, 64)
    finally:
        torch.set_default_dtype(old)
        T.route_modules(False)
    assert ops.gemm is T._D["gemm"]  # the direct path is back


@pytest.mark.gpu
def test_routed_block_equals_the_direct_block():
    import sana_b200
    import sana_b200.torch_ops as T
    from sana_b200 import synthetic

    C, heads, hid, HW = 64, 2, 160, (4, 6)
    blk = sana_b200.SanaMSBlock(C, heads, mlp_ratio=hid / C, attn_type="linear", ffn_type="glumbconv").eval()
    blk.load_state_dict(synthetic.make_block_params(C, hid, 3, std=0.06), strict=True)
    blk = blk.cuda().bfloat16()
    g = torch.Generator().manual_seed(4)
    x = torch.randn(2, 24, C, generator=g).bfloat16().cuda()
    y = torch.randn(2, 5, C, generator=g).bfloat16().cuda()
    t = (torch.randn(2, 6 * C, generator=g) * 0.3).bfloat16().cuda()
    direct = blk(x, y, t, None, HW)
    T.route_modules(True)
    try:
        routed = blk(x, y, t, None, HW)
    finally:
        T.route_modules(False)
    assert torch.equal(routed, direct)


@pytest.mark.gpu
def test_routed_block_traces_as_one_graph():
    """With the kernel calls routed through the operators, torch.compile captures SanaMSBlock.forward as ONE graph
    (fullgraph=True would raise on a graph break) and the result equals the direct path bit for bit.  The backend
    is "eager": what is checked is the tracing, not code generation - the operators are opaque to the compiler."""
    import sana_b200
    import sana_b200.torch_ops as T
    import torch._dynamo as dynamo
    from sana_b200 import synthetic

    C, heads, hid, HW = 64, 2, 160, (4, 6)
    blk = sana_b200.SanaMSBlock(C, heads, mlp_ratio=hid / C, attn_type="linear", ffn_type="glumbconv").eval()
    blk.load_state_dict(synthetic.make_block_params(C, hid, 3, std=0.06), strict=True)
    blk = blk.cuda().bfloat16()
    g = torch.Generator().manual_seed(4)
    x = torch.randn(2, 24, C, generator=g).bfloat16().cuda()
    y = torch.randn(2, 5, C, generator=g).bfloat16().cuda()
    t = (torch.randn(2, 6 * C, generator=g) * 0.3).bfloat16().cuda()
    direct = blk(x, y, t, None, HW)
    T.route_modules(True)
    try:
        dynamo.reset()
        traced = torch.compile(blk, backend="eager", fullgraph=True)
        assert torch.equal(traced(x, y, t, None, HW), direct)
    finally:
        T.route_modules(False)
        dynamo.reset()

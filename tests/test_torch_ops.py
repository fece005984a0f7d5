"""The kernels are also registered as torch custom operators (namespace sana_b200) with fake
implementations: shapes propagate without a GPU; on a GPU they give the direct path's result."""
import pytest
import torch

import sana_b200.torch_ops  # noqa: F401  (registers the operators)
from sana_b200 import ops


def test_operators_are_registered_with_fake_implementations():
    from torch._subclasses.fake_tensor import FakeTensorMode

    for name in ("gemm", "ln_modulate", "la_state", "la_apply", "dwconv_glu", "rmsnorm_"):
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

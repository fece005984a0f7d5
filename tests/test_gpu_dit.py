"""The whole DiT forward (sana_b200.SanaMS) on a B200 against the upstream model's golden
outputs and against the CPU oracle; plus the small kernels either side of the block loop."""
import pytest
import torch

import sana_b200
from oracle import sana_oracle as O
from sana_b200 import dit, ops

from conftest import nmax_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _model(g, dt):
    m = sana_b200.SanaMS(**g["cfg"]).eval()
    missing = m.load_state_dict(g["params"], strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    return m.to(device=DEV, dtype=dt)


def test_state_dict_keys_are_upstreams(golden):
    g = golden("sana_ms_small")
    m = sana_b200.SanaMS(**g["cfg"])
    assert set(m.state_dict().keys()) == set(g["params"].keys())
    for k, v in m.state_dict().items():
        assert tuple(v.shape) == tuple(g["params"][k].shape), k


@pytest.mark.parametrize("masked", [True, False])
def test_whole_forward_fp32_matches_upstream(golden, masked):
    g = golden("sana_ms_small")
    m = _model(g, torch.float32)
    mask = g["mask"] if masked else torch.ones_like(g["mask"])
    out = m(g["x"].to(DEV), g["timestep"].to(DEV), g["y"].to(DEV), mask=mask.to(DEV))
    ref = g["out_f32" if masked else "out_nomask_f32"]
    assert out.shape == ref.shape and out.dtype == torch.float32
    assert nmax_err(out, ref) <= 1e-5


def test_whole_forward_bf16_within_budget(golden):
    """bf16 model against the fp32 evaluation on bf16-rounded parameters and inputs."""
    g = golden("sana_ms_small")
    cfg = g["cfg"]
    m = _model(g, torch.bfloat16)
    out = m(g["x"].to(DEV), g["timestep"].to(DEV), g["y"].to(DEV), mask=g["mask"].to(DEV))
    r = lambda v: v.to(torch.bfloat16).float() if v.is_floating_point() else v
    gold = O.sana_ms_forward(r(g["x"]), g["timestep"], r(g["y"]), {k: r(v) for k, v in g["params"].items()},
                             depth=cfg["depth"], num_heads=cfg["num_heads"], patch_size=1, out_channels=32,
                             base_size=cfg["input_size"], mask=g["mask"], y_norm=True, norm_eps=cfg["norm_eps"])
    assert out.dtype == torch.bfloat16
    ours, ups = nmax_err(out, gold), nmax_err(g["out_bf16"], gold)
    assert ours <= 2e-2, (ours, ups)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("p", [1, 2])
def test_patchify_and_unpatchify_match_conv_and_einsum(dt, p):
    torch.manual_seed(p)
    B, Cin, H, W, E = 2, 8, 4 * p, 6 * p, 16
    x = torch.randn(B, Cin, H, W).to(dt)
    w = torch.randn(E, Cin, p, p).to(dt)
    rows = ops.patchify(x.to(DEV), p)
    ref = torch.nn.functional.conv2d(x.double(), w.double(), stride=p).flatten(2).transpose(1, 2).reshape(-1, E)
    got = rows.double().cpu() @ w.double().reshape(E, -1).t()
    assert nmax_err(got, ref) < 1e-12
    c = 4
    tok = torch.randn(B * (H // p) * (W // p), p * p * c).to(dt)
    img = ops.unpatchify(tok.to(DEV), B, c, H // p, W // p, p)
    t6 = tok.reshape(B, H // p, W // p, p, p, c)
    ref = torch.einsum("nhwpqc->nchpwq", t6).reshape(B, c, H, W)
    assert torch.equal(img.cpu(), ref)


def test_timestep_embedding_and_silu():
    t = torch.tensor([0.0, 1.0, 37.0, 500.5, 999.0])
    ref = O.timestep_embedding(t, 256)
    got = ops.timestep_embedding(t.to(DEV), 256, torch.float32).cpu()
    assert nmax_err(got, ref) < 2e-4  # cos/sin of arguments up to 1000: one ulp of the frequency moves them by 6e-5
    assert (got[0, :128] == 1).all() and (got[0, 128:] == 0).all()
    x = torch.randn(3, 64)
    assert nmax_err(ops.silu(x.to(DEV)).cpu(), torch.nn.functional.silu(x)) < 1e-6


@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_gelu_epilogue_and_final_layer_rows(dt, tol):
    torch.manual_seed(0)
    a = (torch.randn(40, 48) * 0.5).to(dt)
    w = (torch.randn(64, 48) * 0.2).to(dt)
    b = (torch.randn(64) * 0.1).to(dt)
    ref = torch.nn.functional.gelu(a.double() @ w.double().t() + b.double(), approximate="tanh")
    got = ops.gemm(a.to(DEV), w.to(DEV), bias=b.to(DEV), act=ops.ACT_GELU_TANH)
    assert nmax_err(got, ref) < tol
    B, N, C = 3, 7, 64
    x = torch.randn(B, N, C).to(dt)
    table = (torch.randn(2, C) * 0.3).to(dt)
    t = (torch.randn(B, C) * 0.3).to(dt)
    shift, scale = (table.double()[None] + t.double()[:, None]).chunk(2, dim=1)
    ref = O.t2i_modulate(torch.nn.functional.layer_norm(x.double(), (C,), eps=1e-6), shift, scale)
    got = ops.ln_modulate_rows(x.to(DEV), table.to(DEV), t.to(DEV), 0, 1, 0, 0, 1e-6)
    assert nmax_err(got, ref) < tol


def test_position_table_matches_oracle():
    a = dit.sincos_pos_embed_2d(64, (6, 8), base_size=8)
    b = O.sincos_pos_embed_2d(64, (6, 8), base_size=8)
    assert (a == b).all()


def test_graph_replay_matches_eager(golden):
    """One CUDA graph of the whole forward gives the eager result bit for bit, also on new inputs."""
    from sana_b200.graphs import GraphedForward

    g = golden("sana_ms_small")
    m = _model(g, torch.bfloat16)
    x, ts, y = g["x"].to(DEV).bfloat16(), g["timestep"].to(DEV), g["y"].to(DEV).bfloat16()
    mask = g["mask"].to(DEV)
    fwd = GraphedForward(m, x, ts, y, mask=mask)
    assert torch.equal(fwd(x, ts, y), m(x, ts, y, mask=mask))
    x2, ts2 = (x * 0.5 + 0.1).contiguous(), torch.tensor([5.0, 700.0], device=DEV)
    assert torch.equal(fwd(x2, ts2, y), m(x2, ts2, y, mask=mask))


@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_final_layer_per_sample_and_per_frame(golden, dt, tol):
    g = golden("final_layer")
    m = dit.T2IFinalLayer(g["C"], 1, 32).eval()
    m.load_state_dict(g["params"], strict=True)
    m = m.to(DEV, dt)
    r = (lambda v: v.to(dt).float()) if dt != torch.float32 else (lambda v: v)
    p = {k: r(v) for k, v in g["params"].items()}
    for key in ("t", "t_frames"):
        out = m(g["x"].to(DEV, dt), g[key].to(DEV, dt))
        ref = O.final_layer_forward(r(g["x"]), r(g[key]), p)
        assert out.shape == ref.shape and nmax_err(out, ref) < tol

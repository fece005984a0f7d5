"""Sequence-parallel host logic on CPU ranks (gloo, world_size 2, 3, 4 and 8 - at 8 ranks the 15
image rows leave ranks with one or two rows, so a rank's two halos come from both neighbours and
its only row is first and last at once): the row partitioner,
the state all-reduce and the one-row halo exchange of sana_b200.sharding, driving the oracle's
math per shard, must reproduce the single-process oracle (fp64 <= 1e-12, fp32 <= 1e-6; the
sharded sum changes the addition order, so bit equality is not expected).  Also: a rank that
dies before the collective makes the others fail with an error instead of hanging."""
import datetime
import os
import socket
import sys
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, fn, q, timeout_s):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
        q.put((rank, "ok", fn(rank, world)))
    except Exception as e:  # noqa: BLE001
        q.put((rank, "error", f"{type(e).__name__}: {e}\n{traceback.format_exc()[-600:]}"))
    finally:
        try:
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(world, fn, timeout_s=60, join_s=120):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, q, timeout_s)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        try:
            r, status, payload = q.get(timeout=join_s)
            res[r] = (status, payload)
        except Exception:  # noqa: BLE001
            break
    for p in procs:
        p.join(10)
        if p.is_alive():
            p.kill()
    return res


def _seqpar_block(rank, world):
    from oracle import sana_oracle as O
    from sana_b200 import sharding, synthetic

    torch.set_num_threads(2)
    out = {}
    for dt, tag in ((torch.float64, "f64"), (torch.float32, "f32")):
        C, heads, frames, H, W = 64, 2, 3, 5, 4
        shp = synthetic.BlockShape("sp", C, heads, 1, (frames, H, W), text_len=6)
        p = {k: v.to(dt) for k, v in synthetic.make_block_params(C, shp.ffn_hidden, seed=1, std=0.1).items()}
        x, y, t = (v.to(dt) for v in synthetic.make_block_inputs(shp, seed=1, std=0.1, text_dim=32))
        full, a_full, f_full = O.sana_ms_block_forward(x, y, t, p, heads, shp.grid, keep_dtype=True, return_branches=True)
        sh = sharding.SequenceShard(frames, H, W, rank, world)
        a, b = sh.token_range
        xs = sh.scatter_tokens(x)
        # --- the block on this rank's tokens, exchanging only the state and the halo rows ---
        mod = (p["scale_shift_table"][None] + t.reshape(1, 6, -1)).chunk(6, dim=1)
        z = O.t2i_modulate(O.layer_norm(xs), mod[0], mod[1])
        qkv = torch.nn.functional.linear(z, p["attn.qkv.weight"]).reshape(1, sh.tokens, 3, C // 32, 32)
        q, k, v = qkv.unbind(2)
        state = O.lite_la_state(torch.relu(k), v)
        sh.allreduce_state(state)
        o = O.lite_la_apply(torch.relu(q), state, O.BLOCK_LA_EPS).reshape(1, sh.tokens, C)
        att = torch.nn.functional.linear(o, p["attn.proj.weight"], p["attn.proj.bias"])
        x1 = xs + mod[2] * att
        x1 = x1 + O.cross_attention_forward(x1, y, O.sub(p, "cross_attn"), heads)
        z2 = O.t2i_modulate(O.layer_norm(x1), mod[3], mod[4])
        w1 = p["mlp.inverted_conv.conv.weight"].reshape(-1, C)
        u = torch.nn.functional.silu(torch.nn.functional.linear(z2[0], w1, p["mlp.inverted_conv.conv.bias"]))
        top, bot = sh.exchange_halo(u)
        gl = O.depthwise_glu_rows(u.reshape(sh.rows, W, -1), top, bot, p["mlp.depth_conv.conv.weight"],
                                  p["mlp.depth_conv.conv.bias"], sh.row0, H).reshape(sh.tokens, -1)
        f = torch.nn.functional.linear(gl, p["mlp.point_conv.conv.weight"].reshape(C, -1))
        x2 = x1 + mod[5] * f[None]
        ref = full[:, a:b]
        out[tag] = ((x2 - ref).abs().max() / ref.abs().max()).item()
        out[tag + "_attn"] = ((att - a_full[:, a:b]).abs().max() / a_full.abs().max()).item()
    return out


def _dies_before_collective(rank, world):
    from sana_b200 import sharding

    sh = sharding.SequenceShard(1, 8, 4, rank, world)
    if rank == world - 1:
        raise RuntimeError("injected host-side failure before the all-reduce")
    state = torch.ones(1, 2, 33, 32)
    sh.allreduce_state(state)  # must raise (peer gone / timeout), not hang
    return "unexpected success"


def _peer_health(rank, world):
    from sana_b200 import sharding

    store = dist.distributed_c10d._get_default_store()
    h = sharding.PeerHealth(store, rank, world, timeout_s=2.0)
    h.report(0)
    h.require(0)  # everybody reported step 0
    if rank == world - 1:
        return "left"  # leaves between steps
    h.report(1)
    try:
        h.require(1)
    except sharding.PeerLostError as e:
        return f"detected: {e}"
    return "not detected"


def test_peer_health_detects_a_rank_that_left_between_steps():
    res = _run(3, _peer_health, timeout_s=20, join_s=60)
    assert res[2] == ("ok", "left"), res
    for r in (0, 1):
        assert res[r][0] == "ok" and res[r][1].startswith("detected"), res


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_sequence_parallel_block_matches_single_process(world):
    res = _run(world, _seqpar_block, timeout_s=120, join_s=240)
    assert len(res) == world, res
    for r, (status, payload) in res.items():
        assert status == "ok", payload
        assert payload["f64"] < 1e-12 and payload["f64_attn"] < 1e-12, payload
        assert payload["f32"] < 1e-6 and payload["f32_attn"] < 1e-5, payload


def test_rank_failure_surfaces_as_error_not_hang():
    res = _run(2, _dies_before_collective, timeout_s=8, join_s=60)
    assert res[1][0] == "error" and "injected" in res[1][1]
    assert 0 in res and res[0][0] == "error", res


def _seqpar_rotated_attention(rank, world):
    """The video self-attention (ReLU, then rotation) on this rank's tokens: its slice of the rotation
    table, its partial (D+1) x D state, one all-reduce, the apply on its own tokens."""
    from oracle import sana_oracle as O
    from sana_b200 import sharding

    torch.set_num_threads(2)
    C, heads, frames, H, W = 96, 2, 3, 5, 4
    d, N = C // heads, 3 * 5 * 4
    g = torch.Generator().manual_seed(3)
    p = {"qkv.weight": torch.randn(3 * C, C, generator=g, dtype=torch.float64) * 0.1,
         "proj.weight": torch.randn(C, C, generator=g, dtype=torch.float64) * 0.1,
         "proj.bias": torch.randn(C, generator=g, dtype=torch.float64) * 0.1}
    x = torch.randn(1, N, C, generator=g, dtype=torch.float64)
    freqs = O.wan_rotary_freqs(d, (frames, H, W))
    full = O.lite_la_relu_rope_forward(x, p, heads, freqs, eps=O.BLOCK_LA_EPS)
    sh = sharding.SequenceShard(frames, H, W, rank, world)
    a, b = sh.token_range
    xs = sh.scatter_tokens(x)
    q, k, v = torch.nn.functional.linear(xs, p["qkv.weight"]).reshape(1, sh.tokens, 3, heads, d).unbind(2)
    q, k = q.relu(), k.relu()
    fr = freqs[0, 0, a:b][None, :, None, :]
    rot = lambda t: torch.view_as_real(torch.view_as_complex(t.unflatten(-1, (-1, 2)).contiguous()) * fr).flatten(-2)
    state = O.lite_la_rope_state(k, rot(k), v)
    sh.allreduce_state(state)
    o = O.lite_la_rope_apply(q, rot(q), state, O.BLOCK_LA_EPS).reshape(1, sh.tokens, C)
    out = torch.nn.functional.linear(o, p["proj.weight"], p["proj.bias"])
    ref = full[:, a:b]
    return ((out - ref).abs().max() / ref.abs().max()).item()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_parallel_rotated_attention_matches_single_process(world):
    res = _run(world, _seqpar_rotated_attention)
    assert len(res) == world, res
    for r, (status, payload) in res.items():
        assert status == "ok", payload
        assert payload < 1e-12, payload


def _seqpar_temporal_ffn(rank, world, by_frames=False):
    """GLUMBConvTemp per shard: the conv's one-row halo, then one frame of the spatial result from each
    neighbour for the 3-tap convolution along the frame axis (`SequenceShard.exchange_frames`)."""
    from oracle import sana_oracle as O
    from sana_b200 import sharding, synthetic

    torch.set_num_threads(2)
    C, hid, frames, H, W = 32, 80, 4, 5, 4
    hw, dt = H * W, torch.float64
    p = {k[4:]: v.to(dt) for k, v in synthetic.make_block_params(C, hid, seed=4, std=0.1).items() if k.startswith("mlp.")}
    g = torch.Generator().manual_seed(8)
    p["t_conv.weight"] = torch.randn(C, C, 3, 1, generator=g, dtype=dt) * 0.1
    x = torch.randn(1, frames * hw, C, generator=g, dtype=dt)
    full = O.glumbconv_temp_forward(x, p, (frames, H, W))
    sh = sharding.SequenceShard(frames, H, W, rank, world, by_frames=by_frames)
    a, b = sh.token_range
    xs = sh.scatter_tokens(x)[0]
    lin = torch.nn.functional.linear
    u = torch.nn.functional.silu(lin(xs, p["inverted_conv.conv.weight"].reshape(-1, C), p["inverted_conv.conv.bias"]))
    top, bot = sh.exchange_halo(u)
    gl = O.depthwise_glu_rows(u.reshape(sh.rows, W, -1), top, bot, p["depth_conv.conv.weight"], p["depth_conv.conv.bias"],
                              sh.row0, H).reshape(sh.tokens, -1)
    s = lin(gl, p["point_conv.conv.weight"].reshape(C, -1))
    prev, nxt = sh.exchange_frames(s)
    assert (prev is None) == (rank == 0) and (nxt is None) == (rank == world - 1)
    zeros = torch.zeros(hw, C, dtype=dt)
    ext = torch.cat([zeros if prev is None else prev, s, zeros if nxt is None else nxt])
    wt, n = p["t_conv.weight"], sh.tokens
    out = s + lin(ext[:n], wt[:, :, 0, 0]) + lin(ext[hw:hw + n], wt[:, :, 1, 0]) + lin(ext[2 * hw:2 * hw + n], wt[:, :, 2, 0])
    ref = full[0, a:b]
    return ((out - ref).abs().max() / ref.abs().max()).item()


def _seqpar_temporal_ffn_by_frames(rank, world):
    return _seqpar_temporal_ffn(rank, world, by_frames=True)


@pytest.mark.parametrize("world,fn", [(2, _seqpar_temporal_ffn), (3, _seqpar_temporal_ffn), (4, _seqpar_temporal_ffn),
                                      (2, _seqpar_temporal_ffn_by_frames), (4, _seqpar_temporal_ffn_by_frames)])
def test_sequence_parallel_temporal_ffn_matches_single_process(world, fn):
    res = _run(world, fn)
    assert len(res) == world, res
    for r, (status, payload) in res.items():
        assert status == "ok", payload
        assert payload < 1e-12, payload


def test_frame_partition_and_frame_halo_guard():
    from sana_b200 import sharding

    assert sharding.SequenceShard(5, 6, 4, 1, 2, by_frames=True).ranges == [(0, 18), (18, 30)]
    sh = sharding.SequenceShard(2, 6, 4, 0, 4)  # 3 rows per rank < 6 rows per frame
    with pytest.raises(ValueError):
        sh.exchange_frames(torch.zeros(sh.tokens, 8))

"""Multi-GPU tests (need >= 2 B200s on one node; skipped otherwise).  One process per GPU,
NCCL.  The failure test makes the failure on the host, between steps, with nothing in flight,
and with NVLS off; no GPU is ever faulted or hung."""
import datetime
import os
import socket
import sys
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, fn, q, pg_timeout_s):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                                timeout=datetime.timedelta(seconds=pg_timeout_s))
        q.put((rank, "ok", fn(rank, world)))
    except Exception as e:  # noqa: BLE001
        q.put((rank, "error", f"{type(e).__name__}: {e}\n{traceback.format_exc()[-800:]}"))
    finally:
        try:
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def _run(world, fn, pg_timeout_s=120, join_s=300):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, q, pg_timeout_s)) for r in range(world)]
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
        p.join(20)
        if p.is_alive():
            p.kill()
    return res


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _seqpar_vs_single(rank, world):
    import sana_b200
    from sana_b200 import sharding, synthetic

    dev, dt = torch.device("cuda", rank), torch.bfloat16
    C, heads, grid = 512, 8, (3, 10, 16)
    shp = synthetic.BlockShape("sp", C, heads, 1, grid, text_len=24)
    params = synthetic.make_block_params(C, shp.ffn_hidden, seed=2, std=0.05)
    x, y, t = synthetic.make_block_inputs(shp, seed=2, std=0.05, text_dim=64)
    blk = sana_b200.SanaMSBlock(C, heads, mlp_ratio=2.5, attn_type="linear", ffn_type="glumbconv").eval()
    blk.load_state_dict(params, strict=True)
    blk = blk.to(dev, dt)
    xd, yd, td = x.to(dev, dt), y.to(dev, dt), t.to(dev, dt)
    full = blk(xd, yd, td, None, grid)  # unsharded, on this rank's own GPU
    sh = sharding.SequenceShard(*grid, rank, world)
    blk.set_sequence_shard(sh)
    a, b = sh.token_range
    out = blk(sh.scatter_tokens(xd), yd, td, None, grid)
    torch.cuda.synchronize()
    ref = full[:, a:b].float()
    return ((out.float() - ref).abs().max() / full.float().abs().max()).item()


def _seqpar_full_size(rank, world):
    """The sequence-parallel configuration at its stated size - hidden 2240, 21 x 45 x 80 = 75 600
    tokens - with both exchanges over peer memory, against the unsharded block on the same GPU."""
    import sana_b200
    from sana_b200 import sharding, synthetic

    dev, dt = torch.device("cuda", rank), torch.bfloat16
    C, heads, hid, grid = 2240, 20, 5600, (21, 45, 80)
    blk = sana_b200.SanaMSBlock(C, heads, mlp_ratio=2.5, attn_type="linear", ffn_type="glumbconv").eval().to(dev, dt)
    blk.load_state_dict(synthetic.make_block_params_on_device(C, hid, 0, 0.02, dt, dev), strict=True)
    g = torch.Generator(device=dev).manual_seed(11)
    x = torch.randn(1, grid[0] * grid[1] * grid[2], C, generator=g, device=dev).to(dt)
    y = torch.randn(1, 300, C, generator=g, device=dev).to(dt)
    t = (torch.randn(1, 6 * C, generator=g, device=dev) * 0.1).to(dt)
    full = blk(x, y, t, None, grid)
    sh = sharding.SequenceShard(*grid, rank, world)
    blk.set_sequence_shard(sh)
    sh.enable_fused_state_exchange(1, C // 32, dev)
    sh.enable_fused_halo_exchange(grid[2] * 2 * hid, dt, dev)
    a, b = sh.token_range
    worst = 0.0
    for i in range(3):
        out = blk(sh.scatter_tokens(x), y, t, None, grid)
        worst = max(worst, ((out.float() - full[:, a:b].float()).abs().max() / full.float().abs().max()).item())
    sh.check()  # raises if a wait for the peer ran out
    return worst


def _stack_batch_parallel(rank, world):
    import sana_b200
    from sana_b200 import sharding, synthetic

    dev, dt = torch.device("cuda", rank), torch.bfloat16
    C, heads, grid, B = 256, 4, (8, 8), 4
    stack = sana_b200.BlockStack(C, heads, 2).eval().to(dev, dt)
    for i, blk in enumerate(stack.blocks):
        blk.load_state_dict({k: v.to(dt) for k, v in synthetic.make_block_params(C, 640, seed=i, std=0.05).items()})
    shp = synthetic.BlockShape("dp", C, heads, B, grid, text_len=10)
    x, y, t = (v.to(dev, dt) for v in synthetic.make_block_inputs(shp, seed=0, std=0.05, text_dim=32))
    full = stack(x, y, t, None, grid)
    b0, b1 = sharding.batch_partition(B, world)[rank]
    mine = stack(x[b0:b1].contiguous(), y[b0:b1].contiguous(), t[b0:b1].contiguous(), None, grid)
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    return ((torch.cat(gathered).float() - full.float()).abs().max() / full.float().abs().max()).item()


def _peer_leaves_between_steps(rank, world):
    """Rank world-1 leaves after step 0 with nothing in flight; the others notice it on the
    host (store heartbeat) before launching step 1."""
    from sana_b200 import sharding

    store = dist.distributed_c10d._get_default_store()
    health = sharding.PeerHealth(store, rank, world, timeout_s=3.0)
    dev = torch.device("cuda", rank)
    state = torch.ones(1, 2, 33, 32, device=dev)
    sh = sharding.SequenceShard(1, 8, 4, rank, world)
    sh.allreduce_state(state)  # step 0: everybody takes part
    torch.cuda.synchronize()
    assert state[0, 0, 0, 0].item() == world
    health.report(0)
    health.require(0)
    if rank == world - 1:
        return "left"  # leaves between steps; never reports step 1
    health.report(1)
    try:
        health.require(1)
    except sharding.PeerLostError:
        # the context is still usable: a local kernel runs fine after the peer is gone
        return float((state * 2).sum().item())
    return "not detected"


def _fused_exchange_vs_nccl(rank, world):
    """Same sharded block, state all-reduce by NCCL vs fused into the reduction kernel over
    peer memory; several calls in a row exercise the two slot parities."""
    import sana_b200
    from sana_b200 import sharding, synthetic

    dev, dt = torch.device("cuda", rank), torch.bfloat16
    C, heads, grid = 512, 8, (3, 10, 16)
    shp = synthetic.BlockShape("sp", C, heads, 1, grid, text_len=24)
    params = synthetic.make_block_params(C, shp.ffn_hidden, seed=2, std=0.05)
    x, y, t = synthetic.make_block_inputs(shp, seed=2, std=0.05, text_dim=64)
    blk = sana_b200.SanaMSBlock(C, heads, mlp_ratio=2.5, attn_type="linear", ffn_type="glumbconv").eval()
    blk.load_state_dict(params, strict=True)
    blk = blk.to(dev, dt)
    yd, td = y.to(dev, dt), t.to(dev, dt)
    sh = sharding.SequenceShard(*grid, rank, world)
    blk.set_sequence_shard(sh)
    xs = sh.scatter_tokens(x.to(dev, dt))
    ref = blk(xs, yd, td, None, grid)  # NCCL all-reduce
    sh.enable_fused_state_exchange(1, blk.attn.heads, dev)
    worst = 0.0
    for i in range(5):
        xi = xs * (1.0 + 0.25 * i)
        a = blk(xi, yd, td, None, grid)
        sh._sp_ptrs_saved, sh._sp_ptrs = sh._sp_ptrs, None  # same input through the NCCL path
        b = blk(xi, yd, td, None, grid)
        sh._sp_ptrs = sh._sp_ptrs_saved
        worst = max(worst, ((a.float() - b.float()).abs().max() / b.float().abs().max()).item())
    # the fused sum adds the ranks in rank order on every rank: totals are bit-identical
    C2 = C
    qkv = torch.randn(sh.tokens, 3 * C2, device=dev, generator=torch.Generator(device=dev).manual_seed(rank)).to(dt)
    st = sh.fused_state(qkv[:, C2:2 * C2], qkv[:, 2 * C2:], 1, blk.attn.heads)
    gathered = [torch.empty_like(st) for _ in range(world)]
    dist.all_gather(gathered, st)
    same = all(torch.equal(gathered[0], g) for g in gathered)
    torch.cuda.synchronize()
    first = ((blk(xs, yd, td, None, grid).float() - ref.float()).abs().max() / ref.float().abs().max()).item()
    return {"worst": worst, "same": same, "status": sh.fused_exchange_status(), "first": first}


def _fused_rope_state_full_width(rank, world):
    """sana_la_rope_state_sp at the video model's width (20 heads of 112 channels: the reduction kernel's threads
    stride over the 253 120 state elements) on this rank's half of the tokens, against the NCCL all-reduce of the
    per-rank states; bit-identical totals on every rank; three steps in a row (both slot parities)."""
    import sana_b200
    from sana_b200 import ops, sharding

    dev, dt = torch.device("cuda", rank), torch.bfloat16
    heads, D, grid = 20, 112, (4, 10, 16)
    C = heads * D
    sh = sharding.SequenceShard(*grid, rank, world)
    a, b = sh.token_range
    fr = sana_b200.wan_rotary_freqs(D, grid).reshape(grid[0] * grid[1] * grid[2], D // 2)
    cos, sin = fr.real.float().to(dev)[a:b].contiguous(), fr.imag.float().to(dev)[a:b].contiguous()
    sh.enable_fused_state_exchange(1, heads, dev, head_dim=D)
    worst, same = 0.0, True
    for step in range(3):
        g = torch.Generator(device=dev).manual_seed(10 * step + rank)
        kv = torch.randn(sh.tokens, 2 * C, device=dev, generator=g).to(dt)
        k, v = kv[:, :C], kv[:, C:]
        st = sh.fused_rope_state(k, v, cos, sin, 1, heads, D)
        ref = ops.la_rope_state(k, v, cos, sin, 1, sh.tokens, heads, D)
        dist.all_reduce(ref)
        worst = max(worst, ((st - ref).abs().max() / ref.abs().max()).item())
        gathered = [torch.empty_like(st) for _ in range(world)]
        dist.all_gather(gathered, st)
        same = same and all(torch.equal(gathered[0], x) for x in gathered)
    torch.cuda.synchronize()
    return {"worst": worst, "same": same, "status": sh.fused_exchange_status() + ops.take_la_rope_device_status()}


def _fused_halo_and_graph(rank, world):
    """Sharded block with both exchanges over peer memory (state all-reduce fused into the
    reduction kernel, conv halo rows pushed by the halo kernel) against the NCCL paths, then
    the same block replayed from one CUDA graph with the kernels numbering their own steps."""
    import sana_b200
    from sana_b200 import sharding, synthetic
    from sana_b200.graphs import GraphedForward

    dev, dt = torch.device("cuda", rank), torch.bfloat16
    C, heads, grid = 512, 8, (2, 11, 16)  # 22 rows: the cut at row 11 is a frame boundary for world 2 ...
    out = {}
    for name, g in (("frame_cut", (2, 11, 16)), ("inner_cut", (1, 22, 16))):  # ... and inside a frame here
        shp = synthetic.BlockShape("sp", C, heads, 1, g, text_len=24)
        params = synthetic.make_block_params(C, shp.ffn_hidden, seed=3, std=0.05)
        x, y, t = synthetic.make_block_inputs(shp, seed=3, std=0.05, text_dim=64)
        blk = sana_b200.SanaMSBlock(C, heads, mlp_ratio=2.5, attn_type="linear", ffn_type="glumbconv").eval()
        blk.load_state_dict(params, strict=True)
        blk = blk.to(dev, dt)
        yd, td = y.to(dev, dt), t.to(dev, dt)
        sh = sharding.SequenceShard(*g, rank, world)
        blk.set_sequence_shard(sh)
        xs = sh.scatter_tokens(x.to(dev, dt))
        ref = [blk(xs * (1.0 + 0.25 * i), yd, td, None, g) for i in range(3)]  # NCCL all-reduce + send/recv
        sh.enable_fused_state_exchange(1, blk.attn.heads, dev)
        sh.enable_fused_halo_exchange(g[2] * 2 * shp.ffn_hidden, dt, dev)
        worst = 0.0
        for i in range(3):
            a = blk(xs * (1.0 + 0.25 * i), yd, td, None, g)
            worst = max(worst, ((a.float() - ref[i].float()).abs().max() / ref[i].float().abs().max()).item())
        torch.cuda.synchronize()
        dist.barrier()
        # graph replay: fresh shard state so that every rank starts the device-side numbering together
        sh2 = sharding.SequenceShard(*g, rank, world, device_steps=True)
        blk.set_sequence_shard(sh2)
        sh2.enable_fused_state_exchange(1, blk.attn.heads, dev)
        sh2.enable_fused_halo_exchange(g[2] * 2 * shp.ffn_hidden, dt, dev)
        fwd = GraphedForward(lambda a: blk(a, yd, td, None, g), xs)
        gworst = 0.0
        for i in range(3):
            a = fwd(xs * (1.0 + 0.25 * i))
            gworst = max(gworst, ((a.float() - ref[i].float()).abs().max() / ref[i].float().abs().max()).item())
        torch.cuda.synchronize()
        out[name] = {"worst": worst, "graph_worst": gworst, "halo_status": sh.fused_halo_status() + sh2.fused_halo_status(),
                     "state_status": sh.fused_exchange_status() + sh2.fused_exchange_status()}
        dist.barrier()
    return out


def _video_block_shards(rank, world):
    """The video block (rotated linear attention + temporal Mix-FFN) on two ranks: the temporal halo through
    send / receive, then through the peer-memory kernel, against the unsharded block on the same GPU."""
    import sana_b200
    from sana_b200 import sharding, synthetic

    dev, dt = torch.device("cuda", rank), torch.bfloat16
    C, heads, hid, THW, L = 448, 4, 1120, (4, 10, 16), 24
    F_, H, W = THW
    N = F_ * H * W
    g = torch.Generator().manual_seed(5)
    p = synthetic.make_block_params(C, hid, seed=3, std=0.05)
    p["mlp.t_conv.weight"] = torch.randn(C, C, 3, 1, generator=g) * 0.03
    blk = sana_b200.SanaVideoMSBlock(C, heads, mlp_ratio=hid / C, attn_type="LiteLAReLURope", ffn_type="GLUMBConvTemp",
                                     linear_head_dim=C // heads).eval()
    blk.load_state_dict(p, strict=True)
    blk = blk.to(dev, dt)
    x = (torch.randn(1, N, C, generator=g) * 0.5).to(dev, dt)
    y = (torch.randn(1, L, C, generator=g) * 0.5).to(dev, dt)
    fr = sana_b200.wan_rotary_freqs(C // heads, THW)
    out = {}
    for name, by_frames, t in (("rows", False, torch.randn(1, 6 * C, generator=g) * 0.2),
                               ("frames", True, torch.randn(1, 1, F_, 6 * C, generator=g) * 0.2)):
        t = t.to(dev, dt)
        blk.set_sequence_shard(None)
        full = blk(x, y, t, THW=THW, rotary_emb=fr)
        sh = sharding.SequenceShard(*THW, rank, world, by_frames=by_frames)
        a, b = sh.token_range
        tl = t[:, :, a // (H * W):b // (H * W)].contiguous() if by_frames else t
        blk.set_sequence_shard(sh)
        ref = full[:, a:b].float()
        err = lambda o: ((o.float() - ref).abs().max() / full.float().abs().max()).item()
        worst = err(blk(x[:, a:b].contiguous(), y, tl, THW=THW, rotary_emb=fr))
        sh.enable_fused_frame_exchange(C, dt, dev)
        fused = max(err(blk(x[:, a:b].contiguous(), y, tl, THW=THW, rotary_emb=fr)) for _ in range(3))
        # ... and the attention state's all-reduce inside its reduction kernel as well
        sh.enable_fused_state_exchange(1, heads, dev, head_dim=C // heads)
        assert sh.fused_rope_state_exchange
        fused = max([fused] + [err(blk(x[:, a:b].contiguous(), y, tl, THW=THW, rotary_emb=fr)) for _ in range(3)])
        torch.cuda.synchronize()
        out[name] = {"nccl": worst, "fused": fused, "status": sh.fused_frame_status() + sh.fused_exchange_status()}
        sh.check()
        dist.barrier()
    return out


def test_video_block_with_temporal_halo_on_two_gpus():
    _need(2)
    res = _run(2, _video_block_shards)
    assert len(res) == 2, res
    for r, (status, payload) in res.items():
        assert status == "ok", payload
        for name, p in payload.items():
            assert p["status"] == 0 and p["nccl"] < 1e-2 and p["fused"] < 1e-2, (name, p)


def test_fused_rotated_state_exchange_at_full_width_on_two_gpus():
    _need(2)
    res = _run(2, _fused_rope_state_full_width)
    assert len(res) == 2, res
    for r, (status, payload) in res.items():
        assert status == "ok", payload
        assert payload["status"] == 0 and payload["same"] and payload["worst"] < 1e-5, payload  # only the summation order differs


def test_fused_halo_exchange_and_graph_replay_on_two_gpus():
    _need(2)
    res = _run(2, _fused_halo_and_graph)
    assert len(res) == 2, res
    for r, (status, payload) in res.items():
        assert status == "ok", payload
        for name, p in payload.items():
            assert p["halo_status"] == 0 and p["state_status"] == 0, (name, p)
            assert p["worst"] < 2e-3 and p["graph_worst"] < 2e-3, (name, p)  # only the state summation order differs


def test_fused_state_exchange_matches_nccl_on_two_gpus():
    _need(2)
    res = _run(2, _fused_exchange_vs_nccl)
    assert len(res) == 2, res
    for r, (status, payload) in res.items():
        assert status == "ok", payload
        assert payload["status"] == 0 and payload["same"], payload
        assert payload["worst"] < 2e-3 and payload["first"] < 2e-3, payload  # only the summation order differs


def test_sequence_parallel_block_on_two_gpus():
    _need(2)
    res = _run(2, _seqpar_vs_single)
    assert len(res) == 2, res
    for r, (status, payload) in res.items():
        assert status == "ok", payload
        assert payload < 1e-2, payload  # same kernels; only the state summation order differs


def test_sequence_parallel_block_at_full_size_on_two_gpus():
    _need(2)
    res = _run(2, _seqpar_full_size)
    assert len(res) == 2, res
    for r, (status, payload) in res.items():
        assert status == "ok", payload
        assert payload < 1e-2, payload


def test_batch_parallel_stack_on_two_gpus():
    _need(2)
    res = _run(2, _stack_batch_parallel)
    for r, (status, payload) in res.items():
        assert status == "ok", payload
        assert payload < 1e-2, payload


def test_peer_leaving_between_steps_is_detected_on_the_host():
    _need(2)
    res = _run(2, _peer_leaves_between_steps, pg_timeout_s=30)
    assert res[1] == ("ok", "left"), res
    assert res[0][0] == "ok" and isinstance(res[0][1], float), res

"""The sequence-parallel configuration at its stated size on a B200: one SanaMSBlock at hidden 2240
on the 21 x 45 x 80 = 75 600-token grid, bf16.

(1) The unsharded block against the CPU oracle on sampled image rows: every row next to a cut of
    the 8-, 4- and 2-way row partitions, the first and last row of frames, and a few interior rows.
    The oracle is evaluated in fp32 on the bf16-rounded tensors; tolerance 2e-2 (normalised max
    error), the bf16 budget of the block.
(2) The 8-way row shards run one after the other on the one device: their partial attention
    states add up to the unsharded state, and the depthwise conv with neighbour halo rows gives
    bit-identical rows.
"""
import pytest
import torch

import sana_b200
from oracle import sana_oracle as O
from sana_b200 import ops, sharding, synthetic

from conftest import nmax_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
C, HEADS, HID, GRID = 2240, 20, 5600, (21, 45, 80)


def _setup():
    dt = torch.bfloat16
    shp = synthetic.BlockShape("cfg4", C, HEADS, 1, GRID)
    g = torch.Generator().manual_seed(404)
    params = {k: (torch.randn(s, generator=g) * 0.02) for k, s in synthetic.block_param_shapes(C, HID).items()}
    x = torch.randn(1, shp.tokens, C, generator=g)
    y = torch.randn(1, 300, C, generator=g)
    t = torch.randn(1, 6 * C, generator=g) * 0.1
    blk = sana_b200.SanaMSBlock(C, HEADS, mlp_ratio=2.5, attn_type="linear", ffn_type="glumbconv").eval()
    blk.load_state_dict(params, strict=True)
    return shp, params, x, y, t, blk.to(DEV, dt), dt


def test_cfg4_block_rows_against_cpu_oracle():
    shp, params, x, y, t, blk, dt = _setup()
    out = blk(x.to(DEV, dt), y.to(DEV, dt), t.to(DEV, dt), None, GRID).float().cpu()
    assert ops.take_gemm_device_status() == 0 and ops.take_dwconv_glu_device_status() == 0
    frames, H, W = GRID
    rows = {0, 1, H - 1, H, 10 * H + 22, frames * H - 1}
    for world in (2, 4, 8):
        for r0, r1 in sharding.row_partition(frames * H, world)[:-1]:
            rows.update((r1 - 1, r1))
    rows = sorted(rows)
    r = lambda v: v.to(dt).float()
    torch.set_num_threads(torch.get_num_threads())
    ref = O.sana_ms_block_rows(r(x), r(y), r(t), {k: r(v) for k, v in params.items()}, HEADS, GRID, rows)
    scale = max(v.abs().max().item() for v in ref.values())
    worst = max((out[0, g * W:(g + 1) * W] - ref[g]).abs().max().item() / scale for g in rows)
    assert worst < 2e-2, worst


def test_cfg4_eight_shards_emulated_on_one_gpu():
    shp, params, x, y, t, blk, dt = _setup()
    frames, H, W = GRID
    xd, td = x.to(DEV, dt), t.to(DEV, dt)
    la, mlp = blk.attn, blk.mlp
    world = 8
    shards = [sharding.SequenceShard(frames, H, W, r, world) for r in range(world)]
    z = ops.ln_modulate(xd, blk.scale_shift_table, td, 0, 1)
    qkv = ops.gemm(z.reshape(-1, C), la.qkv.weight)
    full_state = ops.la_state(qkv[:, C:2 * C], qkv[:, 2 * C:], 1, shp.tokens, la.heads)
    parts = [ops.la_state(qkv[s.token_range[0]:s.token_range[1], C:2 * C], qkv[s.token_range[0]:s.token_range[1], 2 * C:],
                          1, s.tokens, la.heads) for s in shards]
    assert nmax_err(torch.stack(parts).sum(0), full_state) < 1e-5  # fp32 sums in another order
    # the state itself against the oracle's token-major restatement, fp64 on the bf16 values
    k = torch.relu(qkv[:, C:2 * C].double().cpu()).reshape(1, -1, la.heads, 32)
    v = qkv[:, 2 * C:].double().cpu().reshape(1, -1, la.heads, 32)
    assert nmax_err(full_state, O.lite_la_state(k, v)) < 1e-5
    u = mlp._expand(z.reshape(-1, C))
    rows = u.reshape(frames * H, W, -1)
    c = mlp.depth_conv.conv
    outs = []
    for s in shards:
        top = rows[s.row0 - 1].contiguous() if s.needs_top() else None
        bot = rows[s.row1].contiguous() if s.needs_bot() else None
        outs.append(ops.dwconv_glu(rows[s.row0:s.row1].reshape(-1, rows.shape[-1]).contiguous(), c.weight, c.bias, W, H,
                                   row0=s.row0, halo_top=top, halo_bot=bot))
    assert torch.equal(torch.cat(outs), ops.dwconv_glu(u, c.weight, c.bias, W, H))
    assert ops.take_dwconv_glu_device_status() == 0

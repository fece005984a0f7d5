"""CPU check of the row-sampled block oracle against the full one (it is what the full-size
75 600-token GPU test compares with, so it has to agree with the pinned oracle first)."""
import pytest
import torch

from oracle import sana_oracle as O
from sana_b200 import synthetic


@pytest.mark.parametrize("grid", [(3, 5, 4), (6, 4)])
@pytest.mark.parametrize("dt,tol", [(torch.float64, 1e-12), (torch.float32, 1e-5)])
def test_sampled_rows_equal_the_full_block(grid, dt, tol):
    C, hid, heads = 64, 160, 2
    shp = synthetic.BlockShape("rows", C, heads, 1, grid, text_len=7)
    p = {k: v.to(dt) for k, v in synthetic.make_block_params(C, hid, seed=1, std=0.2).items()}
    x, y, t = (v.to(dt) for v in synthetic.make_block_inputs(shp, seed=1, std=0.2, text_dim=16))
    mask = torch.ones(1, 7, dtype=torch.int64)
    mask[0, 5:] = 0
    full = O.sana_ms_block_forward(x, y, t, p, heads, grid, mask, keep_dtype=True)
    W = grid[-1]
    rows = list(range(shp.tokens // W))
    got = O.sana_ms_block_rows(x, y, t, p, heads, grid, rows, mask)
    worst = max(((got[r] - full[0, r * W:(r + 1) * W]).abs().max() / full.abs().max()).item() for r in rows)
    assert worst < tol

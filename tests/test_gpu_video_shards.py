"""The video block on sequence shards, every rank emulated on ONE GPU.

The ranks run one after the other; a shard object shared through a dictionary stands in for the
collectives (attention state all-reduce, one-row conv halo, one-frame temporal halo).  What a rank
sends does not depend on what it receives in the same exchange, so three passes over the ranks
settle everything: the first records states and conv rows, the second records the spatial results'
edge frames (now computed with the right conv rows), the third is compared - against the CPU oracle
of the unsharded block (fp32) and against the unsharded module on the same GPU (bf16).
"""
import pytest
import torch

import sana_b200
from oracle import sana_oracle as O
from sana_b200 import sharding, synthetic

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def nmax_err(a, ref):
    a, ref = a.detach().double().cpu(), ref.detach().double().cpu()
    return ((a - ref).abs().max() / ref.abs().max().clamp(min=1e-30)).item()


def _r(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


class EmulatedShard(sharding.SequenceShard):
    """One rank of `world`; what the ranks exchange lives in `self.store` (set after construction)."""

    store: dict = None

    def allreduce_state(self, state):
        self.store[("state", self.rank)] = state.clone()
        total = None
        for r in range(self.world):
            part = self.store.get(("state", r))
            if part is not None:
                total = part.clone() if total is None else total + part
        state.copy_(total)
        return state

    def _swap(self, kind, first, last, want_prev, want_next):
        self.store[(kind, self.rank, "first")], self.store[(kind, self.rank, "last")] = first.clone(), last.clone()
        zeros = torch.zeros_like(first)
        prev = self.store.get((kind, self.rank - 1, "last"), zeros) if want_prev else None
        nxt = self.store.get((kind, self.rank + 1, "first"), zeros) if want_next else None
        return prev, nxt

    def exchange_halo(self, u):
        W = self.W
        return self._swap("conv", u[:W], u[-W:], self.needs_top(), self.needs_bot())

    def exchange_frames(self, s):
        hw = self.H * self.W
        assert min(b - a for a, b in self.ranges) >= self.H
        return self._swap("frame", s[:hw], s[-hw:], self.rank > 0, self.rank < self.world - 1)


def _run_sharded(blk, world, THW, by_frames, call):
    """call(shard) -> this rank's output rows; returns the concatenation after three passes."""
    store = {}
    shards = [EmulatedShard(*THW, r, world, by_frames=by_frames) for r in range(world)]
    for sh in shards:
        sh.store = store
    outs = None
    for _ in range(3):
        outs = []
        for sh in shards:
            blk.set_sequence_shard(sh)
            outs.append(call(sh))
    blk.set_sequence_shard(None)
    return torch.cat(outs, dim=1)


def _video_block(C, heads, hid, THW, seed, dt):
    p = synthetic.make_block_params(C, hid, seed, std=0.06)
    p["mlp.t_conv.weight"] = _r(C, C, 3, 1, seed=seed + 1, scale=0.05)
    blk = sana_b200.SanaVideoMSBlock(C, heads, mlp_ratio=hid / C, attn_type="LiteLAReLURope", ffn_type="GLUMBConvTemp",
                                     linear_head_dim=C // heads)
    blk.load_state_dict(p, strict=True)
    return blk.to(DEV, dt).eval(), p


@pytest.mark.parametrize("world,by_frames", [(2, False), (3, False), (2, True), (4, True)])
def test_temporal_ffn_on_shards_matches_the_oracle(world, by_frames):
    """GLUMBConvTemp alone, fp32: mid-frame cuts need the conv row AND the frame halo."""
    C, hid, THW = 64, 160, (4, 5, 4)
    N = THW[0] * THW[1] * THW[2]
    blk, p = _video_block(C, 2, hid, THW, 5, torch.float32)
    x = _r(1, N, C, seed=9, scale=0.7)
    ref = O.glumbconv_temp_forward(x, O.sub(p, "mlp"), THW)
    xd = x.to(DEV)

    def call(sh):
        a, b = sh.token_range
        return blk.mlp(xd[:, a:b].contiguous(), HW=THW)

    out = _run_sharded(blk, world, THW, by_frames, call)
    assert nmax_err(out, ref) < 1e-5


@pytest.mark.parametrize("per_frame,world,by_frames", [(False, 2, False), (False, 3, False), (True, 2, True), (True, 4, True)])
@pytest.mark.parametrize("dt,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_video_block_on_shards_matches_the_oracle(dt, tol, per_frame, world, by_frames):
    """The whole video block (rotated linear attention, cross-attention, temporal Mix-FFN) on shards: one
    modulation vector per sample with cuts anywhere, one per frame with cuts between frames."""
    C, heads, hid, THW, L = 64, 2, 160, (4, 5, 4), 6
    F_, H, W = THW
    N = F_ * H * W
    blk, p = _video_block(C, heads, hid, THW, 7, dt)
    x, y = _r(1, N, C, seed=1, scale=0.7), _r(1, L, C, seed=2, scale=0.7)
    t = _r(1, 1, F_, 6 * C, seed=3, scale=0.3) if per_frame else _r(1, 6 * C, seed=3, scale=0.3)
    fr = sana_b200.wan_rotary_freqs(C // heads, THW)
    ref = O.sana_video_block_forward(x, y, t, p, heads, THW, fr, linear_head_dim=C // heads)
    xd, yd, td = x.to(DEV, dt), y.to(DEV, dt), t.to(DEV, dt)
    with torch.no_grad():
        full = blk(xd, yd, td, THW=THW, rotary_emb=fr)

    def call(sh):
        a, b = sh.token_range
        tl = td[:, :, a // (H * W):b // (H * W)].contiguous() if per_frame else td
        with torch.no_grad():
            return blk(xd[:, a:b].contiguous(), yd, tl, THW=THW, rotary_emb=fr)

    out = _run_sharded(blk, world, THW, by_frames, call)
    assert nmax_err(out, ref) < tol
    assert nmax_err(out, full) < (1e-5 if dt == torch.float32 else 1e-2)  # only the state's summation order differs


def test_per_frame_modulation_needs_cuts_between_frames():
    C, heads, hid, THW = 64, 2, 160, (4, 5, 4)
    blk, _ = _video_block(C, heads, hid, THW, 7, torch.float32)
    sh = EmulatedShard(*THW, 0, 3)  # 7 of 20 rows: the cut lies inside frame 1
    sh.store = {}
    blk.set_sequence_shard(sh)
    a, b = sh.token_range
    x = _r(1, b - a, C, seed=1).to(DEV)
    t = _r(1, 1, 2, 6 * C, seed=3).to(DEV)  # two vectors for 1.4 frames
    with pytest.raises(ValueError):
        blk(x, _r(1, 6, C, seed=2).to(DEV), t, THW=THW, rotary_emb=sana_b200.wan_rotary_freqs(C // heads, THW))

"""Partitioning of the Linear-DiT block over the GPUs of one node.

Two ways to split, both one process per GPU:

* by batch (independent images): no communication in the forward;
* by sequence (long token grids): tokens are row-major ``(frame, row, col)``; the
  ``frames * H`` image rows are cut into contiguous, balanced ranges.  Per block this needs
  one fp32 all-reduce of the linear-attention state ``[B, h, 33, 32]`` (the state is a plain
  sum over tokens) and, for the 3x3 depthwise conv, one image row of halo from each
  neighbour whose boundary row lies inside the same frame.

Upstream has context parallelism only for its video/GDN nets
(diffusion/distributed/context_parallel/: contiguous rank groups config.py:155-178, halo
exchange halo_exchange.py:44-127); plain LiteLA has no sequence-parallel path upstream.  The
halo exchange here follows the same contract (neighbour p2p, zero padding at the ends) at
row instead of frame granularity.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def row_partition(total_rows: int, world: int) -> List[Tuple[int, int]]:
    """Contiguous balanced [start, end) ranges; the first ``total_rows % world`` ranks get one
    extra row."""
    if world <= 0 or total_rows < world:
        raise ValueError(f"cannot split {total_rows} rows over {world} ranks")
    base, extra = divmod(total_rows, world)
    out, s = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((s, s + n))
        s += n
    return out


def batch_partition(batch: int, world: int) -> List[Tuple[int, int]]:
    if batch % world != 0:
        raise ValueError(f"batch {batch} is not divisible by {world} ranks")
    per = batch // world
    return [(r * per, (r + 1) * per) for r in range(world)]


class PeerLostError(RuntimeError):
    """A peer rank did not report the expected step in time."""


class PeerHealth:
    """Host-side failure detector for a group of ranks that step in lock-step.

    After finishing step ``s`` (all of its kernels and collectives complete) a rank calls
    ``report(s)``; before launching step ``s+1`` it calls ``require(s)``, which raises
    ``PeerLostError`` if some peer has not reported step ``s`` within ``timeout_s``.  A rank
    that died between steps is therefore noticed on the host before the next collective is
    launched, instead of inside a kernel or an NCCL call.  Works with any
    ``torch.distributed`` store (TCPStore / FileStore / the default process-group store)."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 5.0, prefix: str = "sana_health"):
        self.store, self.rank, self.world, self.timeout_s, self.prefix = store, rank, world, timeout_s, prefix

    def _key(self, rank: int, step: int) -> str:
        return f"{self.prefix}/{rank}/{step}"

    def report(self, step: int) -> None:
        self.store.set(self._key(self.rank, step), b"1")

    def require(self, step: int) -> None:
        import datetime

        keys = [self._key(r, step) for r in range(self.world) if r != self.rank]
        if not keys:
            return
        try:
            self.store.wait(keys, datetime.timedelta(seconds=self.timeout_s))
        except Exception as e:  # noqa: BLE001 - the store raises backend-specific errors on time-out
            raise PeerLostError(f"rank {self.rank}: a peer did not finish step {step} within {self.timeout_s}s "
                                f"({type(e).__name__})") from e


@dataclass
class SequenceShard:
    """This rank's slice of a ``(frames, H, W)`` token grid (``frames`` = 1 for an image)."""

    frames: int
    H: int
    W: int
    rank: int
    world: int
    group: Optional[dist.ProcessGroup] = None
    # cut between frames only (every rank holds whole frames, like upstream's context parallelism for
    # video): no conv halo is needed then, and per-frame modulation vectors stay aligned with the shard
    by_frames: bool = False

    def __post_init__(self):
        if self.by_frames:
            self.ranges = [(a * self.H, b * self.H) for a, b in row_partition(self.frames, self.world)]
        else:
            self.ranges = row_partition(self.frames * self.H, self.world)
        self.row0, self.row1 = self.ranges[self.rank]

    @property
    def rows(self) -> int:
        return self.row1 - self.row0

    @property
    def tokens(self) -> int:
        return self.rows * self.W

    @property
    def token_range(self) -> Tuple[int, int]:
        return self.row0 * self.W, self.row1 * self.W

    def needs_top(self) -> bool:
        """True when the row above this shard's first row belongs to the same frame."""
        return self.row0 % self.H != 0

    def needs_bot(self) -> bool:
        return self.row1 % self.H != 0

    # ---- fused exchange over peer memory ------------------------------------------------
    def enable_fused_state_exchange(self, B: int, heads: int, device, head_dim: Optional[int] = None) -> None:
        """Allocates this rank's exchange buffer in symmetric (peer-mapped) memory and maps the
        peers' buffers, so that the linear-attention state reduction kernel can do the
        all-reduce itself (`ops.la_state_sp`) instead of calling NCCL.  Collective over the
        group; call once, on every rank, before the first forward.  With ``head_dim`` the buffer is sized for the
        rotated attention's [head_dim + 1, head_dim] states (`ops.la_rope_state_sp`, `fused_rope_state`); without,
        for the 32-channel heads of the plain linear attention (`fused_state`)."""
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer loads/stores only
        import torch.distributed._symmetric_memory as symm_mem

        from . import ops

        nbytes = (ops.la_state_sp_buffer_bytes(B, heads) if head_dim is None
                  else ops.la_rope_state_sp_buffer_bytes(B, heads, head_dim))
        if nbytes <= 0:
            raise ValueError(f"no fused state exchange for B = {B}, heads = {heads}, head_dim = {head_dim}")
        buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        buf.zero_()
        group = self.group if self.group is not None else dist.group.WORLD
        hdl = symm_mem.rendezvous(buf, group)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)  # every buffer is zeroed before anybody's first step
        self._sp_buf, self._sp_handle = buf, hdl
        self._sp_ptrs = [int(p) for p in hdl.buffer_ptrs]
        self._sp_shape = (B, heads) if head_dim is None else (B, heads, head_dim)
        self._sp_step = 0

    @property
    def fused_state_exchange(self) -> bool:
        return getattr(self, "_sp_ptrs", None) is not None

    def enable_fused_halo_exchange(self, row_elems: int, dtype: torch.dtype, device) -> None:
        """Allocates this rank's halo buffer in symmetric memory and maps the neighbours', so
        that `exchange_halo` moves the conv halo rows with one kernel over peer memory
        (`ops.halo_exchange`) instead of NCCL send/recv.  ``row_elems`` = W * 2 * hid elements of
        ``dtype`` per image row.  Collective over the group; call once on every rank."""
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer loads/stores only
        import torch.distributed._symmetric_memory as symm_mem

        from . import ops

        row_bytes = row_elems * torch.empty((), dtype=dtype).element_size()
        buf = symm_mem.empty(ops.halo_exchange_buffer_bytes(row_bytes), dtype=torch.uint8, device=device)
        buf.zero_()
        group = self.group if self.group is not None else dist.group.WORLD
        hdl = symm_mem.rendezvous(buf, group)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        self._halo_buf, self._halo_handle = buf, hdl
        self._halo_ptrs = [int(p) for p in hdl.buffer_ptrs]
        self._halo_row = (row_elems, dtype, row_bytes)
        self._halo_step = 0

    @property
    def fused_halo_exchange(self) -> bool:
        return getattr(self, "_halo_ptrs", None) is not None

    def enable_fused_frame_exchange(self, channels: int, dtype: torch.dtype, device) -> None:
        """Like :meth:`enable_fused_halo_exchange` for the temporal Mix-FFN's halo (`exchange_frames`): one
        frame, H * W * channels elements, from each neighbour.  A buffer of its own, so the conv rows and the
        frames of one block never share a slot.  Collective over the group; call once on every rank.
        Like the conv rows' buffer it has ONE slot per side, which is safe inside a block (between two
        exchanges lies the attention's state all-reduce, which no rank passes before every rank has consumed
        the previous step's slot) but not for a Mix-FFN called on its own in a loop: use the send / receive
        path there."""
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer loads/stores only
        import torch.distributed._symmetric_memory as symm_mem

        from . import ops

        elems = self.H * self.W * channels
        row_bytes = elems * torch.empty((), dtype=dtype).element_size()
        buf = symm_mem.empty(ops.halo_exchange_buffer_bytes(row_bytes), dtype=torch.uint8, device=device)
        buf.zero_()
        group = self.group if self.group is not None else dist.group.WORLD
        hdl = symm_mem.rendezvous(buf, group)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        self._frame_buf, self._frame_handle = buf, hdl
        self._frame_ptrs = [int(p) for p in hdl.buffer_ptrs]
        self._frame_row = (channels, dtype, row_bytes)
        self._frame_step = 0

    @property
    def fused_frame_exchange(self) -> bool:
        return getattr(self, "_frame_ptrs", None) is not None

    def fused_frame_status(self) -> int:
        """Soft-error word of the frame exchange (bits as in :meth:`fused_halo_status`).  Synchronises."""
        return int(self._frame_buf[20:24].view(torch.int32).item())

    def fused_halo_status(self) -> int:
        """Soft-error word of the halo kernel (0 = every wait completed; bit 0 = the upper, bit 1 =
        the lower neighbour did not arrive in time).  Synchronises."""
        return int(self._halo_buf[20:24].view(torch.int32).item())

    def check(self) -> None:
        """Raises :class:`PeerLostError` when a wait for a peer inside one of the fused exchange
        kernels ran out since the buffers were set up (the kernel then carried on with this rank's
        data only, so every result since is wrong).  Reads two words from the device, i.e.
        synchronises: call it where the host waits for the device anyway (after a denoising step,
        before results leave the GPU), not per block."""
        state = self.fused_exchange_status() if self.fused_state_exchange else 0
        halo = self.fused_halo_status() if self.fused_halo_exchange else 0
        frame = self.fused_frame_status() if self.fused_frame_exchange else 0
        if state or halo or frame:
            who = []
            if frame & 1:
                who.append(f"rank {self.rank - 1} did not deliver its last frame")
            if frame & 2:
                who.append(f"rank {self.rank + 1} did not deliver its first frame")
            if state:
                who.append(f"rank {state - 1} did not publish its attention state")
            if halo & 1:
                who.append(f"rank {self.rank - 1} did not deliver its conv halo row")
            if halo & 2:
                who.append(f"rank {self.rank + 1} did not deliver its conv halo row")
            raise PeerLostError(f"rank {self.rank}: " + "; ".join(who) + " within the exchange wait limit")

    @property
    def fused_rope_state_exchange(self) -> bool:
        """True when the exchange buffer was sized for the rotated attention's states (``head_dim`` given)."""
        return self.fused_state_exchange and len(self._sp_shape) == 3

    # With `device_steps` the exchange kernels number their steps themselves (a word in the
    # exchange buffer) instead of taking the number as a launch argument: required for CUDA-graph
    # replay, where the host does not run between steps.  Set it on every rank or on none.
    device_steps: bool = False

    def fused_state(self, k: torch.Tensor, v: torch.Tensor, B: int, heads: int) -> torch.Tensor:
        """State of the whole sequence from this rank's k, v (fused reduction + all-reduce)."""
        from . import ops

        if (B, heads) != self._sp_shape:
            raise ValueError(f"fused exchange was sized for (B, heads) = {self._sp_shape}, got {(B, heads)}")
        self._sp_step += 1
        return ops.la_state_sp(k, v, B, self.tokens, heads, self._sp_ptrs, self.rank, self.world,
                               0 if self.device_steps else self._sp_step)

    def fused_rope_state(self, k: torch.Tensor, v: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, B: int, heads: int,
                         head_dim: int) -> torch.Tensor:
        """The rotated attention's state of the whole sequence from this rank's k, v and table rows."""
        from . import ops

        if (B, heads, head_dim) != self._sp_shape:
            raise ValueError(f"fused exchange was sized for (B, heads, head_dim) = {self._sp_shape}, "
                             f"got {(B, heads, head_dim)}")
        self._sp_step += 1
        return ops.la_rope_state_sp(k, v, cos, sin, B, self.tokens, heads, head_dim, self._sp_ptrs, self.rank, self.world,
                                    0 if self.device_steps else self._sp_step)

    def fused_exchange_status(self) -> int:
        """Soft-error word of the exchange kernel (0 = every wait completed).  Synchronises."""
        return int(self._sp_buf[320:324].view(torch.int32).item())

    # ---- collectives -------------------------------------------------------------------
    def allreduce_state(self, state: torch.Tensor) -> torch.Tensor:
        """Sums the per-rank partial linear-attention states in place (fp32)."""
        if self.world > 1:
            dist.all_reduce(state, op=dist.ReduceOp.SUM, group=self.group)
        return state

    def exchange_halo(self, u: torch.Tensor) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        """u [rows*W, C2] local rows.  Returns (halo_top, halo_bot) = the neighbour's last /
        first row ([W, C2]) where that row is in the same frame, else None."""
        W = self.W
        if self.world > 1 and self.fused_halo_exchange:
            from . import ops as K

            row_elems, dtype, row_bytes = self._halo_row
            if W * u.shape[1] != row_elems or u.dtype != dtype:
                raise ValueError("fused halo exchange was sized for another row")
            up = self._halo_ptrs[self.rank - 1] if self.needs_top() else None
            down = self._halo_ptrs[self.rank + 1] if self.needs_bot() else None
            self._halo_step += 1
            K.halo_exchange(u[:W].reshape(-1) if up else None, u[-W:].reshape(-1) if down else None, row_bytes,
                            self._halo_ptrs[self.rank], up, down, 0 if self.device_steps else self._halo_step)
            rows = self._halo_buf[1024:1024 + 2 * row_bytes].view(dtype).view(2, W, u.shape[1])
            return (rows[0] if up else None), (rows[1] if down else None)
        top = torch.empty(W, u.shape[1], dtype=u.dtype, device=u.device) if self.needs_top() else None
        bot = torch.empty(W, u.shape[1], dtype=u.dtype, device=u.device) if self.needs_bot() else None
        if self.world == 1:
            return top, bot
        ops = []
        peer = lambda r: r if self.group is None else dist.get_global_rank(self.group, r)
        if self.needs_top():  # my first row is the neighbour's halo_bot and vice versa
            ops.append(dist.P2POp(dist.isend, u[:W].contiguous(), peer(self.rank - 1), self.group))
            ops.append(dist.P2POp(dist.irecv, top, peer(self.rank - 1), self.group))
        if self.needs_bot():
            ops.append(dist.P2POp(dist.isend, u[-W:].contiguous(), peer(self.rank + 1), self.group))
            ops.append(dist.P2POp(dist.irecv, bot, peer(self.rank + 1), self.group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        return top, bot

    def exchange_frames(self, s: torch.Tensor) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        """s [tokens, C]: this rank's rows of a per-token tensor (batch 1).  Returns (prev, next): the H * W
        tokens that precede this rank's first token and those that follow its last one, i.e. what a 3-tap
        convolution along the frame axis needs from the neighbours ([H*W, C] each; None at the two ends of
        the grid, where the convolution pads with zeros).  Every rank must hold at least one frame's worth
        of rows, so that both pieces come from the adjacent ranks (upstream exchanges whole frames the same
        way: basic_modules.py:252-263 through halo_exchange.py:44-127)."""
        hw = self.H * self.W
        if min(b - a for a, b in self.ranges) < self.H:
            raise ValueError(f"a rank holds fewer than {self.H} image rows: the frame halo would span several ranks")
        if s.shape[0] != self.tokens:
            raise ValueError("exchange_frames: s must hold this rank's tokens")
        has_prev, has_next = self.rank > 0, self.rank < self.world - 1
        if self.world == 1:
            return None, None
        if self.fused_frame_exchange:
            from . import ops as K

            channels, dtype, row_bytes = self._frame_row
            if s.shape[1] != channels or s.dtype != dtype or not s.is_contiguous():
                raise ValueError("fused frame exchange was sized for another tensor")
            up = self._frame_ptrs[self.rank - 1] if has_prev else None
            down = self._frame_ptrs[self.rank + 1] if has_next else None
            self._frame_step += 1
            K.halo_exchange(s[:hw].reshape(-1) if up else None, s[-hw:].reshape(-1) if down else None, row_bytes,
                            self._frame_ptrs[self.rank], up, down, 0 if self.device_steps else self._frame_step)
            rows = self._frame_buf[1024:1024 + 2 * row_bytes].view(dtype).view(2, hw, channels)
            return (rows[0] if up else None), (rows[1] if down else None)
        prev = torch.empty(hw, s.shape[1], dtype=s.dtype, device=s.device) if has_prev else None
        nxt = torch.empty(hw, s.shape[1], dtype=s.dtype, device=s.device) if has_next else None
        ops = []
        peer = lambda r: r if self.group is None else dist.get_global_rank(self.group, r)
        if has_prev:
            ops.append(dist.P2POp(dist.isend, s[:hw].contiguous(), peer(self.rank - 1), self.group))
            ops.append(dist.P2POp(dist.irecv, prev, peer(self.rank - 1), self.group))
        if has_next:
            ops.append(dist.P2POp(dist.isend, s[-hw:].contiguous(), peer(self.rank + 1), self.group))
            ops.append(dist.P2POp(dist.irecv, nxt, peer(self.rank + 1), self.group))
        for req in dist.batch_isend_irecv(ops):
            req.wait()
        return prev, nxt

    def scatter_tokens(self, x_full: torch.Tensor) -> torch.Tensor:
        """[B, N, C] full sequence -> this rank's [B, tokens, C] slice (a copy)."""
        a, b = self.token_range
        return x_full[:, a:b].contiguous()

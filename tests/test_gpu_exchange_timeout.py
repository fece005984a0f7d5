"""The give-up path of the two sequence-parallel exchange kernels, on ONE GPU.

Each kernel waits - for a bounded time - until a peer GPU has written a step number into this
rank's exchange buffer.  Here the "peer" is a second, zero-filled buffer on the same device that
nobody ever writes: the wait (shortened to 20 ms through sana_exchange_set_wait_limit_ns) runs
out, the kernel records which peer it gave up on in the buffer's soft-error word and returns.
Nothing hangs or faults, the context stays usable, and a later call without peers gives the
usual result."""
import ctypes as C

import pytest
import torch

from oracle import sana_oracle as O
from sana_b200 import _lib, ops

from conftest import nmax_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture()
def short_wait():
    ops.set_exchange_wait_limit(0.02)
    yield
    ops.set_exchange_wait_limit(0.0)  # back to the default


def test_state_exchange_gives_up_on_a_silent_peer(short_wait):
    B, N, H = 1, 640, 8
    g = torch.Generator(device=DEV).manual_seed(0)
    kv = torch.randn(N, 2 * H * 32, generator=g, device=DEV).bfloat16()
    k, v = kv[:, :H * 32], kv[:, H * 32:]
    nbytes = ops.la_state_sp_buffer_bytes(B, H)
    mine = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    silent = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    ops.la_state_sp(k, v, B, N, H, [mine.data_ptr(), silent.data_ptr()], 0, 2, 1)
    t1.record()
    torch.cuda.synchronize()
    assert int(mine[320:324].view(torch.int32).item()) == 1 + 1  # gave up on rank 1
    assert 15.0 < t0.elapsed_time(t1) < 1500.0  # about the 20 ms limit, far from the 2 s default
    assert int(silent[0:4].view(torch.int32).item()) == 1  # our own flag did reach the peer's buffer
    # the device is fine: the same reduction without peers, on fresh buffers
    solo = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    st = ops.la_state_sp(k, v, B, N, H, [solo.data_ptr()], 0, 1, 1)
    ref = O.lite_la_state(torch.relu(k.double().cpu()).reshape(1, N, H, 32), v.double().cpu().reshape(1, N, H, 32))
    assert nmax_err(st, ref) < 1e-5
    assert int(solo[320:324].view(torch.int32).item()) == 0


def test_rotated_state_exchange_gives_up_on_a_silent_peer(short_wait):
    """The same for the rotated attention's wider state (the reduction kernel's threads stride over it)."""
    B, N, H, D = 1, 520, 20, 112
    g = torch.Generator(device=DEV).manual_seed(1)
    kv = torch.randn(N, 2 * H * D, generator=g, device=DEV).bfloat16()
    k, v = kv[:, :H * D], kv[:, H * D:]
    ang = torch.randn(N, D // 2, generator=g, device=DEV) * 3.0
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    nbytes = ops.la_rope_state_sp_buffer_bytes(B, H, D)
    mine, silent0, silent2 = (torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(3))
    ops.la_rope_state_sp(k, v, cos, sin, B, N, H, D, [silent0.data_ptr(), mine.data_ptr(), silent2.data_ptr()], 1, 3, 1)
    torch.cuda.synchronize()
    assert int(mine[320:324].view(torch.int32).item()) == 1 + 0  # gave up on rank 0, the first it waits for
    assert int(silent0[4:8].view(torch.int32).item()) == 1 and int(silent2[4:8].view(torch.int32).item()) == 1
    solo = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    st = ops.la_rope_state_sp(k, v, cos, sin, B, N, H, D, [solo.data_ptr()], 0, 1, 1)
    assert torch.equal(st, ops.la_rope_state(k, v, cos, sin, B, N, H, D))
    assert int(solo[320:324].view(torch.int32).item()) == 0 and ops.take_la_rope_device_status() == 0


def test_halo_exchange_gives_up_per_side(short_wait):
    row_bytes = 4096
    nbytes = ops.halo_exchange_buffer_bytes(row_bytes)
    mine, upper, lower = (torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(3))
    first = torch.arange(row_bytes // 2, device=DEV, dtype=torch.int16).view(torch.uint8)
    last = (torch.arange(row_bytes // 2, device=DEV, dtype=torch.int16) + 7).view(torch.uint8)
    ops.halo_exchange(first, last, row_bytes, mine.data_ptr(), upper.data_ptr(), lower.data_ptr(), 1)
    torch.cuda.synchronize()
    assert int(mine[20:24].view(torch.int32).item()) == 3  # both neighbours silent: bit 0 | bit 1
    # our rows did arrive in the neighbours' slots: first row -> upper's `bot`, last row -> lower's `top`
    assert torch.equal(upper[1024 + row_bytes:1024 + 2 * row_bytes], first)
    assert torch.equal(lower[1024:1024 + row_bytes], last)
    # only a lower neighbour, and it "delivers" (its flag word is pre-set): no error
    mine2, lower2 = (torch.zeros(nbytes, dtype=torch.uint8, device=DEV) for _ in range(2))
    mine2[4:8].view(torch.int32).fill_(1)  # word 1 = last step delivered by the lower neighbour
    ops.halo_exchange(None, last, row_bytes, mine2.data_ptr(), None, lower2.data_ptr(), 1)
    torch.cuda.synchronize()
    assert int(mine2[20:24].view(torch.int32).item()) == 0

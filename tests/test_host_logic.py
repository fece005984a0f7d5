"""Host-side logic: partitioning, module construction / checkpoint keys, loud failures."""
import pytest
import torch

import sana_b200
from sana_b200 import SanaLibraryError, ops, sharding, synthetic


def test_row_partition_balanced():
    for total, world in [(945, 2), (945, 4), (945, 8), (128, 8), (7, 7)]:
        r = sharding.row_partition(total, world)
        assert r[0][0] == 0 and r[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
        sizes = [b - a for a, b in r]
        assert max(sizes) - min(sizes) <= 1
    assert [b - a for a, b in sharding.row_partition(945, 8)] == [119] + [118] * 7
    with pytest.raises(ValueError):
        sharding.row_partition(3, 4)
    with pytest.raises(ValueError):
        sharding.batch_partition(8, 3)
    assert sharding.batch_partition(8, 4)[3] == (6, 8)


def test_sequence_shard_halo_flags_match_between_neighbours():
    for world in (2, 4, 8):
        shards = [sharding.SequenceShard(21, 45, 80, r, world) for r in range(world)]
        assert sum(s.tokens for s in shards) == 21 * 45 * 80
        for a, b in zip(shards, shards[1:]):
            assert a.needs_bot() == b.needs_top()
        assert not shards[0].needs_top() and not shards[-1].needs_bot()
    # a boundary that falls between two frames needs no halo
    s = sharding.SequenceShard(2, 4, 4, 1, 2)
    assert s.row0 == 4 and not s.needs_top()


def test_state_dict_keys_match_upstream(golden):
    g = golden("small_block_a")
    blk = sana_b200.SanaMSBlock(g["C"], g["heads"], mlp_ratio=2.5, attn_type="linear", ffn_type="glumbconv")
    assert {k: tuple(v.shape) for k, v in blk.state_dict().items()} == {k: tuple(v.shape) for k, v in g["params"].items()}
    blk.load_state_dict(g["params"], strict=True)
    assert set(synthetic.block_param_shapes(64, 160)) == set(g["params"])
    la = blk.attn
    for attr in ("qkv", "proj", "q_norm", "k_norm", "kernel_func", "heads", "dim", "eps", "in_dim", "out_dim"):
        assert hasattr(la, attr)
    assert la.eps == 1e-8 and la.dim == 32 and la.heads == 2


def test_unsupported_features_raise():
    with pytest.raises(NotImplementedError):
        sana_b200.SanaMSBlock(64, 4, attn_type="flash", ffn_type="glumbconv")
    with pytest.raises(NotImplementedError):
        sana_b200.SanaMSBlock(64, 4, attn_type="linear", ffn_type="mlp")
    with pytest.raises(NotImplementedError):
        sana_b200.GLUMBConv(64, 160, dilation=2)
    with pytest.raises(NotImplementedError):
        sana_b200.LiteLA(64, 64, heads=4)  # head dimension 16


def test_qk_norm_state_dict_keys_match_upstream(golden):
    g = golden("small_block_qknorm")
    blk = sana_b200.SanaMSBlock(g["C"], g["heads"], mlp_ratio=2.5, attn_type="linear", ffn_type="glumbconv",
                                qk_norm=True, cross_norm=True)
    assert set(blk.state_dict()) == set(g["params"])
    blk.load_state_dict(g["params"], strict=True)


def test_no_cpu_path():
    m = sana_b200.LiteLA(64, 64, heads=2, eps=1e-8)
    with pytest.raises(SanaLibraryError, match="CUDA tensors only"):
        m(torch.randn(1, 8, 64), HW=(2, 4))
    f = sana_b200.GLUMBConv(64, 160, use_bias=(True, True, False))
    with pytest.raises(SanaLibraryError):
        f(torch.randn(1, 8, 64), HW=(2, 4))
    with pytest.raises(SanaLibraryError, match="unsupported dtype"):
        ops._dtype_code(torch.float16)


def test_synthetic_is_seeded():
    a = synthetic.make_block_params(64, 160, seed=3)
    b = synthetic.make_block_params(64, 160, seed=3)
    assert all(torch.equal(a[k], b[k]) for k in a)
    x1, y1, t1 = synthetic.make_block_inputs(synthetic.BlockShape("s", 64, 4, 2, (4, 4), text_len=5), seed=1)
    assert x1.shape == (2, 16, 64) and y1.shape == (2, 5, 64) and t1.shape == (2, 384)
    assert synthetic.CFG3.la_heads == 70 and synthetic.CFG3.ffn_hidden == 5600 and synthetic.CFG4.tokens == 75600

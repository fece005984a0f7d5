"""Host-side checks of the whole-forward modules that need no GPU: state-dict compatibility
with upstream's SanaMS, the position table, constructor guards, partitioning of the halo buffer."""
import pytest
import torch

import sana_b200
from oracle import sana_oracle as O
from sana_b200 import dit


def test_state_dict_keys_and_shapes_are_upstreams(golden):
    g = golden("sana_ms_small")
    m = sana_b200.SanaMS(**g["cfg"])
    sd = m.state_dict()
    assert set(sd.keys()) == set(g["params"].keys())
    for k, v in sd.items():
        assert tuple(v.shape) == tuple(g["params"][k].shape), k
    res = m.load_state_dict(g["params"], strict=True)
    assert not res.missing_keys and not res.unexpected_keys


@pytest.mark.parametrize("hw,base", [((6, 8), 8), ((8, 6), 8), ((32, 32), 32), ((5, 3), 4)])
def test_position_table_matches_oracle(hw, base):
    a = dit.sincos_pos_embed_2d(64, hw, pe_interpolation=1.0, base_size=base)
    b = O.sincos_pos_embed_2d(64, hw, pe_interpolation=1.0, base_size=base)
    assert a.shape == (hw[0] * hw[1], 64) and (a == b).all()
    c = dit.sincos_pos_embed_2d(64, hw, pe_interpolation=2.0, base_size=base)
    assert (c == O.sincos_pos_embed_2d(64, hw, pe_interpolation=2.0, base_size=base)).all() and not (a == c).all()


def test_constructor_guards():
    kw = dict(input_size=8, patch_size=1, in_channels=32, hidden_size=64, depth=1, num_heads=2, mlp_ratio=2.5,
              caption_channels=48, model_max_length=10)
    with pytest.raises(NotImplementedError):
        sana_b200.SanaMS(pos_embed_type="flux_rope", **kw)
    with pytest.raises(NotImplementedError):
        sana_b200.SanaMS(logvar=True, **kw)
    with pytest.raises(NotImplementedError):
        sana_b200.SanaMS(attn_type="flash", **kw)
    with pytest.raises(NotImplementedError):
        sana_b200.PatchEmbedMS(patch_size=2, in_chans=4, embed_dim=64, kernel_size=3)
    with pytest.raises(NotImplementedError):
        sana_b200.GLUMBConvTemp(64, 160, t_kernel_size=5)
    m = sana_b200.SanaMS(y_norm=True, y_norm_scale_factor=0.01, **kw)
    assert torch.allclose(m.attention_y_norm.weight, torch.full((64,), 0.01))
    assert m.out_channels == 64 and sana_b200.SanaMS(pred_sigma=False, **kw).out_channels == 32


def test_video_ffn_keeps_upstreams_keys(golden):
    g = golden("glumbconv_temp")
    m = sana_b200.GLUMBConvTemp(in_features=g["C"], hidden_features=g["hid"], use_bias=(True, True, False),
                                norm=(None, None, None), act=("silu", "silu", None))
    assert set(m.state_dict().keys()) == set(g["params"].keys())
    assert float(m.t_conv.weight.detach().abs().sum()) == 0.0  # zero-initialised like upstream


def test_video_block_state_dict_keys_and_guards():
    import sana_b200
    blk = sana_b200.SanaVideoMSBlock(96, 2, mlp_ratio=2.5, attn_type="LiteLAReLURope", ffn_type="GLUMBConvTemp",
                                     linear_head_dim=48)
    assert set(blk.state_dict()) == {
        "scale_shift_table", "attn.qkv.weight", "attn.proj.weight", "attn.proj.bias", "cross_attn.q_linear.weight",
        "cross_attn.q_linear.bias", "cross_attn.kv_linear.weight", "cross_attn.kv_linear.bias", "cross_attn.proj.weight",
        "cross_attn.proj.bias", "mlp.inverted_conv.conv.weight", "mlp.inverted_conv.conv.bias",
        "mlp.depth_conv.conv.weight", "mlp.depth_conv.conv.bias", "mlp.point_conv.conv.weight", "mlp.t_conv.weight"}
    assert blk.attn.dim == 48 and blk.attn.heads == 2
    import pytest
    with pytest.raises(NotImplementedError):
        sana_b200.SanaVideoMSBlock(96, 2, attn_type="flash", ffn_type="GLUMBConvTemp")
    with pytest.raises(NotImplementedError):
        sana_b200.SanaVideoMSBlock(96, 2, attn_type="LiteLAReLURope", ffn_type="GLUMBConvTemp", linear_head_dim=48,
                                   additional_flash_attn="flash")
    with pytest.raises(NotImplementedError):
        sana_b200.LiteLAReLURope(80, 80, heads=2)  # heads of 40 channels


def test_video_block_refuses_uncovered_call_options():
    import pytest
    import torch
    import sana_b200
    blk = sana_b200.SanaVideoMSBlock(96, 2, mlp_ratio=2.5, attn_type="LiteLAReLURope", ffn_type="GLUMBConvTemp",
                                     linear_head_dim=48)
    x, y, t = torch.zeros(1, 24, 96), torch.zeros(1, 3, 96), torch.zeros(1, 6 * 96)
    with pytest.raises(NotImplementedError):
        blk(x, y, t, THW=(2, 3, 4), chunk_index=[0, 1])
    with pytest.raises(NotImplementedError):
        blk(x, y, t, THW=(2, 3, 4), kv_cache=[None])
    with pytest.raises(ValueError):
        blk(x, y, torch.zeros(1, 1, 5, 6 * 96), THW=(2, 3, 4))  # 24 tokens are not 5 frames
    with pytest.raises(ValueError):
        blk(x, y, torch.zeros(1, 1, 4, 6 * 96), THW=(2, 3, 4))  # 4 modulation vectors for a 2-frame grid
    sh1 = sana_b200.sharding.SequenceShard(2, 3, 4, 0, 1)
    blk.set_sequence_shard(sh1)  # the temporal Mix-FFN runs on shards (one frame from each neighbour) ...
    assert blk.mlp.seq_shard is sh1
    cached = sana_b200.SanaVideoMSBlock(96, 2, mlp_ratio=2.5, attn_type="cachedcausal", ffn_type="CachedGLUMBConvTemp",
                                        linear_head_dim=48)
    with pytest.raises(NotImplementedError):
        cached.set_sequence_shard(sh1)  # ... its cached variant does not
    plain = sana_b200.SanaVideoMSBlock(96, 2, mlp_ratio=2.5, attn_type="LiteLAReLURope", ffn_type="glumbconv",
                                       linear_head_dim=48)
    sh = sana_b200.sharding.SequenceShard(2, 3, 4, 0, 1)
    plain.set_sequence_shard(sh)
    assert plain.attn.seq_shard is sh and plain.mlp.seq_shard is sh

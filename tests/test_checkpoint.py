"""Checkpoint reading on CPU: synthetic files written in upstream's three on-disk layouts
(.pth wrapper dict, safetensors with upstream keys, the diffusers key layout) load into the
drop-in model with the semantics of upstream's load_checkpoint_ddp."""
import json
import os

import pytest
import torch

import sana_b200
from sana_b200 import checkpoint as ck

CFG = dict(input_size=8, patch_size=1, in_channels=4, hidden_size=64, depth=2, num_heads=2, mlp_ratio=2.5,
           class_dropout_prob=0.0, pred_sigma=False, caption_channels=24, model_max_length=6, y_norm=True,
           qk_norm=True, cross_norm=True, linear_head_dim=32)


def _model(seed):
    torch.manual_seed(seed)
    m = sana_b200.SanaMS(**CFG).eval()
    for p in m.parameters():
        torch.nn.init.normal_(p, std=0.1)
    return m


def _same(a, b):
    return all(torch.equal(a[k], b[k]) for k in a) and set(a) == set(b)


def test_pth_wrapper_ema_pos_embed_and_reshape(tmp_path):
    src, ema = _model(0), _model(1)
    sd = {k: v.clone() for k, v in src.state_dict().items()}
    sd["pos_embed"] = torch.zeros(1, 64, 64)  # upstream drops position tables on load
    sd["blocks.0.mlp.point_conv.conv.weight"] = sd["blocks.0.mlp.point_conv.conv.weight"][:, :, 0, 0]  # [out, in] only
    sd["extra.key"] = torch.zeros(3)
    path = str(tmp_path / "epoch_3_step_100.pth")
    torch.save({"state_dict": sd, "state_dict_ema": ema.state_dict(), "image_step": 100}, path)
    dst = _model(2)
    missing, unexpected = ck.load_checkpoint(path, dst)
    assert missing == ["pos_embed"] and unexpected == ["extra.key"]  # the position table is rebuilt, never loaded
    assert _same(dst.state_dict(), src.state_dict())
    dst = _model(2)
    ck.load_checkpoint(path, dst, load_ema=True)
    assert _same(dst.state_dict(), ema.state_dict())
    # the official releases are bare state dicts; a null caption embedding can be swapped in
    torch.save(src.state_dict(), str(tmp_path / "bare.pth"))
    dst = _model(2)
    null = torch.full_like(src.state_dict()["y_embedder.y_embedding"], 0.5)
    ck.load_checkpoint(str(tmp_path / "bare.pth"), dst, null_embed=null)
    assert torch.equal(dst.y_embedder.y_embedding, null)
    assert torch.equal(dst.blocks[1].attn.qkv.weight, src.blocks[1].attn.qkv.weight)
    with pytest.raises(KeyError):
        ck.load_checkpoint(str(tmp_path / "bare.pth"), dst, load_ema=True)
    with pytest.raises(FileNotFoundError):
        ck.load_checkpoint(str(tmp_path / "absent.pth"), dst)


def test_safetensors_single_file_and_index(tmp_path):
    src = _model(3)
    sd = {k: v.to(torch.bfloat16) if v.dim() > 1 else v for k, v in src.state_dict().items()}
    one = str(tmp_path / "model.safetensors")
    ck.save_safetensors(sd, one, metadata={"format": "pt"})
    back = ck.load_safetensors(one)
    assert _same(back, sd) and all(back[k].dtype == sd[k].dtype for k in sd)
    # sharded: two files + an index, as the hub stores large models
    keys = sorted(sd)
    a, b = keys[: len(keys) // 2], keys[len(keys) // 2:]
    ck.save_safetensors({k: sd[k] for k in a}, str(tmp_path / "m-00001-of-00002.safetensors"))
    ck.save_safetensors({k: sd[k] for k in b}, str(tmp_path / "m-00002-of-00002.safetensors"))
    index = {"weight_map": {**{k: "m-00001-of-00002.safetensors" for k in a}, **{k: "m-00002-of-00002.safetensors" for k in b}}}
    ipath = str(tmp_path / "m.safetensors.index.json")
    json.dump(index, open(ipath, "w"))
    dst = _model(4).to(torch.bfloat16)
    missing, unexpected = ck.load_checkpoint(ipath, dst)
    assert missing == ["pos_embed"] and unexpected == []
    assert all(torch.equal(dst.state_dict()[k], sd[k].to(torch.bfloat16)) for k in sd)
    # a truncated file is refused, not misread
    raw = open(one, "rb").read()
    open(str(tmp_path / "cut.safetensors"), "wb").write(raw[: len(raw) - 16])
    with pytest.raises(ValueError):
        ck.load_safetensors(str(tmp_path / "cut.safetensors"))


def test_diffusers_layout_round_trip(tmp_path):
    src = _model(5)
    sd = src.state_dict()
    dif = ck.to_diffusers_keys(sd)
    assert "transformer_blocks.1.attn1.to_k.weight" in dif and "blocks.1.attn.qkv.weight" not in dif
    assert torch.equal(dif["transformer_blocks.0.attn2.to_v.bias"], sd["blocks.0.cross_attn.kv_linear.bias"][64:])
    assert torch.equal(dif["scale_shift_table"], sd["final_layer.scale_shift_table"])
    assert _same(ck.from_diffusers_keys(dif), dict(sd))
    path = str(tmp_path / "diffusion_pytorch_model.safetensors")
    ck.save_safetensors(dif, path)
    dst = _model(6)
    missing, unexpected = ck.load_checkpoint(path, dst)  # layout detected from the keys
    assert missing == ["pos_embed"] and unexpected == []
    assert _same(dst.state_dict(), sd)

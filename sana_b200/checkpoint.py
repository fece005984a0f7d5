"""On-disk formats of Sana checkpoints, read without third-party packages.

Upstream ships its transformer weights three ways:

* ``.pth``: a pickled dict ``{"state_dict": ..., "state_dict_ema": ..., ...}`` (or the bare state
  dict of the official releases), read by ``find_model`` (tools/download.py:31-62) and applied by
  ``load_checkpoint_ddp`` (diffusion/utils/checkpoint.py:264-345): position tables are dropped,
  ``state_dict_ema`` is taken with ``load_ema``, the null caption embedding may be replaced, tensors
  with missing trailing dimensions are reshaped, and the load is non-strict;
* ``.safetensors`` / ``.safetensors.index.json`` with upstream's keys (tools/download.py:43-59);
* the diffusers layout written by tools/convert_scripts/convert_sana_to_diffusers.py:72-228
  (``transformer_blocks.N.attn1.to_q`` ...), which splits the fused q|k|v and k|v projections.

The modules of this package keep upstream's state-dict keys, so loading is a matter of reading
the file and, for the diffusers layout, undoing the key map.  The safetensors container (8-byte
little-endian header length, JSON header, raw little-endian tensor bytes) is parsed here directly.
"""
from __future__ import annotations

import json
import os
import struct
from collections import OrderedDict
from typing import Dict, Iterable, List, Optional, Tuple

import torch

StateDict = Dict[str, torch.Tensor]

_ST_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_ST_NAMES = {v: k for k, v in _ST_DTYPES.items()}
if hasattr(torch, "float8_e4m3fn"):
    _ST_DTYPES["F8_E4M3"] = torch.float8_e4m3fn
    _ST_NAMES[torch.float8_e4m3fn] = "F8_E4M3"


def load_safetensors(path: str) -> StateDict:
    """Tensors of one ``.safetensors`` file (CPU, own memory)."""
    with open(path, "rb") as fh:
        head = fh.read(8)
        if len(head) != 8:
            raise ValueError(f"{path}: not a safetensors file (shorter than its length field)")
        (hlen,) = struct.unpack("<Q", head)
        if hlen > 100 * 1024 * 1024:
            raise ValueError(f"{path}: implausible safetensors header of {hlen} bytes")
        header = json.loads(fh.read(hlen).decode("utf-8"))
        data = fh.read()
    out: StateDict = OrderedDict()
    for name, info in header.items():
        if name == "__metadata__":
            continue
        dt = _ST_DTYPES.get(info["dtype"])
        if dt is None:
            raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {info['dtype']}")
        a, b = info["data_offsets"]
        shape = tuple(info["shape"])
        n = 1
        for s in shape:
            n *= s
        esize = torch.empty((), dtype=dt).element_size()
        if not (0 <= a <= b <= len(data)) or b - a != n * esize:
            raise ValueError(f"{path}: tensor {name!r} has inconsistent offsets {a}..{b} for shape {shape}")
        if n == 0:
            out[name] = torch.empty(shape, dtype=dt)
        else:
            out[name] = torch.frombuffer(bytearray(data[a:b]), dtype=dt).reshape(shape)
    return out


def save_safetensors(tensors: StateDict, path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    """Writes ``tensors`` as one ``.safetensors`` file (contiguous, little-endian, 8-byte aligned header)."""
    header, blobs, off = OrderedDict(), [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _ST_NAMES:
            raise ValueError(f"tensor {name!r}: dtype {t.dtype} has no safetensors name")
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _ST_NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hbytes = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hbytes += b" " * (-len(hbytes) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(hbytes)))
        fh.write(hbytes)
        for raw in blobs:
            fh.write(raw)


def find_model(path: str, trusted_pickle: bool = False) -> dict:
    """Reads a checkpoint file into ``{"state_dict": ...}`` form (tools/download.py:31-62 without
    the download step).  ``.pth`` files are unpickled with ``weights_only=True`` unless
    ``trusted_pickle`` is set (needed only for files that carry optimizer or RNG objects)."""
    if not os.path.isfile(path):
        raise FileNotFoundError(f"Could not find Sana checkpoint at {path}")
    if path.endswith(".safetensors"):
        return {"state_dict": load_safetensors(path)}
    if path.endswith(".safetensors.index.json"):
        with open(path) as fh:
            index = json.load(fh)["weight_map"]
        sd: StateDict = OrderedDict()
        for shard in sorted(set(index.values())):
            sd.update(load_safetensors(os.path.join(os.path.dirname(path), shard)))
        return {"state_dict": sd}
    ck = torch.load(path, map_location="cpu", weights_only=not trusted_pickle)
    if not isinstance(ck, dict):
        raise ValueError(f"{path}: expected a dict checkpoint, got {type(ck).__name__}")
    return ck


POS_EMBED_KEYS = ("pos_embed", "base_model.pos_embed", "model.pos_embed")


def load_checkpoint(path: str, model: torch.nn.Module, load_ema: bool = False, null_embed: Optional[torch.Tensor] = None,
                    remove_state_dict_keys: Optional[Iterable[str]] = None, diffusers_layout: Optional[bool] = None,
                    trusted_pickle: bool = False) -> Tuple[List[str], List[str]]:
    """Loads the weights of ``path`` into ``model`` the way ``load_checkpoint_ddp`` does
    (diffusion/utils/checkpoint.py:264-325): the position tables and ``remove_state_dict_keys`` are
    dropped, ``state_dict_ema`` is used with ``load_ema``, a bare state dict is accepted,
    ``null_embed`` (the unconditional caption embedding) replaces ``y_embedder.y_embedding``,
    tensors with fewer dimensions than the parameter get trailing 1s, keys the model does not have
    are ignored.  Files in the diffusers layout (detected by their keys, or forced with
    ``diffusers_layout``) are mapped back to upstream's keys first.  Returns (missing, unexpected)."""
    ck = find_model(path, trusted_pickle)
    drop = list(remove_state_dict_keys or []) + list(POS_EMBED_KEYS)
    if load_ema:
        if "state_dict_ema" not in ck:
            raise KeyError(f"{path} has no state_dict_ema")
        sd = ck["state_dict_ema"]
    else:
        sd = ck.get("state_dict", ck)
    sd = OrderedDict((k, v) for k, v in sd.items() if k not in drop and torch.is_tensor(v))
    if diffusers_layout or (diffusers_layout is None and any(k.startswith("transformer_blocks.") for k in sd)):
        sd = from_diffusers_keys(sd)
    if null_embed is not None:
        sd["y_embedder.y_embedding"] = null_embed
    own = model.state_dict()
    picked: StateDict = OrderedDict()
    for k, v in own.items():
        if k in sd:
            w = sd[k]
            if w.dim() < v.dim():  # e.g. a [out, in] matrix for a 1x1 convolution
                w = w.reshape(*w.shape, *([1] * (v.dim() - w.dim())))
            picked[k] = w
    missing, unexpected = model.load_state_dict(picked, strict=False)
    unexpected = list(unexpected) + [k for k in sd if k not in own]
    return list(missing), unexpected


# ---- diffusers layout <-> upstream layout ---------------------------------------------------------
_TOP = [  # (diffusers, upstream)
    ("patch_embed.proj.weight", "x_embedder.proj.weight"), ("patch_embed.proj.bias", "x_embedder.proj.bias"),
    ("caption_projection.linear_1.weight", "y_embedder.y_proj.fc1.weight"),
    ("caption_projection.linear_1.bias", "y_embedder.y_proj.fc1.bias"),
    ("caption_projection.linear_2.weight", "y_embedder.y_proj.fc2.weight"),
    ("caption_projection.linear_2.bias", "y_embedder.y_proj.fc2.bias"),
    ("time_embed.emb.timestep_embedder.linear_1.weight", "t_embedder.mlp.0.weight"),
    ("time_embed.emb.timestep_embedder.linear_1.bias", "t_embedder.mlp.0.bias"),
    ("time_embed.emb.timestep_embedder.linear_2.weight", "t_embedder.mlp.2.weight"),
    ("time_embed.emb.timestep_embedder.linear_2.bias", "t_embedder.mlp.2.bias"),
    ("time_embed.linear.weight", "t_block.1.weight"), ("time_embed.linear.bias", "t_block.1.bias"),
    ("caption_norm.weight", "attention_y_norm.weight"),
    ("proj_out.weight", "final_layer.linear.weight"), ("proj_out.bias", "final_layer.linear.bias"),
    ("scale_shift_table", "final_layer.scale_shift_table"),
]
_BLOCK = [  # one-to-one keys of a block
    ("scale_shift_table", "scale_shift_table"),
    ("attn1.norm_q.weight", "attn.q_norm.weight"), ("attn1.norm_k.weight", "attn.k_norm.weight"),
    ("attn1.to_out.0.weight", "attn.proj.weight"), ("attn1.to_out.0.bias", "attn.proj.bias"),
    ("ff.conv_inverted.weight", "mlp.inverted_conv.conv.weight"), ("ff.conv_inverted.bias", "mlp.inverted_conv.conv.bias"),
    ("ff.conv_depth.weight", "mlp.depth_conv.conv.weight"), ("ff.conv_depth.bias", "mlp.depth_conv.conv.bias"),
    ("ff.conv_point.weight", "mlp.point_conv.conv.weight"),
    ("attn2.to_q.weight", "cross_attn.q_linear.weight"), ("attn2.to_q.bias", "cross_attn.q_linear.bias"),
    ("attn2.norm_q.weight", "cross_attn.q_norm.weight"), ("attn2.norm_k.weight", "cross_attn.k_norm.weight"),
    ("attn2.to_out.0.weight", "cross_attn.proj.weight"), ("attn2.to_out.0.bias", "cross_attn.proj.bias"),
]


def to_diffusers_keys(sd: StateDict) -> StateDict:
    """Upstream keys -> the diffusers transformer layout (convert_sana_to_diffusers.py:72-228): the
    fused ``attn.qkv`` splits into to_q / to_k / to_v and ``cross_attn.kv_linear`` into to_k / to_v."""
    sd = dict(sd)
    out: StateDict = OrderedDict()
    for d, u in _TOP:
        if u in sd:
            out[d] = sd.pop(u)
    depth = 1 + max([int(k.split(".")[1]) for k in sd if k.startswith("blocks.")], default=-1)
    for i in range(depth):
        b, t = f"blocks.{i}.", f"transformer_blocks.{i}."
        q, k, v = torch.chunk(sd.pop(b + "attn.qkv.weight"), 3, dim=0)
        out[t + "attn1.to_q.weight"], out[t + "attn1.to_k.weight"], out[t + "attn1.to_v.weight"] = q, k, v
        kw, vw = torch.chunk(sd.pop(b + "cross_attn.kv_linear.weight"), 2, dim=0)
        kb, vb = torch.chunk(sd.pop(b + "cross_attn.kv_linear.bias"), 2, dim=0)
        out[t + "attn2.to_k.weight"], out[t + "attn2.to_v.weight"] = kw, vw
        out[t + "attn2.to_k.bias"], out[t + "attn2.to_v.bias"] = kb, vb
        for d, u in _BLOCK:
            if b + u in sd:
                out[t + d] = sd.pop(b + u)
    out.update(sd)  # keys the map does not know travel unchanged
    return out


def from_diffusers_keys(sd: StateDict) -> StateDict:
    """The inverse of :func:`to_diffusers_keys`: a diffusers-layout transformer state dict with
    upstream's keys and fused projections (rows q | k | v and k | v)."""
    sd = dict(sd)
    out: StateDict = OrderedDict()
    for d, u in _TOP:
        if d in sd:
            out[u] = sd.pop(d)
    depth = 1 + max([int(k.split(".")[1]) for k in sd if k.startswith("transformer_blocks.")], default=-1)
    for i in range(depth):
        b, t = f"blocks.{i}.", f"transformer_blocks.{i}."
        out[b + "attn.qkv.weight"] = torch.cat([sd.pop(t + f"attn1.to_{n}.weight") for n in "qkv"], dim=0)
        out[b + "cross_attn.kv_linear.weight"] = torch.cat([sd.pop(t + f"attn2.to_{n}.weight") for n in "kv"], dim=0)
        out[b + "cross_attn.kv_linear.bias"] = torch.cat([sd.pop(t + f"attn2.to_{n}.bias") for n in "kv"], dim=0)
        for d, u in _BLOCK:
            if t + d in sd:
                out[b + u] = sd.pop(t + d)
    out.update(sd)
    return out

"""Offline NVFP4 weight pack: quantise the projection weights of a model once, store the
codes and scales, and load them into another process so that no weight is quantised at run
time (activations still are, per call).

Format (a flat dict of tensors, ``torch.save``-able; one group per quantised projection, keyed
by the module's name inside the model and the projection's name):

    <module>.<proj>.nvfp4.q       uint8 [N, K/2]   E2M1 codes, element 2j in the low nibble
    <module>.<proj>.nvfp4.sf      uint8 [...]      E4M3 scales, one per 16 elements along K, in the
                                                   512-byte tiles the tensor core reads
                                                   (offset (r%32)*16 + ((r%128)/32)*4 + kb%4 inside
                                                   tile (r/128, kb/4), K tiles padded to x4)
    <module>.<proj>.nvfp4.scales  fp32 [4]         (amax, tensor scale = amax / (6 * 448), 0, 0)
    <module>.<proj>.nvfp4.shape   int64 [2]        (N, K)

The projections are the four that ``SanaMSBlock.set_nvfp4`` switches to FP4: ``attn`` qkv and
proj, ``mlp`` inverted_conv and point_conv.  Upstream has no such file format (it quantises
through Transformer Engine at run time, inference_video_scripts/wm/inference_sana_wm.py:388-406).
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn as nn

from . import ops
from .modules import GLUMBConv, LiteLA


def _projections(module: nn.Module):
    """(key used by modules._project, 2-D weight view) of every NVFP4-capable projection."""
    if isinstance(module, LiteLA):
        yield "qkv", module.qkv.weight
        yield "proj", module.proj.weight
    elif isinstance(module, GLUMBConv):
        ic, pc = module.inverted_conv.conv, module.point_conv.conv
        yield "inverted_conv", ic.weight.reshape(ic.out_channels, ic.in_channels)
        yield "point_conv", pc.weight.reshape(pc.out_channels, pc.in_channels)


@torch.no_grad()
def pack_nvfp4_weights(model: nn.Module) -> Dict[str, torch.Tensor]:
    """Quantises every NVFP4-capable projection weight of ``model`` (bf16, on a CUDA device) and
    returns the pack (tensors on the CPU)."""
    pack: Dict[str, torch.Tensor] = {}
    for name, module in model.named_modules():
        for key, w in _projections(module):
            if w.dtype != torch.bfloat16 or not w.is_cuda:
                raise ValueError(f"{name}.{key}: NVFP4 packing needs bf16 weights on a CUDA device")
            t = ops.nvfp4_quantize(w.contiguous())
            base = f"{name}.{key}.nvfp4"
            pack[base + ".q"] = t.q.cpu()
            pack[base + ".sf"] = t.sf.cpu()
            pack[base + ".scales"] = t.scales.cpu()
            pack[base + ".shape"] = torch.tensor([t.rows, t.K], dtype=torch.int64)
    if not pack:
        raise ValueError("the model has no NVFP4-capable projection (LiteLA / GLUMBConv)")
    return pack


@torch.no_grad()
def load_nvfp4_weights(model: nn.Module, pack: Dict[str, torch.Tensor], enable: bool = True) -> int:
    """Installs the packed weights on the matching modules of ``model`` (moved to each module's
    device) so that their NVFP4 projections use them instead of quantising the bf16 weights, and
    (``enable``) switches those modules to NVFP4.  Every NVFP4-capable projection of the model must
    be in the pack with the right shape.  Returns the number of projections installed."""
    n = 0
    for name, module in model.named_modules():
        for key, w in _projections(module):
            base = f"{name}.{key}.nvfp4"
            if base + ".q" not in pack:
                raise KeyError(f"{base}.* missing from the weight pack")
            rows, K = (int(v) for v in pack[base + ".shape"])
            if (rows, K) != tuple(w.shape):
                raise ValueError(f"{base}: packed shape {(rows, K)} does not match the model's {tuple(w.shape)}")
            dev = w.device
            t = ops.NvFp4Tensor(pack[base + ".q"].to(dev), pack[base + ".sf"].to(dev), pack[base + ".scales"].to(dev),
                                rows, K)
            module.__dict__.setdefault("_nvfp4_packed", {})[key] = t
            n += 1
        if enable and isinstance(module, (LiteLA, GLUMBConv)):
            module.nvfp4 = True
    return n

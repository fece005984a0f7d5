"""Import the upstream Sana hot-path modules unmodified, on CPU, without their package tree.

Used only by ``make_golden.py`` (fixture generation) on a machine that has a checkout of
NVlabs/Sana; nothing in the test-suite, the benchmark or the package imports this file at
run time.  The upstream package ``__init__`` files import every scheduler and every net
(diffusers, mmcv, xformers, ...), so this loader

1. registers empty namespace modules for the ``diffusion.*`` packages whose ``__path__``
   points at the real directories (sub-modules then load from the real files while the
   package ``__init__``s never run),
2. provides minimal stand-ins for the third-party names the hot path touches
   (``timm.models.vision_transformer.Attention`` / ``Mlp``, ``timm.models.layers.DropPath``,
   ``mmcv.Registry``, ``termcolor.colored``) - these contribute no arithmetic beyond
   ``torch.nn.Linear``,
3. replaces three heavy in-repo modules by stubs exposing only the names that
   ``sana.py`` / ``sana_multi_scale.py`` use.
"""
from __future__ import annotations

import importlib
import importlib.machinery
import os
import sys
import types

import torch.nn as nn

_LOADED = {}


def _ns(name: str, path: str | None = None) -> types.ModuleType:
    mod = types.ModuleType(name)
    mod.__spec__ = importlib.machinery.ModuleSpec(name, loader=None, is_package=True)
    mod.__path__ = [path] if path else []
    if path:
        mod.__spec__.submodule_search_locations = [path]
    sys.modules[name] = mod
    return mod


def _install_third_party_shims() -> None:
    if "timm" not in sys.modules:
        timm = _ns("timm")
        models = _ns("timm.models")
        vt = _ns("timm.models.vision_transformer")
        layers = _ns("timm.models.layers")

        class Attention(nn.Module):
            # constructor contract of timm 0.6.x vision_transformer.Attention
            def __init__(self, dim, num_heads=8, qkv_bias=False, attn_drop=0.0, proj_drop=0.0, **kw):
                super().__init__()
                self.num_heads = num_heads
                self.scale = (dim // num_heads) ** -0.5
                self.qkv = nn.Linear(dim, dim * 3, bias=qkv_bias)
                self.attn_drop = nn.Dropout(attn_drop)
                self.proj = nn.Linear(dim, dim)
                self.proj_drop = nn.Dropout(proj_drop)

        class Mlp(nn.Module):
            def __init__(self, in_features, hidden_features=None, out_features=None, act_layer=nn.GELU, drop=0.0):
                super().__init__()
                out_features = out_features or in_features
                hidden_features = hidden_features or in_features
                self.fc1 = nn.Linear(in_features, hidden_features)
                self.act = act_layer()
                self.drop1 = nn.Dropout(drop)
                self.fc2 = nn.Linear(hidden_features, out_features)
                self.drop2 = nn.Dropout(drop)

            def forward(self, x):
                return self.drop2(self.fc2(self.drop1(self.act(self.fc1(x)))))

        class DropPath(nn.Module):
            def __init__(self, drop_prob=0.0):
                super().__init__()
                self.drop_prob = drop_prob

            def forward(self, x):
                assert self.drop_prob == 0.0 or not self.training
                return x

        vt.Attention, vt.Mlp = Attention, Mlp
        layers.DropPath = DropPath
        timm.models, models.vision_transformer, models.layers = models, vt, layers

    if "mmcv" not in sys.modules:
        mmcv = _ns("mmcv")

        class Registry:
            def __init__(self, name):
                self.name, self._d = name, {}

            def register_module(self, name=None, force=False, module=None):
                def deco(cls):
                    self._d[name or cls.__name__] = cls
                    return cls

                return deco if module is None else deco(module)

            def get(self, key):
                return self._d.get(key)

        mmcv.Registry = Registry

    if "termcolor" not in sys.modules:
        tc = _ns("termcolor")
        tc.colored = lambda s, *a, **k: s


def load_reference(root: str):
    """Returns a namespace with the upstream ``LiteLA``, ``GLUMBConv``, ``SanaMSBlock``,
    ``MultiHeadCrossAttention``, ``TimestepEmbedder`` and ``t2i_modulate``."""
    if root in _LOADED:
        return _LOADED[root]
    if not os.path.isdir(os.path.join(root, "diffusion")):
        raise FileNotFoundError(f"no Sana checkout at {root}")
    _install_third_party_shims()
    d = os.path.join(root, "diffusion")
    _ns("diffusion", d)
    _ns("diffusion.model", os.path.join(d, "model"))
    _ns("diffusion.model.nets", os.path.join(d, "model", "nets"))
    _ns("diffusion.utils", os.path.join(d, "utils"))
    _ns("diffusion.distributed", os.path.join(d, "distributed"))
    _ns("diffusion.distributed.context_parallel", os.path.join(d, "distributed", "context_parallel"))

    builder = types.ModuleType("diffusion.model.builder")
    builder.MODELS = sys.modules["mmcv"].Registry("models")
    sys.modules["diffusion.model.builder"] = builder
    du = types.ModuleType("diffusion.utils.dist_utils")
    du.get_rank = lambda: 0
    sys.modules["diffusion.utils.dist_utils"] = du
    lg = types.ModuleType("diffusion.utils.logger")
    import logging

    lg.get_root_logger = lambda *a, **k: logging.getLogger("sana-ref")
    sys.modules["diffusion.utils.logger"] = lg

    blocks = importlib.import_module("diffusion.model.nets.sana_blocks")
    basic = importlib.import_module("diffusion.model.nets.basic_modules")
    ms = importlib.import_module("diffusion.model.nets.sana_multi_scale")
    ns = types.SimpleNamespace(
        LiteLA=blocks.LiteLA,
        GLUMBConv=basic.GLUMBConv,
        SanaMSBlock=ms.SanaMSBlock,
        MultiHeadCrossAttention=blocks.MultiHeadCrossAttention,
        TimestepEmbedder=blocks.TimestepEmbedder,
        t2i_modulate=blocks.t2i_modulate,
        sana_blocks=blocks,
        basic_modules=basic,
        sana_multi_scale=ms,
    )
    _LOADED[root] = ns
    return ns


def load_video_module(root: str):
    """Upstream's ``sana_multi_scale_video`` (SanaVideoMSBlock).  Its one import outside the nets,
    ``diffusion.model.wan.model.BlockHook`` (a type annotation), is stubbed: the real module needs
    diffusers."""
    load_reference(root)
    if "diffusion.model.wan.model" not in sys.modules:
        _ns("diffusion.model.wan")
        wm = types.ModuleType("diffusion.model.wan.model")
        wm.BlockHook = object
        sys.modules["diffusion.model.wan.model"] = wm
    return importlib.import_module("diffusion.model.nets.sana_multi_scale_video")


def set_fp32_attention(module: nn.Module) -> None:
    """What upstream ``build_model(use_fp32_attention=True)`` does for every shipped config."""
    for m in module.modules():
        m.fp32_attention = True

"""Seeded synthetic weights and inputs with the shapes of the five benchmark configurations.

The reference evaluates on public image/video suites; a block benchmark depends only on
tensor shapes, so seeded N(0,1) activations and N(0, 0.02) weights of the same shapes stand
in for them (no dataset item or checkpoint is used or reproduced).

All generators draw on the CPU from one ``torch.Generator`` so that the same numbers are
obtained on every machine, then move to the requested device/dtype.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

Params = Dict[str, torch.Tensor]


@dataclass(frozen=True)
class BlockShape:
    name: str
    hidden: int          # C
    cross_heads: int     # heads of the softmax cross-attention
    batch: int
    grid: Tuple[int, ...]  # (H, W) or (T, H, W)
    text_len: int = 300
    mlp_ratio: float = 2.5
    blocks: int = 1

    @property
    def tokens(self) -> int:
        return math.prod(self.grid)

    @property
    def ffn_hidden(self) -> int:
        return int(self.hidden * self.mlp_ratio)

    @property
    def la_heads(self) -> int:
        return self.hidden // 32


# the five configurations of the benchmark definition
CFG1 = BlockShape("cfg1-litela-fp32", 1152, 16, 1, (32, 32))
CFG2 = BlockShape("cfg2-block-600m-bf16", 1152, 16, 4, (32, 32))
CFG3 = BlockShape("cfg3-stack-1600m-bf16", 2240, 20, 1, (128, 128), blocks=20)
CFG4 = BlockShape("cfg4-seqpar-1600m-bf16", 2240, 20, 1, (21, 45, 80))
CFG5 = BlockShape("cfg5-nvfp4-1600m", 2240, 20, 8, (64, 64))


def block_param_shapes(C: int, hid: int) -> Dict[str, Tuple[int, ...]]:
    """State-dict keys/shapes of upstream's SanaMSBlock(attn_type='linear', ffn_type='glumbconv')."""
    return {
        "scale_shift_table": (6, C),
        "attn.qkv.weight": (3 * C, C),
        "attn.proj.weight": (C, C),
        "attn.proj.bias": (C,),
        "cross_attn.q_linear.weight": (C, C),
        "cross_attn.q_linear.bias": (C,),
        "cross_attn.kv_linear.weight": (2 * C, C),
        "cross_attn.kv_linear.bias": (2 * C,),
        "cross_attn.proj.weight": (C, C),
        "cross_attn.proj.bias": (C,),
        "mlp.inverted_conv.conv.weight": (2 * hid, C, 1, 1),
        "mlp.inverted_conv.conv.bias": (2 * hid,),
        "mlp.depth_conv.conv.weight": (2 * hid, 1, 3, 3),
        "mlp.depth_conv.conv.bias": (2 * hid,),
        "mlp.point_conv.conv.weight": (C, hid, 1, 1),
    }


def make_block_params(C: int, hid: int, seed: int, std: float = 0.02, dtype=torch.float32,
                      device="cpu") -> Params:
    """Every parameter ~ N(0, std), drawn in state-dict order from Generator(seed)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for k, shp in block_param_shapes(C, hid).items():
        out[k] = (torch.randn(shp, generator=g) * std).to(dtype=dtype, device=device)
    return out


def make_block_params_on_device(C: int, hid: int, seed: int, std: float, dtype, device) -> Params:
    """Same distribution drawn with the device generator (fast path for the 20-block
    benchmark stack; values differ from the CPU generator's)."""
    g = torch.Generator(device=device).manual_seed(seed)
    return {k: (torch.randn(shp, generator=g, device=device) * std).to(dtype)
            for k, shp in block_param_shapes(C, hid).items()}


def timestep_embedding(t: torch.Tensor, dim: int = 256, max_period: int = 10000) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(0, half, dtype=torch.float32) / half)
    args = t[:, None].float() * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


def make_block_inputs(shape: BlockShape, seed: int = 0, std: float = 0.02, text_dim: int = 2304,
                      batch: Optional[int] = None):
    """x ~ N(0,1) [B, N, C]; y = text ~ N(0,1) [B, L, text_dim] projected to C by a seeded
    N(0, std) linear; t [B, 6C] from t_scalar ~ U[0,1000) through sinusoidal embedding ->
    Linear/SiLU/Linear -> SiLU -> Linear(C, 6C), all N(0, std).  fp32 CPU tensors."""
    B = batch or shape.batch
    C, N, L = shape.hidden, shape.tokens, shape.text_len
    g = torch.Generator().manual_seed(10_000 + seed)
    x = torch.randn(B, N, C, generator=g)
    text = torch.randn(B, L, text_dim, generator=g)
    w_y = torch.randn(C, text_dim, generator=g) * std
    y = text @ w_y.t()
    t_scalar = torch.rand(B, generator=g) * 1000.0
    w0 = torch.randn(C, 256, generator=g) * std
    b0 = torch.randn(C, generator=g) * std
    w2 = torch.randn(C, C, generator=g) * std
    b2 = torch.randn(C, generator=g) * std
    wt = torch.randn(6 * C, C, generator=g) * std
    bt = torch.randn(6 * C, generator=g) * std
    e = timestep_embedding(t_scalar) @ w0.t() + b0
    e = torch.nn.functional.silu(e) @ w2.t() + b2
    t = torch.nn.functional.silu(e) @ wt.t() + bt
    return x, y, t


def make_litela_cfg1(seed: int = 0):
    """cfg 1: x ~ N(0,1) [1, 1024, 1152]; qkv/proj weights Xavier-uniform, proj bias zero."""
    C = CFG1.hidden
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(1, CFG1.tokens, C, generator=g)

    def xavier(out_f, in_f):
        bound = math.sqrt(6.0 / (in_f + out_f))
        return (torch.rand(out_f, in_f, generator=g) * 2 - 1) * bound

    p = {"qkv.weight": xavier(3 * C, C), "proj.weight": xavier(C, C), "proj.bias": torch.zeros(C)}
    return x, p


def load_block_params(block: torch.nn.Module, params: Params) -> None:
    """Copies a state-dict-keyed parameter dict into a block (strict)."""
    missing, unexpected = block.load_state_dict(params, strict=True)
    assert not missing and not unexpected

"""Perturbed-attention-guidance processors for LiteLA on the library's kernels.

Upstream's samplers install a processor on selected blocks with
``model.blocks[i].attn.forward = Processor(model.blocks[i].attn)``
(diffusion/model/dpm_solver.py:486-499); ``SanaMSBlock.forward`` here honours a ``forward``
installed on the attention instance.  These two classes are drop-ins for upstream's
``PAGIdentitySelfAttnProcessorLiteLA`` / ``PAGCFGIdentitySelfAttnProcessorLiteLA``
(diffusion/model/nets/sana_blocks.py:573-675): the batch is [.., original.., perturbed]; the
original chunks go through linear attention, the perturbed chunk through "identity attention",
i.e. its value projection straight into the output projection.  Upstream's own classes also
work on this package's LiteLA (they only use its attributes), but run the projections through
``nn.Linear``; these run them on the GEMM kernel.
"""
from __future__ import annotations

import torch

from . import ops
from .modules import LiteLA, _as2d


class _PAGProcessor:
    chunks = 2

    def __init__(self, attn: LiteLA):
        self.attn = attn

    @torch.no_grad()
    def __call__(self, x: torch.Tensor, mask=None, HW=None, rotary_emb=None, block_id=None, block_mask=None,
                 **kwargs) -> torch.Tensor:
        attn = self.attn
        if x.shape[0] % self.chunks:
            raise ValueError(f"the batch must hold {self.chunks} equal chunks")
        nb = x.shape[0] // self.chunks
        x_org, x_ptb = x[: nb * (self.chunks - 1)], x[nb * (self.chunks - 1):]
        out = LiteLA.forward(attn, x_org, HW=HW, rotary_emb=rotary_emb)
        C = attn.out_dim
        bias = attn.qkv.bias[2 * C:3 * C] if attn.qkv.bias is not None else None
        v = ops.gemm(_as2d(x_ptb.contiguous()), attn.qkv.weight[2 * C:3 * C], bias=bias)
        p = ops.gemm(v, attn.proj.weight, bias=attn.proj.bias).reshape(x_ptb.shape[0], x_ptb.shape[1], -1)
        return torch.cat([out, p])


class PAGIdentitySelfAttnProcessorLiteLA(_PAGProcessor):
    """Batch = [original, perturbed] (guidance scale 1)."""

    chunks = 2


class PAGCFGIdentitySelfAttnProcessorLiteLA(_PAGProcessor):
    """Batch = [unconditional, original, perturbed]."""

    chunks = 3

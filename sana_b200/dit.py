"""The whole multi-scale Linear-DiT forward on libsana_b200's kernels: the steps either side of
the block loop of upstream's ``SanaMS.forward`` plus the loop itself.

  PatchEmbedMS      diffusion/model/nets/sana_blocks.py:1235-1268
  TimestepEmbedder  diffusion/model/nets/sana_blocks.py:967-1012
  CaptionEmbedder   diffusion/model/nets/sana_blocks.py:1083-1138
  T2IFinalLayer     diffusion/model/nets/sana_blocks.py:893-925
  SanaMS            diffusion/model/nets/sana_multi_scale.py:160-421 (on Sana, sana.py:163-300)

Constructor arguments, attribute names, state-dict keys and the ``forward`` signature are
upstream's, so a checkpoint written by upstream loads with ``load_state_dict(strict=True)``.
Inference only.  The sin-cos position table is built on the host once per latent size (as
upstream does, in numpy) and added inside the patch-embedding projection's epilogue.
"""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch
import torch.nn as nn

from . import ops
from .modules import RMSNorm, SanaMSBlock, _as2d


def _sincos_1d(embed_dim: int, pos: np.ndarray) -> np.ndarray:
    """sana.py:447-465: [M] positions -> [M, embed_dim] = sin | cos of pos * 10000^(-2i/embed_dim)
    (float64 frequencies, so the product and the result are float64)."""
    if embed_dim % 2:
        raise ValueError("the sin-cos table needs an even number of channels per axis")
    omega = np.arange(embed_dim // 2, dtype=np.float64)
    omega /= embed_dim / 2.0
    omega = 1.0 / 10000 ** omega
    out = np.einsum("m,d->md", pos.reshape(-1), omega)
    return np.concatenate([np.sin(out), np.cos(out)], axis=1)


def sincos_pos_embed_2d(embed_dim: int, grid_hw, pe_interpolation: float = 1.0, base_size: int = 16) -> np.ndarray:
    """sana.py:416-444: [h*w, embed_dim] float64 table.  Coordinates are float32
    ``arange(n) / (n / base_size) / pe_interpolation``; the meshgrid puts w first and is then
    *reshaped* (not transposed) to [2, 1, w, h], exactly as upstream does."""
    h, w = grid_hw
    gh = np.arange(h, dtype=np.float32) / (h / base_size) / pe_interpolation
    gw = np.arange(w, dtype=np.float32) / (w / base_size) / pe_interpolation
    grid = np.stack(np.meshgrid(gw, gh), axis=0).reshape([2, 1, w, h])
    first = _sincos_1d(embed_dim // 2, grid[0])
    second = _sincos_1d(embed_dim // 2, grid[1])
    return np.concatenate([first, second], axis=1)


class Mlp(nn.Module):
    """Two linears with an activation between them (state-dict keys ``fc1`` / ``fc2`` of
    timm's Mlp, which upstream's CaptionEmbedder uses); the activation is fused into the first
    projection's epilogue."""

    def __init__(self, in_features, hidden_features=None, out_features=None, act: int = ops.ACT_GELU_TANH):
        super().__init__()
        self.fc1 = nn.Linear(in_features, hidden_features or in_features)
        self.fc2 = nn.Linear(hidden_features or in_features, out_features or in_features)
        self.act_code = act

    @torch.no_grad()
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = ops.gemm(_as2d(x.contiguous()), self.fc1.weight, bias=self.fc1.bias, act=self.act_code)
        o = ops.gemm(h, self.fc2.weight, bias=self.fc2.bias)
        return o.reshape(*x.shape[:-1], o.shape[-1])


class PatchEmbedMS(nn.Module):
    """Patch convolution (kernel = stride = patch size) as unfold + projection; ``forward``
    optionally adds a per-token table [N, embed] (the position embedding) in the same kernel."""

    def __init__(self, patch_size=16, in_chans=3, embed_dim=768, kernel_size=None, padding=0, norm_layer=None,
                 flatten=True, bias=True):
        super().__init__()
        kernel_size = kernel_size or patch_size
        if isinstance(kernel_size, (tuple, list)):
            kernel_size = kernel_size[0]
        if kernel_size != patch_size or padding or norm_layer is not None or not flatten:
            raise NotImplementedError("PatchEmbedMS here covers kernel_size == patch_size, no padding, no norm")
        self.patch_size = (patch_size, patch_size)
        self.flatten = flatten
        self.proj = nn.Conv2d(in_chans, embed_dim, kernel_size=kernel_size, stride=patch_size, bias=bias)
        self.norm = nn.Identity()

    @torch.no_grad()
    def forward(self, x: torch.Tensor, pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, Cin, H, W = x.shape
        p = self.patch_size[0]
        N = (H // p) * (W // p)
        rows = ops.patchify(x, p)
        w2d = self.proj.weight.reshape(self.proj.out_channels, -1)
        if pos is None:
            out = ops.gemm(rows, w2d, bias=self.proj.bias)
        else:
            out = torch.empty(B * N, w2d.shape[0], dtype=x.dtype, device=x.device)
            pos2d = pos.reshape(N, -1)
            for b in range(B):  # the table repeats per sample: one launch each, the add rides in the epilogue
                ops.gemm(rows[b * N:(b + 1) * N], w2d, bias=self.proj.bias, residual=pos2d, out=out[b * N:(b + 1) * N])
        return out.view(B, N, -1)


class TimestepEmbedder(nn.Module):
    """Sinusoidal features -> Linear -> SiLU -> Linear."""

    def __init__(self, hidden_size, frequency_embedding_size=256):
        super().__init__()
        self.mlp = nn.Sequential(nn.Linear(frequency_embedding_size, hidden_size, bias=True), nn.SiLU(),
                                 nn.Linear(hidden_size, hidden_size, bias=True))
        self.frequency_embedding_size = frequency_embedding_size

    @property
    def dtype(self):
        return next(self.parameters()).dtype

    @torch.no_grad()
    def forward(self, t: torch.Tensor) -> torch.Tensor:
        f = ops.timestep_embedding(t, self.frequency_embedding_size, self.dtype)
        h = ops.gemm(f, self.mlp[0].weight, bias=self.mlp[0].bias, act=ops.ACT_SILU)
        return ops.gemm(h, self.mlp[2].weight, bias=self.mlp[2].bias)


class CaptionEmbedder(nn.Module):
    """Caption features [B, 1, L, Cc] -> [B, 1, L, hidden] through a GELU(tanh) MLP.  The
    ``y_embedding`` buffer (the unconditional caption) is kept for checkpoints and for forced
    drops; random label dropout is a training feature and is not covered."""

    def __init__(self, in_channels, hidden_size, uncond_prob, act_layer=None, token_num=120):
        super().__init__()
        self.y_proj = Mlp(in_channels, hidden_size, hidden_size, act=ops.ACT_GELU_TANH)
        self.register_buffer("y_embedding", torch.randn(token_num, in_channels) / in_channels ** 0.5)
        self.uncond_prob = uncond_prob

    @torch.no_grad()
    def forward(self, caption, train=False, force_drop_ids=None, mask=None):
        if train:
            raise NotImplementedError("training-time label dropout is not covered")
        if force_drop_ids is not None:
            drop = (force_drop_ids == 1)[:, None, None, None]
            caption = torch.where(drop, self.y_embedding.to(caption.dtype), caption)
        return self.y_proj(caption)


class T2IFinalLayer(nn.Module):
    """LayerNorm + 2-way modulate + linear to patch pixels."""

    def __init__(self, hidden_size, patch_size, out_channels):
        super().__init__()
        if isinstance(patch_size, int):
            patch_size = [patch_size, patch_size]
        self.norm_final = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=1e-6)
        self.linear = nn.Linear(hidden_size, math.prod(patch_size) * out_channels, bias=True)
        self.scale_shift_table = nn.Parameter(torch.randn(2, hidden_size) / hidden_size ** 0.5)
        self.out_channels = out_channels

    @torch.no_grad()
    def forward(self, x: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        B, N, C = x.shape
        if t.dim() > 2:
            # frame-aware (sana_blocks.py:907-917): t [B, 1, F, C], one modulation vector per frame;
            # the frames of a sample are contiguous token ranges, so (sample, frame) acts as the batch
            F_ = t.shape[2]
            if N % F_:
                raise ValueError("the token count must be a multiple of the number of frames")
            z = ops.ln_modulate_rows(x.reshape(B * F_, N // F_, C), self.scale_shift_table,
                                     t.reshape(B * F_, 1, C), 0, 1, 0, 0, 1e-6).reshape(B, N, C)
            return ops.gemm(_as2d(z), self.linear.weight, bias=self.linear.bias).view(B, N, -1)
        z = ops.ln_modulate_rows(x, self.scale_shift_table, t.reshape(B, 1, C), 0, 1, 0, 0, 1e-6)
        return ops.gemm(_as2d(z), self.linear.weight, bias=self.linear.bias).view(B, N, -1)


class SanaMS(nn.Module):
    """Multi-scale Linear-DiT (Sana) forward, inference only."""

    def __init__(self, input_size=32, patch_size=2, in_channels=4, hidden_size=1152, depth=28, num_heads=16,
                 mlp_ratio=4.0, class_dropout_prob=0.1, learn_sigma=True, pred_sigma=True, drop_path: float = 0.0,
                 caption_channels=2304, pe_interpolation=1.0, config=None, model_max_length=300, qk_norm=False,
                 y_norm=False, norm_eps=1e-5, attn_type="linear", ffn_type="glumbconv", use_pe=True,
                 y_norm_scale_factor=1.0, patch_embed_kernel=None, mlp_acts=("silu", "silu", None), linear_head_dim=32,
                 cross_norm=False, cross_attn_type="flash", logvar=False, logvar_scale_factor=1.0, cfg_embed=False,
                 cfg_embed_scale=1.0, lr_scale=None, timestep_norm_scale_factor=1.0, pos_embed_type="sincos", **kwargs):
        super().__init__()
        if pos_embed_type != "sincos":
            raise NotImplementedError("only the sin-cos position embedding is covered")
        if logvar:
            raise NotImplementedError("the log-variance head (training) is not covered")
        self.pred_sigma = pred_sigma
        self.in_channels = in_channels
        self.out_channels = in_channels * 2 if pred_sigma else in_channels
        self.hidden_size = hidden_size
        self.patch_size = patch_size[0] if isinstance(patch_size, tuple) else patch_size
        self.num_heads = num_heads
        self.linear_head_dim = linear_head_dim
        self.pe_interpolation = pe_interpolation
        self.depth = depth
        self.use_pe = use_pe
        self.pos_embed_type = pos_embed_type
        self.y_norm = y_norm
        self.config = config
        self.timestep_norm_scale_factor = timestep_norm_scale_factor
        self.cfg_embed_scale = cfg_embed_scale
        self.base_size = input_size // self.patch_size
        self.h = self.w = 0

        self.x_embedder = PatchEmbedMS(self.patch_size, in_channels, hidden_size,
                                       kernel_size=patch_embed_kernel or self.patch_size, bias=True)
        self.t_embedder = TimestepEmbedder(hidden_size)
        self.cfg_embedder = TimestepEmbedder(hidden_size) if cfg_embed else None
        self.register_buffer("pos_embed", torch.zeros(1, self.base_size ** 2, hidden_size))
        self.t_block = nn.Sequential(nn.SiLU(), nn.Linear(hidden_size, 6 * hidden_size, bias=True))
        self.y_embedder = CaptionEmbedder(caption_channels, hidden_size, class_dropout_prob, token_num=model_max_length)
        if y_norm:
            self.attention_y_norm = RMSNorm(hidden_size, scale_factor=y_norm_scale_factor, eps=norm_eps)
        self.blocks = nn.ModuleList([
            SanaMSBlock(hidden_size, num_heads, mlp_ratio=mlp_ratio, drop_path=0.0, qk_norm=qk_norm,
                        attn_type=attn_type, ffn_type=ffn_type, mlp_acts=mlp_acts, linear_head_dim=linear_head_dim,
                        cross_norm=cross_norm, cross_attn_type=cross_attn_type) for _ in range(depth)])
        self.final_layer = T2IFinalLayer(hidden_size, self.patch_size, self.out_channels)
        self.logvar_linear = None
        self.pos_embed_ms = None
        # The blocks' key / value projections of the caption depend on nothing the block loop
        # computes: with this flag they are all launched on a second stream when the forward
        # starts and each block waits only for its own (at small latents the GPU has idle SMs for
        # them; captured in a CUDA graph they become a parallel branch).
        self.overlap_caption_projections = True
        self._side_stream = None

    @property
    def dtype(self):
        return next(self.parameters()).dtype

    def _position_table(self, x: torch.Tensor) -> torch.Tensor:
        """[1, N, C] sin-cos table for the current latent size, cached like upstream's
        ``pos_embed_ms`` (sana_multi_scale.py:296-312)."""
        if self.pos_embed_ms is None or self.pos_embed_ms.shape[1] != self.h * self.w or \
                self.pos_embed_ms.device != x.device or self.pos_embed_ms.dtype != self.dtype or \
                getattr(self, "_pos_hw", None) != (self.h, self.w):
            table = sincos_pos_embed_2d(self.pos_embed.shape[-1], (self.h, self.w),
                                        pe_interpolation=self.pe_interpolation, base_size=self.base_size)
            self.pos_embed_ms = torch.from_numpy(table).unsqueeze(0).to(x.device).to(self.dtype)
            self._pos_hw = (self.h, self.w)
        return self.pos_embed_ms

    @torch.no_grad()
    def forward(self, x, timestep, y, mask=None, data_info=None, return_logvar=False, jvp=False, **kwargs):
        """x [B, Cin, H, W] latents, timestep [B], y [B, 1, L, caption_channels], mask [B, L] (or
        [B, 1, 1, L]) of 0/1 -> [B, out_channels, H, W]."""
        if jvp or return_logvar:
            raise NotImplementedError("JVP / log-variance outputs (training) are not covered")
        bs = x.shape[0]
        x = x.to(self.dtype)
        if self.timestep_norm_scale_factor != 1.0:
            timestep = (timestep.float() / self.timestep_norm_scale_factor).to(torch.float32)
        else:
            timestep = timestep.long().to(torch.float32)
        y = y.to(self.dtype)
        p = self.patch_size
        self.h, self.w = x.shape[-2] // p, x.shape[-1] // p
        x = self.x_embedder(x, self._position_table(x) if self.use_pe else None)

        t = self.t_embedder(timestep)  # [B, C]
        if self.cfg_embedder is not None:
            t = t + self.cfg_embedder(data_info["cfg_scale"] * self.cfg_embed_scale)
        lin = self.t_block[1]
        t0 = ops.gemm(ops.silu(t), lin.weight, bias=lin.bias)  # [B, 6C]

        y = self.y_embedder(y, False, mask=mask)
        if self.y_norm:
            y = self.attention_y_norm(y)
        if mask is not None:
            mask = mask.to(torch.int16)
            if mask.shape[0] != y.shape[0]:
                mask = mask.repeat(y.shape[0] // mask.shape[0], 1)
            mask = mask.squeeze(1).squeeze(1)

        caption_kv = [None] * len(self.blocks)
        ready = None
        if self.overlap_caption_projections and "caption_kv" not in kwargs:
            cur = torch.cuda.current_stream()
            if self._side_stream is None or self._side_stream.device != x.device:
                self._side_stream = torch.cuda.Stream(device=x.device)
            side = self._side_stream
            side.wait_stream(cur)  # y is ready
            ready = []
            with torch.cuda.stream(side):
                for i, block in enumerate(self.blocks):
                    caption_kv[i] = block.cross_attn.project_kv(y)
                    caption_kv[i].record_stream(cur)
                    ev = torch.cuda.Event()
                    ev.record(side)
                    ready.append(ev)
        for i, block in enumerate(self.blocks):
            if ready is not None:
                torch.cuda.current_stream().wait_event(ready[i])
                x = block(x, y, t0, mask, (self.h, self.w), None, caption_kv=caption_kv[i], **kwargs)
            else:
                x = block(x, y, t0, mask, (self.h, self.w), None, **kwargs)
        if ready is not None:
            torch.cuda.current_stream().wait_stream(self._side_stream)  # rejoin (needed under graph capture)

        x = self.final_layer(x, t)  # [B, N, p*p*out]
        return ops.unpatchify(_as2d(x), bs, self.out_channels, self.h, self.w, p)

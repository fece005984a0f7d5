"""CPU restatement of the Sana Linear-DiT block arithmetic.  TEST INFRASTRUCTURE ONLY.

This file is the checker the CUDA path is compared with.  Only the test-suite, the
smoke entry and the CPU-baseline / reference legs of the benchmark may import it; the
product package never does, and fails loudly when its CUDA library is missing.

Every function follows one upstream function (path inside NVlabs/Sana given in its
docstring) op by op and dtype by dtype, so that running it in bf16 rounds at exactly the
places upstream rounds and running it in fp32/fp64 gives the "golden" result.  Parity of
this restatement is PINNED: ``tests/golden/make_golden.py`` runs the unmodified upstream
modules (imported on CPU) on seeded inputs and commits inputs/outputs as fixtures;
``tests/test_oracle_golden.py`` requires this file to reproduce those outputs bit for bit
(fp32 and bf16) on the same CPU kernels.

Parameters are passed as plain ``dict[str, Tensor]`` using upstream's state-dict keys:

    scale_shift_table                      [6, C]
    attn.qkv.weight                        [3C, C]      (rows q | k | v, head-major, 32/head)
    attn.proj.weight / attn.proj.bias      [C, C] / [C]
    cross_attn.q_linear.weight / .bias     [C, C] / [C]
    cross_attn.kv_linear.weight / .bias    [2C, C] / [2C]   (rows k | v)
    cross_attn.proj.weight / .bias         [C, C] / [C]
    mlp.inverted_conv.conv.weight / .bias  [2*hid, C, 1, 1] / [2*hid]
    mlp.depth_conv.conv.weight / .bias     [2*hid, 1, 3, 3] / [2*hid]
    mlp.point_conv.conv.weight             [C, hid, 1, 1]
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

Params = Dict[str, torch.Tensor]

LN_EPS = 1e-6  # nn.LayerNorm(hidden, elementwise_affine=False, eps=1e-6), sana_multi_scale.py:76,111
BLOCK_LA_EPS = 1e-8  # LiteLA(..., eps=1e-8) as built by the block, sana_multi_scale.py:90
PAD_VAL = 1  # LiteLA.PAD_VAL, sana_blocks.py:214


def sub(params: Params, prefix: str) -> Params:
    """Sub-dictionary of ``params`` under ``prefix.`` with the prefix removed."""
    p = prefix + "."
    return {k[len(p):]: v for k, v in params.items() if k.startswith(p)}


def t2i_modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """diffusion/model/nets/sana_blocks.py:44-45"""
    return x * (1 + scale) + shift


def layer_norm(x: torch.Tensor) -> torch.Tensor:
    """norm1 / norm2 of the block: affine-free LayerNorm over C, eps 1e-6
    (diffusion/model/nets/sana_multi_scale.py:76,111)."""
    return F.layer_norm(x, (x.shape[-1],), None, None, LN_EPS)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm.forward, diffusion/model/norms.py:216-231 (norm over the last dimension, computed
    in fp32 - or in x's dtype when that is wider - then cast back)."""
    xf = x.float() if x.dtype in (torch.float16, torch.bfloat16) else x
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (weight.view(*([1] * (x.dim() - 1)), -1) * n).type_as(x)


def lite_la_attn_matmul(q, k, v, eps: float, fp32_attention: bool = True) -> torch.Tensor:
    """LiteLA.attn_matmul, diffusion/model/nets/sana_blocks.py:245-263.

    q, v: [B, h, d, N]; k: [B, h, N, d].  Returns fp32 (or input dtype for fp32/fp64 inputs)
    [B, h, d, N]."""
    q = F.relu(q)
    k = F.relu(k)
    if fp32_attention:
        q, k, v = q.float(), k.float(), v.float()
    v = F.pad(v, (0, 0, 0, 1), mode="constant", value=PAD_VAL)
    vk = torch.matmul(v, k)
    out = torch.matmul(vk, q)
    if out.dtype in (torch.float16, torch.bfloat16):
        out = out.float()
    return out[:, :, :-1] / (out[:, :, -1:] + eps)


def apply_rotary_emb(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """apply_rotary_emb(..., use_real=True, use_real_unbind_dim=-2), sana_blocks.py:1549-1586:
    x [B, h, D, S], cos / sin [S, D]."""
    cos = cos[None, None].transpose(-1, -2)
    sin = sin[None, None].transpose(-1, -2)
    x_real, x_imag = x.reshape(*x.shape[:-2], -1, 2, x.shape[-1]).unbind(-2)  # [B, h, D/2, S]
    x_rotated = torch.stack([-x_imag, x_real], dim=-2).flatten(2, 3)
    return (x.float() * cos + x_rotated.float() * sin).to(x.dtype)


def lite_la_forward(x, p: Params, heads: Optional[int] = None, dim: int = 32, eps: float = 1e-15,
                    fp32_attention: bool = True, keep_dtype: bool = False, quant_fn=None,
                    norm_eps: float = 1e-5, rotary_emb=None) -> torch.Tensor:
    """LiteLA.forward, diffusion/model/nets/sana_blocks.py:265-291; ``rotary_emb`` = (cos, sin)
    [N, dim] rotates q and k before the ReLU (:282-284).

    ``p`` holds ``qkv.weight`` (+ optional ``qkv.bias``), ``proj.weight``, ``proj.bias``.
    ``keep_dtype`` runs the fp32_attention region in the input dtype instead of fp32 - used
    only to produce fp64 golden values (upstream's ``.float()`` would truncate them).
    ``quant_fn`` (e.g. :func:`nvfp4_fake_quant`) replaces input and weight of both Linear
    layers by their quantise-dequantise image along the contraction dimension - the
    "upstream run on the dequantised tensors" reference of the FP4 configuration."""
    B, N, C = x.shape
    heads = heads or C // dim
    hd = C // heads
    qf = quant_fn or (lambda v: v)
    qkv = F.linear(qf(x), qf(p["qkv.weight"]), p.get("qkv.bias")).reshape(B, N, 3, C)
    q, k, v = qkv.unbind(2)
    dtype = q.dtype
    if "q_norm.weight" in p:  # qk_norm=True: RMSNorm over the full C, sana_blocks.py:238-243,274-275
        q = rms_norm(q, p["q_norm.weight"], norm_eps)
        k = rms_norm(k, p["k_norm.weight"], norm_eps)
    q = q.transpose(-1, -2).reshape(B, C // hd, hd, N)
    k = k.transpose(-1, -2).reshape(B, C // hd, hd, N)
    v = v.transpose(-1, -2).reshape(B, C // hd, hd, N)
    if rotary_emb is not None:
        q = apply_rotary_emb(q, rotary_emb[0], rotary_emb[1])
        k = apply_rotary_emb(k, rotary_emb[0], rotary_emb[1])
    out = lite_la_attn_matmul(q, k.transpose(-1, -2), v, eps, fp32_attention and not keep_dtype).to(dtype)
    out = out.view(B, C, N).permute(0, 2, 1)
    return F.linear(qf(out), qf(p["proj.weight"]), p["proj.bias"])


def pag_identity_forward(x, p: Params, chunks: int, heads: Optional[int] = None, eps: float = 1e-15,
                         rotary_emb=None) -> torch.Tensor:
    """PAGIdentitySelfAttnProcessorLiteLA (chunks = 2) / PAGCFGIdentitySelfAttnProcessorLiteLA
    (chunks = 3), diffusion/model/nets/sana_blocks.py:573-675: the last chunk of the batch takes
    "identity attention" (value projection straight into ``proj``), the others LiteLA."""
    parts = x.chunk(chunks)
    x_org, x_ptb = torch.cat(parts[:-1]), parts[-1]
    C = x.shape[-1]
    out = lite_la_forward(x_org, p, heads=heads, eps=eps, rotary_emb=rotary_emb)
    v_weight = p["qkv.weight"][C * 2:C * 3, :]
    x_ptb = torch.matmul(x_ptb, v_weight.t()).to(out.dtype)
    if p.get("qkv.bias") is not None:
        x_ptb = (x_ptb + p["qkv.bias"][C * 2:C * 3]).to(out.dtype)
    x_ptb = F.linear(x_ptb, p["proj.weight"], p["proj.bias"])
    return torch.cat([out, x_ptb])


def lite_la_state(k_relu: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Token-major restatement of the first product of attn_matmul (sana_blocks.py:255-256):
    k_relu, v: [B, N, h, d] -> state [B, h, d+1, d] with state[b,h,i,j] = sum_n v1[n,i] k[n,j],
    v1 = [v ; 1].  Used to check the sharded (sequence-parallel) sum: a state over a token
    range is a plain sum, so shards add."""
    ones = torch.ones_like(v[..., :1])
    v1 = torch.cat([v, ones], dim=-1)
    return torch.einsum("bnhi,bnhj->bhij", v1, k_relu)


def lite_la_apply(q_relu: torch.Tensor, state: torch.Tensor, eps: float) -> torch.Tensor:
    """Second product + normalisation (sana_blocks.py:257-261), token-major:
    q_relu [B, N, h, d], state [B, h, d+1, d] -> [B, N, h, d]."""
    out = torch.einsum("bhij,bnhj->bnhi", state, q_relu)
    return out[..., :-1] / (out[..., -1:] + eps)


def wan_rotary_freqs(head_dim: int, fhw: Sequence[int], theta: float = 10000.0, max_seq_len: int = 1024,
                     fhw_dim: Optional[Sequence[int]] = None) -> torch.Tensor:
    """WanRotaryPosEmbed, diffusion/model/nets/sana_blocks.py:1361-1410 (with
    get_1d_rotary_pos_embed(use_real=False, freqs_dtype=float64), :1483-1547): complex128
    [1, 1, f*h*w, head_dim/2]; the head's channel pairs are split into a frame, a row and a column
    group, each rotating by its own coordinate."""
    if fhw_dim is not None:
        t_dim, h_dim, w_dim = fhw_dim
    else:
        h_dim = w_dim = 2 * (head_dim // 6)
        t_dim = head_dim - h_dim - w_dim
    f, h, w = fhw
    parts = []
    for dim, count, shape in ((t_dim, f, (f, 1, 1)), (h_dim, h, (1, h, 1)), (w_dim, w, (1, 1, w))):
        inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64)[: dim // 2] / dim))
        ang = torch.outer(torch.arange(max_seq_len)[:count], inv)
        parts.append(torch.polar(torch.ones_like(ang), ang).view(*shape, -1).expand(f, h, w, -1))
    return torch.cat(parts, dim=-1).reshape(1, 1, f * h * w, -1)


def rotate_pairs_complex(x: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """The inner `apply_rotary_emb` of LiteLAReLURope.forward, sana_blocks.py:359-362:
    x [B, h, D, N], freqs complex [1, 1, N, D/2]; channel pairs (2p, 2p+1) multiply, as complex
    numbers in float64, by freqs[n, p]; the result is cast back to x's dtype."""
    xr = torch.view_as_complex(x.permute(0, 1, 3, 2).to(torch.float64).unflatten(3, (-1, 2)))
    out = torch.view_as_real(xr * freqs).flatten(3, 4).permute(0, 1, 3, 2)
    return out.type_as(x)


def lite_la_relu_rope_forward(x, p: Params, heads: int, rotary_emb: torch.Tensor, eps: float = 1e-15,
                              fp32_attention: bool = False, norm_eps: float = 1e-5) -> torch.Tensor:
    """LiteLAReLURope.forward, diffusion/model/nets/sana_blocks.py:339-388: ReLU feature map first,
    then the rotation on the numerator's q and k only; the normaliser uses the unrotated ones.
    Rounds where upstream rounds (in bf16 the two matmuls and `z` run in bf16 unless
    ``fp32_attention``)."""
    B, N, C = x.shape
    hd = C // heads
    qkv = F.linear(x, p["qkv.weight"], p.get("qkv.bias")).reshape(B, N, 3, C)
    q, k, v = qkv.unbind(2)
    dtype = q.dtype
    if "q_norm.weight" in p:  # qk_norm=True, sana_blocks.py:329-331,346-347
        q = rms_norm(q, p["q_norm.weight"], norm_eps)
        k = rms_norm(k, p["k_norm.weight"], norm_eps)
    q = F.relu(q.transpose(-1, -2).reshape(B, heads, hd, N))
    k = F.relu(k.transpose(-1, -2).reshape(B, heads, hd, N))
    v = v.transpose(-1, -2).reshape(B, heads, hd, N)
    q_rot = rotate_pairs_complex(q, rotary_emb)
    k_rot = rotate_pairs_complex(k, rotary_emb)
    if fp32_attention:
        q_rot, k_rot, v = q_rot.float(), k_rot.float(), v.float()
    z = 1 / (k.sum(dim=-1, keepdim=True).transpose(-2, -1) @ q + eps)
    vk = torch.matmul(v, k_rot.transpose(-1, -2))
    out = torch.matmul(vk, q_rot)
    out = (out * z).to(dtype)
    out = out.view(B, C, N).permute(0, 2, 1)
    return F.linear(out, p["proj.weight"], p["proj.bias"])


def _relu_rope_qkv(x, p: Params, heads: int, rotary_emb: torch.Tensor, fp32_attention: bool, norm_eps: float):
    """The part the three rotated attentions share (sana_blocks.py:413-450): projections, optional q / k norm,
    head split, ReLU, rotation.  Returns q, k, v, q_rot, k_rot as [B, h, d, N] and the activation dtype."""
    B, N, C = x.shape
    hd = C // heads
    qkv = F.linear(x, p["qkv.weight"], p.get("qkv.bias")).reshape(B, N, 3, C)
    q, k, v = qkv.unbind(2)
    dtype = q.dtype
    if "q_norm.weight" in p:
        q = rms_norm(q, p["q_norm.weight"], norm_eps)
        k = rms_norm(k, p["k_norm.weight"], norm_eps)
    q = F.relu(q.transpose(-1, -2).reshape(B, heads, hd, N))
    k = F.relu(k.transpose(-1, -2).reshape(B, heads, hd, N))
    v = v.transpose(-1, -2).reshape(B, heads, hd, N)
    q_rot = rotate_pairs_complex(q, rotary_emb)
    k_rot = rotate_pairs_complex(k, rotary_emb)
    if fp32_attention:
        q_rot, k_rot, v = q_rot.float(), k_rot.float(), v.float()
    return q, k, v, q_rot, k_rot, dtype


def chunk_causal_forward(x, p: Params, heads: int, rotary_emb: torch.Tensor, HW: Sequence[int], chunk_index=None,
                         eps: float = 1e-15, fp32_attention: bool = False, norm_eps: float = 1e-5) -> torch.Tensor:
    """ChunkCausalAttention.forward, diffusion/model/nets/sana_blocks.py:408-496: the frames are cut at
    ``chunk_index``; a chunk's queries see the state summed over its own and all earlier chunks."""
    B, N, C = x.shape
    q, k, v, q_rot, k_rot, dtype = _relu_rope_qkv(x, p, heads, rotary_emb, fp32_attention, norm_eps)
    f, h, w = HW
    idx = (list(chunk_index) if chunk_index is not None else [0]) + [f]
    sizes = [(b - a) * h * w for a, b in zip(idx[:-1], idx[1:])]
    hd = C // heads
    cum_vk = torch.zeros(B, heads, hd, hd, dtype=k_rot.dtype)
    cum_ks = torch.zeros(B, heads, 1, hd, dtype=k_rot.dtype)
    outs = []
    for _qr, _kr, _v, _q, _k in zip(q_rot.split(sizes, -1), k_rot.split(sizes, -1), v.split(sizes, -1), q.split(sizes, -1),
                                    k.split(sizes, -1)):
        cum_vk += torch.matmul(_v, _kr.transpose(-1, -2))
        cum_ks += _k.sum(dim=-1, keepdim=True).transpose(-2, -1)
        z = 1 / (cum_ks @ _q + eps)
        outs.append((torch.matmul(cum_vk, _qr) * z).to(dtype))
    out = torch.cat(outs, dim=-1).view(B, C, N).permute(0, 2, 1)
    return F.linear(out, p["proj.weight"], p["proj.bias"])


def cached_causal_forward(x, p: Params, heads: int, rotary_emb: torch.Tensor, kv_cache=None, save_kv_cache: bool = False,
                          eps: float = 1e-15, fp32_attention: bool = False, norm_eps: float = 1e-5):
    """CachedCausalAttention.forward, diffusion/model/nets/sana_blocks.py:502-572: this chunk's vk and key sum,
    plus the pair found in ``kv_cache[0:2]``; with ``save_kv_cache`` the cache takes THIS chunk's own pair
    (before the addition).  Returns (out, kv_cache) when a cache list is given, else out."""
    B, N, C = x.shape
    q, k, v, q_rot, k_rot, dtype = _relu_rope_qkv(x, p, heads, rotary_emb, fp32_attention, norm_eps)
    k_sum = k.sum(dim=-1, keepdim=True).transpose(-2, -1)
    vk = torch.matmul(v, k_rot.transpose(-1, -2))
    if kv_cache is not None:
        prev_vk, prev_ks = kv_cache[0], kv_cache[1]
        if save_kv_cache:
            kv_cache[0], kv_cache[1] = vk.detach().clone(), k_sum.detach().clone()
        if prev_vk is not None and prev_ks is not None:
            vk = vk + prev_vk
            k_sum = k_sum + prev_ks
    z = 1 / (k_sum @ q + eps)
    out = (torch.matmul(vk, q_rot) * z).to(dtype)
    out = F.linear(out.view(B, C, N).permute(0, 2, 1), p["proj.weight"], p["proj.bias"])
    return (out, kv_cache) if kv_cache is not None else out


def cached_glumbconv_temp_forward(x, p: Params, HW: Sequence[int], kv_cache=None, save_kv_cache: bool = False):
    """CachedGLUMBConvTemp.forward, diffusion/model/nets/basic_modules.py:364-397: GLUMBConv per frame, then the
    3-tap temporal convolution whose left context is the last frame of the previous chunk (``kv_cache[-1]``,
    [B, C, 1, H*W]) instead of zero padding; the right side is zero-padded."""
    B, N, C = x.shape
    T, H, W = HW
    s = glumbconv_forward(x, p, HW)
    xr = s.reshape(B, T, H * W, C).permute(0, 3, 1, 2)  # [B, C, T, HW]
    wt = p["t_conv.weight"]
    pad = wt.shape[2] // 2
    x_in, padded = xr, 0
    if kv_cache is not None:
        if kv_cache[-1] is not None:
            x_in = torch.cat([kv_cache[-1][:, :, -pad:], xr], dim=2)
            padded = x_in.shape[2] - xr.shape[2]
        if save_kv_cache:
            kv_cache[-1] = xr[:, :, -pad:, :].detach().clone()
    t_out = F.conv2d(x_in, wt, None, padding=(pad, 0))[:, :, padded:]
    out = (xr + t_out).permute(0, 2, 3, 1).reshape(B, N, C)
    return (out, kv_cache) if kv_cache is not None else out


def chunk_glumbconv_temp_forward(x, p: Params, HW: Sequence[int], chunk_index=None) -> torch.Tensor:
    """ChunkGLUMBConvTemp.forward without frame mask and context parallelism,
    diffusion/model/nets/basic_modules.py:273-351: GLUMBConv per frame, then the 3-tap temporal convolution
    applied chunk by chunk - the frames are cut at ``chunk_index``; a chunk sees the last frame of the chunk
    before it on its left (zeros before the first chunk) and zeros on its right, so the previous-frame tap
    crosses chunk boundaries and the next-frame tap does not.  As upstream does, the padded chunks are laid
    end to end and convolved in one call."""
    B, N, C = x.shape
    T, H, W = HW
    hw = H * W
    s = glumbconv_forward(x, p, HW)
    xr = s.reshape(B, T, hw, C).permute(0, 3, 1, 2)  # [B, C, T, HW]
    wt = p["t_conv.weight"]
    pad = wt.shape[2] // 2
    cuts = sorted({0, T, *(int(i) for i in (chunk_index or [0]) if 0 < int(i) < T)})
    zeros = xr.new_zeros(B, C, pad, hw)
    pieces, keep, pos = [], [], 0
    for k, (a, b) in enumerate(zip(cuts, cuts[1:])):
        left = [] if k == 0 else [xr[:, :, a - pad:a]]
        pieces += left + [xr[:, :, a:b], zeros]
        start = pos + (0 if k == 0 else pad)
        keep.append((start, start + (b - a)))
        pos = start + (b - a) + pad
    conv = F.conv2d(torch.cat(pieces, dim=2), wt, None, padding=(pad, 0))
    t_out = torch.cat([conv[:, :, a:b] for a, b in keep], dim=2)
    return (xr + t_out).permute(0, 2, 3, 1).reshape(B, N, C)


def lite_la_rope_state(k_relu: torch.Tensor, k_rot: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Token-major restatement of `vk` and of the key sum of LiteLAReLURope (sana_blocks.py:380-382):
    k_relu, k_rot, v [B, N, h, d] -> state [B, h, d+1, d]; rows 0..d-1 hold
    sum_n v[n, i] k_rot[n, j], row d holds sum_n k_relu[n, j] (unrotated)."""
    vk = torch.einsum("bnhi,bnhj->bhij", v, k_rot)
    return torch.cat([vk, k_relu.sum(1)[:, :, None, :]], dim=2)


def lite_la_rope_apply(q_relu: torch.Tensor, q_rot: torch.Tensor, state: torch.Tensor, eps: float) -> torch.Tensor:
    """Second product and normalisation (sana_blocks.py:380,383-385), token-major:
    q_relu, q_rot [B, N, h, d], state [B, h, d+1, d] -> [B, N, h, d]."""
    num = torch.einsum("bhij,bnhj->bnhi", state[:, :, :-1], q_rot)
    den = torch.einsum("bhj,bnhj->bnh", state[:, :, -1], q_relu)
    return num / (den[..., None] + eps)


def glumbconv_forward(x, p: Params, HW: Sequence[int], quant_fn=None) -> torch.Tensor:
    """GLUMBConv.forward / _apply_spatial, diffusion/model/nets/basic_modules.py:161-199.

    ``HW`` = (H, W) or (T, H, W); with three entries the depthwise conv runs per frame.
    In-place SiLU after the 1x1 expand (act.py:31), separate SiLU for the gate.  ``quant_fn``
    quantise-dequantises input and weight of the two 1x1 convs along the channel dimension."""
    B, N, C = x.shape
    qf = quant_fn or (lambda v: v)
    qw = (lambda w: qf(w.reshape(w.shape[0], -1)).reshape(w.shape)) if quant_fn else (lambda w: w)
    qc = (lambda v: qf(v.permute(0, 2, 3, 1)).permute(0, 3, 1, 2)) if quant_fn else (lambda v: v)
    if len(HW) == 2:
        H, W = HW
        BT = B
    elif len(HW) == 3:
        T, H, W = HW
        BT = B * T
    else:
        raise ValueError("HW must have 2 or 3 entries")
    x = qf(x).reshape(BT, H, W, C).permute(0, 3, 1, 2)
    x = F.conv2d(x, qw(p["inverted_conv.conv.weight"]), p.get("inverted_conv.conv.bias"))
    x = F.silu(x)
    wd = p["depth_conv.conv.weight"]
    x = F.conv2d(x, wd, p.get("depth_conv.conv.bias"), padding=wd.shape[-1] // 2, groups=wd.shape[0])
    a, g = torch.chunk(x, 2, dim=1)
    g = F.silu(g)
    x = F.conv2d(qc(a * g), qw(p["point_conv.conv.weight"]), p.get("point_conv.conv.bias"))
    Cout = x.shape[1]
    if len(HW) == 3:
        return x.reshape(BT, Cout, H * W).permute(0, 2, 1).reshape(B, N, Cout)
    return x.reshape(B, Cout, N).permute(0, 2, 1)


def glumbconv_temp_forward(x, p: Params, HW: Sequence[int]) -> torch.Tensor:
    """GLUMBConvTemp.forward without frame mask and context parallelism,
    diffusion/model/nets/basic_modules.py:238-266: GLUMBConv per frame, then
    ``x + t_conv(x)`` with t_conv a (3, 1) convolution over (frames, pixels)."""
    B, N, C = x.shape
    T, H, W = HW
    s = glumbconv_forward(x, p, HW)  # [B, N, C], frames stacked along N
    xr = s.reshape(B, T, H * W, C).permute(0, 3, 1, 2)  # [B, C, T, HW]
    wt = p["t_conv.weight"]
    t_out = F.conv2d(xr, wt, None, padding=(wt.shape[2] // 2, 0))
    out = xr + t_out
    return out.permute(0, 2, 3, 1).reshape(B, N, C)


def cross_attention_forward(x, cond, p: Params, num_heads: int, mask=None) -> torch.Tensor:
    """MultiHeadCrossAttention.forward, SDPA branch (no xformers),
    diffusion/model/nets/sana_blocks.py:69-98.  ``mask``: None or [B, L] of 0/1."""
    B, N, C = x.shape
    hd = C // num_heads
    q = F.linear(x, p["q_linear.weight"], p["q_linear.bias"])
    kv = F.linear(cond, p["kv_linear.weight"], p["kv_linear.bias"]).view(B, -1, 2, C)
    k, v = kv.unbind(2)
    if "q_norm.weight" in p:  # cross_norm=True: RMSNorm(d_model, eps=1e-6), sana_blocks.py:62-64,77-78
        q = rms_norm(q, p["q_norm.weight"], 1e-6)
        k = rms_norm(k, p["k_norm.weight"], 1e-6)
    q = q.view(B, -1, num_heads, hd).transpose(1, 2)
    k = k.view(B, -1, num_heads, hd).transpose(1, 2)
    v = v.view(B, -1, num_heads, hd).transpose(1, 2)
    if mask is not None and mask.ndim == 2:
        mask = (1 - mask.to(q.dtype)) * -10000.0
        mask = mask[:, None, None].repeat(1, num_heads, 1, 1)
    o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, dropout_p=0.0, is_causal=False)
    o = o.transpose(1, 2).reshape(B, -1, C)
    return F.linear(o, p["proj.weight"], p["proj.bias"])


def sana_ms_block_forward(x, y, t, p: Params, num_heads: int, HW: Sequence[int], mask=None,
                          linear_head_dim: int = 32, fp32_attention: bool = True,
                          keep_dtype: bool = False, return_branches: bool = False, quant_fn=None, rotary_emb=None):
    """SanaMSBlock.forward with attn_type="linear", ffn_type="glumbconv", drop_path 0,
    diffusion/model/nets/sana_multi_scale.py:145-157.

    x [B, N, C], y [B, L, C], t [B, 6C].  With ``return_branches`` also returns the outputs
    of LiteLA.forward and GLUMBConv.forward (before gate and residual), the two places where
    parity is asserted besides the block output."""
    B, N, C = x.shape
    mod = (p["scale_shift_table"][None] + t.reshape(B, 6, -1)).chunk(6, dim=1)
    shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = mod
    a = lite_la_forward(t2i_modulate(layer_norm(x), shift_msa, scale_msa), sub(p, "attn"),
                        heads=C // linear_head_dim, eps=BLOCK_LA_EPS,
                        fp32_attention=fp32_attention, keep_dtype=keep_dtype, quant_fn=quant_fn,
                        rotary_emb=rotary_emb)
    x = x + gate_msa * a
    x = x + cross_attention_forward(x, y, sub(p, "cross_attn"), num_heads, mask)
    f = glumbconv_forward(t2i_modulate(layer_norm(x), shift_mlp, scale_mlp), sub(p, "mlp"), HW, quant_fn=quant_fn)
    x = x + gate_mlp * f
    if return_branches:
        return x, a, f
    return x


def sana_video_block_forward(x, y, t, p: Params, num_heads: int, THW: Sequence[int], rotary_emb, mask=None,
                             linear_head_dim: int = 112) -> torch.Tensor:
    """SanaVideoMSBlock.forward with attn_type="LiteLAReLURope", ffn_type="GLUMBConvTemp" (or
    "glumbconv" when ``p`` has no ``mlp.t_conv.weight``), drop_path 0, no additional attention,
    diffusion/model/nets/sana_multi_scale_video.py:256-333; a ``t`` of more than two dimensions
    ([B, 1, F, 6C]: one modulation per frame) takes forward_frame_aware (:204-254)."""
    B, N, C = x.shape
    heads = C // linear_head_dim
    mlp = glumbconv_temp_forward if "mlp.t_conv.weight" in p else glumbconv_forward
    if t.dim() > 2:
        Fr = t.shape[2]
        tt = t.reshape(B, Fr, 6, -1)
        mod = (p["scale_shift_table"][None, None, :, :] + tt).chunk(6, dim=-2)  # each [B, F, 1, C]
        shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = mod
        z = t2i_modulate(layer_norm(x).reshape(B, Fr, -1, C), shift_msa, scale_msa).reshape(B, N, C)
        a = lite_la_relu_rope_forward(z, sub(p, "attn"), heads, rotary_emb, eps=BLOCK_LA_EPS)
        x = x + (gate_msa * a.reshape(B, Fr, -1, C)).reshape(B, N, C)
        x = x + cross_attention_forward(x, y, sub(p, "cross_attn"), num_heads, mask)
        z = t2i_modulate(layer_norm(x).reshape(B, Fr, -1, C), shift_mlp, scale_mlp).reshape(B, N, C)
        return x + (gate_mlp * mlp(z, sub(p, "mlp"), THW).reshape(B, Fr, -1, C)).reshape(B, N, C)
    mod = (p["scale_shift_table"][None] + t.reshape(B, 6, -1)).chunk(6, dim=1)
    shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = mod
    a = lite_la_relu_rope_forward(t2i_modulate(layer_norm(x), shift_msa, scale_msa), sub(p, "attn"), heads, rotary_emb,
                                  eps=BLOCK_LA_EPS)
    x = x + gate_msa * a
    x = x + cross_attention_forward(x, y, sub(p, "cross_attn"), num_heads, mask)
    return x + gate_mlp * mlp(t2i_modulate(layer_norm(x), shift_mlp, scale_mlp), sub(p, "mlp"), THW)


def timestep_embedding(t: torch.Tensor, dim: int = 256, max_period: int = 10000) -> torch.Tensor:
    """TimestepEmbedder.timestep_embedding, diffusion/model/nets/sana_blocks.py:980-999."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(0, half, dtype=torch.float32) / half)
    args = t[:, None].float() * freqs[None]
    emb = torch.cat([torch.cos(args), torch.sin(args)], dim=-1)
    if dim % 2:
        emb = torch.cat([emb, torch.zeros_like(emb[:, :1])], dim=-1)
    return emb


def adaln_single(t_scalar: torch.Tensor, p: Params, dtype=torch.float32) -> torch.Tensor:
    """t -> [B, 6C]: TimestepEmbedder.forward (sana_blocks.py:1001-1004) followed by
    t_block = SiLU -> Linear(C, 6C) (sana_multi_scale.py:240).  Keys: ``mlp.0.*``,
    ``mlp.2.*`` (embedder) and ``t_block.1.*``."""
    e = timestep_embedding(t_scalar, p["mlp.0.weight"].shape[1]).to(dtype)
    e = F.linear(e, p["mlp.0.weight"], p["mlp.0.bias"])
    e = F.linear(F.silu(e), p["mlp.2.weight"], p["mlp.2.bias"])
    return F.linear(F.silu(e), p["t_block.1.weight"], p["t_block.1.bias"])


# ----------------------------------------------------------------------------------------
# The whole multi-scale DiT forward (the steps either side of the block loop).
# ----------------------------------------------------------------------------------------
def sincos_1d(embed_dim: int, pos):
    """get_1d_sincos_pos_embed_from_grid, diffusion/model/nets/sana.py:447-465 (numpy, float64
    frequencies; sin half first, then cos)."""
    import numpy as np

    omega = np.arange(embed_dim // 2, dtype=np.float64)
    omega /= embed_dim / 2.0
    omega = 1.0 / 10000**omega
    out = np.einsum("m,d->md", pos.reshape(-1), omega)
    return np.concatenate([np.sin(out), np.cos(out)], axis=1)


def sincos_pos_embed_2d(embed_dim: int, grid_size, pe_interpolation: float = 1.0, base_size: int = 16):
    """get_2d_sincos_pos_embed (+ _from_grid), sana.py:416-444: float32 coordinates, meshgrid
    with w first, reshape to [2, 1, w, h]; the first half of the channels encodes grid[0]."""
    import numpy as np

    grid_h = np.arange(grid_size[0], dtype=np.float32) / (grid_size[0] / base_size) / pe_interpolation
    grid_w = np.arange(grid_size[1], dtype=np.float32) / (grid_size[1] / base_size) / pe_interpolation
    grid = np.meshgrid(grid_w, grid_h)
    grid = np.stack(grid, axis=0)
    grid = grid.reshape([2, 1, grid_size[1], grid_size[0]])
    return np.concatenate([sincos_1d(embed_dim // 2, grid[0]), sincos_1d(embed_dim // 2, grid[1])], axis=1)


def final_layer_forward(x, t, p: Params) -> torch.Tensor:
    """T2IFinalLayer.forward / forward_frame_aware, diffusion/model/nets/sana_blocks.py:907-925:
    t [B, C], or [B, 1, F, C] with one modulation vector per frame.  Keys: scale_shift_table,
    linear.weight, linear.bias."""
    B, N, C = x.shape
    if t.dim() > 2:
        num_frames = t.shape[2]
        shift, scale = (p["scale_shift_table"][None, None, :, :] + t.transpose(1, 2)).chunk(2, dim=-2)
        x = t2i_modulate(layer_norm(x).reshape(B, num_frames, -1, C), shift, scale).reshape(B, N, C)
    else:
        shift, scale = (p["scale_shift_table"][None] + t[:, None]).chunk(2, dim=1)
        x = t2i_modulate(layer_norm(x), shift, scale)
    return F.linear(x, p["linear.weight"], p["linear.bias"])


def sana_ms_forward(x, timestep, y, p: Params, *, depth: int, num_heads: int, patch_size: int, out_channels: int,
                    base_size: int, mask=None, pe_interpolation: float = 1.0, y_norm: bool = False,
                    norm_eps: float = 1e-5, timestep_norm_scale_factor: float = 1.0, use_pe: bool = True,
                    linear_head_dim: int = 32, return_parts: bool = False):
    """SanaMS.forward, diffusion/model/nets/sana_multi_scale.py:326-393, without xformers (the
    2-D mask goes to every block), sin-cos positions, no cfg embedder, no log-variance head.

    x [B, Cin, H, W]; timestep [B]; y [B, 1, L, Cc]; mask [B, L] or None.  Parameters use the
    model's state-dict keys (x_embedder.proj.*, t_embedder.mlp.{0,2}.*, t_block.1.*,
    y_embedder.y_proj.fc{1,2}.*, attention_y_norm.weight, blocks.<i>.*, final_layer.*)."""
    import torch as _t

    dtype = p["t_block.1.weight"].dtype
    x = x.to(dtype)
    if timestep_norm_scale_factor != 1.0:
        timestep = (timestep.float() / timestep_norm_scale_factor).to(_t.float32)
    else:
        timestep = timestep.long().to(_t.float32)
    y = y.to(dtype)
    h, w = x.shape[-2] // patch_size, x.shape[-1] // patch_size
    # PatchEmbedMS.forward, sana_blocks.py:1263-1268
    x = F.conv2d(x, p["x_embedder.proj.weight"], p["x_embedder.proj.bias"], stride=patch_size)
    x = x.flatten(2).transpose(1, 2)
    C = x.shape[-1]
    if use_pe:
        pos = _t.from_numpy(sincos_pos_embed_2d(C, (h, w), pe_interpolation=pe_interpolation, base_size=base_size))
        x = x + pos.unsqueeze(0).to(dtype)
    # TimestepEmbedder.forward, sana_blocks.py:1002-1005
    t = timestep_embedding(timestep, p["t_embedder.mlp.0.weight"].shape[1]).to(dtype)
    t = F.linear(t, p["t_embedder.mlp.0.weight"], p["t_embedder.mlp.0.bias"])
    t = F.linear(F.silu(t), p["t_embedder.mlp.2.weight"], p["t_embedder.mlp.2.bias"])
    t0 = F.linear(F.silu(t), p["t_block.1.weight"], p["t_block.1.bias"])
    # CaptionEmbedder.forward in eval mode (sana_blocks.py:1123-1138): the GELU(tanh) MLP only
    y = F.linear(y, p["y_embedder.y_proj.fc1.weight"], p["y_embedder.y_proj.fc1.bias"])
    y = F.linear(F.gelu(y, approximate="tanh"), p["y_embedder.y_proj.fc2.weight"], p["y_embedder.y_proj.fc2.bias"])
    if y_norm:
        y = rms_norm(y, p["attention_y_norm.weight"], norm_eps)
    if mask is not None:
        mask = mask.to(_t.int16)
        mask = mask.repeat(y.shape[0] // mask.shape[0], 1) if mask.shape[0] != y.shape[0] else mask
        mask = mask.squeeze(1).squeeze(1)
    parts = {"x_embed": x, "t": t, "t0": t0, "y": y}
    for i in range(depth):
        x = sana_ms_block_forward(x, y, t0, sub(p, f"blocks.{i}"), num_heads, (h, w), mask,
                                  linear_head_dim=linear_head_dim)
    parts["x_blocks"] = x
    # T2IFinalLayer.forward, sana_blocks.py:919-925
    shift, scale = (p["final_layer.scale_shift_table"][None] + t[:, None]).chunk(2, dim=1)
    x = t2i_modulate(layer_norm(x), shift, scale)
    x = F.linear(x, p["final_layer.linear.weight"], p["final_layer.linear.bias"])
    # unpatchify, sana_multi_scale.py:409-421
    c, ps = out_channels, patch_size
    x = x.reshape(shape=(x.shape[0], h, w, ps, ps, c))
    x = _t.einsum("nhwpqc->nchpwq", x)
    imgs = x.reshape(shape=(x.shape[0], c, h * ps, w * ps))
    if return_parts:
        return imgs, parts
    return imgs


# ----------------------------------------------------------------------------------------
# Sequence-parallel restatement (no upstream counterpart for LiteLA: the state is a plain
# sum over tokens, so shards add; the depthwise conv needs one row of halo inside a frame).
# The partition rule mirrors the contiguous-rank layout of upstream's context-parallel
# groups (diffusion/distributed/context_parallel/config.py:155-178) but splits image rows,
# not frames.
# ----------------------------------------------------------------------------------------
def row_partition(total_rows: int, world: int) -> Sequence[Tuple[int, int]]:
    """Contiguous, balanced [start, end) row ranges; the first ``total_rows % world`` ranks
    get one extra row."""
    base, extra = divmod(total_rows, world)
    out, s = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((s, s + n))
        s += n
    return out


def depthwise_glu_rows(u_rows, halo_top, halo_bot, wd, bd, row0: int, H: int) -> torch.Tensor:
    """3x3 depthwise conv + bias + SiLU-GLU on a contiguous range of image rows.

    u_rows [R, W, 2*hid] are global rows ``row0 .. row0+R`` of a stack of frames that are
    ``H`` rows tall; halo_top / halo_bot [W, 2*hid] are global rows ``row0-1`` / ``row0+R``
    (ignored when that row lies in another frame, where upstream zero-pads).  Same math as
    basic_modules.py:164-167 applied per frame."""
    R, W, C2 = u_rows.shape
    out = torch.empty(R, W, C2 // 2, dtype=u_rows.dtype, device=u_rows.device)
    zero = torch.zeros(W, C2, dtype=u_rows.dtype, device=u_rows.device)
    for r in range(R):
        g = row0 + r
        fr = g % H
        up = zero if fr == 0 else (u_rows[r - 1] if r > 0 else halo_top)
        dn = zero if fr == H - 1 else (u_rows[r + 1] if r < R - 1 else halo_bot)
        tile = torch.stack([up, u_rows[r], dn], 0).permute(2, 0, 1)[None]  # [1, C2, 3, W]
        w = F.conv2d(F.pad(tile, (1, 1, 0, 0)), wd, bd, groups=C2)  # [1, C2, 1, W]
        a, gt = torch.chunk(w[0, :, 0], 2, dim=0)
        out[r] = (a * F.silu(gt)).permute(1, 0)
    return out


def sana_ms_block_rows(x, y, t, p: Params, num_heads: int, HW: Sequence[int], rows: Sequence[int], mask=None,
                       linear_head_dim: int = 32) -> Dict[int, torch.Tensor]:
    """Rows of :func:`sana_ms_block_forward`'s output for one sample, without evaluating the whole
    block: ``rows`` are global image rows (frame * H + row) of the (T, H, W) or (H, W) grid and the
    result maps each to its [W, C] output.  Only the linear-attention state needs every token (k and v
    of the whole sequence); everything after it is local to a token, except the 3x3 depthwise conv,
    which reads the rows above and below inside the same frame.  Same operations in the same order as
    the full function (sana_multi_scale.py:145-157), so in fp64 the two agree to rounding; it exists
    so that a 75 600-token block can be checked on sampled rows in seconds of CPU time."""
    B, N, C = x.shape
    assert B == 1
    H, W = HW[-2], HW[-1]
    heads = C // linear_head_dim
    mod = (p["scale_shift_table"][None] + t.reshape(B, 6, -1)).chunk(6, dim=1)
    shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = mod
    pa, pm = sub(p, "attn"), sub(p, "mlp")
    z = t2i_modulate(layer_norm(x), shift_msa, scale_msa)
    wqkv = pa["qkv.weight"]
    kv = F.linear(z, wqkv[C:])
    k = F.relu(kv[..., :C]).reshape(B, N, heads, linear_head_dim)
    v = kv[..., C:].reshape(B, N, heads, linear_head_dim)
    state = lite_la_state(k, v)
    w1 = pm["inverted_conv.conv.weight"]
    w3 = pm["point_conv.conv.weight"]
    wd, bd = pm["depth_conv.conv.weight"], pm.get("depth_conv.conv.bias")
    out = {}
    for r in rows:
        fr = r % H
        need = [g for g in (r - 1, r, r + 1) if 0 <= fr + (g - r) < H]
        tok = torch.cat([torch.arange(g * W, (g + 1) * W) for g in need])
        q = F.relu(F.linear(z[:, tok], wqkv[:C])).reshape(B, -1, heads, linear_head_dim)
        o = lite_la_apply(q, state, BLOCK_LA_EPS).reshape(B, -1, C)
        x1 = x[:, tok] + gate_msa * F.linear(o, pa["proj.weight"], pa["proj.bias"])
        x2 = x1 + cross_attention_forward(x1, y, sub(p, "cross_attn"), num_heads, mask)
        z2 = t2i_modulate(layer_norm(x2), shift_mlp, scale_mlp)
        u = F.silu(F.linear(z2, w1.reshape(w1.shape[0], C), pm.get("inverted_conv.conv.bias")))
        u = {g: u[0, i * W:(i + 1) * W] for i, g in enumerate(need)}
        gl = depthwise_glu_rows(u[r][None], u.get(r - 1), u.get(r + 1), wd, bd, r, H)[0]  # [W, hid]
        f = F.linear(gl, w3.reshape(w3.shape[0], -1), pm.get("point_conv.conv.bias"))
        i0 = need.index(r) * W
        out[r] = x2[0, i0:i0 + W] + gate_mlp[0] * f
    return out


# ----------------------------------------------------------------------------------------
# NVFP4 fake quantisation (E2M1 values, one E4M3 scale per 16 contiguous elements of the
# contraction dimension, one fp32 scale per tensor).  Upstream holds no FP4 arithmetic of
# its own (it calls Transformer Engine, which is not vendored), so nothing upstream pins
# these numbers: parity of this section is UNPINNED; the block-level check is "upstream
# block run on the dequantised tensors".
# ----------------------------------------------------------------------------------------
E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
E2M1_MAX = 6.0
E4M3_MAX = 448.0


def _round_to_e2m1(x: torch.Tensor) -> torch.Tensor:
    """Round-to-nearest-even onto the E2M1 grid {0,.5,1,1.5,2,3,4,6} with sign, saturating."""
    s = torch.sign(x)
    a = x.abs().clamp(max=E2M1_MAX)
    # midpoints: ties go to the value with even mantissa (0, 1, 2, 4 | .5->0? see below)
    # grid index by thresholds; ties resolved to even code (codes 0..7; even codes 0,2,4,6)
    grid = E2M1_VALUES.to(x.dtype)
    mids = (grid[:-1] + grid[1:]) / 2  # .25 .75 1.25 1.75 2.5 3.5 5
    idx = torch.zeros_like(a, dtype=torch.long)
    for i in range(7):
        lower_code_even = (i % 2 == 0)
        if lower_code_even:
            idx = idx + (a > mids[i]).long()  # tie stays at the lower (even) code
        else:
            idx = idx + (a >= mids[i]).long()  # tie goes up to the even code
    return s * grid[idx]


def _round_to_e4m3(x: torch.Tensor) -> torch.Tensor:
    """Positive values -> nearest E4M3 (fn variant, max 448) via torch's float8_e4m3fn."""
    return x.clamp(max=E4M3_MAX).to(torch.float8_e4m3fn).to(torch.float32)


def nvfp4_quantize(x: torch.Tensor, amax: Optional[float] = None):
    """Quantise along the last dimension (length a multiple of 16).  ``amax``: scale for this
    maximum magnitude instead of the tensor's own (values beyond it saturate).

    Returns (codes_value fp32 on the E2M1 grid, block_scale fp32 holding E4M3 values
    [..., K/16], tensor_scale python float) with
    ``dequant = codes_value * block_scale[..., None] * tensor_scale``.

    tensor_scale = amax / (6 * 448); block scale = E4M3(block_amax * (1 / (6 * tensor_scale)));
    code = E2M1(x * (1 / (block_scale * tensor_scale))) - reciprocals and products in fp32, rounded to
    nearest, the formulation a device quantiser uses (one multiply per element instead of a division)."""
    xf = x.float()
    K = xf.shape[-1]
    assert K % 16 == 0
    amax = xf.abs().max().clamp(min=1e-30) if amax is None else torch.tensor(float(amax), dtype=torch.float32).clamp(min=1e-30)
    ts32 = amax / torch.tensor(E2M1_MAX * E4M3_MAX, dtype=torch.float32)  # fp32 throughout, as on the device
    inv6ts = 1.0 / (torch.tensor(E2M1_MAX, dtype=torch.float32) * ts32)
    blocks = xf.reshape(*xf.shape[:-1], K // 16, 16)
    bamax = blocks.abs().amax(dim=-1)
    bs = _round_to_e4m3(bamax * inv6ts)
    denom = (bs * ts32)[..., None]
    inv = torch.where(denom > 0, 1.0 / denom, torch.zeros_like(denom))
    vals = _round_to_e2m1(blocks * inv)
    return vals.reshape(xf.shape), bs, ts32.item()


def nvfp4_dequantize(vals: torch.Tensor, bs: torch.Tensor, ts: float) -> torch.Tensor:
    K = vals.shape[-1]
    return (vals.reshape(*vals.shape[:-1], K // 16, 16) * (bs * ts)[..., None]).reshape(vals.shape)


def nvfp4_fake_quant(x: torch.Tensor) -> torch.Tensor:
    """dequant(quant(x)) along the last dimension, returned in x's dtype."""
    return nvfp4_dequantize(*nvfp4_quantize(x)).to(x.dtype)

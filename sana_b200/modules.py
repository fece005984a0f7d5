"""Drop-in PyTorch modules with upstream's constructor arguments, attribute names, state-dict
keys and forward signatures, computing through libsana_b200's CUDA kernels.

  LiteLA                   diffusion/model/nets/sana_blocks.py:211-301
  GLUMBConv (+ ConvLayer)  diffusion/model/nets/basic_modules.py:32-199
  MultiHeadCrossAttention  diffusion/model/nets/sana_blocks.py:48-98
  SanaMSBlock              diffusion/model/nets/sana_multi_scale.py:54-157

Inference only (no autograd through the kernels).  Feature combinations the kernels do not
cover raise; nothing falls back to eager PyTorch arithmetic.  The cross-attention's softmax core
runs on the library's own kernel (``cross_attn.softmax_core = "sdpa"`` selects torch SDPA, the
vendor flash kernel, for comparison; it is also what a head dimension the kernel does not cover
- not a multiple of 8, or above 128 - takes).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .sharding import SequenceShard

LN_EPS = 1e-6


def val2tuple(x, min_len: int = 1):
    """diffusion/model/utils.py val2tuple: scalar -> tuple repeated to ``min_len``."""
    x = tuple(x) if isinstance(x, (list, tuple)) else (x,)
    return x + (x[-1],) * max(0, min_len - len(x))


def _as2d(x: torch.Tensor) -> torch.Tensor:
    return x.reshape(-1, x.shape[-1])


def _fp4_weight(owner: nn.Module, key: str, w2d: torch.Tensor) -> "ops.NvFp4Tensor":
    """The NVFP4 image of a projection weight: a packed weight installed by
    ``weight_pack.load_nvfp4_weights``, else quantised once and cached on the module until the
    parameter is modified or moved."""
    packed = owner.__dict__.get("_nvfp4_packed")
    if packed is not None and key in packed:
        return packed[key]
    cache = owner.__dict__.setdefault("_nvfp4_weights", {})
    tag = (w2d.data_ptr(), w2d._version, tuple(w2d.shape))
    entry = cache.get(key)
    if entry is None or entry[0] != tag:
        entry = (tag, ops.nvfp4_quantize(w2d.contiguous()))
        cache[key] = entry
    return entry[1]


def _project(owner: nn.Module, key: str, x2d, w2d: torch.Tensor, **epilogue) -> torch.Tensor:
    """``x2d @ w2d.T`` with the fused epilogue of :func:`ops.gemm`.  When ``owner.nvfp4`` is set
    both operands are NVFP4: the weight through :func:`_fp4_weight`; the activation is either
    already quantised by the kernel that produced it (an ``ops.NvFp4Tensor``) or quantised here,
    with a measuring pass, on every call."""
    if isinstance(x2d, ops.NvFp4Tensor):
        return ops.gemm_nvfp4(x2d, _fp4_weight(owner, key, w2d), **epilogue)
    if not getattr(owner, "nvfp4", False):
        return ops.gemm(x2d, w2d, **epilogue)
    if x2d.dtype != torch.bfloat16:
        raise NotImplementedError("NVFP4 projections take bf16 activations and weights")
    qa = ops.nvfp4_quantize(x2d)
    seen = owner.__dict__.get("_fp4_seen")
    if seen is not None:  # a calibrating forward: remember the measured scales of this projection's input
        seen[key] = qa.scales
    return ops.gemm_nvfp4(qa, _fp4_weight(owner, key, w2d), **epilogue)


class RMSNorm(nn.Module):
    """Parameter holder with upstream's RMSNorm state-dict key (``weight``,
    diffusion/model/norms.py:182-231); the attention modules apply it in place on their
    q / k projections through the CUDA kernel."""

    def __init__(self, dim: int, scale_factor=1.0, eps: float = 1e-6, norm_dim: int = -1):
        super().__init__()
        if norm_dim != -1:
            raise NotImplementedError("RMSNorm over a dimension other than the last is not covered")
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim) * scale_factor)
        self.norm_dim = norm_dim

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = x.reshape(-1, x.shape[-1]).clone()
        return ops.rmsnorm_(y, self.weight, float(self.eps)).reshape(x.shape)


class LiteLA(nn.Module):
    """ReLU linear attention.  Same arguments and attributes as upstream's LiteLA (which
    derives from timm's Attention: ``qkv``, ``proj``, ``num_heads``, ``scale``,
    ``attn_drop``, ``proj_drop``)."""

    PAD_VAL = 1

    def __init__(self, in_dim: int, out_dim: int, heads: Optional[int] = None, heads_ratio: float = 1.0, dim=32,
                 eps=1e-15, use_bias=False, qk_norm=False, norm_eps=1e-5):
        super().__init__()
        heads = heads or int(out_dim // dim * heads_ratio)
        if in_dim != out_dim or out_dim // heads != ops.HEAD_DIM or out_dim % heads != 0:
            raise NotImplementedError("the linear-attention kernels need in_dim == out_dim and head dimension 32")
        self.num_heads = heads
        self.scale = (in_dim // heads) ** -0.5
        self.qkv = nn.Linear(in_dim, in_dim * 3, bias=use_bias)
        self.attn_drop = nn.Dropout(0.0)
        self.proj = nn.Linear(in_dim, in_dim)
        self.proj_drop = nn.Dropout(0.0)
        self.in_dim = in_dim
        self.out_dim = out_dim
        self.heads = heads
        self.dim = out_dim // heads
        self.eps = eps
        self.kernel_func = nn.ReLU(inplace=False)
        if qk_norm:  # RMSNorm over the full channel dimension, before the head split
            self.q_norm = RMSNorm(in_dim, scale_factor=1.0, eps=norm_eps)
            self.k_norm = RMSNorm(in_dim, scale_factor=1.0, eps=norm_eps)
        else:
            self.q_norm = nn.Identity()
            self.k_norm = nn.Identity()
        self.seq_shard: Optional[SequenceShard] = None
        self.nvfp4 = False  # quantise the qkv / proj projections to NVFP4

    # -- pieces shared with the fused block path --------------------------------------------
    def _core(self, qkv: torch.Tensor, B: int, N: int, rotary_emb=None, fp4_buf=None):
        """qkv [B*N, 3C] -> normalised attention output [B*N, C] (before ``proj``).
        ``rotary_emb`` = (cos, sin), each [N, head_dim]: rotates q and k before the ReLU.
        With ``fp4_buf`` (an ``ops.Fp4Buffers``) the output is written as NVFP4 by the apply kernel
        and an ``ops.NvFp4Tensor`` is returned."""
        C = self.out_dim
        if isinstance(self.q_norm, RMSNorm):  # in place on the q and k column blocks
            ops.rmsnorm_(qkv[:, :C], self.q_norm.weight, float(self.q_norm.eps))
            ops.rmsnorm_(qkv[:, C:2 * C], self.k_norm.weight, float(self.k_norm.eps))
        if rotary_emb is not None:
            if self.seq_shard is not None:
                raise NotImplementedError("rotary embeddings on a sequence shard are not covered")
            cos, sin = rotary_emb
            ops.rope_(qkv[:, :C], cos, sin, B, N, self.dim)
            ops.rope_(qkv[:, C:2 * C], cos, sin, B, N, self.dim)
        sh = self.seq_shard
        if sh is not None and sh.fused_state_exchange:
            # reduction kernel sums the ranks' partial states itself, over peer memory
            state = sh.fused_state(qkv[:, C:2 * C], qkv[:, 2 * C:], B, self.heads)
        else:
            state = ops.la_state(qkv[:, C:2 * C], qkv[:, 2 * C:], B, N, self.heads)
            if sh is not None:
                sh.allreduce_state(state)
        if fp4_buf is not None:
            return ops.la_apply_fp4(qkv[:, :C], state, B, N, self.heads, float(self.eps), fp4_buf)
        return ops.la_apply(qkv[:, :C], state, B, N, self.heads, float(self.eps))

    def attn_matmul(self, q, k, v: torch.Tensor) -> torch.Tensor:
        """Upstream layout (sana_blocks.py:245-263): q, v [B, h, d, N], k [B, h, N, d]; returns
        fp32 [B, h, d, N].  Kept for the guidance processors that call it directly."""
        B, h, d, N = q.shape
        dt = q.dtype
        qt = q.permute(0, 3, 1, 2).reshape(B * N, h * d).contiguous()
        kt = k.permute(0, 2, 1, 3).reshape(B * N, h * d).contiguous()
        vt = v.permute(0, 3, 1, 2).reshape(B * N, h * d).contiguous()
        state = ops.la_state(kt, vt, B, N, h)
        o = ops.la_apply(qt, state, B, N, h, float(self.eps))
        # contiguous like upstream's result: callers .view() it as [B, C, N]
        return o.to(dt).float().reshape(B, N, h, d).permute(0, 2, 3, 1).contiguous()

    def forward(self, x: torch.Tensor, mask=None, HW=None, rotary_emb=None, block_id=None, block_mask=None):
        B, N, C = x.shape
        qkv = _project(self, "qkv", _as2d(x), self.qkv.weight, bias=self.qkv.bias)
        o = self._core(qkv, B, N, rotary_emb)
        return _project(self, "proj", o, self.proj.weight, bias=self.proj.bias).reshape(B, N, C)

    @property
    def module_str(self) -> str:
        return f"{type(self).__name__}(i={self.in_dim},o={self.out_dim},h={self.heads},d={self.dim},eps={self.eps:.1E}"

    def __repr__(self):
        return f"EPS{self.eps}-" + super().__repr__()


def wan_rotary_freqs(head_dim: int, fhw: Sequence[int], theta: float = 10000.0, max_seq_len: int = 1024,
                     fhw_dim: Optional[Sequence[int]] = None, device=None) -> torch.Tensor:
    """Frequencies of upstream's WanRotaryPosEmbed (sana_blocks.py:1361-1410): complex128
    [1, 1, f*h*w, head_dim/2].  The channel pairs of a head split into a frame, a row and a column
    group; group g of a token at (f, h, w) rotates by coordinate * theta^(-2i / dim_g)."""
    if fhw_dim is not None:
        t_dim, h_dim, w_dim = fhw_dim
        if t_dim + h_dim + w_dim != head_dim:
            raise ValueError(f"head_dim {head_dim} must equal sum(fhw_dim) {t_dim + h_dim + w_dim}")
    else:
        h_dim = w_dim = 2 * (head_dim // 6)
        t_dim = head_dim - h_dim - w_dim
    f, h, w = (int(v) for v in fhw)
    if max(f, h, w) > max_seq_len:
        raise ValueError("a grid side exceeds max_seq_len")
    groups = []
    for dim, shape in ((t_dim, (f, 1, 1)), (h_dim, (1, h, 1)), (w_dim, (1, 1, w))):
        rate = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float64, device=device)[: dim // 2] / dim))
        angle = torch.outer(torch.arange(max(shape), device=device), rate)
        groups.append(torch.polar(torch.ones_like(angle), angle).view(*shape, -1).expand(f, h, w, -1))
    return torch.cat(groups, dim=-1).reshape(1, 1, f * h * w, -1)


class LiteLAReLURope(nn.Module):
    """Linear attention with the ReLU feature map first and the rotation after it, on the
    numerator's q and k only (upstream's LiteLAReLURope, sana_blocks.py:304-388; self-attention of
    Sana-Video).  Same constructor arguments, attributes and state-dict keys as upstream.
    ``rotary_emb`` is upstream's complex tensor [1, 1, N, head_dim/2] (or a (cos, sin) pair of fp32
    [N, head_dim/2] tables); its fp32 tables are cached per tensor."""

    PAD_VAL = 1

    def __init__(self, in_dim: int, out_dim: int, heads: Optional[int] = None, heads_ratio: float = 1.0, dim=32,
                 eps=1e-15, use_bias=False, qk_norm=False, norm_eps=1e-5):
        super().__init__()
        heads = heads or int(out_dim // dim * heads_ratio)
        head_dim = out_dim // heads
        if in_dim != out_dim or out_dim % heads != 0 or head_dim % 16 != 0 or not 16 <= head_dim <= 128:
            raise NotImplementedError("the kernels need in_dim == out_dim and a head dimension that is a multiple "
                                      "of 16 in [16, 128]")
        self.num_heads = heads
        self.scale = (in_dim // heads) ** -0.5
        self.qkv = nn.Linear(in_dim, in_dim * 3, bias=use_bias)
        self.attn_drop = nn.Dropout(0.0)
        self.proj = nn.Linear(in_dim, in_dim)
        self.proj_drop = nn.Dropout(0.0)
        self.in_dim = in_dim
        self.out_dim = out_dim
        self.heads = heads
        self.dim = head_dim
        self.eps = eps
        self.kernel_func = nn.ReLU(inplace=False)
        if qk_norm:
            self.q_norm = RMSNorm(in_dim, scale_factor=1.0, eps=norm_eps)
            self.k_norm = RMSNorm(in_dim, scale_factor=1.0, eps=norm_eps)
        else:
            self.q_norm = nn.Identity()
            self.k_norm = nn.Identity()
        self.qkv_store_buffer = None
        self.nvfp4 = False
        self.seq_shard: Optional[SequenceShard] = None
        self._tables = None  # (key, cos, sin)

    def rotary_tables(self, rotary_emb, N: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        """fp32 [N, head_dim/2] cos / sin tables of ``rotary_emb`` on ``device``."""
        if isinstance(rotary_emb, (tuple, list)):
            cos, sin = rotary_emb
            return (cos.to(device=device, dtype=torch.float32).contiguous(),
                    sin.to(device=device, dtype=torch.float32).contiguous())
        key = (rotary_emb.data_ptr(), rotary_emb._version, tuple(rotary_emb.shape), str(device))
        if self._tables is None or self._tables[0] != key:
            if not rotary_emb.is_complex() or rotary_emb.numel() != N * (self.dim // 2):
                raise ValueError("rotary_emb must be complex [1, 1, N, head_dim / 2]")
            fr = rotary_emb.reshape(N, self.dim // 2)
            self._tables = (key, fr.real.to(device=device, dtype=torch.float32).contiguous(),
                            fr.imag.to(device=device, dtype=torch.float32).contiguous())
        return self._tables[1], self._tables[2]

    def _core(self, qkv: torch.Tensor, B: int, N: int, rotary_emb) -> torch.Tensor:
        """qkv [B*N, 3C] -> normalised attention output [B*N, C] (before ``proj``)."""
        C = self.out_dim
        if rotary_emb is None:
            raise ValueError("LiteLAReLURope needs rotary_emb")
        if isinstance(self.q_norm, RMSNorm):  # in place on the q and k column blocks
            ops.rmsnorm_(qkv[:, :C], self.q_norm.weight, float(self.q_norm.eps))
            ops.rmsnorm_(qkv[:, C:2 * C], self.k_norm.weight, float(self.k_norm.eps))
        sh = self.seq_shard
        if sh is None:
            cos, sin = self.rotary_tables(rotary_emb, N, qkv.device)
        else:
            # this rank holds tokens [a, b) of every sample; ``rotary_emb`` covers the whole grid.  The state is
            # a plain sum over tokens, so the ranks' partial states add.
            a, b = sh.token_range
            if b - a != N:
                raise ValueError("the token count does not match this rank's share of the grid")
            cos, sin = self.rotary_tables(rotary_emb, sh.frames * sh.H * sh.W, qkv.device)
            # this rank's rows of the tables, kept until the tables or the range change
            cached = getattr(self, "_shard_tables", None)
            if cached is None or cached[0] is not cos or cached[1] != (a, b):
                cached = self._shard_tables = (cos, (a, b), cos[a:b].contiguous(), sin[a:b].contiguous())
            cos, sin = cached[2], cached[3]
        if sh is not None and sh.fused_rope_state_exchange:  # all-reduce inside the reduction kernel
            state = sh.fused_rope_state(qkv[:, C:2 * C], qkv[:, 2 * C:], cos, sin, B, self.heads, self.dim)
        else:
            state = ops.la_rope_state(qkv[:, C:2 * C], qkv[:, 2 * C:], cos, sin, B, N, self.heads, self.dim)
            if sh is not None:
                sh.allreduce_state(state)
        return ops.la_rope_apply(qkv[:, :C], cos, sin, state, B, N, self.heads, self.dim, float(self.eps))

    def forward(self, x: torch.Tensor, mask=None, HW=None, rotary_emb=None, block_mask=None, **kwargs):
        B, N, C = x.shape
        qkv = _project(self, "qkv", _as2d(x), self.qkv.weight, bias=self.qkv.bias)
        o = self._core(qkv, B, N, rotary_emb)
        return _project(self, "proj", o, self.proj.weight, bias=self.proj.bias).reshape(B, N, C)


class ChunkedLiteLAReLURope(LiteLAReLURope):
    """Upstream's ChunkedLiteLAReLURope (sana_blocks.py:1790-1914) sums ``vk`` over chunks of
    ``chunk_size`` tokens to bound its temporaries; the result is the same sum.  The state kernel here
    already walks the tokens in tiles and keeps nothing token-sized, so ``chunk_size`` is accepted and
    has no effect."""

    def __init__(self, *args, chunk_size=200_000, **kwargs):
        super().__init__(*args, **kwargs)
        self.chunk_size = chunk_size


class ChunkCausalAttention(LiteLAReLURope):
    """Upstream's ChunkCausalAttention (sana_blocks.py:391-496): the frames of the (T, H, W) grid are cut at
    ``chunk_index``; the queries of a chunk see the state summed over their own and all earlier chunks.  Per
    sample and chunk one state launch (added on top of the running state) and one apply launch."""

    def _core(self, qkv: torch.Tensor, B: int, N: int, rotary_emb, HW=None, chunk_index=None) -> torch.Tensor:
        C, D, H = self.out_dim, self.dim, self.heads
        if rotary_emb is None or HW is None or len(HW) != 3:
            raise ValueError("ChunkCausalAttention needs rotary_emb and HW = (T, H, W)")
        if self.seq_shard is not None:
            raise NotImplementedError("chunk-causal attention on a sequence shard is not covered")
        f, h, w = HW
        if N != f * h * w:
            raise ValueError(f"N={N} does not match HW={tuple(HW)}")
        if isinstance(self.q_norm, RMSNorm):
            ops.rmsnorm_(qkv[:, :C], self.q_norm.weight, float(self.q_norm.eps))
            ops.rmsnorm_(qkv[:, C:2 * C], self.k_norm.weight, float(self.k_norm.eps))
        cos, sin = self.rotary_tables(rotary_emb, N, qkv.device)
        bounds = (list(chunk_index) if chunk_index is not None else [0]) + [f]
        out = torch.empty(B * N, C, dtype=qkv.dtype, device=qkv.device)
        for b in range(B):
            state = None
            for f0, f1 in zip(bounds[:-1], bounds[1:]):
                n0, n1 = int(f0) * h * w, int(f1) * h * w
                if n1 <= n0:
                    continue
                rows = slice(b * N + n0, b * N + n1)
                c, sn = cos[n0:n1], sin[n0:n1]
                state = ops.la_rope_state(qkv[rows, C:2 * C], qkv[rows, 2 * C:], c, sn, 1, n1 - n0, H, D, prior=state)
                ops.la_rope_apply(qkv[rows, :C], c, sn, state, 1, n1 - n0, H, D, float(self.eps), out=out[rows])
        return out

    def forward(self, x: torch.Tensor, mask=None, HW=None, rotary_emb=None, block_mask=None, chunk_index=None, **kwargs):
        B, N, C = x.shape
        qkv = _project(self, "qkv", _as2d(x), self.qkv.weight, bias=self.qkv.bias)
        o = self._core(qkv, B, N, rotary_emb, HW=HW, chunk_index=[0] if chunk_index is None else chunk_index)
        return _project(self, "proj", o, self.proj.weight, bias=self.proj.bias).reshape(B, N, C)


class CachedCausalAttention(LiteLAReLURope):
    """Upstream's CachedCausalAttention (sana_blocks.py:498-572): one chunk of frames per call; the state of
    this chunk's tokens is added to the pair found in ``kv_cache[0:2]`` (vk [B, h, d, d] and the key sum
    [B, h, 1, d], fp32 here), and with ``save_kv_cache`` the cache takes THIS chunk's own pair.  Returns
    (out, kv_cache) when a cache list is given, like upstream."""

    def _core_cached(self, qkv: torch.Tensor, B: int, N: int, rotary_emb, kv_cache, save_kv_cache: bool) -> torch.Tensor:
        C, D, H = self.out_dim, self.dim, self.heads
        if rotary_emb is None:
            raise ValueError("CachedCausalAttention needs rotary_emb (the frequencies of this chunk's tokens)")
        if self.seq_shard is not None:
            raise NotImplementedError("cached attention on a sequence shard is not covered")
        if isinstance(self.q_norm, RMSNorm):
            ops.rmsnorm_(qkv[:, :C], self.q_norm.weight, float(self.q_norm.eps))
            ops.rmsnorm_(qkv[:, C:2 * C], self.k_norm.weight, float(self.k_norm.eps))
        cos, sin = self.rotary_tables(rotary_emb, N, qkv.device)
        cur = ops.la_rope_state(qkv[:, C:2 * C], qkv[:, 2 * C:], cos, sin, B, N, H, D)
        state = cur
        if kv_cache is not None:
            prev_vk, prev_ks = kv_cache[0], kv_cache[1]
            if save_kv_cache:
                kv_cache[0], kv_cache[1] = cur[:, :, :D].clone(), cur[:, :, D:].clone()
            if prev_vk is not None and prev_ks is not None:
                prior = torch.cat([prev_vk.to(torch.float32), prev_ks.to(torch.float32)], dim=2).contiguous()  # layout only
                state = ops.add_f32(cur, prior)
        return ops.la_rope_apply(qkv[:, :C], cos, sin, state, B, N, H, D, float(self.eps))

    def forward(self, x: torch.Tensor, mask=None, HW=None, rotary_emb=None, block_mask=None, save_kv_cache=False,
                kv_cache=None, **kwargs):
        B, N, C = x.shape
        qkv = _project(self, "qkv", _as2d(x), self.qkv.weight, bias=self.qkv.bias)
        o = self._core_cached(qkv, B, N, rotary_emb, kv_cache, bool(save_kv_cache))
        out = _project(self, "proj", o, self.proj.weight, bias=self.proj.bias).reshape(B, N, C)
        return (out, kv_cache) if kv_cache is not None else out


class ConvLayer(nn.Module):
    """Parameter holder with upstream's ``conv`` / ``norm`` / ``act`` attributes
    (basic_modules.py:32-99) so checkpoints load unchanged; GLUMBConv reads the weights and
    runs the fused kernels instead of calling this layer."""

    def __init__(self, in_dim: int, out_dim: int, kernel_size=3, stride=1, dilation=1, groups=1, padding=None,
                 use_bias=False, dropout=0.0, conv_type="2d", norm=None, act=None):
        super().__init__()
        if stride != 1 or dilation != 1 or dropout > 0 or conv_type != "2d" or norm is not None:
            raise NotImplementedError("ConvLayer: only stride 1, dilation 1, no dropout, no norm, 2-D is covered")
        if padding is None:
            padding = kernel_size // 2
        self.in_dim, self.out_dim, self.kernel_size = in_dim, out_dim, kernel_size
        self.stride, self.dilation, self.groups, self.padding, self.use_bias = stride, dilation, groups, padding, use_bias
        self.dropout = None
        self.conv = nn.Conv2d(in_dim, out_dim, kernel_size=(kernel_size, kernel_size), stride=(stride, stride),
                              padding=padding, dilation=(dilation, dilation), groups=groups, bias=use_bias)
        self.norm = None
        self.act_name = act
        self.act = nn.SiLU(inplace=True) if act == "silu" else None
        if act not in (None, "silu"):
            raise NotImplementedError(f"ConvLayer: activation {act!r} is not covered")

    def forward(self, x):
        raise NotImplementedError("ConvLayer is a parameter holder here; call GLUMBConv.forward")


class GLUMBConv(nn.Module):
    """Mix-FFN: 1x1 expand + SiLU, 3x3 depthwise, SiLU-GLU, 1x1 project."""

    def __init__(self, in_features: int, hidden_features: int, out_feature=None, kernel_size=3, stride=1,
                 padding=None, use_bias=False, norm=(None, None, None), act=("silu", "silu", None), dilation=1):
        super().__init__()
        out_feature = out_feature or in_features
        use_bias = val2tuple(use_bias, 3)
        norm = val2tuple(norm, 3)
        act = val2tuple(act, 3)
        if kernel_size != 3 or stride != 1 or dilation != 1 or any(n is not None for n in norm):
            raise NotImplementedError("GLUMBConv: only kernel 3, stride 1, dilation 1, no norms is covered")
        if tuple(act) != ("silu", "silu", None):
            raise NotImplementedError("GLUMBConv: only act=('silu','silu',None) is covered")
        if hidden_features % 8 != 0 or in_features % 8 != 0 or out_feature % 8 != 0:
            raise NotImplementedError("GLUMBConv: feature sizes must be multiples of 8")
        self.glu_act = nn.SiLU(inplace=False)
        self.inverted_conv = ConvLayer(in_features, hidden_features * 2, 1, use_bias=use_bias[0], act=act[0])
        self.depth_conv = ConvLayer(hidden_features * 2, hidden_features * 2, kernel_size, groups=hidden_features * 2,
                                    padding=padding, use_bias=use_bias[1], act=None)
        self.point_conv = ConvLayer(hidden_features, out_feature, 1, use_bias=use_bias[2], act=act[2])
        self.in_features, self.hidden_features, self.out_feature = in_features, hidden_features, out_feature
        self.seq_shard: Optional[SequenceShard] = None
        self.nvfp4 = False  # quantise the two 1x1 projections to NVFP4

    def _expand(self, z2d: torch.Tensor) -> torch.Tensor:
        c = self.inverted_conv.conv
        return _project(self, "inverted_conv", z2d, c.weight.reshape(c.out_channels, c.in_channels), bias=c.bias,
                        act=ops.ACT_SILU)

    def _depthwise_glu(self, u: torch.Tensor, B: int, N: int, HW: Sequence[int], amax_out=None) -> torch.Tensor:
        if HW is None or len(HW) not in (2, 3):
            raise ValueError("GLUMBConv.forward needs HW=(H, W) or (T, H, W)")
        H, W = HW[-2], HW[-1]
        c = self.depth_conv.conv
        sh = self.seq_shard
        if sh is not None:
            if B != 1 or N != sh.tokens or (H, W) != (sh.H, sh.W):
                raise ValueError("sequence-parallel GLUMBConv: batch must be 1 and x the local token shard")
            top, bot = sh.exchange_halo(u)
            return ops.dwconv_glu(u, c.weight, c.bias, W, H, row0=sh.row0, halo_top=top, halo_bot=bot)
        frames = HW[0] if len(HW) == 3 else 1
        if N != frames * H * W:
            raise ValueError(f"GLUMBConv: N={N} does not match HW={tuple(HW)}")
        return ops.dwconv_glu(u, c.weight, c.bias, W, H, amax_out=amax_out)

    def forward(self, x: torch.Tensor, HW=None) -> torch.Tensor:
        B, N, C = x.shape
        u = self._expand(_as2d(x))
        g = self._depthwise_glu(u, B, N, HW)
        c = self.point_conv.conv
        out = _project(self, "point_conv", g, c.weight.reshape(c.out_channels, c.in_channels), bias=c.bias)
        return out.reshape(B, N, -1)


class GLUMBConvTemp(GLUMBConv):
    """Mix-FFN of the video blocks: GLUMBConv per frame, then a 3-tap convolution along the
    frame axis that mixes channels (``t_conv``: Conv2d(C, C, (3, 1)), no bias, zero padding in
    time) added to the spatial result (diffusion/model/nets/basic_modules.py:200-257).  Token-
    major, the three taps are three projections of the same tensor shifted by one frame, each
    accumulated through the GEMM's residual epilogue."""

    def __init__(self, in_features: int, hidden_features: int, out_feature=None, kernel_size=3, stride=1,
                 padding=None, use_bias=False, norm=(None, None, None), act=("silu", "silu", None), t_kernel_size=3):
        super().__init__(in_features, hidden_features, out_feature=out_feature, kernel_size=kernel_size, stride=stride,
                         padding=padding, use_bias=use_bias, norm=norm, act=act)
        if t_kernel_size != 3:
            raise NotImplementedError("GLUMBConvTemp: only the 3-tap temporal convolution is covered")
        C = self.out_feature
        self.t_conv = nn.Conv2d(C, C, kernel_size=(t_kernel_size, 1), stride=1, padding=(t_kernel_size // 2, 0), bias=False)
        nn.init.zeros_(self.t_conv.weight)

    def _taps(self):
        """The three [C, C] tap matrices as contiguous copies, rebuilt when the weight changes."""
        w = self.t_conv.weight
        tag = (w.data_ptr(), w._version, w.dtype, w.device)
        cached = self.__dict__.get("_tap_cache")
        if cached is None or cached[0] != tag:
            cached = (tag, [w[:, :, k, 0].contiguous() for k in range(3)])
            self.__dict__["_tap_cache"] = cached
        return cached[1]

    def _next_tap_ranges(self, T: int, chunk_index=None):
        """Frame ranges [a, b) inside which a frame sees the frame after it: the whole sample here."""
        return [(0, T)]

    def _frame_halo(self, s: torch.Tensor, B: int):
        """On a sequence shard: the frame before this rank's first token and the one after its last token,
        fetched from the neighbours (upstream: cp_halo_exchange of one frame each side,
        basic_modules.py:252-263).  (None, None) on one GPU."""
        sh = self.seq_shard
        if sh is None:
            return None, None
        if B != 1:
            raise ValueError("sequence-parallel GLUMBConvTemp: batch must be 1")
        return sh.exchange_frames(s)

    @torch.no_grad()
    def forward(self, x: torch.Tensor, HW=None, chunk_index=None, **kwargs) -> torch.Tensor:
        if HW is None or len(HW) != 3:
            raise ValueError("HW must be a tuple of (T, H, W)")
        if kwargs.get("frame_valid_mask") is not None:
            raise NotImplementedError("frame_valid_mask is not covered")
        B, N, C = x.shape
        T, H, W = HW
        hw = H * W
        ranges = self._next_tap_ranges(T, chunk_index)
        if self.seq_shard is not None and ranges != [(0, T)]:
            raise NotImplementedError("the chunked temporal Mix-FFN on a sequence shard is not covered")
        s = _as2d(GLUMBConv.forward(self, x, HW=HW))  # spatial result, token-major [B*N, C]
        halo_prev, halo_next = self._frame_halo(s, B)
        w_prev, w_mid, w_next = self._taps()
        y = ops.gemm(s, w_mid, residual=s)  # x + centre tap
        # a token takes the token H*W places before it through the previous-frame tap and the one H*W places
        # after it through the next-frame tap (zero padding at the ends of a sample); every row gets its
        # previous-frame term before its next-frame term, on one GPU and on shards alike
        for b in range(B):
            lo, hi = b * N, (b + 1) * N
            if N > hw:
                ops.gemm(s[lo:hi - hw], w_prev, residual=y[lo + hw:hi], out=y[lo + hw:hi])
        if halo_prev is not None:
            ops.gemm(halo_prev, w_prev, residual=y[:hw], out=y[:hw])
        for b in range(B):
            lo = b * N
            # frames fa .. fb-2 of a range take frames fa+1 .. fb-1; a shard (one range) counts in tokens, its
            # cuts need not lie between frames
            for ta, tb in ([(0, N)] if self.seq_shard is not None else [(fa * hw, fb * hw) for fa, fb in ranges]):
                if tb - ta > hw:
                    dst = y[lo + ta:lo + tb - hw]
                    ops.gemm(s[lo + ta + hw:lo + tb], w_next, residual=dst, out=dst)
        if halo_next is not None:
            ops.gemm(halo_next, w_next, residual=y[N - hw:N], out=y[N - hw:N])
        return y.reshape(B, N, C)

    @torch.no_grad()
    def forward_gated(self, z: torch.Tensor, HW, x2: torch.Tensor, table: torch.Tensor, t2: torch.Tensor, row: int,
                      rows_per_vec: int, kv_cache=None, save_kv_cache: bool = False, chunk_index=None) -> torch.Tensor:
        """``x2 + gate * forward(z)`` for the video block, [B*N, C]: ``gate`` = table[row] + t2[v, row] for
        the v-th run of ``rows_per_vec`` tokens (one modulation vector per sample, or per frame).  The
        spatial result enters through one fused multiply-add, the three temporal taps through the
        gate + residual epilogue of their projections."""
        if HW is None or len(HW) != 3:
            raise ValueError("HW must be a tuple of (T, H, W)")
        B, N, C = z.shape
        T, H, W = HW
        hw = H * W
        sh = self.seq_shard
        ranges = self._next_tap_ranges(T, chunk_index)
        if sh is not None and (kv_cache is not None or ranges != [(0, T)]):
            raise NotImplementedError("the cached / chunked temporal Mix-FFN on a sequence shard is not covered")
        whole = N == (T * hw if sh is None else sh.tokens)
        per_frame_ok = N % hw == 0 and (sh is None or sh.row0 % H == 0)
        if not whole or not (rows_per_vec == N or (rows_per_vec == hw and per_frame_ok)):
            # the taps of the previous / next frame take their gates by shifting t2 one vector, which is
            # only right when a vector covers a whole sample or exactly one frame (on a shard: whole frames)
            raise ValueError(f"GLUMBConvTemp: modulation runs of {rows_per_vec} tokens fit neither a sample ({N}) "
                             f"nor a frame ({hw}) of the {tuple(HW)} grid")
        s = _as2d(GLUMBConv.forward(self, z, HW=HW))
        halo_prev, halo_next = self._frame_halo(s, B)
        prev = None
        if kv_cache is not None:  # CachedGLUMBConvTemp: the previous chunk's last frame is the left context
            prev = self._left_context(kv_cache, B, hw, C, s.dtype)
            if save_kv_cache:
                self._save_context(kv_cache, s, B, T, hw, C)
        vecs = (B * N) // rows_per_vec
        gate = (table[row].float()[None] + t2.reshape(vecs, 6, C)[:, row].float()).to(s.dtype)  # [vecs, C]
        y = torch.addcmul(x2.view(vecs, rows_per_vec, C), gate[:, None, :], s.view(vecs, rows_per_vec, C)).view(B * N, C)
        w_prev, w_mid, w_next = self._taps()
        per_sample = N // rows_per_vec  # modulation vectors per sample: 1, or the number of frames held
        y = ops.gemm(s, w_mid, gate=(table, t2, row, rows_per_vec), residual=y, out=y)
        for b in range(B):
            lo, hi = b * N, (b + 1) * N
            v0 = b * per_sample
            if N > hw:
                # output frames 1 .. take frame t-1: their vectors start one frame later when per frame
                t_hi = t2[v0 + (1 if per_sample > 1 else 0):v0 + per_sample]
                ops.gemm(s[lo:hi - hw], w_prev, gate=(table, t_hi, row, rows_per_vec), residual=y[lo + hw:hi],
                         out=y[lo + hw:hi])
            if prev is not None:  # frame 0 takes the cached frame through the previous-frame tap, under frame 0's gate
                ops.gemm(prev[b], w_prev, gate=(table, t2[v0:v0 + 1], row, hw), residual=y[lo:lo + hw], out=y[lo:lo + hw])
        if halo_prev is not None:  # the first frame's worth of rows takes the left neighbour's last one
            ops.gemm(halo_prev, w_prev, gate=(table, t2[0:1], row, hw), residual=y[:hw], out=y[:hw])
        for b in range(B):
            lo = b * N
            v0 = b * per_sample
            for ta, tb in ([(0, N)] if sh is not None else [(fa * hw, fb * hw) for fa, fb in ranges]):
                if tb - ta > hw:  # the rows of a range except its last frame's worth, under their own frames' gates
                    tv = t2[v0 + ta // hw:v0 + per_sample] if per_sample > 1 else t2[v0:v0 + 1]
                    dst = y[lo + ta:lo + tb - hw]
                    ops.gemm(s[lo + ta + hw:lo + tb], w_next, gate=(table, tv, row, rows_per_vec), residual=dst, out=dst)
        if halo_next is not None:  # ... and the last frame's worth the right neighbour's first one
            ops.gemm(halo_next, w_next, gate=(table, t2[per_sample - 1:per_sample], row, hw), residual=y[N - hw:N],
                     out=y[N - hw:N])
        return y


class ChunkGLUMBConvTemp(GLUMBConvTemp):
    """Upstream's ChunkGLUMBConvTemp (basic_modules.py:273-351), the Mix-FFN that goes with the chunk-causal
    attention: the frames are cut at ``chunk_index``; the previous-frame tap crosses the cuts (a chunk's first frame
    sees the last frame of the chunk before it), the next-frame tap does not (a chunk's last frame sees zeros).
    Here that is the plain temporal Mix-FFN with the next-frame projection issued per chunk."""

    def _next_tap_ranges(self, T: int, chunk_index=None):
        cuts = sorted({0, T, *(int(i) for i in (chunk_index or [0]) if 0 < int(i) < T)})
        return list(zip(cuts, cuts[1:]))


class CachedGLUMBConvTemp(GLUMBConvTemp):
    """Upstream's CachedGLUMBConvTemp (basic_modules.py:359-397): the temporal convolution's left context is
    the last frame of the previous chunk, kept in ``kv_cache[-1]`` as [B, C, 1, H*W] (upstream's layout), instead
    of zero padding; the right side stays zero-padded.  The cached frame is one more projection (the tap of the
    previous frame) accumulated into the first frame's rows.  Returns (out, kv_cache) when a cache list is given."""

    def _left_context(self, kv_cache, B: int, hw: int, C: int, dtype):
        """The cached frame as token-major rows [B, hw, C], or None."""
        if kv_cache is None or kv_cache[-1] is None:
            return None
        prev = kv_cache[-1][:, :, -1]  # [B, C, hw]
        if prev.shape != (B, C, hw):
            raise ValueError(f"cached frame has shape {tuple(prev.shape)}, expected {(B, C, hw)}")
        return prev.to(dtype).permute(0, 2, 1).contiguous()

    @staticmethod
    def _save_context(kv_cache, s: torch.Tensor, B: int, T: int, hw: int, C: int) -> None:
        kv_cache[-1] = s.view(B, T, hw, C)[:, -1].permute(0, 2, 1)[:, :, None].contiguous()

    @torch.no_grad()
    def forward(self, x: torch.Tensor, HW=None, save_kv_cache=False, kv_cache=None, **kwargs):
        if HW is None or len(HW) != 3:
            raise ValueError("HW must be a tuple of (T, H, W)")
        B, N, C = x.shape
        T, H, W = HW
        hw = H * W
        s = _as2d(GLUMBConv.forward(self, x, HW=HW))
        prev = self._left_context(kv_cache, B, hw, C, s.dtype)
        if kv_cache is not None and save_kv_cache:
            self._save_context(kv_cache, s, B, T, hw, C)
        w_prev, w_mid, w_next = self._taps()
        y = ops.gemm(s, w_mid, residual=s)
        for b in range(B):
            lo, hi = b * N, (b + 1) * N
            if T > 1:
                ops.gemm(s[lo:hi - hw], w_prev, residual=y[lo + hw:hi], out=y[lo + hw:hi])
                ops.gemm(s[lo + hw:hi], w_next, residual=y[lo:hi - hw], out=y[lo:hi - hw])
            if prev is not None:
                ops.gemm(prev[b], w_prev, residual=y[lo:lo + hw], out=y[lo:lo + hw])
        out = y.reshape(B, N, C)
        return (out, kv_cache) if kv_cache is not None else out


class MultiHeadCrossAttention(nn.Module):
    """Softmax attention of image tokens over the text tokens (upstream's SDPA branch), with
    the projections on the GEMM kernel and the softmax core on its own kernel."""

    def __init__(self, d_model, num_heads, attn_drop=0.0, proj_drop=0.0, qk_norm=False, **block_kwargs):
        super().__init__()
        assert d_model % num_heads == 0, "d_model must be divisible by num_heads"
        self.d_model, self.num_heads, self.head_dim = d_model, num_heads, d_model // num_heads
        self.q_linear = nn.Linear(d_model, d_model)
        self.kv_linear = nn.Linear(d_model, d_model * 2)
        self.attn_drop = nn.Dropout(attn_drop)
        self.proj = nn.Linear(d_model, d_model)
        self.proj_drop = nn.Dropout(proj_drop)
        # softmax core: "kernel" / "auto" = sana_cross_attention (bf16: the tcgen05 kernel for 17..304 text
        # tokens, 84 us per 16 384-token image at 1.6B width; the warp-level kernel otherwise), "sdpa" =
        # torch's scaled_dot_product_attention (the vendor flash kernel, 57 us on the same box), kept
        # selectable for comparison only
        self.softmax_core = "auto"
        if qk_norm:
            self.q_norm = RMSNorm(d_model, scale_factor=1.0, eps=1e-6)
            self.k_norm = RMSNorm(d_model, scale_factor=1.0, eps=1e-6)
        else:
            self.q_norm = nn.Identity()
            self.k_norm = nn.Identity()

    def project_kv(self, cond: torch.Tensor) -> torch.Tensor:
        """Key / value projection of the text tokens, [B*L, 2C] (k | v), with the optional k norm
        applied.  It depends on the caption only, so a caller may compute it ahead of the block
        (on another stream, or once for several denoising steps) and pass it to ``_attend``."""
        C = self.d_model
        kv2d = ops.gemm(_as2d(cond), self.kv_linear.weight, bias=self.kv_linear.bias)
        if isinstance(self.k_norm, RMSNorm):
            ops.rmsnorm_(kv2d[:, :C], self.k_norm.weight, float(self.k_norm.eps))
        return kv2d

    def _attend(self, x2d: torch.Tensor, cond: torch.Tensor, mask, B: int, kv2d: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Returns the attention output [B*N, C] before ``proj``.  ``kv2d``: the result of
        :meth:`project_kv` when it was computed ahead of time."""
        C, h, hd = self.d_model, self.num_heads, self.head_dim
        q = ops.gemm(x2d, self.q_linear.weight, bias=self.q_linear.bias)
        if kv2d is None:
            kv2d = self.project_kv(cond)
        if isinstance(self.q_norm, RMSNorm):
            ops.rmsnorm_(q, self.q_norm.weight, float(self.q_norm.eps))
        if mask is not None and (not torch.is_tensor(mask) or mask.ndim != 2):
            raise NotImplementedError("cross-attention mask must be None or a [B, L] 0/1 tensor")
        L = kv2d.shape[0] // B
        core = self.softmax_core
        if core == "auto":
            core = "kernel" if hd % 8 == 0 and hd <= 128 else "sdpa"
        if core == "kernel":
            if hd % 8 != 0 or hd > 128:
                raise NotImplementedError("the cross-attention kernel needs a head dimension that is a multiple of 8, <= 128")
            return ops.cross_attention(q, kv2d[:, :C], kv2d[:, C:], mask, B, x2d.shape[0] // B, L, h, hd)
        kv = kv2d.view(B, L, 2, h, hd)
        bias = None
        if mask is not None:
            bias = ((1 - mask.to(q.dtype)) * -10000.0)[:, None, None].expand(B, h, 1, L)
        o = F.scaled_dot_product_attention(q.view(B, -1, h, hd).transpose(1, 2), kv[:, :, 0].transpose(1, 2),
                                           kv[:, :, 1].transpose(1, 2), attn_mask=bias, dropout_p=0.0, is_causal=False)
        return o.transpose(1, 2).reshape(-1, C)

    def forward(self, x, cond, mask=None):
        B, N, C = x.shape
        o = self._attend(_as2d(x), cond, mask, B)
        return ops.gemm(o, self.proj.weight, bias=self.proj.bias).reshape(B, N, C)


class SanaMSBlock(nn.Module):
    """adaLN-single Linear-DiT block: modulate -> LiteLA -> gate+residual -> cross-attention
    + residual -> modulate -> GLUMBConv -> gate+residual.  Eight GEMM launches with fused
    bias / SiLU / gate / residual epilogues, plus LN-modulate, linear-attention state/apply and
    depthwise-GLU kernels."""

    def __init__(self, hidden_size, num_heads, mlp_ratio=4.0, drop_path=0.0, qk_norm=False, attn_type="flash",
                 ffn_type="mlp", mlp_acts=("silu", "silu", None), linear_head_dim=32, cross_norm=False,
                 cross_attn_type="flash", **block_kwargs):
        super().__init__()
        if attn_type != "linear" or ffn_type != "glumbconv":
            raise NotImplementedError("SanaMSBlock here covers attn_type='linear' with ffn_type='glumbconv' only")
        if drop_path != 0.0:
            raise NotImplementedError("drop_path > 0 (training) is not covered")
        if cross_attn_type not in ("flash", "linear"):
            raise ValueError(f"{cross_attn_type} type is not defined.")
        self.hidden_size = hidden_size
        self.norm1 = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=LN_EPS)
        self.attn = LiteLA(hidden_size, hidden_size, heads=hidden_size // linear_head_dim, eps=1e-8, qk_norm=qk_norm)
        self.cross_attn = MultiHeadCrossAttention(hidden_size, num_heads, qk_norm=cross_norm, **block_kwargs)
        self.norm2 = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=LN_EPS)
        self.mlp = GLUMBConv(in_features=hidden_size, hidden_features=int(hidden_size * mlp_ratio),
                             use_bias=(True, True, False), norm=(None, None, None), act=mlp_acts)
        self.drop_path = nn.Identity()
        self.scale_shift_table = nn.Parameter(torch.randn(6, hidden_size) / hidden_size ** 0.5)

    def set_sequence_shard(self, shard: Optional[SequenceShard]) -> None:
        """Run this block on one rank's slice of the token grid (see sharding.SequenceShard)."""
        self.attn.seq_shard = shard
        self.mlp.seq_shard = shard

    def set_nvfp4(self, enabled: bool = True, delayed_scaling: bool = False, margin: float = 1.0) -> None:
        """Run the qkv, attention-output and the two FFN 1x1 projections on the block-scaled FP4
        tensor cores (E2M1 values, E4M3 scales per 16 channels, fp32 scale per tensor, for both
        weights and activations).  Linear-attention state, depthwise conv, LayerNorm and the
        cross-attention stay in bf16/fp32.

        By default every activation is quantised with its own measured maximum, which costs two more
        passes over it.  With ``delayed_scaling`` the kernels that produce the four activations write
        FP4 directly (LayerNorm-modulate, attention apply) or note their maximum on the way (depthwise
        conv), using per-tensor scales measured on the previous forward (times ``margin``); the first
        forward after enabling it, and any forward after :meth:`recalibrate_nvfp4`, measures."""
        self.attn.nvfp4 = enabled
        self.mlp.nvfp4 = enabled
        self.__dict__["_fp4_delayed"] = bool(enabled and delayed_scaling)
        self.__dict__["_fp4_margin"] = float(margin)
        self.__dict__["_fp4_state"] = None  # records + buffers, built by the calibrating forward

    def recalibrate_nvfp4(self) -> None:
        """The next forward measures the activation maxima again (delayed scaling)."""
        self.__dict__["_fp4_state"] = None

    _FP4_KEYS = (("attn", "qkv"), ("attn", "proj"), ("mlp", "inverted_conv"), ("mlp", "point_conv"))

    def _fp4_calibrate(self, x, y, t, mask, HW, image_rotary_emb, kwargs):
        """A measuring forward: the four activations' scales are copied into the records."""
        seen_a, seen_m = {}, {}
        self.attn.__dict__["_fp4_seen"], self.mlp.__dict__["_fp4_seen"] = seen_a, seen_m
        self.__dict__["_fp4_delayed"] = False
        try:
            out = self.forward(x, y, t, mask, HW, image_rotary_emb, **kwargs)
        finally:
            self.__dict__["_fp4_delayed"] = True
            del self.attn.__dict__["_fp4_seen"], self.mlp.__dict__["_fp4_seen"]
        records = torch.zeros(4, 4, dtype=torch.float32, device=x.device)
        for i, (owner, key) in enumerate(self._FP4_KEYS):
            records[i, :2] = (seen_a if owner == "attn" else seen_m)[key][:2]
        self.__dict__["_fp4_state"] = {"records": records, "bufs": {}}
        return out

    def _fp4_buf(self, idx: int, rows: int, K: int, device) -> "ops.Fp4Buffers":
        st = self.__dict__["_fp4_state"]
        buf = st["bufs"].get((idx, rows, K))
        if buf is None:
            buf = ops.Fp4Buffers(rows, K, device, record=st["records"][idx])
            st["bufs"][(idx, rows, K)] = buf
        return buf

    @torch.no_grad()
    def forward(self, x, y, t, mask=None, HW=None, image_rotary_emb=None, **kwargs):
        B, N, C = x.shape
        x2 = _as2d(x.contiguous())
        table = self.scale_shift_table
        t = t.reshape(B, 6 * C)
        attn, mlp, ca = self.attn, self.mlp, self.cross_attn
        delayed = (self.__dict__.get("_fp4_delayed", False) and x.dtype == torch.bfloat16 and "forward" not in attn.__dict__
                   and attn.seq_shard is None)
        if delayed and self.__dict__.get("_fp4_state") is None:
            return self._fp4_calibrate(x, y, t, mask, HW, image_rotary_emb, kwargs)
        if delayed:
            # activations quantised where they are produced, scales from the previous forward
            rows, hid = B * N, mlp.hidden_features
            ops.nvfp4_scale_roll(self.__dict__["_fp4_state"]["records"], self.__dict__["_fp4_margin"])
            zq = ops.ln_modulate_fp4(x, table, t, 0, 1, self._fp4_buf(0, rows, C, x.device), LN_EPS)
            qkv = _project(attn, "qkv", zq, attn.qkv.weight, bias=attn.qkv.bias)
            oq = attn._core(qkv, B, N, image_rotary_emb, fp4_buf=self._fp4_buf(1, rows, C, x.device))
            x2 = _project(attn, "proj", oq, attn.proj.weight, bias=attn.proj.bias, gate=(table, t, 2, N), residual=x2)
            o = ca._attend(x2, y, mask, B, kwargs.get("caption_kv"))
            x2 = ops.gemm(o, ca.proj.weight, bias=ca.proj.bias, residual=x2)
            zq = ops.ln_modulate_fp4(x2.view(B, N, C), table, t, 3, 4, self._fp4_buf(2, rows, C, x.device), LN_EPS)
            c1 = mlp.inverted_conv.conv
            u = _project(mlp, "inverted_conv", zq, c1.weight.reshape(c1.out_channels, c1.in_channels), bias=c1.bias,
                         act=ops.ACT_SILU)
            buf = self._fp4_buf(3, rows, hid, x.device)
            g = mlp._depthwise_glu(u, B, N, HW, amax_out=buf.record[2:3])
            gq = ops.nvfp4_quantize_scaled(g, buf)
            pc = mlp.point_conv.conv
            x2 = _project(mlp, "point_conv", gq, pc.weight.reshape(pc.out_channels, pc.in_channels), bias=pc.bias,
                          gate=(table, t, 5, N), residual=x2)
            return x2.view(B, N, C)
        if "forward" in attn.__dict__:
            # an attention processor was installed on this instance (guidance code does that):
            # keep its semantics, at the cost of the fused epilogues
            z = ops.ln_modulate(x, table, t, 0, 1, LN_EPS)
            a = attn.forward(z, HW=HW, rotary_emb=image_rotary_emb)
            gate = (table[2][None] + t.reshape(B, 6, C)[:, 2])[:, None]
            x2 = _as2d((x + gate * a).contiguous())
        else:
            z = ops.ln_modulate(x, table, t, 0, 1, LN_EPS)
            qkv = _project(attn, "qkv", _as2d(z), attn.qkv.weight, bias=attn.qkv.bias)
            o = attn._core(qkv, B, N, image_rotary_emb)
            x2 = _project(attn, "proj", o, attn.proj.weight, bias=attn.proj.bias, gate=(table, t, 2, N), residual=x2)
        o = ca._attend(x2, y, mask, B, kwargs.get("caption_kv"))
        x2 = ops.gemm(o, ca.proj.weight, bias=ca.proj.bias, residual=x2)
        z = ops.ln_modulate(x2.view(B, N, C), table, t, 3, 4, LN_EPS)
        u = mlp._expand(_as2d(z))
        g = mlp._depthwise_glu(u, B, N, HW)
        pc = mlp.point_conv.conv
        x2 = _project(mlp, "point_conv", g, pc.weight.reshape(pc.out_channels, pc.in_channels), bias=pc.bias,
                      gate=(table, t, 5, N), residual=x2)
        return x2.view(B, N, C)


class SanaVideoMSBlock(nn.Module):
    """The block of Sana-Video (upstream's SanaVideoMSBlock, sana_multi_scale_video.py:65-333):
    modulate -> self-attention (``LiteLAReLURope`` or ``LiteLA``) -> gate + residual -> cross-attention
    + residual -> modulate -> Mix-FFN (``GLUMBConvTemp`` or ``GLUMBConv``) -> gate + residual, on a
    (T, H, W) token grid.  ``t`` is [B, 6C] (one modulation per sample) or [B, 1, F, 6C] (one per
    frame, upstream's forward_frame_aware).  Same constructor arguments and state-dict keys as
    upstream for the covered options."""

    def __init__(self, hidden_size, num_heads, mlp_ratio=4.0, drop_path=0.0, qk_norm=False, attn_type="flash",
                 ffn_type="mlp", mlp_acts=("silu", "silu", None), linear_head_dim=32, cross_norm=False,
                 cross_attn_image_embeds=False, t_kernel_size=3, additional_flash_attn=False,
                 flash_attn_window_count=None, **block_kwargs):
        super().__init__()
        attn_classes = {"linear": LiteLA, "LiteLAReLURope": LiteLAReLURope, "ChunkedLiteLAReLURope": ChunkedLiteLAReLURope,
                        "ChunkCausalAttention": ChunkCausalAttention, "CachedCausalAttention": CachedCausalAttention}
        # upstream's own names for the two autoregressive attentions are the lower-case ones
        attn_classes.update({"chunkcausal": ChunkCausalAttention, "cachedcausal": CachedCausalAttention})
        ffn_classes = {"glumbconv": GLUMBConv, "GLUMBConvTemp": GLUMBConvTemp, "ChunkGLUMBConvTemp": ChunkGLUMBConvTemp,
                       "CachedGLUMBConvTemp": CachedGLUMBConvTemp}
        if attn_type not in attn_classes or ffn_type not in ffn_classes:
            raise NotImplementedError(f"SanaVideoMSBlock here covers attn_type {sorted(attn_classes)} with ffn_type "
                                      f"{sorted(ffn_classes)}")
        if drop_path != 0.0 or cross_attn_image_embeds or additional_flash_attn:
            raise NotImplementedError("drop_path, image-embedding cross-attention and the additional softmax "
                                      "attention are not covered")
        self.hidden_size = hidden_size
        self.norm1 = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=LN_EPS)
        self.attn = attn_classes[attn_type](hidden_size, hidden_size, heads=hidden_size // linear_head_dim, eps=1e-8, qk_norm=qk_norm)
        self.flash_attn_additional = None
        self.cross_attn_image_embeds = False
        self.cross_attn = MultiHeadCrossAttention(hidden_size, num_heads, qk_norm=cross_norm, **block_kwargs)
        self.norm2 = nn.LayerNorm(hidden_size, elementwise_affine=False, eps=LN_EPS)
        ffn = dict(in_features=hidden_size, hidden_features=int(hidden_size * mlp_ratio), use_bias=(True, True, False),
                   norm=(None, None, None), act=mlp_acts)
        self.mlp = GLUMBConv(**ffn) if ffn_type == "glumbconv" else ffn_classes[ffn_type](t_kernel_size=t_kernel_size, **ffn)
        self.drop_path = nn.Identity()
        self.scale_shift_table = nn.Parameter(torch.randn(6, hidden_size) / hidden_size ** 0.5)
        self.block_hook = None

    def set_sequence_shard(self, shard: Optional[SequenceShard]) -> None:
        """Run this block on one rank's slice of the token grid (see sharding.SequenceShard): the partial
        attention states are summed over the ranks, the depthwise conv takes its halo rows from the
        neighbours, the temporal Mix-FFN one frame from each neighbour (every rank must then hold at least one
        frame's worth of rows; with one modulation vector per frame the cuts must lie between frames:
        ``SequenceShard(..., by_frames=True)``)."""
        if shard is not None and isinstance(self.mlp, CachedGLUMBConvTemp):
            raise NotImplementedError("the cached temporal Mix-FFN on a sequence shard is not covered")
        self.attn.seq_shard = shard
        self.mlp.seq_shard = shard

    @torch.no_grad()
    def forward(self, x, y, t, mask=None, THW=None, rotary_emb=None, chunk_index=None, **kwargs):
        kv_cache, save_kv_cache = kwargs.get("kv_cache"), bool(kwargs.get("save_kv_cache"))
        if chunk_index is not None and not isinstance(self.attn, ChunkCausalAttention):
            raise NotImplementedError("chunk_index needs attn_type 'ChunkCausalAttention'")
        plain_temporal = isinstance(self.mlp, GLUMBConvTemp) and not isinstance(self.mlp, CachedGLUMBConvTemp)
        if kv_cache is not None and (not isinstance(self.attn, CachedCausalAttention) or plain_temporal):
            raise NotImplementedError("kv_cache needs attn_type 'CachedCausalAttention' (and 'CachedGLUMBConvTemp' or "
                                      "'glumbconv' as ffn_type)")
        if self.block_hook is not None:
            raise NotImplementedError("block hooks are not covered")
        B, N, C = x.shape
        if t.dim() > 2:  # [B, 1, F, 6C]: one modulation per frame = per run of N / F tokens
            frames = t.shape[2]
            if N % frames:
                raise ValueError("the token count is not a multiple of the frame count of t")
            rows = N // frames
            sh = self.mlp.seq_shard
            held = None if THW is None else (THW[0] if sh is None else sh.rows // sh.H)  # frames in x
            if isinstance(self.mlp, GLUMBConvTemp) and frames != held:
                raise ValueError(f"t carries {frames} modulation vectors per sample but x holds "
                                 f"{held} frames: the temporal Mix-FFN needs one per frame")
        else:
            rows = N
        t2 = t.reshape(B * (N // rows), 6 * C)
        x2 = _as2d(x.contiguous())
        table = self.scale_shift_table
        attn, mlp, ca = self.attn, self.mlp, self.cross_attn
        z = ops.ln_modulate(x2.view(-1, rows, C), table, t2, 0, 1, LN_EPS)
        qkv = _project(attn, "qkv", _as2d(z), attn.qkv.weight, bias=attn.qkv.bias)
        if isinstance(attn, ChunkCausalAttention):
            o = attn._core(qkv, B, N, rotary_emb, HW=THW, chunk_index=[0] if chunk_index is None else list(chunk_index))
        elif isinstance(attn, CachedCausalAttention):
            o = attn._core_cached(qkv, B, N, rotary_emb, kv_cache, save_kv_cache)
        else:
            o = attn._core(qkv, B, N, rotary_emb)
        x2 = _project(attn, "proj", o, attn.proj.weight, bias=attn.proj.bias, gate=(table, t2, 2, rows), residual=x2)
        o = ca._attend(x2, y, mask, B, kwargs.get("caption_kv"))
        x2 = ops.gemm(o, ca.proj.weight, bias=ca.proj.bias, residual=x2)
        z = ops.ln_modulate(x2.view(-1, rows, C), table, t2, 3, 4, LN_EPS)
        if isinstance(mlp, GLUMBConvTemp):
            cached = isinstance(mlp, CachedGLUMBConvTemp) and kv_cache is not None
            x2 = mlp.forward_gated(z.view(B, N, C), THW, x2, table, t2, 5, rows, kv_cache=kv_cache if cached else None,
                                   save_kv_cache=save_kv_cache, chunk_index=chunk_index)
        else:
            u = mlp._expand(_as2d(z))
            g = mlp._depthwise_glu(u, B, N, THW)
            pc = mlp.point_conv.conv
            x2 = _project(mlp, "point_conv", g, pc.weight.reshape(pc.out_channels, pc.in_channels), bias=pc.bias,
                          gate=(table, t2, 5, rows), residual=x2)
        if kv_cache is not None:
            return x2.view(B, N, C), kv_cache
        return x2.view(B, N, C)


class BlockStack(nn.Module):
    """``depth`` SanaMSBlocks applied in sequence with a shared (y, t, mask, HW): the block loop
    of upstream's SanaMS.forward (diffusion/model/nets/sana_multi_scale.py:368-383)."""

    def __init__(self, hidden_size, num_heads, depth, mlp_ratio=2.5, **block_kwargs):
        super().__init__()
        self.blocks = nn.ModuleList([
            SanaMSBlock(hidden_size, num_heads, mlp_ratio=mlp_ratio, attn_type="linear", ffn_type="glumbconv",
                        **block_kwargs) for _ in range(depth)])

    def set_sequence_shard(self, shard: Optional[SequenceShard]) -> None:
        for b in self.blocks:
            b.set_sequence_shard(shard)

    def set_nvfp4(self, enabled: bool = True, delayed_scaling: bool = False, margin: float = 1.0) -> None:
        for b in self.blocks:
            b.set_nvfp4(enabled, delayed_scaling, margin)

    @torch.no_grad()
    def forward(self, x, y, t, mask=None, HW=None, **kwargs):
        for block in self.blocks:
            x = block(x, y, t, mask, HW, **kwargs)
        return x

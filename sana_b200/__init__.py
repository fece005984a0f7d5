"""sana_b200: the Sana Linear-DiT block (LiteLA + GLUMBConv inside SanaMSBlock) on B200.

CUDA kernels for sm_100a behind a C ABI (include/sana_b200.h, built into
sana_b200/lib/libsana_b200.so by ``python -m sana_b200.build``) and drop-in PyTorch modules
that keep upstream's signatures.  There is no CPU path.
"""
from . import checkpoint, graphs, ops, sharding, synthetic  # noqa: F401
from ._lib import SanaLibraryError, load as load_library  # noqa: F401
from .modules import (BlockStack, CachedCausalAttention, CachedGLUMBConvTemp, ChunkCausalAttention, ChunkGLUMBConvTemp, ChunkedLiteLAReLURope, ConvLayer, GLUMBConv, GLUMBConvTemp, LiteLA, LiteLAReLURope,  # noqa: F401
                      MultiHeadCrossAttention, RMSNorm, SanaMSBlock, SanaVideoMSBlock, wan_rotary_freqs)
from .checkpoint import load_checkpoint  # noqa: F401
from .weight_pack import load_nvfp4_weights, pack_nvfp4_weights  # noqa: F401
from .dit import CaptionEmbedder, PatchEmbedMS, SanaMS, T2IFinalLayer, TimestepEmbedder  # noqa: F401

__all__ = ["LiteLA", "LiteLAReLURope", "ChunkedLiteLAReLURope", "ChunkCausalAttention", "CachedCausalAttention", "CachedGLUMBConvTemp", "ChunkGLUMBConvTemp", "wan_rotary_freqs", "GLUMBConv", "GLUMBConvTemp", "ConvLayer", "MultiHeadCrossAttention", "SanaMSBlock", "SanaVideoMSBlock", "BlockStack", "RMSNorm",
           "SanaMS", "pack_nvfp4_weights", "load_nvfp4_weights", "PatchEmbedMS", "TimestepEmbedder", "CaptionEmbedder", "T2IFinalLayer", "ops",
           "sharding", "synthetic", "checkpoint", "load_checkpoint", "load_library", "SanaLibraryError"]

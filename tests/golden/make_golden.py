"""Generates tests/golden/*.pt by running the UNMODIFIED upstream modules on CPU.

Run on a machine with a checkout of NVlabs/Sana:

    python tests/golden/make_golden.py --ref <checkout of NVlabs/Sana>   (or SANA_REFERENCE=<checkout>)

Each fixture stores the seeded inputs, the parameters (upstream state-dict keys) and the
outputs of upstream's LiteLA / GLUMBConv / SanaMSBlock forward, in fp32 and (for the block)
bf16, at shapes small enough to commit (a few hundred KB in total).  Full-size
configurations are pinned through sub-sampled outputs: the inputs are regenerated from the
seed by sana_b200.synthetic, only every `stride`-th token row of the output is stored.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from ref_loader import load_reference, load_video_module, set_fp32_attention  # noqa: E402

from sana_b200 import synthetic  # noqa: E402


def _block(R, C, heads, params, dtype):
    qk = "attn.q_norm.weight" in params
    blk = R.SanaMSBlock(C, heads, mlp_ratio=2.5, attn_type="linear", ffn_type="glumbconv", qk_norm=qk,
                        cross_norm=qk).eval()
    blk.load_state_dict(params, strict=True)
    set_fp32_attention(blk)
    return blk.to(dtype)


def small_block_case(R, name, C, heads, B, HW, L, seed, with_mask=False, qk_norm=False, rope=False):
    hid = int(C * 2.5)
    shape = synthetic.BlockShape(name, C, heads, B, tuple(HW), text_len=L)
    params = synthetic.make_block_params(C, hid, seed, std=0.05)
    if qk_norm:  # learned RMSNorm weights on q / k of both attentions (qk_norm=True, cross_norm=True)
        g = torch.Generator().manual_seed(1000 + seed)
        for k in ("attn.q_norm.weight", "attn.k_norm.weight", "cross_attn.q_norm.weight", "cross_attn.k_norm.weight"):
            params[k] = 1.0 + 0.2 * torch.randn(C, generator=g)
    x, y, t = synthetic.make_block_inputs(shape, seed=seed, std=0.05, text_dim=96)
    mask = None
    if with_mask:
        mask = torch.ones(B, L)
        for b in range(B):
            mask[b, L - 1 - b:] = 0
    out = {"C": C, "heads": heads, "B": B, "HW": tuple(HW), "L": L, "params": params, "x": x, "y": y, "t": t,
           "mask": mask}
    rot = None
    if rope:  # per-position rotation tables [N, 32] (any angles; pairs need not share an angle upstream)
        g = torch.Generator().manual_seed(2000 + seed)
        ang = torch.rand(shape.tokens, 32, generator=g) * 6.28
        rot = (torch.cos(ang), torch.sin(ang))
        out["rope_cos"], out["rope_sin"] = rot
    with torch.no_grad():
        for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            blk = _block(R, C, heads, params, dt)
            xx, yy, tt = x.to(dt), y.to(dt), t.to(dt)
            # branch outputs: what LiteLA.forward / GLUMBConv.forward return inside the block
            mod = (blk.scale_shift_table[None] + tt.reshape(B, 6, -1)).chunk(6, dim=1)
            z1 = R.t2i_modulate(blk.norm1(xx), mod[0], mod[1])
            out[f"attn_in_{tag}"] = z1
            out[f"attn_out_{tag}"] = blk.attn(z1, HW=tuple(HW), rotary_emb=rot)
            out[f"mlp_out_{tag}"] = blk.mlp(z1, HW=tuple(HW))  # GLUMBConv on the same modulated input
            out[f"cross_out_{tag}"] = blk.cross_attn(xx, yy, mask)
            out[f"block_out_{tag}"] = blk(xx, yy, tt, mask, tuple(HW), rot)
    return out


def litela_cfg1_case(R, stride=64):
    x, p = synthetic.make_litela_cfg1(seed=0)
    C = x.shape[-1]
    m = R.LiteLA(C, C, heads=C // 32, eps=1e-8).eval()
    m.load_state_dict(p, strict=True)
    set_fp32_attention(m)
    with torch.no_grad():
        o32 = m(x, HW=(32, 32))
        m64 = m.double()
        # fp64 golden: upstream's .float() inside attn_matmul is bypassed by clearing the flag
        for mod in m64.modules():
            mod.fp32_attention = False
        o64 = m64(x.double(), HW=(32, 32))
    return {"stride": stride, "out_f32_rows": o32[:, ::stride].clone(), "out_f64_rows": o64[:, ::stride].clone(),
            "out_f32_absmax": o32.abs().max().item(), "out_f32_sum": o32.double().sum().item()}


def block_cfg2_case(R, stride=256):
    shp = synthetic.CFG2
    C, hid = shp.hidden, shp.ffn_hidden
    params = synthetic.make_block_params(C, hid, seed=0)
    x, y, t = synthetic.make_block_inputs(shp, seed=0)
    out = {"stride": stride}
    with torch.no_grad():
        # golden: fp32 math on the bf16-rounded tensors; native: upstream run in bf16
        pb = {k: v.bfloat16() for k, v in params.items()}
        xb, yb, tb = x.bfloat16(), y.bfloat16(), t.bfloat16()
        blk = _block(R, C, shp.cross_heads, {k: v.float() for k, v in pb.items()}, torch.float32)
        xx, yy, tt = xb.float(), yb.float(), tb.float()
        mod = (blk.scale_shift_table[None] + tt.reshape(shp.batch, 6, -1)).chunk(6, dim=1)
        z1 = R.t2i_modulate(blk.norm1(xx), mod[0], mod[1]).bfloat16().float()
        out["attn_in_rows"] = z1[:, ::stride].clone()
        out["attn_out_golden_rows"] = blk.attn(z1, HW=shp.grid)[:, ::stride].clone()
        out["mlp_out_golden_rows"] = blk.mlp(z1, HW=shp.grid)[:, ::stride].clone()
        full = blk(xx, yy, tt, None, shp.grid)
        out["block_out_golden_rows"] = full[:, ::stride].clone()
        out["block_out_golden_absmax"] = full.abs().max().item()
        blk16 = _block(R, C, shp.cross_heads, pb, torch.bfloat16)
        full16 = blk16(xb, yb, tb, None, shp.grid)
        out["block_out_bf16_rows"] = full16[:, ::stride].clone()
    return out


def video_case(R, seed=3):
    """3-tuple HW (per-frame depthwise conv), small."""
    return small_block_case(R, "video", 64, 4, 1, (3, 5, 8), 7, seed)


def pag_case(R, seed=8):
    """Upstream's two perturbed-attention-guidance processors on a LiteLA (eps of the block)."""
    C, N = 64, 30
    g = torch.Generator().manual_seed(seed)
    params = {k[len("attn."):]: v for k, v in synthetic.make_block_params(C, 160, seed, std=0.05).items()
              if k.startswith("attn.")}
    x = torch.randn(6, N, C, generator=g) * 0.5
    out = {"C": C, "params": params, "x": x}
    with torch.no_grad():
        for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            m = R.LiteLA(C, C, heads=C // 32, eps=1e-8).eval()
            m.load_state_dict(params, strict=True)
            set_fp32_attention(m)
            m = m.to(dt)
            out[f"pag_{tag}"] = R.sana_blocks.PAGIdentitySelfAttnProcessorLiteLA(m)(x.to(dt))
            out[f"pagcfg_{tag}"] = R.sana_blocks.PAGCFGIdentitySelfAttnProcessorLiteLA(m)(x.to(dt))
    return out


def glumbconv_temp_case(R, seed=9):
    """Upstream's GLUMBConvTemp (video Mix-FFN) on 3 frames of 5 x 8 tokens, two samples."""
    C, hid, HW, B = 64, 160, (3, 5, 8), 2
    g = torch.Generator().manual_seed(seed)
    params = {k[len("mlp."):]: v for k, v in synthetic.make_block_params(C, hid, seed, std=0.05).items()
              if k.startswith("mlp.")}
    params["t_conv.weight"] = torch.randn(C, C, 3, 1, generator=g) * 0.05
    x = torch.randn(B, HW[0] * HW[1] * HW[2], C, generator=g) * 0.5
    out = {"C": C, "hid": hid, "HW": HW, "params": params, "x": x}
    with torch.no_grad():
        for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            m = R.basic_modules.GLUMBConvTemp(in_features=C, hidden_features=hid, use_bias=(True, True, False),
                                              norm=(None, None, None), act=("silu", "silu", None)).eval()
            m.load_state_dict(params, strict=True)
            out[f"out_{tag}"] = m.to(dt)(x.to(dt), HW=HW)
    return out


def litela_relu_rope_case(R, seed=11):
    """Upstream's LiteLAReLURope (Sana-Video self-attention: ReLU, then a complex rotation of the
    numerator's q and k) with WanRotaryPosEmbed frequencies; heads of 48 channels, with and
    without qk_norm."""
    C, heads, fhw, B = 96, 2, (2, 3, 5), 2
    N = fhw[0] * fhw[1] * fhw[2]
    g = torch.Generator().manual_seed(seed)
    params = {"qkv.weight": torch.randn(3 * C, C, generator=g) * 0.08,
              "proj.weight": torch.randn(C, C, generator=g) * 0.08,
              "proj.bias": torch.randn(C, generator=g) * 0.05}
    norm = {"q_norm.weight": 1.0 + 0.1 * torch.randn(C, generator=g),
            "k_norm.weight": 1.0 + 0.1 * torch.randn(C, generator=g)}
    x = torch.randn(B, N, C, generator=g) * 0.7
    rope = R.sana_blocks.WanRotaryPosEmbed(attention_head_dim=C // heads, patch_size=(1, 1, 1), max_seq_len=1024)
    freqs = rope(fhw, torch.device("cpu"))
    out = {"C": C, "heads": heads, "fhw": fhw, "params": params, "norm_params": norm, "x": x, "freqs": freqs}
    with torch.no_grad():
        for qk_norm, tag_n in ((False, ""), (True, "_qknorm")):
            for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
                m = R.sana_blocks.LiteLAReLURope(C, C, heads=heads, eps=1e-8, qk_norm=qk_norm).eval()
                m.load_state_dict({**params, **(norm if qk_norm else {})}, strict=True)
                out[f"out{tag_n}_{tag}"] = m.to(dt)(x.to(dt), rotary_emb=freqs)
    return out


def causal_video_case(R, seed=13):
    """Upstream's autoregressive variants of the Sana-Video block parts: ChunkCausalAttention (frames cut into
    chunks, state cumulative over chunks) with its Mix-FFN ChunkGLUMBConvTemp, CachedCausalAttention and
    CachedGLUMBConvTemp (one chunk per call, the state of the previous chunk handed over in a cache list)."""
    C, heads, fhw, B, hid = 96, 2, (4, 3, 5), 2, 240
    hw = fhw[1] * fhw[2]
    N = fhw[0] * hw
    g = torch.Generator().manual_seed(seed)
    params = {"qkv.weight": torch.randn(3 * C, C, generator=g) * 0.08,
              "proj.weight": torch.randn(C, C, generator=g) * 0.08,
              "proj.bias": torch.randn(C, generator=g) * 0.05}
    mlp = {k[len("mlp."):]: v for k, v in synthetic.make_block_params(C, hid, seed, std=0.05).items() if k.startswith("mlp.")}
    mlp["t_conv.weight"] = torch.randn(C, C, 3, 1, generator=g) * 0.05
    x = torch.randn(B, N, C, generator=g) * 0.7
    rope = R.sana_blocks.WanRotaryPosEmbed(attention_head_dim=C // heads, patch_size=(1, 1, 1), max_seq_len=1024)
    freqs = rope(fhw, torch.device("cpu"))
    chunk_index = [0, 1, 3]  # chunks of 1, 2 and 1 frames
    out = {"C": C, "heads": heads, "fhw": fhw, "hid": hid, "params": params, "mlp_params": mlp, "x": x, "freqs": freqs,
           "chunk_index": chunk_index}
    with torch.no_grad():
        for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            m = R.sana_blocks.ChunkCausalAttention(C, C, heads=heads, eps=1e-8).eval()
            m.load_state_dict(params, strict=True)
            out[f"chunk_{tag}"] = m.to(dt)(x.to(dt), HW=fhw, rotary_emb=freqs, chunk_index=list(chunk_index))
            cf = R.basic_modules.ChunkGLUMBConvTemp(in_features=C, hidden_features=hid, use_bias=(True, True, False),
                                                    norm=(None, None, None), act=("silu", "silu", None)).eval()
            cf.load_state_dict(mlp, strict=True)
            out[f"chunk_ffn_{tag}"] = cf.to(dt)(x.to(dt), HW=fhw, chunk_index=list(chunk_index))
            # two calls of two frames each: the second sees the first one's state through the cache
            m = R.sana_blocks.CachedCausalAttention(C, C, heads=heads, eps=1e-8).eval()
            m.load_state_dict(params, strict=True)
            m = m.to(dt)
            f = R.basic_modules.CachedGLUMBConvTemp(in_features=C, hidden_features=hid, use_bias=(True, True, False),
                                                    norm=(None, None, None), act=("silu", "silu", None)).eval()
            f.load_state_dict(mlp, strict=True)
            f = f.to(dt)
            cache = [None, None, None]
            half, fr = 2 * hw, freqs.reshape(1, 1, N, -1)
            for i in range(2):
                xs = x[:, i * half:(i + 1) * half].to(dt)
                o, cache = m(xs, HW=(2, fhw[1], fhw[2]), rotary_emb=fr[:, :, i * half:(i + 1) * half], save_kv_cache=True,
                             kv_cache=cache)
                out[f"cached_attn{i}_{tag}"] = o
                o, cache = f(xs, HW=(2, fhw[1], fhw[2]), save_kv_cache=True, kv_cache=cache)
                out[f"cached_ffn{i}_{tag}"] = o
    return out


def video_block_case(ref_root, R, seed=12):
    """Upstream's SanaVideoMSBlock (LiteLAReLURope + cross-attention + GLUMBConvTemp) on 3 frames of
    4 x 5 tokens, with one modulation per sample and with one per frame."""
    V = load_video_module(ref_root)
    C, heads, lin_dim, hid, THW, B, L = 96, 2, 48, 240, (3, 4, 5), 2, 7
    N = THW[0] * THW[1] * THW[2]
    g = torch.Generator().manual_seed(seed)
    params = synthetic.make_block_params(C, hid, seed, std=0.06)
    params["mlp.t_conv.weight"] = torch.randn(C, C, 3, 1, generator=g) * 0.05
    x = torch.randn(B, N, C, generator=g) * 0.7
    y = torch.randn(B, L, C, generator=g) * 0.7
    t = torch.randn(B, 6 * C, generator=g) * 0.3
    t_frames = torch.randn(B, 1, THW[0], 6 * C, generator=g) * 0.3
    mask = torch.ones(B, L)
    mask[1, 5:] = 0
    rope = R.sana_blocks.WanRotaryPosEmbed(attention_head_dim=lin_dim, patch_size=(1, 1, 1), max_seq_len=1024)
    freqs = rope(THW, torch.device("cpu"))
    # the block parameters are regenerated from the seed (sana_b200.synthetic.make_block_params); only t_conv is stored
    out = {"C": C, "heads": heads, "linear_head_dim": lin_dim, "hid": hid, "THW": THW, "param_seed": seed, "param_std": 0.06,
           "t_conv": params["mlp.t_conv.weight"], "x": x, "y": y, "t": t, "t_frames": t_frames, "mask": mask, "freqs": freqs}
    with torch.no_grad():
        for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            m = V.SanaVideoMSBlock(C, heads, mlp_ratio=hid / C, attn_type="LiteLAReLURope", ffn_type="GLUMBConvTemp",
                                   linear_head_dim=lin_dim).eval()
            m.load_state_dict(params, strict=True)
            m = m.to(dt)
            out[f"out_{tag}"] = m(x.to(dt), y.to(dt), t.to(dt), mask=mask, THW=THW, rotary_emb=freqs)
            out[f"out_frames_{tag}"] = m(x.to(dt), y.to(dt), t_frames.to(dt), mask=mask, THW=THW, rotary_emb=freqs)
    return out


def final_layer_case(R, seed=10):
    """Upstream's T2IFinalLayer with one modulation vector per sample and per frame."""
    C, B, Fr, P = 64, 2, 3, 10
    g = torch.Generator().manual_seed(seed)
    m = R.sana_blocks.T2IFinalLayer(C, 1, 32).eval()
    params = {k: torch.randn(v.shape, generator=g) * 0.2 for k, v in m.state_dict().items()}
    m.load_state_dict(params, strict=True)
    x = torch.randn(B, Fr * P, C, generator=g)
    t = torch.randn(B, C, generator=g) * 0.3
    tf = torch.randn(B, 1, Fr, C, generator=g) * 0.3
    with torch.no_grad():
        return {"C": C, "params": params, "x": x, "t": t, "t_frames": tf, "out": m(x, t), "out_frames": m(x, tf)}


SANA_MS_SMALL = dict(input_size=8, patch_size=1, in_channels=32, hidden_size=64, depth=2, num_heads=2, mlp_ratio=2.5,
                     class_dropout_prob=0.0, pred_sigma=False, caption_channels=48, model_max_length=10, y_norm=True,
                     attn_type="linear", ffn_type="glumbconv", mlp_acts=("silu", "silu", None), linear_head_dim=32,
                     use_pe=True, norm_eps=1e-5, y_norm_scale_factor=0.01)


def sana_ms_case(R, seed=5):
    """The whole SanaMS.forward of a two-block model on a 6 x 8 latent (non-square on purpose:
    the position table depends on the h / w order), every parameter drawn at random so that no
    zero-initialised projection hides an error.  Stores the inputs, the state dict and the output
    in fp32 and bf16."""
    cfg = dict(SANA_MS_SMALL)
    g = torch.Generator().manual_seed(seed)
    m = R.sana_multi_scale.SanaMS(**cfg, use_fp32_attention=True).eval()
    sd = m.state_dict()
    params = {}
    for k, v in sd.items():
        if k == "pos_embed":
            params[k] = v.clone()  # unused buffer of the base class at a fixed size
        elif k.endswith("norm.weight") or k.endswith("attention_y_norm.weight"):
            params[k] = v + 0.2 * v * torch.randn(v.shape, generator=g)
        elif k == "y_embedder.y_embedding":
            params[k] = v.clone()
        else:
            params[k] = torch.randn(v.shape, generator=g) * (0.3 if v.dim() == 1 else 1.5 / v[0].numel() ** 0.5)
    B, L = 2, 10
    x = torch.randn(B, 32, 6, 8, generator=g)
    timestep = torch.tensor([37.0, 912.0])
    y = torch.randn(B, 1, L, 48, generator=g)
    mask = torch.ones(B, L, dtype=torch.int64)
    mask[1, 6:] = 0
    out = {"cfg": cfg, "params": params, "x": x, "timestep": timestep, "y": y, "mask": mask}
    with torch.no_grad():
        for dt, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            m.load_state_dict(params, strict=True)
            set_fp32_attention(m)
            mm = m.to(dt)
            mm.pos_embed_ms = None  # upstream caches the position table by shape only, not by dtype
            out[f"out_{tag}"] = mm(x, timestep, y, mask=mask)
            out[f"out_nomask_{tag}"] = mm(x, timestep, y, mask=torch.ones(B, L, dtype=torch.int64))
            m = m.float()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("SANA_REFERENCE"), required="SANA_REFERENCE" not in os.environ,
                    help="checkout of NVlabs/Sana")
    ap.add_argument("--only", default=None, help="regenerate just this fixture")
    a = ap.parse_args()
    torch.manual_seed(0)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    R = load_reference(a.ref)
    makers = {
        "small_block_a": lambda: small_block_case(R, "a", 64, 4, 2, (6, 5), 9, seed=1),
        "small_block_masked": lambda: small_block_case(R, "m", 64, 2, 2, (4, 7), 11, seed=2, with_mask=True),
        "small_block_video": lambda: video_case(R),
        "small_block_qknorm": lambda: small_block_case(R, "q", 64, 4, 2, (5, 6), 8, seed=4, with_mask=True, qk_norm=True),
        "small_block_rope": lambda: small_block_case(R, "r", 64, 4, 2, (4, 6), 8, seed=6, rope=True),
        "litela_cfg1": lambda: litela_cfg1_case(R),
        "block_cfg2": lambda: block_cfg2_case(R),
        "sana_ms_small": lambda: sana_ms_case(R),
        "pag_litela": lambda: pag_case(R),
        "glumbconv_temp": lambda: glumbconv_temp_case(R),
        "final_layer": lambda: final_layer_case(R),
        "litela_relu_rope": lambda: litela_relu_rope_case(R),
        "video_block": lambda: video_block_case(a.ref, R),
        "causal_video": lambda: causal_video_case(R),
    }
    cases = {k: mk() for k, mk in makers.items() if a.only in (None, k)}
    for name, c in cases.items():
        path = os.path.join(HERE, name + ".pt")
        torch.save(c, path)
        print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB")


if __name__ == "__main__":
    main()

"""SDXL UNet (eps-prediction), channels-last convolutions through cuDNN and transformer blocks
through the fused ops.

Configuration (src/models/sdxl_unet_complete.rs:53-93; crates/training/src/sdxl/keymap.rs:6-77):
block channels (320, 640, 1280), transformer depth per level (0, 2, 10), head_dim 64,
cross-attention width 2048, GroupNorm 32, ``text_time`` additional embedding (pooled 1280 + six
256-d sinusoidal size/crop ids = 2816 -> 1280), 70 transformer blocks in total. A transformer block
is LN -> self-attn -> LN -> cross-attn -> LN -> GEGLU feed-forward with residuals, wrapped by
proj_in / proj_out (crates/training/src/sdxl/runtime.rs:1393-1565); conditioning assembly follows
crates/training/src/conditioning/make_conditioning.rs:4-25 and time_ids.rs:9.
Convolutions stay a library call (cuDNN), as in the reference (cudnn-sys).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F
from .layers import Linear, timestep_embedding
from .registry import register_model


@dataclass
class SDXLConfig:
    in_channels: int = 4
    out_channels: int = 4
    block_channels: tuple = (320, 640, 1280)
    transformer_depth: tuple = (0, 2, 10)
    layers_per_block: int = 2
    head_dim: int = 64
    context_dim: int = 2048
    groups: int = 32
    addition_time_embed_dim: int = 256
    pooled_dim: int = 1280                  # 0: no additional (pooled text + size ids) embedding
    num_heads: int | None = None            # set: a fixed head count per level instead of a fixed head size
    mid_transformer_depth: int | None = None   # default: the last level's depth


# Stable Diffusion 1.5: four levels, one transformer block per attention level (none at the deepest),
# 8 heads at every width, CLIP-L context (768), no pooled / size conditioning
# (crates/training/src/pipelines/sd15_pipeline.rs:12-275; src/models/unet_2d.rs).
SD15_CONFIG = dict(block_channels=(320, 640, 1280, 1280), transformer_depth=(1, 1, 1, 0), context_dim=768,
                   num_heads=8, pooled_dim=0, mid_transformer_depth=1)


class LayerNormAffine(nn.Module):
    def __init__(self, dim, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device))

    def forward(self, x):
        return F.norm_modulate(x, weight=self.weight, bias=self.bias, eps=1e-5)


class CrossAttention(nn.Module):
    def __init__(self, dim, ctx_dim, head_dim, dtype, device):
        super().__init__()
        self.heads = dim // head_dim
        self.self_attn = ctx_dim is None
        if self.self_attn:
            self.to_qkv = Linear(dim, 3 * dim, bias=False, dtype=dtype, device=device)
        else:
            self.to_q = Linear(dim, dim, bias=False, dtype=dtype, device=device)
            self.to_kv = Linear(ctx_dim, 2 * dim, bias=False, dtype=dtype, device=device)
        self.to_out = Linear(dim, dim, dtype=dtype, device=device)

    def forward(self, x, ctx=None, residual=None):
        B, L, D = x.shape
        H = self.heads
        if self.self_attn:
            q, k, v = F.qknorm_rope(self.to_qkv(x), None, None, None, None, H)
        else:
            q = self.to_q(x).view(B, L, H, D // H)
            kv = self.to_kv(ctx).view(B, ctx.shape[1], 2, H, D // H)
            k, v = kv[:, :, 0].contiguous(), kv[:, :, 1].contiguous()
        o = F.attention(q, k, v).reshape(B, L, D)
        return self.to_out(o, residual=residual)


class BasicTransformerBlock(nn.Module):
    def __init__(self, dim, ctx_dim, head_dim, dtype, device):
        super().__init__()
        self.norm1 = LayerNormAffine(dim, dtype, device)
        self.attn1 = CrossAttention(dim, None, head_dim, dtype, device)
        self.norm2 = LayerNormAffine(dim, dtype, device)
        self.attn2 = CrossAttention(dim, ctx_dim, head_dim, dtype, device)
        self.norm3 = LayerNormAffine(dim, dtype, device)
        self.ff_in = Linear(dim, 8 * dim, dtype=dtype, device=device)       # GEGLU: [act | gate]
        self.ff_out = Linear(4 * dim, dim, dtype=dtype, device=device)

    def forward(self, x, ctx):
        x = self.attn1(self.norm1(x), residual=x)
        x = self.attn2(self.norm2(x), ctx, residual=x)
        h = F.linear_glu(self.norm3(x), self.ff_in, "gelu", act_first=False)       # value * gelu(gate)
        return self.ff_out(h, residual=x)


class GroupNormAct(nn.GroupNorm):
    """``nn.GroupNorm`` parameters (same state-dict keys) with the channels-last GroupNorm(+SiLU)
    kernel as the forward; the result keeps the input's NCHW shape in channels-last format, which
    is what the cuDNN convolutions that follow want."""

    def __init__(self, groups, ch, eps, silu, dtype=None, device=None):
        super().__init__(groups, ch, eps=eps, dtype=dtype, device=device)
        self.silu = silu

    def forward(self, x):
        return F.group_norm_silu(x, self.weight, self.bias, self.num_groups, self.eps, self.silu)


class Transformer2D(nn.Module):
    def __init__(self, ch, depth, cfg: SDXLConfig, dtype, device):
        super().__init__()
        self.norm = GroupNormAct(cfg.groups, ch, 1e-6, False, dtype=dtype, device=device)
        self.proj_in = Linear(ch, ch, dtype=dtype, device=device)
        head_dim = ch // cfg.num_heads if cfg.num_heads else cfg.head_dim
        self.blocks = nn.ModuleList(BasicTransformerBlock(ch, cfg.context_dim, head_dim, dtype, device)
                                    for _ in range(depth))
        self.proj_out = Linear(ch, ch, dtype=dtype, device=device)

    def forward(self, x, ctx):
        B, C, H, W = x.shape
        h = self.norm(x).permute(0, 2, 3, 1).reshape(B, H * W, C)            # NHWC tokens
        h = self.proj_in(h)
        for blk in self.blocks:
            h = blk(h, ctx)
        h = self.proj_out(h)
        return x + h.view(B, H, W, C).permute(0, 3, 1, 2)


class ResBlock(nn.Module):
    def __init__(self, cin, cout, temb, cfg, dtype, device):
        super().__init__()
        self.norm1 = GroupNormAct(cfg.groups, cin, 1e-5, True, dtype=dtype, device=device)
        self.conv1 = nn.Conv2d(cin, cout, 3, padding=1, dtype=dtype, device=device)
        self.temb = nn.Linear(temb, cout, dtype=dtype, device=device)
        self.norm2 = GroupNormAct(cfg.groups, cout, 1e-5, True, dtype=dtype, device=device)
        self.conv2 = nn.Conv2d(cout, cout, 3, padding=1, dtype=dtype, device=device)
        self.skip = nn.Conv2d(cin, cout, 1, dtype=dtype, device=device) if cin != cout else None

    def forward(self, x, emb):
        h = self.conv1(self.norm1(x))                                       # GroupNorm + SiLU fused
        h = h + self.temb(TF.silu(emb))[:, :, None, None]
        h = self.conv2(self.norm2(h))
        return (x if self.skip is None else self.skip(x)) + h


class SDXLUNet(nn.Module):
    def __init__(self, cfg: SDXLConfig = SDXLConfig(), dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        ch = cfg.block_channels
        te = ch[0] * 4
        kw = dict(dtype=dtype, device=device)
        self.time_embed = nn.Sequential(nn.Linear(ch[0], te, **kw), nn.SiLU(), nn.Linear(te, te, **kw))
        add_in = cfg.pooled_dim + 6 * cfg.addition_time_embed_dim
        self.add_embed = nn.Sequential(nn.Linear(add_in, te, **kw), nn.SiLU(), nn.Linear(te, te, **kw)) \
            if cfg.pooled_dim else None
        self.conv_in = nn.Conv2d(cfg.in_channels, ch[0], 3, padding=1, **kw)
        self.down = nn.ModuleList()
        self.down_kinds = []
        skips = [ch[0]]
        cin = ch[0]
        for lvl, c in enumerate(ch):
            for _ in range(cfg.layers_per_block):
                self.down.append(nn.ModuleList([ResBlock(cin, c, te, cfg, dtype, device),
                                                Transformer2D(c, cfg.transformer_depth[lvl], cfg, dtype, device)
                                                if cfg.transformer_depth[lvl] else nn.Identity()]))
                self.down_kinds.append("block")
                cin = c
                skips.append(c)
            if lvl < len(ch) - 1:
                self.down.append(nn.Conv2d(c, c, 3, stride=2, padding=1, **kw))
                self.down_kinds.append("down")
                skips.append(c)
        mid_depth = cfg.transformer_depth[-1] if cfg.mid_transformer_depth is None else cfg.mid_transformer_depth
        self.mid = nn.ModuleList([ResBlock(cin, cin, te, cfg, dtype, device),
                                  Transformer2D(cin, mid_depth, cfg, dtype, device),
                                  ResBlock(cin, cin, te, cfg, dtype, device)])
        self.up = nn.ModuleList()
        self.up_kinds = []
        for lvl in reversed(range(len(ch))):
            c = ch[lvl]
            for i in range(cfg.layers_per_block + 1):
                sk = skips.pop()
                self.up.append(nn.ModuleList([ResBlock(cin + sk, c, te, cfg, dtype, device),
                                              Transformer2D(c, cfg.transformer_depth[lvl], cfg, dtype, device)
                                              if cfg.transformer_depth[lvl] else nn.Identity()]))
                self.up_kinds.append("block")
                cin = c
            if lvl > 0:
                self.up.append(nn.Conv2d(c, c, 3, padding=1, **kw))
                self.up_kinds.append("up")
        self.norm_out = GroupNormAct(cfg.groups, ch[0], 1e-5, True, **kw)
        self.conv_out = nn.Conv2d(ch[0], cfg.out_channels, 3, padding=1, **kw)

    def conditioning(self, t, pooled, time_ids):
        """emb = time_mlp(sin(t)) + add_mlp([pooled | sin(time_ids)]) (2816 -> 1280)."""
        cfg = self.cfg
        dt = self.conv_in.weight.dtype
        temb = self.time_embed(timestep_embedding(t, cfg.block_channels[0], time_factor=1.0).to(dt))
        if self.add_embed is None:
            return temb
        ids = timestep_embedding(time_ids.flatten(), cfg.addition_time_embed_dim, time_factor=1.0)
        ids = ids.view(time_ids.shape[0], -1).to(dt)
        return temb + self.add_embed(torch.cat([pooled.to(dt), ids], dim=-1))

    def encode(self, x, emb, ctx, adapter_features=None):
        """conv_in + down path + middle: returns (mid, skips). ``adapter_features`` (T2I-Adapter):
        one tensor per resolution level, added to the last feature of that level."""
        h = self.conv_in(x.contiguous(memory_format=torch.channels_last))
        hs = [h]
        level, in_level = 0, 0
        per_level = self.cfg.layers_per_block
        for kind, m in zip(self.down_kinds, self.down):
            if kind == "down":
                h = m(h)
                level, in_level = level + 1, 0
            else:
                h = m[0](h, emb)
                h = m[1](h, ctx) if not isinstance(m[1], nn.Identity) else h
                in_level += 1
                if adapter_features is not None and in_level == per_level and level < len(adapter_features):
                    h = h + adapter_features[level].to(h.dtype)
            hs.append(h)
        h = self.mid[0](h, emb)
        h = self.mid[1](h, ctx)
        h = self.mid[2](h, emb)
        return h, hs

    def forward(self, x, t, ctx, pooled=None, time_ids=None, control=None, adapter_features=None):
        """x [B, 4, H, W]; t [B] timesteps (0..999); ctx [B, 77, 2048]; pooled [B, 1280];
        time_ids [B, 6] = (orig_h, orig_w, crop_y, crop_x, tgt_h, tgt_w). ``control`` =
        (skip residuals, mid residual) from a ControlNet; ``adapter_features`` from a T2I-Adapter."""
        emb = self.conditioning(t, pooled, time_ids)
        h, hs = self.encode(x, emb, ctx, adapter_features)
        if control is not None:
            down_res, mid_res = control
            hs = [a + r.to(a.dtype) for a, r in zip(hs, down_res)]
            h = h + mid_res.to(h.dtype)
        for kind, m in zip(self.up_kinds, self.up):
            if kind == "up":
                h = m(TF.interpolate(h, scale_factor=2.0, mode="nearest"))
            else:
                h = m[0](torch.cat([h, hs.pop()], dim=1), emb)
                h = m[1](h, ctx) if not isinstance(m[1], nn.Identity) else h
        return self.conv_out(self.norm_out(h))

    def lora_targets(self):
        return [r"\.attn[12]\.(to_qkv|to_q|to_kv|to_out)$", r"\.ff_(in|out)$"]

    def num_transformer_blocks(self):
        return sum(1 for m in self.modules() if isinstance(m, BasicTransformerBlock))


def sdxl_forward(model, xt, t, batch, cfg):
    """Trainer forward hook for the UNet (latents are not patchified: trainer patch = 1 gives
    [B, H*W, C] tokens, which are folded back to NCHW here)."""
    B, L, C = xt.shape
    hh = batch["latents"].shape[-2]
    x = xt.view(B, hh, L // hh, C).permute(0, 3, 1, 2)
    out = model(x, t, batch["txt"], batch.get("pooled"), batch.get("time_ids"))
    return out.permute(0, 2, 3, 1).reshape(B, L, C)


@register_model("sdxl")
def build_sdxl(dtype=torch.bfloat16, device=None, **overrides):
    cfg = SDXLConfig(**{**SDXLConfig().__dict__, **overrides})
    return SDXLUNet(cfg, dtype=dtype, device=device)


@register_model("sd15")
def build_sd15(dtype=torch.bfloat16, device=None, **overrides):
    cfg = SDXLConfig(**{**SDXLConfig().__dict__, **SD15_CONFIG, **overrides})
    return SDXLUNet(cfg, dtype=dtype, device=device)

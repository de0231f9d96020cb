"""Auxiliary conditioning networks: ControlNet, IP-Adapter, T2I-Adapter and the Flux control-latent
concatenation.

Reference: crates/networks/src/controlnet.rs (``ControlNetConfig`` :13-25, ``process_conditioning``
:375, ``apply_control`` :416 with ``conditioning_scale`` and ``global_pool_conditions``),
ip_adapter.rs (``IPAdapterConfig`` :13-24 with the plus / full / faceid variants, decoupled image
cross-attention :313), t2i_adapter.rs (``T2IAdapterConfig`` :13-20, ``extract_features`` :301,
``apply_features`` :331) and crates/training/src/pipelines/flux_pipeline.rs:278-294 (control
latents concatenated on the channel dimension, 16 + 16). The reference modules are partial
(adapter forwards exist, wiring into the UNet does not); here they plug into ``SDXLUNet``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..models.layers import Linear, timestep_embedding
from ..ops import functional as F


# ----------------------------------------------------------------------------- ControlNet
@dataclass
class ControlNetConfig:
    conditioning_channels: int = 3
    conditioning_embedding_channels: tuple = (16, 32, 96, 256)
    conditioning_scale: float = 1.0
    global_pool_conditions: bool = False


class ControlNet(nn.Module):
    """A trainable copy of the UNet encoder plus zero-initialised 1x1 output convolutions; the
    hint image enters through a small strided conv stack and is added after ``conv_in``."""

    def __init__(self, unet, cfg: ControlNetConfig = ControlNetConfig()):
        super().__init__()
        self.cfg = cfg
        p = unet.conv_in.weight
        kw = dict(dtype=p.dtype, device=p.device)
        self.unet_cfg = unet.cfg
        # encoder copy (shares nothing with the base UNet after construction)
        self.time_embed = copy.deepcopy(unet.time_embed)
        self.add_embed = copy.deepcopy(unet.add_embed)
        self.conv_in = copy.deepcopy(unet.conv_in)
        self.down = copy.deepcopy(unet.down)
        self.down_kinds = list(unet.down_kinds)
        self.mid = copy.deepcopy(unet.mid)
        ch0 = unet.cfg.block_channels[0]
        emb_ch = tuple(cfg.conditioning_embedding_channels)
        layers = [nn.Conv2d(cfg.conditioning_channels, emb_ch[0], 3, padding=1, **kw), nn.SiLU()]
        for c_in, c_out in zip(emb_ch[:-1], emb_ch[1:]):
            layers += [nn.Conv2d(c_in, c_in, 3, padding=1, **kw), nn.SiLU(),
                       nn.Conv2d(c_in, c_out, 3, padding=1, stride=2, **kw), nn.SiLU()]
        self.hint = nn.Sequential(*layers)          # three stride-2 convs: pixel -> latent resolution
        self.hint_out = nn.Conv2d(emb_ch[-1], ch0, 3, padding=1, **kw)
        nn.init.zeros_(self.hint_out.weight)
        nn.init.zeros_(self.hint_out.bias)
        # one zero conv per skip (conv_in output + every down entry) and one for the middle
        skip_ch = [ch0]
        c = ch0
        for kind, m in zip(self.down_kinds, self.down):
            if kind != "down":
                c = m[0].conv2.out_channels
            skip_ch.append(c)
        self.zero_convs = nn.ModuleList(nn.Conv2d(sc, sc, 1, **kw) for sc in skip_ch)
        self.mid_out = nn.Conv2d(c, c, 1, **kw)
        for z in list(self.zero_convs) + [self.mid_out]:
            nn.init.zeros_(z.weight)
            nn.init.zeros_(z.bias)

    def forward(self, x, t, ctx, pooled, time_ids, hint, scale=None):
        """``hint`` [B, 3, 8H, 8W] (pixel space, 0..1). Returns (skip residuals, mid residual) for
        ``SDXLUNet.forward(control=...)``."""
        s = self.cfg.conditioning_scale if scale is None else scale
        emb = self.conditioning(t, pooled, time_ids)
        h = self.conv_in(x.contiguous(memory_format=torch.channels_last))
        h = h + self.hint_out(self.hint(hint.to(h.dtype)))
        hs = [h]
        for kind, m in zip(self.down_kinds, self.down):
            if kind == "down":
                h = m(h)
            else:
                h = m[0](h, emb)
                h = m[1](h, ctx) if not isinstance(m[1], nn.Identity) else h
            hs.append(h)
        h = self.mid[0](h, emb)
        h = self.mid[1](h, ctx)
        h = self.mid[2](h, emb)
        down = [z(a) * s for z, a in zip(self.zero_convs, hs)]
        mid = self.mid_out(h) * s
        if self.cfg.global_pool_conditions:
            down = [d.mean(dim=(2, 3), keepdim=True) for d in down]
            mid = mid.mean(dim=(2, 3), keepdim=True)
        return down, mid

    def conditioning(self, t, pooled, time_ids):
        ucfg = self.unet_cfg
        dt = self.conv_in.weight.dtype
        temb = self.time_embed(timestep_embedding(t, ucfg.block_channels[0], time_factor=1.0).to(dt))
        ids = timestep_embedding(time_ids.flatten(), ucfg.addition_time_embed_dim, time_factor=1.0)
        ids = ids.view(time_ids.shape[0], -1).to(dt)
        return temb + self.add_embed(torch.cat([pooled.to(dt), ids], dim=-1))


def preprocess_control_image(img: torch.Tensor, height: int, width: int) -> torch.Tensor:
    """uint8 / float image [B, 3, h, w] -> float [B, 3, height, width] in 0..1."""
    x = img.float()
    if img.dtype == torch.uint8:
        x = x / 255.0
    if x.shape[-2:] != (height, width):
        x = TF.interpolate(x, size=(height, width), mode="bilinear", align_corners=False)
    return x.clamp(0.0, 1.0)


def multiscale_control(down, mid, scales):
    """Per-resolution conditioning scales (``create_multiscale_control``)."""
    return [d * s for d, s in zip(down, list(scales) + [scales[-1]] * (len(down) - len(scales)))], mid * scales[-1]


def flux_control_concat(latents: torch.Tensor, control_latents: torch.Tensor) -> torch.Tensor:
    """Flux control: VAE latents of the control image concatenated on channels (16 + 16)."""
    if latents.shape[0] != control_latents.shape[0] or latents.shape[2:] != control_latents.shape[2:]:
        raise ValueError("control latents must match the latent batch and spatial size")
    return torch.cat([latents, control_latents.to(latents.dtype)], dim=1)


def widen_input_projection(linear: Linear, extra_in: int) -> Linear:
    """Widen ``img_in`` for control-conditioned Flux: the new input columns start at zero so the
    model's output is unchanged before training."""
    w = linear.weight
    new = Linear(w.shape[1] + extra_in, w.shape[0], bias=linear.bias is not None, dtype=w.dtype, device=w.device)
    with torch.no_grad():
        new.weight.zero_()
        new.weight[:, : w.shape[1]].copy_(w)
        if linear.bias is not None:
            new.bias.copy_(linear.bias)
    return new


# ----------------------------------------------------------------------------- IP-Adapter
@dataclass
class IPAdapterConfig:
    image_embed_dim: int = 1280          # pooled CLIP-ViT-H image embedding
    cross_attention_dim: int = 2048
    num_tokens: int = 4
    scale: float = 1.0
    plus: bool = False                   # perceiver resampler over patch embeddings
    hidden_dim: int = 1280
    depth: int = 4
    heads: int = 20
    mlp_ratio: float = 4.0

    @staticmethod
    def plus_config():
        return IPAdapterConfig(plus=True, num_tokens=16)

    @staticmethod
    def faceid_config():
        return IPAdapterConfig(image_embed_dim=512, num_tokens=4)


class ImageProjection(nn.Module):
    """Pooled image embedding -> ``num_tokens`` context tokens (linear + LayerNorm)."""

    def __init__(self, cfg: IPAdapterConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.proj = nn.Linear(cfg.image_embed_dim, cfg.num_tokens * cfg.cross_attention_dim, dtype=dtype, device=device)
        self.norm = nn.LayerNorm(cfg.cross_attention_dim, dtype=dtype, device=device)

    def forward(self, e):
        return self.norm(self.proj(e).view(e.shape[0], self.cfg.num_tokens, self.cfg.cross_attention_dim))


class PerceiverResampler(nn.Module):
    """IP-Adapter Plus: learned latent queries attend over the image patch embeddings."""

    def __init__(self, cfg: IPAdapterConfig, dtype, device):
        super().__init__()
        kw = dict(dtype=dtype, device=device)
        d = cfg.hidden_dim
        self.latents = nn.Parameter(torch.randn(1, cfg.num_tokens, d, **kw) / d ** 0.5)
        self.proj_in = nn.Linear(cfg.image_embed_dim, d, **kw)
        self.layers = nn.ModuleList()
        for _ in range(cfg.depth):
            self.layers.append(nn.ModuleDict(dict(
                norm_x=nn.LayerNorm(d, **kw), norm_l=nn.LayerNorm(d, **kw),
                to_q=nn.Linear(d, d, bias=False, **kw), to_kv=nn.Linear(d, 2 * d, bias=False, **kw),
                to_out=nn.Linear(d, d, bias=False, **kw),
                ff=nn.Sequential(nn.LayerNorm(d, **kw), nn.Linear(d, int(d * cfg.mlp_ratio), bias=False, **kw),
                                 nn.GELU(), nn.Linear(int(d * cfg.mlp_ratio), d, bias=False, **kw)))))
        self.proj_out = nn.Linear(d, cfg.cross_attention_dim, **kw)
        self.norm_out = nn.LayerNorm(cfg.cross_attention_dim, **kw)
        self.heads = cfg.heads

    def forward(self, x):
        B = x.shape[0]
        x = self.proj_in(x)
        lat = self.latents.expand(B, -1, -1)
        H = self.heads
        for ly in self.layers:
            xn, ln = ly["norm_x"](x), ly["norm_l"](lat)
            q = ly["to_q"](ln).view(B, -1, H, ln.shape[-1] // H)
            kv = ly["to_kv"](torch.cat([xn, ln], dim=1))
            k, v = kv.chunk(2, dim=-1)
            k = k.reshape(B, -1, H, q.shape[-1])
            v = v.reshape(B, -1, H, q.shape[-1])
            lat = lat + ly["to_out"](F.attention(q, k.contiguous(), v.contiguous()).reshape(B, -1, ln.shape[-1]))
            lat = lat + ly["ff"](lat)
        return self.norm_out(self.proj_out(lat))


class _DecoupledCrossAttention(nn.Module):
    """Wraps one text cross-attention: out = attn(q, K_txt, V_txt) + scale * attn(q, K_img, V_img)
    with its own image key/value projections (``to_k_ip`` / ``to_v_ip``)."""

    def __init__(self, base, cross_dim, adapter):
        super().__init__()
        self.base = base
        w = base.to_q.weight
        dim = w.shape[0]
        self.to_kv_ip = Linear(cross_dim, 2 * dim, bias=False, dtype=w.dtype, device=w.device)
        self._adapter = [adapter]            # not a submodule (avoids a reference cycle in state dicts)

    def forward(self, x, ctx=None, residual=None):
        ad = self._adapter[0]
        out = self.base(x, ctx, residual=residual)
        tokens = ad.image_tokens
        if tokens is None or ad.scale == 0.0:
            return out
        B, L, D = x.shape
        H = self.base.heads
        q = self.base.to_q(x).view(B, L, H, D // H)
        kv = self.to_kv_ip(tokens.to(x.dtype)).view(B, tokens.shape[1], 2, H, D // H)
        o = F.attention(q, kv[:, :, 0].contiguous(), kv[:, :, 1].contiguous()).reshape(B, L, D)
        return out + ad.scale * TF.linear(o, self.base.to_out.weight)


class IPAdapter(nn.Module):
    """Image-prompt adapter: projects image embeddings to context tokens and adds a decoupled
    image cross-attention to every text cross-attention (``attn2``) of the UNet."""

    def __init__(self, unet, cfg: IPAdapterConfig = IPAdapterConfig()):
        super().__init__()
        self.cfg = cfg
        p = unet.conv_in.weight
        self.image_proj = (PerceiverResampler if cfg.plus else ImageProjection)(cfg, p.dtype, p.device)
        self.scale = cfg.scale
        self.image_tokens = None
        self.wrapped = nn.ModuleList()
        for mod in unet.modules():
            if hasattr(mod, "attn2") and not isinstance(mod.attn2, _DecoupledCrossAttention):
                w = _DecoupledCrossAttention(mod.attn2, cfg.cross_attention_dim, self)
                mod.attn2 = w
                self.wrapped.append(w.to_kv_ip)

    def set_image(self, image_embeds: torch.Tensor | None):
        """Pooled [B, E] (or patch [B, N, E] for the plus variant) embeddings; None switches the
        image branch off."""
        self.image_tokens = None if image_embeds is None else self.image_proj(image_embeds)
        return self.image_tokens

    def trainable_parameters(self):
        return list(self.image_proj.parameters()) + [p for m in self.wrapped for p in m.parameters()]


# ----------------------------------------------------------------------------- T2I-Adapter
@dataclass
class T2IAdapterConfig:
    in_channels: int = 3
    channels: tuple = (320, 640, 1280)
    num_res_blocks: int = 2
    downscale_factor: int = 8
    adapter_type: str = "full"           # "full" | "light"

    @staticmethod
    def lightweight():
        return T2IAdapterConfig(num_res_blocks=1, adapter_type="light")


class _AdapterResBlock(nn.Module):
    def __init__(self, ch, dtype, device):
        super().__init__()
        self.c1 = nn.Conv2d(ch, ch, 3, padding=1, dtype=dtype, device=device)
        self.c2 = nn.Conv2d(ch, ch, 1, dtype=dtype, device=device)

    def forward(self, x):
        return x + self.c2(TF.relu(self.c1(x)))


class T2IAdapter(nn.Module):
    """Pixel-unshuffle the condition image to latent resolution, then one stage per UNet level;
    each stage's output is added to the UNet encoder feature of that level."""

    def __init__(self, cfg: T2IAdapterConfig = T2IAdapterConfig(), dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        kw = dict(dtype=dtype, device=device)
        cin = cfg.in_channels * cfg.downscale_factor ** 2
        self.unshuffle = nn.PixelUnshuffle(cfg.downscale_factor)
        self.conv_in = nn.Conv2d(cin, cfg.channels[0], 3, padding=1, **kw)
        self.stages = nn.ModuleList()
        prev = cfg.channels[0]
        for i, ch in enumerate(cfg.channels):
            layers = []
            if i > 0:
                layers.append(nn.AvgPool2d(2) if cfg.adapter_type == "light" else nn.Conv2d(prev, prev, 3, stride=2, padding=1, **kw))
            if ch != prev:
                layers.append(nn.Conv2d(prev, ch, 1, **kw))
            layers += [_AdapterResBlock(ch, dtype, device) for _ in range(cfg.num_res_blocks)]
            self.stages.append(nn.Sequential(*layers))
            prev = ch

    def forward(self, cond, scale: float = 1.0):
        """cond [B, C, 8H, 8W] in 0..1 -> list of features [B, ch_i, H / 2^i, W / 2^i]."""
        p = self.conv_in.weight
        h = self.conv_in(self.unshuffle(cond.to(p.dtype)))
        feats = []
        for st in self.stages:
            h = st(h)
            feats.append(h * scale)
        return feats

    @staticmethod
    def for_condition_type(kind: str, dtype=torch.bfloat16, device=None):
        """Canny / sketch / depth / pose maps are single- or three-channel images."""
        cin = {"canny": 1, "sketch": 1, "depth": 3, "pose": 3, "color": 3, "seg": 3}.get(kind)
        if cin is None:
            raise ValueError(f"unknown condition type {kind!r}")
        return T2IAdapter(T2IAdapterConfig(in_channels=cin), dtype=dtype, device=device)

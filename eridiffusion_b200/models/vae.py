"""Image autoencoders (KL-VAE): SDXL (4 latent channels, scale 0.13025) and the FLUX AE (16
channels, scale 0.3611, shift 0.1159), with tiled encode / decode for large images.

Reference: crates/common/vae/src/sdxl.rs (native NHWC SDXL VAE encode / decode, ``VaeSpec{kind,
path, latent_div, latent_channels, scale}``), crates/models/src/flux/ae.rs:14-59, src/models/
klein_vae.rs, src/trainers/vae_tiling.rs (overlapping tiles blended linearly). Convolutions are
cuDNN calls (channels-last), GroupNorm+SiLU is the fused channels-last kernel, the single
mid-block attention goes through the flash-attention op. Training runs on cached latents, so the
VAE sits on the pre-processing and sampling paths.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F
from .registry import register_model


@dataclass
class VaeConfig:
    in_channels: int = 3
    latent_channels: int = 4
    base: int = 128
    mult: tuple = (1, 2, 4, 4)
    layers_per_block: int = 2
    groups: int = 32
    scaling_factor: float = 0.13025
    shift_factor: float = 0.0
    latent_div: int = 8

    @staticmethod
    def sdxl():
        return VaeConfig()

    @staticmethod
    def flux():
        return VaeConfig(latent_channels=16, scaling_factor=0.3611, shift_factor=0.1159)


class _GN(nn.GroupNorm):
    def __init__(self, groups, ch, silu, kw):
        super().__init__(groups, ch, eps=1e-6, **kw)
        self.silu = silu

    def forward(self, x):
        return F.group_norm_silu(x, self.weight, self.bias, self.num_groups, self.eps, self.silu)


class _Res(nn.Module):
    def __init__(self, cin, cout, groups, kw):
        super().__init__()
        self.n1, self.c1 = _GN(groups, cin, True, kw), nn.Conv2d(cin, cout, 3, padding=1, **kw)
        self.n2, self.c2 = _GN(groups, cout, True, kw), nn.Conv2d(cout, cout, 3, padding=1, **kw)
        self.skip = nn.Conv2d(cin, cout, 1, **kw) if cin != cout else None

    def forward(self, x):
        h = self.c2(self.n2(self.c1(self.n1(x))))
        return (x if self.skip is None else self.skip(x)) + h


class _Attn(nn.Module):
    """Single-head spatial self-attention of the VAE middle block."""

    def __init__(self, ch, groups, kw):
        super().__init__()
        self.norm = _GN(groups, ch, False, kw)
        self.qkv = nn.Linear(ch, 3 * ch, **kw)
        self.out = nn.Linear(ch, ch, **kw)

    def forward(self, x):
        B, C, H, W = x.shape
        t = self.norm(x).permute(0, 2, 3, 1).reshape(B, H * W, C)
        q, k, v = self.qkv(t).view(B, H * W, 3, 1, C).unbind(2)
        o = F.attention(q.contiguous(), k.contiguous(), v.contiguous()).reshape(B, H * W, C)
        return x + self.out(o).view(B, H, W, C).permute(0, 3, 1, 2)


class Encoder(nn.Module):
    def __init__(self, cfg: VaeConfig, kw):
        super().__init__()
        ch = [cfg.base * m for m in cfg.mult]
        self.conv_in = nn.Conv2d(cfg.in_channels, ch[0], 3, padding=1, **kw)
        blocks, c = [], ch[0]
        for i, co in enumerate(ch):
            for _ in range(cfg.layers_per_block):
                blocks.append(_Res(c, co, cfg.groups, kw))
                c = co
            if i < len(ch) - 1:
                blocks.append(nn.Conv2d(c, c, 3, stride=2, padding=0, **kw))     # asymmetric pad in forward
        self.down = nn.ModuleList(blocks)
        self.mid = nn.ModuleList([_Res(c, c, cfg.groups, kw), _Attn(c, cfg.groups, kw), _Res(c, c, cfg.groups, kw)])
        self.norm_out = _GN(cfg.groups, c, True, kw)
        self.conv_out = nn.Conv2d(c, 2 * cfg.latent_channels, 3, padding=1, **kw)

    def forward(self, x):
        h = self.conv_in(x.contiguous(memory_format=torch.channels_last))
        for b in self.down:
            h = b(TF.pad(h, (0, 1, 0, 1))) if isinstance(b, nn.Conv2d) else b(h)
        for b in self.mid:
            h = b(h)
        return self.conv_out(self.norm_out(h))


class Decoder(nn.Module):
    def __init__(self, cfg: VaeConfig, kw):
        super().__init__()
        ch = [cfg.base * m for m in cfg.mult]
        c = ch[-1]
        self.conv_in = nn.Conv2d(cfg.latent_channels, c, 3, padding=1, **kw)
        self.mid = nn.ModuleList([_Res(c, c, cfg.groups, kw), _Attn(c, cfg.groups, kw), _Res(c, c, cfg.groups, kw)])
        blocks = []
        for i, co in enumerate(reversed(ch)):
            for _ in range(cfg.layers_per_block + 1):
                blocks.append(_Res(c, co, cfg.groups, kw))
                c = co
            if i < len(ch) - 1:
                blocks.append(nn.Conv2d(c, c, 3, padding=1, **kw))               # after 2x nearest upsample
        self.up = nn.ModuleList(blocks)
        self.norm_out = _GN(cfg.groups, c, True, kw)
        self.conv_out = nn.Conv2d(c, cfg.in_channels, 3, padding=1, **kw)

    def forward(self, z):
        h = self.conv_in(z.contiguous(memory_format=torch.channels_last))
        for b in self.mid:
            h = b(h)
        for b in self.up:
            h = b(TF.interpolate(h, scale_factor=2.0, mode="nearest")) if isinstance(b, nn.Conv2d) else b(h)
        return self.conv_out(self.norm_out(h))


class AutoencoderKL(nn.Module):
    def __init__(self, cfg: VaeConfig = VaeConfig(), dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        kw = dict(dtype=dtype, device=device)
        self.encoder, self.decoder = Encoder(cfg, kw), Decoder(cfg, kw)
        self.quant_conv = nn.Conv2d(2 * cfg.latent_channels, 2 * cfg.latent_channels, 1, **kw)
        self.post_quant_conv = nn.Conv2d(cfg.latent_channels, cfg.latent_channels, 1, **kw)

    def moments(self, img):
        """img [B, 3, H, W] in [-1, 1] -> (mean, logvar) of the latent posterior."""
        m = self.quant_conv(self.encoder(img.to(self.quant_conv.weight.dtype)))
        mean, logvar = m.chunk(2, dim=1)
        return mean, logvar.clamp(-30.0, 20.0)

    def encode(self, img, sample=True, generator=None):
        """Scaled latents ready for the diffusion model: (z - shift) * scale."""
        mean, logvar = self.moments(img)
        z = mean
        if sample:
            z = mean + torch.exp(0.5 * logvar) * torch.randn(mean.shape, generator=generator,
                                                              device=mean.device, dtype=mean.dtype)
        return (z - self.cfg.shift_factor) * self.cfg.scaling_factor

    def decode(self, latents):
        """Scaled latents -> image in [-1, 1] (not clamped)."""
        z = latents / self.cfg.scaling_factor + self.cfg.shift_factor
        return self.decoder(self.post_quant_conv(z.to(self.post_quant_conv.weight.dtype)))

    # ----------------------------------------------------------------------------- tiling
    @staticmethod
    def _blend(a, b, overlap, dim):
        """Linear cross-fade of ``overlap`` rows/cols between the trailing edge of a and the leading
        edge of b (in place on b)."""
        w = torch.linspace(0, 1, overlap, device=a.device, dtype=a.dtype)
        shape = [1, 1, 1, 1]
        shape[dim] = overlap
        w = w.view(shape)
        sl_a = [slice(None)] * 4
        sl_b = [slice(None)] * 4
        sl_a[dim] = slice(a.shape[dim] - overlap, None)
        sl_b[dim] = slice(0, overlap)
        b[tuple(sl_b)] = a[tuple(sl_a)] * (1 - w) + b[tuple(sl_b)] * w
        return b

    def _tiled(self, fn, x, tile, overlap, scale):
        """Run ``fn`` on overlapping tiles of ``x`` and stitch the outputs, whose spatial size is
        ``scale`` times the input's (8 for decode, 1/8 for encode)."""
        B, C, H, W = x.shape
        stride = tile - overlap
        o_ov = max(1, int(round(overlap * scale)))
        o_stride = int(round(stride * scale))
        rows = []
        for y in range(0, max(1, H - overlap), stride):
            row = []
            for xx in range(0, max(1, W - overlap), stride):
                row.append(fn(x[:, :, y:y + tile, xx:xx + tile]))
            rows.append(row)
        out_rows = []
        for i, row in enumerate(rows):
            pieces = []
            for j, t in enumerate(row):
                if i > 0:
                    t = self._blend(rows[i - 1][j], t, min(o_ov, t.shape[2], rows[i - 1][j].shape[2]), 2)
                if j > 0:
                    t = self._blend(row[j - 1], t, min(o_ov, t.shape[3], row[j - 1].shape[3]), 3)
                row[j] = t
                last_r, last_c = i == len(rows) - 1, j == len(row) - 1
                pieces.append(t[:, :, : (t.shape[2] if last_r else o_stride), : (t.shape[3] if last_c else o_stride)])
            out_rows.append(torch.cat(pieces, dim=3))
        return torch.cat(out_rows, dim=2)

    def tiled_decode(self, latents, tile=64, overlap=16):
        if max(latents.shape[-2:]) <= tile:
            return self.decode(latents)
        return self._tiled(self.decode, latents, tile, overlap, float(self.cfg.latent_div))

    def tiled_encode(self, img, tile=512, overlap=128):
        if max(img.shape[-2:]) <= tile:
            return self.encode(img, sample=False)
        return self._tiled(lambda t: self.encode(t, sample=False), img, tile, overlap, 1.0 / self.cfg.latent_div)


@register_model("vae_sdxl")
def build_vae_sdxl(dtype=torch.bfloat16, device=None, **ov):
    return AutoencoderKL(VaeConfig(**{**VaeConfig.sdxl().__dict__, **ov}), dtype, device)


@register_model("vae_flux")
def build_vae_flux(dtype=torch.bfloat16, device=None, **ov):
    return AutoencoderKL(VaeConfig(**{**VaeConfig.flux().__dict__, **ov}), dtype, device)

"""Z-Image (NextDiT / Lumina-2 family) and Wan 2.2 video DiT definitions.

Z-Image (src/models/zimage_model.rs:32-76): dim 3840, 30 heads x 128, 30 joint layers preceded by
2 noise-refiner and 2 context-refiner layers, SwiGLU hidden 10240, 3-axis RoPE [32, 48, 48] with
theta 256, caption width 2560. Blocks are single-stream over [caption | image] tokens with
sandwich RMSNorms and a 4-way adaLN (scale / tanh-gate for attention and for the MLP).

Wan 2.2 A14B (src/models/wan22_model.rs:92-170, 1040-1077, 1186-1304): dim 5120, 40 heads, 40
layers, FFN 13824 (GELU-tanh), patch (1, 2, 2), text 4096 x 512, 3-D RoPE over (frame, row, col),
6-way modulation from a learned table plus the time embedding, self-attention + text
cross-attention + FFN per block; two full experts (high-noise / low-noise) switched at
``boundary_ratio`` (0.875 T2V, 0.900 I2V): ``t > boundary -> high-noise expert``.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ..ops import functional as F
from .layers import Linear, MLPEmbedder, RMSNormScale, SmallLinear, image_ids, rope_table, timestep_embedding
from .registry import register_model


# ------------------------------------------------------------------------------ Z-Image
@dataclass
class NextDiTConfig:
    in_channels: int = 64            # 16-ch latent, 2x2 patches
    dim: int = 3840
    num_heads: int = 30
    depth: int = 30
    refiner_depth: int = 2
    mlp_hidden: int = 10240
    caption_dim: int = 2560
    axes_dim: tuple = (32, 48, 48)
    theta: float = 256.0
    time_embed_dim: int = 256
    adaln_dim: int = 256


class RMSNorm(nn.Module):
    def __init__(self, dim, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x, scale=None):
        return F.norm_modulate(x, scale=scale, weight=self.weight, rms=True)


class NextDiTBlock(nn.Module):
    def __init__(self, cfg: NextDiTConfig, modulated: bool, dtype, device):
        super().__init__()
        D = cfg.dim
        self.heads = cfg.num_heads
        self.qkv = Linear(D, 3 * D, bias=False, dtype=dtype, device=device)
        self.q_norm = RMSNormScale(D // cfg.num_heads, dtype=dtype, device=device)
        self.k_norm = RMSNormScale(D // cfg.num_heads, dtype=dtype, device=device)
        self.out = Linear(D, D, bias=False, dtype=dtype, device=device)
        self.w13 = Linear(D, 2 * cfg.mlp_hidden, bias=False, dtype=dtype, device=device)    # SwiGLU
        self.w2 = Linear(cfg.mlp_hidden, D, bias=False, dtype=dtype, device=device)
        self.attn_norm1, self.attn_norm2 = RMSNorm(D, dtype, device), RMSNorm(D, dtype, device)
        self.ffn_norm1, self.ffn_norm2 = RMSNorm(D, dtype, device), RMSNorm(D, dtype, device)
        self.adaln = SmallLinear(cfg.adaln_dim, 4 * D, dtype=dtype, device=device) if modulated else None

    def forward(self, x, cos, sin, cond=None):
        if self.adaln is not None:
            sc_a, g_a, sc_m, g_m = self.adaln(cond, silu_in=True).chunk(4, dim=-1)
            g_a, g_m = torch.tanh(g_a), torch.tanh(g_m)
        else:
            sc_a = g_a = sc_m = g_m = None
        h = self.attn_norm1(x, sc_a)
        q, k, v = F.qknorm_rope(self.qkv(h), self.q_norm.scale, self.k_norm.scale, cos, sin, self.heads)
        a = self.attn_norm2(self.out(F.attention(q, k, v).flatten(2)))
        x = F.gate_residual(x, a, g_a)
        h = self.ffn_norm1(x, sc_m)
        m = self.ffn_norm2(self.w2(F.linear_glu(h, self.w13, "silu", act_first=True)))
        return F.gate_residual(x, m, g_m)


class NextDiT(nn.Module):
    def __init__(self, cfg: NextDiTConfig = NextDiTConfig(), dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.dim
        self.x_embedder = Linear(cfg.in_channels, D, dtype=dtype, device=device)
        self.cap_norm = RMSNorm(cfg.caption_dim, dtype, device)
        self.cap_embedder = Linear(cfg.caption_dim, D, dtype=dtype, device=device)
        self.t_embedder = MLPEmbedder(cfg.time_embed_dim, cfg.adaln_dim, dtype=dtype, device=device)
        self.noise_refiner = nn.ModuleList(NextDiTBlock(cfg, True, dtype, device) for _ in range(cfg.refiner_depth))
        self.context_refiner = nn.ModuleList(NextDiTBlock(cfg, False, dtype, device) for _ in range(cfg.refiner_depth))
        self.layers = nn.ModuleList(NextDiTBlock(cfg, True, dtype, device) for _ in range(cfg.depth))
        self.final_adaln = SmallLinear(cfg.adaln_dim, D, dtype=dtype, device=device)
        self.final_linear = Linear(D, cfg.in_channels, dtype=dtype, device=device)
        self._rope = {}

    def rope(self, lt, h, w, device):
        key = (lt, h, w, str(device))
        if key not in self._rope:
            cap = torch.zeros(lt, 3, device=device)
            cap[:, 0] = torch.arange(lt, device=device)
            img = image_ids(h, w, device, t=lt)
            self._rope[key] = rope_table(torch.cat([cap, img], 0), self.cfg.axes_dim, self.cfg.theta)
        return self._rope[key]

    def forward(self, img, txt, t, y=None, guidance=None, grid_hw=None):
        B, Li, _ = img.shape
        Lt = txt.shape[1]
        if grid_hw is None:
            s = int(round(Li ** 0.5))
            grid_hw = (s, Li // s)
        dt = self.x_embedder.weight.dtype
        cond = self.t_embedder(timestep_embedding(t, self.cfg.time_embed_dim).to(dt))
        cos, sin = self.rope(Lt, grid_hw[0], grid_hw[1], img.device)
        x = self.x_embedder(img)
        c = self.cap_embedder(self.cap_norm(txt))
        for blk in self.context_refiner:
            c = blk(c, cos[:Lt], sin[:Lt])
        for blk in self.noise_refiner:
            x = blk(x, cos[Lt:], sin[Lt:], cond)
        h = torch.cat([c, x], dim=1)
        for blk in self.layers:
            h = blk(h, cos, sin, cond)
        h = h[:, Lt:]
        scale = self.final_adaln(cond, silu_in=True)
        return self.final_linear(F.norm_modulate(h, scale=scale))

    def lora_targets(self):
        return [r"(layers|noise_refiner|context_refiner)\.\d+\.(qkv|out|w13|w2)$"]


@register_model("zimage")
def build_zimage(dtype=torch.bfloat16, device=None, **overrides):
    return NextDiT(NextDiTConfig(**{**NextDiTConfig().__dict__, **overrides}), dtype=dtype, device=device)


# ------------------------------------------------------------------------------ Wan 2.2
@dataclass
class WanConfig:
    in_channels: int = 16
    dim: int = 5120
    num_heads: int = 40
    depth: int = 40
    ffn_dim: int = 13824
    text_dim: int = 4096
    patch: tuple = (1, 2, 2)
    theta: float = 10000.0
    time_embed_dim: int = 256
    boundary_ratio: float = 0.875

    @property
    def head_dim(self):
        return self.dim // self.num_heads

    @property
    def axes_dim(self):
        d = self.head_dim
        a = d // 3 // 2 * 2
        return (d - 2 * a, a, a)


class WanBlock(nn.Module):
    def __init__(self, cfg: WanConfig, dtype, device):
        super().__init__()
        D = cfg.dim
        self.heads = cfg.num_heads
        self.modulation = nn.Parameter(torch.randn(6, D, device=device).mul_(D ** -0.5).to(dtype))
        self.self_qkv = Linear(D, 3 * D, dtype=dtype, device=device)
        self.self_qn, self.self_kn = RMSNorm(D, dtype, device), RMSNorm(D, dtype, device)
        self.self_out = Linear(D, D, dtype=dtype, device=device)
        self.norm3 = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
        self.norm3_b = nn.Parameter(torch.zeros(D, dtype=dtype, device=device))
        self.cross_q = Linear(D, D, dtype=dtype, device=device)
        self.cross_kv = Linear(D, 2 * D, dtype=dtype, device=device)
        self.cross_qn, self.cross_kn = RMSNorm(D, dtype, device), RMSNorm(D, dtype, device)
        self.cross_out = Linear(D, D, dtype=dtype, device=device)
        self.ffn_in = Linear(D, cfg.ffn_dim, dtype=dtype, device=device)
        self.ffn_out = Linear(cfg.ffn_dim, D, dtype=dtype, device=device)

    def forward(self, x, ctx, e6, cos, sin):
        B, L, D = x.shape
        H = self.heads
        mod = self.modulation.unsqueeze(0) + e6
        sh_a, sc_a, g_a, sh_m, sc_m, g_m = (mod[:, i] for i in range(6))
        h = F.norm_modulate(x, sc_a, sh_a)
        q, k, v = self.self_qkv(h).split(D, dim=-1)
        q, k = self.self_qn(q.contiguous()), self.self_kn(k.contiguous())
        qkv = torch.cat([q, k, v], dim=-1)
        q, k, v = F.qknorm_rope(qkv, None, None, cos, sin, H)
        x = self.self_out(F.attention(q, k, v).flatten(2), residual=x, gate=g_a)
        h = F.norm_modulate(x, weight=self.norm3, bias=self.norm3_b)
        cq = self.cross_qn(self.cross_q(h)).view(B, L, H, D // H)
        ck, cv = self.cross_kv(ctx).split(D, dim=-1)
        ck = self.cross_kn(ck.contiguous()).view(B, -1, H, D // H)
        x = self.cross_out(F.attention(cq, ck, cv.contiguous().view(B, -1, H, D // H)).flatten(2), residual=x)
        h = F.norm_modulate(x, sc_m, sh_m)
        return self.ffn_out(self.ffn_in(h, act="gelu"), residual=x, gate=g_m)


class WanDiT(nn.Module):
    def __init__(self, cfg: WanConfig = WanConfig(), dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.dim
        pdim = cfg.in_channels * cfg.patch[0] * cfg.patch[1] * cfg.patch[2]
        self.patch_embedding = Linear(pdim, D, dtype=dtype, device=device)     # Conv3d with kernel == stride
        self.text_in = Linear(cfg.text_dim, D, dtype=dtype, device=device)
        self.text_out = Linear(D, D, dtype=dtype, device=device)
        self.time_embedding = MLPEmbedder(cfg.time_embed_dim, D, dtype=dtype, device=device)
        self.time_projection = SmallLinear(D, 6 * D, dtype=dtype, device=device)
        self.blocks = nn.ModuleList(WanBlock(cfg, dtype, device) for _ in range(cfg.depth))
        self.head_mod = nn.Parameter(torch.randn(2, D, device=device).mul_(D ** -0.5).to(dtype))
        self.head = Linear(D, pdim, dtype=dtype, device=device)
        self._rope = {}

    def rope(self, f, h, w, device):
        key = (f, h, w, str(device))
        if key not in self._rope:
            ff, yy, xx = torch.meshgrid(torch.arange(f, device=device), torch.arange(h, device=device),
                                        torch.arange(w, device=device), indexing="ij")
            ids = torch.stack([ff, yy, xx], -1).reshape(-1, 3).float()
            self._rope[key] = rope_table(ids, self.cfg.axes_dim, self.cfg.theta)
        return self._rope[key]

    def forward(self, tokens, txt, t, grid_fhw):
        """tokens [B, L, C*pf*ph*pw] (patchified video latent); txt [B, 512, 4096]; t [B]."""
        cfg = self.cfg
        dt = self.patch_embedding.weight.dtype
        e = self.time_embedding(timestep_embedding(t, cfg.time_embed_dim).to(dt))
        e6 = self.time_projection(e, silu_in=True).view(-1, 6, cfg.dim)
        ctx = self.text_out(self.text_in(txt, act="gelu"))
        cos, sin = self.rope(*grid_fhw, tokens.device)
        x = self.patch_embedding(tokens)
        for blk in self.blocks:
            x = blk(x, ctx, e6, cos, sin)
        mod = self.head_mod.unsqueeze(0) + e.unsqueeze(1)
        return self.head(F.norm_modulate(x, mod[:, 1], mod[:, 0]))

    def lora_targets(self):
        return [r"blocks\.\d+\.(self_qkv|self_out|cross_q|cross_kv|cross_out|ffn_in|ffn_out)$"]


class WanDualExpert(nn.Module):
    """Two full models; the high-noise expert handles t > boundary_ratio (flow time in [0, 1])."""

    def __init__(self, cfg: WanConfig = WanConfig(), dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        self.high_noise = WanDiT(cfg, dtype, device)
        self.low_noise = WanDiT(cfg, dtype, device)

    def select(self, t):
        return self.high_noise if float(t.flatten()[0]) > self.cfg.boundary_ratio else self.low_noise

    def forward(self, tokens, txt, t, grid_fhw):
        return self.select(t)(tokens, txt, t, grid_fhw)


def patchify_video(x, patch=(1, 2, 2)):
    """[B, C, F, H, W] -> [B, (F/pf)(H/ph)(W/pw), C*pf*ph*pw] and the token grid."""
    B, C, Fr, H, W = x.shape
    pf, ph, pw = patch
    x = x.view(B, C, Fr // pf, pf, H // ph, ph, W // pw, pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
    return x.reshape(B, (Fr // pf) * (H // ph) * (W // pw), C * pf * ph * pw), (Fr // pf, H // ph, W // pw)


@register_model("wan22")
def build_wan(dtype=torch.bfloat16, device=None, dual=False, **overrides):
    cfg = WanConfig(**{**WanConfig().__dict__, **overrides})
    return (WanDualExpert if dual else WanDiT)(cfg, dtype=dtype, device=device)

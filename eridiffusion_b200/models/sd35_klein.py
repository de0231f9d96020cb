"""SD3.5 MMDiT and Flux-2 "Klein" definitions built from the same fused ops.

SD3.5 (src/models/mmdit_blocks.rs:202-220, 1794-1850; crates/models/src/sd35/keymap.rs:3-9):
38 joint blocks, hidden 2432 (38 heads x 64), MLP 9728, 6-way adaLN per stream, 16-channel
latent with 2x2 patches, joint attention over [image | text] tokens, per-head RMS QK-norm, a fixed
2-D sin-cos position embedding instead of rotary embedding, pooled vector 2048 (CLIP-L + CLIP-G)
and text width 4096 (T5 / padded CLIP concatenation).

Klein (src/models/klein_model.rs:28-76, 156-187, 261-306): 4B = dim 3072, 24 x 128, 5 double +
20 single blocks, input 128, text width 7680; 9B = dim 4096, 32 x 128, 8 + 24, text 12288.
SwiGLU MLP with hidden 3*dim, no biases, ONE set of modulation vectors computed at model level
and shared by every block, 4-axis rotary embedding [32, 32, 32, 32] with theta 2000.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from ..ops import functional as F
from .layers import Linear, MLPEmbedder, Modulation, RMSNormScale, rope_table, timestep_embedding
from .mmdit import DoubleStreamBlock, LastLayer, MMDiTConfig, SelfAttentionProj
from .registry import register_model


def sincos_2d(dim, h, w, device=None, top=0, left=0):
    """SD3 position table for an h x w patch grid whose first patch sits at (top, left) of the full
    grid: per token ``[emb(column) | emb(row)]`` with ``emb(p) = [sin(p f), cos(p f)]``,
    ``f_i = 10000^(-i / (dim / 4))`` — the column half comes FIRST, as in the released ``pos_embed``
    tables and in ``RoPE2D::embed`` (src/models/mmdit_blocks.rs:2107-2136)."""
    def one(d, pos):
        om = 1.0 / (10000 ** (torch.arange(d // 2, dtype=torch.float64, device=device) / (d / 2)))
        out = pos.double().reshape(-1)[:, None] * om[None]
        return torch.cat([torch.sin(out), torch.cos(out)], dim=1)
    yy, xx = torch.meshgrid(torch.arange(top, top + h, device=device),
                            torch.arange(left, left + w, device=device), indexing="ij")
    return torch.cat([one(dim // 2, xx), one(dim // 2, yy)], dim=1).float()


class SD35JointBlock(nn.Module):
    """Joint block with the two SD3.5 variations of the plain two-stream block
    (src/models/mmdit_blocks.rs:2393-2394):

    * ``context_pre_only`` (the last block): the text stream only feeds the joint attention. It has
      a 2-way modulation and a q/k/v projection, no output projection and no MLP, and leaves the
      block unchanged.
    * ``x_self_attn`` (the "dual attention" blocks of SD3.5-medium): a second, image-only
      self-attention. The image modulation is 9-way; the second attention reads the same
      normalised input with its own shift / scale and is added with its own gate.
    """

    def __init__(self, cfg: MMDiTConfig, dtype, device, context_pre_only=False, x_self_attn=False):
        super().__init__()
        D, H = cfg.hidden, cfg.num_heads
        mlp = int(D * cfg.mlp_ratio)
        self.heads, self.context_pre_only, self.x_self_attn = H, context_pre_only, x_self_attn
        self.img_mod = Modulation(D, 9 if x_self_attn else 6, dtype=dtype, device=device)
        self.txt_mod = Modulation(D, 2 if context_pre_only else 6, dtype=dtype, device=device)
        self.img_attn = SelfAttentionProj(D, H, cfg.qkv_bias, dtype, device)
        self.txt_attn = SelfAttentionProj(D, H, cfg.qkv_bias, dtype, device)
        if context_pre_only:
            self.txt_attn.proj = None
        self.img_attn2 = SelfAttentionProj(D, H, cfg.qkv_bias, dtype, device) if x_self_attn else None
        self.img_mlp_0 = Linear(D, mlp, dtype=dtype, device=device)
        self.img_mlp_2 = Linear(mlp, D, dtype=dtype, device=device)
        if not context_pre_only:
            self.txt_mlp_0 = Linear(D, mlp, dtype=dtype, device=device)
            self.txt_mlp_2 = Linear(mlp, D, dtype=dtype, device=device)

    def forward(self, img, txt, vec, cos=None, sin=None):
        im = self.img_mod(vec)
        i_sh1, i_sc1, i_g1, i_sh2, i_sc2, i_g2 = im[:6]
        tm = self.txt_mod(vec)
        t_sh1, t_sc1 = tm[0], tm[1]
        Lt = txt.shape[1]
        img_qkv = self.img_attn.qkv(F.norm_modulate(img, i_sc1, i_sh1))
        txt_qkv = self.txt_attn.qkv(F.norm_modulate(txt, t_sc1, t_sh1))
        q, k, v = F.qknorm_rope_joint(
            [(txt_qkv, self.txt_attn.q_norm.scale, self.txt_attn.k_norm.scale),
             (img_qkv, self.img_attn.q_norm.scale, self.img_attn.k_norm.scale)],
            cos, sin, self.heads)
        attn = F.attention(q, k, v).flatten(2)
        txt_a, img_a = attn[:, :Lt], attn[:, Lt:]
        x = self.img_attn.proj(img_a, residual=img, gate=i_g1)
        if self.x_self_attn:
            i_sh3, i_sc3, i_g3 = im[6:9]
            qkv2 = self.img_attn2.qkv(F.norm_modulate(img, i_sc3, i_sh3))
            q2, k2, v2 = F.qknorm_rope_joint(
                [(qkv2, self.img_attn2.q_norm.scale, self.img_attn2.k_norm.scale)], None, None, self.heads)
            x = self.img_attn2.proj(F.attention(q2, k2, v2).flatten(2), residual=x, gate=i_g3)
        img = self.img_mlp_2(self.img_mlp_0(F.norm_modulate(x, i_sc2, i_sh2), act="gelu"),
                             residual=x, gate=i_g2)
        if self.context_pre_only:
            return img, txt
        t_g1, t_sh2, t_sc2, t_g2 = tm[2:6]
        txt = self.txt_attn.proj(txt_a, residual=txt, gate=t_g1)
        txt = self.txt_mlp_2(self.txt_mlp_0(F.norm_modulate(txt, t_sc2, t_sh2), act="gelu"),
                             residual=txt, gate=t_g2)
        return img, txt


class SD35MMDiT(nn.Module):
    def __init__(self, hidden=2432, num_heads=38, depth=38, in_channels=64, context_dim=4096,
                 pooled_dim=2048, mlp_ratio=4.0, dtype=torch.bfloat16, device=None,
                 context_pre_only_last=False, x_self_attn_layers=(), pos_embed_max_size=None):
        super().__init__()
        self.cfg = MMDiTConfig(in_channels=in_channels, hidden=hidden, num_heads=num_heads,
                               depth_double=depth, depth_single=0, mlp_ratio=mlp_ratio,
                               context_dim=context_dim, vec_dim=pooled_dim, guidance_embed=False,
                               axes_dim=(hidden // num_heads,))
        D = hidden
        self.x_embedder = Linear(in_channels, D, dtype=dtype, device=device)
        self.context_embedder = Linear(context_dim, D, dtype=dtype, device=device)
        self.t_embedder = MLPEmbedder(256, D, dtype=dtype, device=device)
        self.y_embedder = MLPEmbedder(pooled_dim, D, dtype=dtype, device=device)
        dual = set(x_self_attn_layers)

        def block(i):
            pre_only = context_pre_only_last and i == depth - 1
            if pre_only or i in dual:
                return SD35JointBlock(self.cfg, dtype, device, context_pre_only=pre_only, x_self_attn=i in dual)
            return DoubleStreamBlock(self.cfg, dtype, device)
        self.joint_blocks = nn.ModuleList(block(i) for i in range(depth))
        self.final_layer = LastLayer(D, in_channels, dtype, device)
        self._pos = {}
        # Released checkpoints carry a ``pos_embed`` table over the largest patch grid (192 x 192 for
        # SD3.5-large, 384 x 384 for medium); a smaller image uses the CENTRE crop of it. With a
        # table size the model keeps the table as a buffer (filled with the closed form, replaced by
        # the file's tensor on load); without one positions start at 0 for every grid.
        self.pos_embed_max_size = pos_embed_max_size
        if pos_embed_max_size:
            m = int(pos_embed_max_size)
            self.register_buffer("pos_embed", sincos_2d(D, m, m, device).to(dtype), persistent=True)

    def pos_table(self, h, w, device, dtype):
        """[h*w, hidden] position rows for an h x w patch grid."""
        m = self.pos_embed_max_size
        if m:
            if h > m or w > m:
                raise ValueError(f"patch grid {h}x{w} exceeds the position table ({m}x{m})")
            top, left = (m - h) // 2, (m - w) // 2
            tab = self.pos_embed.view(m, m, -1)[top:top + h, left:left + w]
            return tab.reshape(h * w, -1).to(device=device, dtype=dtype)
        key = (h, w, str(device))
        if key not in self._pos:
            self._pos[key] = sincos_2d(self.cfg.hidden, h, w, device).to(dtype)
        return self._pos[key]

    def forward(self, img, txt, t, y, guidance=None, grid_hw=None):
        B, Li, _ = img.shape
        if grid_hw is None:
            s = int(round(Li ** 0.5))
            grid_hw = (s, Li // s)
        dt = self.x_embedder.weight.dtype
        vec = self.t_embedder(timestep_embedding(t, 256).to(dt)) + self.y_embedder(y.to(dt))
        x = self.x_embedder(img) + self.pos_table(grid_hw[0], grid_hw[1], img.device, dt)
        c = self.context_embedder(txt)
        for blk in self.joint_blocks:
            x, c = blk(x, c, vec, None, None)
        return self.final_layer(x, vec)

    def lora_targets(self):
        return [r"joint_blocks\.\d+\.(img|txt)_attn2?\.(qkv|proj)$", r"joint_blocks\.\d+\.(img|txt)_mlp_[02]$"]


@register_model("sd35")
def build_sd35(dtype=torch.bfloat16, device=None, **kw):
    """SD3.5-large layout; as in the released weights the last block's text stream stops after its
    attention (adaLN width 2 x hidden there: crates/models/src/sd35/keymap.rs ``ADA_DIM_LAST_CONTEXT``)."""
    kw.setdefault("context_pre_only_last", True)
    if kw.get("hidden", 2432) == 2432:
        kw.setdefault("pos_embed_max_size", 192)
    return SD35MMDiT(dtype=dtype, device=device, **kw)


@register_model("sd35_medium")
def build_sd35_medium(dtype=torch.bfloat16, device=None, **kw):
    """SD3.5-medium layout: 24 blocks, hidden 1536 (24 x 64), image-only second attention in blocks
    0-12, text stream dropped after the last block's attention."""
    base = dict(hidden=1536, num_heads=24, depth=24, context_pre_only_last=True,
                x_self_attn_layers=tuple(range(13)))
    base.update(kw)
    if base["hidden"] == 1536:
        base.setdefault("pos_embed_max_size", 384)
    return SD35MMDiT(dtype=dtype, device=device, **base)


# ------------------------------------------------------------------------------ Klein
@dataclass
class KleinConfig:
    in_channels: int = 128
    dim: int = 3072
    num_heads: int = 24
    depth_double: int = 5
    depth_single: int = 20
    context_dim: int = 7680
    axes_dim: tuple = (32, 32, 32, 32)
    theta: float = 2000.0


KLEIN_4B = KleinConfig()
KLEIN_9B = KleinConfig(dim=4096, num_heads=32, depth_double=8, depth_single=24, context_dim=12288)


class KleinStream(nn.Module):
    def __init__(self, D, H, dtype, device):
        super().__init__()
        self.qkv = Linear(D, 3 * D, bias=False, dtype=dtype, device=device)
        self.q_norm, self.k_norm = RMSNormScale(D // H, dtype=dtype, device=device), RMSNormScale(D // H, dtype=dtype, device=device)
        self.proj = Linear(D, D, bias=False, dtype=dtype, device=device)
        self.mlp_in = Linear(D, 6 * D, bias=False, dtype=dtype, device=device)      # SwiGLU, hidden 3D
        self.mlp_out = Linear(3 * D, D, bias=False, dtype=dtype, device=device)


class KleinDouble(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        self.heads = cfg.num_heads
        self.img, self.txt = KleinStream(cfg.dim, cfg.num_heads, dtype, device), KleinStream(cfg.dim, cfg.num_heads, dtype, device)

    def forward(self, img, txt, mod_img, mod_txt, cos, sin):
        Lt = txt.shape[1]
        (i_sh1, i_sc1, i_g1, i_sh2, i_sc2, i_g2), (t_sh1, t_sc1, t_g1, t_sh2, t_sc2, t_g2) = mod_img, mod_txt
        q, k, v = F.qknorm_rope_joint(
            [(self.txt.qkv(F.norm_modulate(txt, t_sc1, t_sh1)), self.txt.q_norm.scale, self.txt.k_norm.scale),
             (self.img.qkv(F.norm_modulate(img, i_sc1, i_sh1)), self.img.q_norm.scale, self.img.k_norm.scale)],
            cos, sin, self.heads)
        a = F.attention(q, k, v).flatten(2)
        img = self.img.proj(a[:, Lt:], residual=img, gate=i_g1)
        txt = self.txt.proj(a[:, :Lt], residual=txt, gate=t_g1)
        img = self.img.mlp_out(F.linear_glu(F.norm_modulate(img, i_sc2, i_sh2), self.img.mlp_in, "silu"), residual=img, gate=i_g2)
        txt = self.txt.mlp_out(F.linear_glu(F.norm_modulate(txt, t_sc2, t_sh2), self.txt.mlp_in, "silu"), residual=txt, gate=t_g2)
        return img, txt


class KleinSingle(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        D = cfg.dim
        self.dim, self.heads = D, cfg.num_heads
        self.linear1 = Linear(D, 3 * D + 6 * D, bias=False, dtype=dtype, device=device)
        self.linear2 = Linear(D + 3 * D, D, bias=False, dtype=dtype, device=device)
        self.q_norm, self.k_norm = RMSNormScale(D // cfg.num_heads, dtype=dtype, device=device), RMSNormScale(D // cfg.num_heads, dtype=dtype, device=device)

    def forward(self, x, mod, cos, sin):
        shift, scale, gate = mod
        h = self.linear1(F.norm_modulate(x, scale, shift))
        qkv, mlp = h[..., : 3 * self.dim], h[..., 3 * self.dim:]
        q, k, v = F.qknorm_rope_joint([(qkv, self.q_norm.scale, self.k_norm.scale)], cos, sin, self.heads)
        cat = torch.cat((F.attention(q, k, v).flatten(2), F.glu(mlp.contiguous(), "silu")), dim=-1)
        return self.linear2(cat, residual=x, gate=gate)


class Klein(nn.Module):
    def __init__(self, cfg: KleinConfig = KLEIN_4B, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.dim
        self.img_in = Linear(cfg.in_channels, D, bias=False, dtype=dtype, device=device)
        self.txt_in = Linear(cfg.context_dim, D, bias=False, dtype=dtype, device=device)
        self.time_in = MLPEmbedder(256, D, dtype=dtype, device=device)
        self.double_mod_img = Modulation(D, 6, dtype=dtype, device=device)
        self.double_mod_txt = Modulation(D, 6, dtype=dtype, device=device)
        self.single_mod = Modulation(D, 3, dtype=dtype, device=device)
        self.double_blocks = nn.ModuleList(KleinDouble(cfg, dtype, device) for _ in range(cfg.depth_double))
        self.single_blocks = nn.ModuleList(KleinSingle(cfg, dtype, device) for _ in range(cfg.depth_single))
        self.final_layer = LastLayer(D, cfg.in_channels, dtype, device)

    def forward(self, img, txt, t, y=None, guidance=None, ids=None, grid_hw=None):
        """ids: [Lt + Li, 4] positions for the 4-axis rotary table (defaults: text index on axis 3,
        image (row, col) on axes 1, 2)."""
        B, Li, _ = img.shape
        Lt = txt.shape[1]
        dev = img.device
        if ids is None:
            if grid_hw is None:
                s = int(round(Li ** 0.5))
                grid_hw = (s, Li // s)
            ti = torch.zeros(Lt, 4, device=dev)
            ti[:, 3] = torch.arange(Lt, device=dev)
            ii = torch.zeros(grid_hw[0], grid_hw[1], 4, device=dev)
            ii[..., 1] = torch.arange(grid_hw[0], device=dev)[:, None]
            ii[..., 2] = torch.arange(grid_hw[1], device=dev)[None, :]
            ids = torch.cat([ti, ii.view(-1, 4)], 0)
        cos, sin = rope_table(ids, self.cfg.axes_dim, self.cfg.theta)
        dt = self.img_in.weight.dtype
        vec = self.time_in(timestep_embedding(t, 256).to(dt))
        mi, mt, ms = self.double_mod_img(vec), self.double_mod_txt(vec), self.single_mod(vec)
        x, c = self.img_in(img), self.txt_in(txt)
        for blk in self.double_blocks:
            x, c = blk(x, c, mi, mt, cos, sin)
        h = torch.cat((c, x), dim=1)
        for blk in self.single_blocks:
            h = blk(h, ms, cos, sin)
        return self.final_layer(h[:, Lt:], vec)

    def lora_targets(self):
        return [r"double_blocks\.\d+\.(img|txt)\.(qkv|proj|mlp_in|mlp_out)$", r"single_blocks\.\d+\.linear[12]$"]


@register_model("klein")
def build_klein(dtype=torch.bfloat16, device=None, variant="4b", **overrides):
    base = KLEIN_9B if str(variant).lower() == "9b" else KLEIN_4B
    return Klein(KleinConfig(**{**base.__dict__, **overrides}), dtype=dtype, device=device)

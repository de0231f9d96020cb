"""FLUX-style MMDiT: double-stream blocks (separate text / image weights, joint attention) followed
by single-stream blocks (fused QKV+MLP projection), adaLN modulation from a conditioning vector,
per-head RMS QK-norm and N-axis rotary embedding.

The architecture constants come from the reference's FLUX config
(src/models/flux_model_complete.rs:424-449: hidden 3072, 24 heads x 128, 19 double + 38 single,
mlp_ratio 4, axes_dim [16, 56, 56], theta 10000) and block math
``x + gate * f(LN(x) * (1 + scale) + shift)`` (crates/training/src/flux/runtime.rs:383-398);
joint attention concatenates text then image tokens as the Klein model does
(src/models/klein_model.rs:403-416). The reference's training runtime simplifies FLUX to
independent streams (flux/runtime.rs:155-159); this model implements the full block.

Every dense op goes through ``ops.functional`` so that CUDA bf16 tensors hit the sm_100a kernels:
norm+modulate, QKV GEMM (+LoRA), QK-norm+RoPE written straight into the joint q/k/v, flash
attention, output GEMM with the gate+residual epilogue, MLP GEMMs with GELU / gate+residual
epilogues.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn

from ..ops import functional as F
from .layers import (Linear, MLPEmbedder, Modulation, RMSNormScale, SmallLinear, image_ids,
                     linear_pair, mlp_pair, rope_table, timestep_embedding)
from .registry import register_model


@dataclass
class MMDiTConfig:
    in_channels: int = 64            # patchified latent channels (16 * 2 * 2)
    out_channels: int | None = None
    hidden: int = 3072
    num_heads: int = 24
    depth_double: int = 19
    depth_single: int = 38
    mlp_ratio: float = 4.0
    context_dim: int = 4096          # T5 width
    vec_dim: int = 768               # pooled CLIP width
    guidance_embed: bool = True
    qkv_bias: bool = True
    axes_dim: tuple = (16, 56, 56)
    theta: float = 10000.0
    time_embed_dim: int = 256
    txt_rmsnorm: bool = False        # RMSNorm on the text embeddings before txt_in (Qwen-Image)

    @property
    def head_dim(self):
        return self.hidden // self.num_heads


FLUX_DEV = MMDiTConfig()
TINY = MMDiTConfig(in_channels=64, hidden=256, num_heads=4, depth_double=2, depth_single=2,
                   context_dim=128, vec_dim=64, guidance_embed=False, axes_dim=(16, 24, 24))


class SelfAttentionProj(nn.Module):
    def __init__(self, dim, heads, qkv_bias, dtype, device):
        super().__init__()
        self.qkv = Linear(dim, 3 * dim, bias=qkv_bias, dtype=dtype, device=device)
        self.q_norm = RMSNormScale(dim // heads, dtype=dtype, device=device)
        self.k_norm = RMSNormScale(dim // heads, dtype=dtype, device=device)
        self.proj = Linear(dim, dim, dtype=dtype, device=device)


class DoubleStreamBlock(nn.Module):
    def __init__(self, cfg: MMDiTConfig, dtype, device):
        super().__init__()
        D, H = cfg.hidden, cfg.num_heads
        mlp = int(D * cfg.mlp_ratio)
        self.heads = H
        self.img_mod = Modulation(D, 6, dtype=dtype, device=device)
        self.txt_mod = Modulation(D, 6, dtype=dtype, device=device)
        self.img_attn = SelfAttentionProj(D, H, cfg.qkv_bias, dtype, device)
        self.txt_attn = SelfAttentionProj(D, H, cfg.qkv_bias, dtype, device)
        self.img_mlp_0 = Linear(D, mlp, dtype=dtype, device=device)
        self.img_mlp_2 = Linear(mlp, D, dtype=dtype, device=device)
        self.txt_mlp_0 = Linear(D, mlp, dtype=dtype, device=device)
        self.txt_mlp_2 = Linear(mlp, D, dtype=dtype, device=device)

    def forward(self, img, txt, vec, cos, sin):
        i_sh1, i_sc1, i_g1, i_sh2, i_sc2, i_g2 = self.img_mod(vec)
        t_sh1, t_sc1, t_g1, t_sh2, t_sc2, t_g2 = self.txt_mod(vec)
        Lt = txt.shape[1]
        # each norm also hands back its input for the residual branch around it: the two gradients of the
        # stream are then summed inside the norm's backward kernel
        img_n, img = F.norm_modulate_skip(img, i_sc1, i_sh1)
        txt_n, txt = F.norm_modulate_skip(txt, t_sc1, t_sh1)
        img_qkv, txt_qkv = linear_pair(self.img_attn.qkv, img_n, self.txt_attn.qkv, txt_n)
        q, k, v = F.qknorm_rope_joint(
            [(txt_qkv, self.txt_attn.q_norm.scale, self.txt_attn.k_norm.scale),
             (img_qkv, self.img_attn.q_norm.scale, self.img_attn.k_norm.scale)],
            cos, sin, self.heads)
        attn = F.attention(q, k, v).flatten(2)               # [B, Lt+Li, D]
        txt_a, img_a = F.split_tokens(attn, Lt)
        img, txt = linear_pair(self.img_attn.proj, img_a, self.txt_attn.proj, txt_a,
                               residual=(img, txt), gate=(i_g1, t_g1))
        img_n, img = F.norm_modulate_skip(img, i_sc2, i_sh2)
        txt_n, txt = F.norm_modulate_skip(txt, t_sc2, t_sh2)
        img, txt = mlp_pair(self.img_mlp_0, self.img_mlp_2, img_n, self.txt_mlp_0, self.txt_mlp_2, txt_n, act="gelu",
                            residual=(img, txt), gate=(i_g2, t_g2))
        return img, txt


class SingleStreamBlock(nn.Module):
    def __init__(self, cfg: MMDiTConfig, dtype, device):
        super().__init__()
        D, H = cfg.hidden, cfg.num_heads
        self.dim, self.heads = D, H
        self.mlp_dim = int(D * cfg.mlp_ratio)
        self.modulation = Modulation(D, 3, dtype=dtype, device=device)
        self.linear1 = Linear(D, 3 * D + self.mlp_dim, dtype=dtype, device=device)
        self.linear2 = Linear(D + self.mlp_dim, D, dtype=dtype, device=device)
        self.q_norm = RMSNormScale(D // H, dtype=dtype, device=device)
        self.k_norm = RMSNormScale(D // H, dtype=dtype, device=device)

    def forward(self, x, vec, cos, sin):
        shift, scale, gate = self.modulation(vec)
        from ..ops import fused_blocks as FB
        xm, x = F.norm_modulate_skip(x, scale, shift)
        if FB.single_stream_supported(xm, gate, self.linear1, self.linear2, self.heads):
            return FB.single_stream(xm, x, gate, self.linear1, self.linear2, self.q_norm.scale,
                                    self.k_norm.scale, cos, sin, self.heads)
        h = self.linear1(xm)                                          # [B, L, 3D + mlp]
        qkv, mlp = h[..., : 3 * self.dim], h[..., 3 * self.dim:]
        q, k, v = F.qknorm_rope_joint([(qkv, self.q_norm.scale, self.k_norm.scale)], cos, sin,
                                      self.heads)
        attn = F.attention(q, k, v).flatten(2)
        cat = torch.cat((attn, F.gelu_tanh(mlp)), dim=-1)
        return self.linear2(cat, residual=x, gate=gate)


class LastLayer(nn.Module):
    def __init__(self, hidden, out_dim, dtype, device):
        super().__init__()
        self.adaLN = Modulation(hidden, 2, dtype=dtype, device=device)
        self.linear = Linear(hidden, out_dim, dtype=dtype, device=device)

    def forward(self, x, vec):
        shift, scale = self.adaLN(vec)
        return self.linear(F.norm_modulate(x, scale, shift))


class MMDiT(nn.Module):
    def __init__(self, cfg: MMDiTConfig = FLUX_DEV, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        assert sum(cfg.axes_dim) == cfg.head_dim, "rotary axes must cover the head dimension"
        self.img_in = Linear(cfg.in_channels, D, dtype=dtype, device=device)
        self.txt_in = Linear(cfg.context_dim, D, dtype=dtype, device=device)
        self.time_in = MLPEmbedder(cfg.time_embed_dim, D, dtype=dtype, device=device)
        self.vector_in = MLPEmbedder(cfg.vec_dim, D, dtype=dtype, device=device) if cfg.vec_dim else None
        self.txt_norm = RMSNormScale(cfg.context_dim, dtype=dtype, device=device) if cfg.txt_rmsnorm else None
        self.guidance_in = MLPEmbedder(cfg.time_embed_dim, D, dtype=dtype, device=device) \
            if cfg.guidance_embed else None
        self.double_blocks = nn.ModuleList(DoubleStreamBlock(cfg, dtype, device)
                                           for _ in range(cfg.depth_double))
        self.single_blocks = nn.ModuleList(SingleStreamBlock(cfg, dtype, device)
                                           for _ in range(cfg.depth_single))
        self.final_layer = LastLayer(D, cfg.out_channels or cfg.in_channels, dtype, device)
        self._rope_cache = {}
        # train.act_checkpoint.BlockRunner: activation policy, layer streaming and TREAD routing of
        # the block stacks (None: the blocks are simply called in order)
        self.runner = None

    def rope(self, txt_len, h, w, device):
        key = (txt_len, h, w, str(device))
        if key not in self._rope_cache:
            ids = torch.cat([torch.zeros(txt_len, 3, device=device), image_ids(h, w, device)], 0)
            self._rope_cache[key] = rope_table(ids, self.cfg.axes_dim, self.cfg.theta)
        return self._rope_cache[key]

    def forward(self, img, txt, t, y, guidance=None, grid_hw=None):
        """img [B, Li, C] patchified latents; txt [B, Lt, ctx]; t [B] in [0, 1]; y [B, vec];
        guidance [B]; grid_hw = (h, w) token grid of the image (defaults to a square)."""
        cfg = self.cfg
        B, Li, _ = img.shape
        Lt = txt.shape[1]
        if grid_hw is None:
            s = int(round(Li ** 0.5))
            grid_hw = (s, Li // s)
        dt = self.img_in.weight.dtype
        vec = self.time_in(timestep_embedding(t, cfg.time_embed_dim).to(dt))
        if self.guidance_in is not None:
            g = guidance if guidance is not None else torch.ones_like(t)
            vec = vec + self.guidance_in(timestep_embedding(g, cfg.time_embed_dim).to(dt))
        if self.vector_in is not None:
            vec = vec + self.vector_in(y.to(dt))
        cos, sin = self.rope(Lt, grid_hw[0], grid_hw[1], img.device)
        img = self.img_in(img)
        if self.txt_norm is not None:
            txt = F.norm_modulate(txt, weight=self.txt_norm.scale, rms=True)
        txt = self.txt_in(txt)
        run = self.runner
        for i, blk in enumerate(self.double_blocks):
            img, txt = blk(img, txt, vec, cos, sin) if run is None else run.double(i, blk, img, txt, vec, cos, sin)
        if len(self.single_blocks) == 0:
            return self.final_layer(img, vec)
        x = torch.cat((txt, img), dim=1)
        if run is None:
            for blk in self.single_blocks:
                x = blk(x, vec, cos, sin)
        else:
            x = run.single_stack(self.single_blocks, x, vec, cos, sin, Lt, first_index=len(self.double_blocks))
        return self.final_layer(x[:, Lt:], vec)

    def lora_targets(self):
        """Module-path regexes of 'all attention and MLP linears'."""
        return [r"double_blocks\.\d+\.(img|txt)_attn\.(qkv|proj)$",
                r"double_blocks\.\d+\.(img|txt)_mlp_[02]$",
                r"single_blocks\.\d+\.linear[12]$"]

    def block_list(self):
        return list(self.double_blocks) + list(self.single_blocks)


@register_model("flux")
def build_flux(dtype=torch.bfloat16, device=None, **overrides):
    cfg = MMDiTConfig(**{**FLUX_DEV.__dict__, **overrides})
    return MMDiT(cfg, dtype=dtype, device=device)


QWEN_IMAGE = MMDiTConfig(in_channels=64, hidden=3072, num_heads=24, depth_double=60, depth_single=0,
                         context_dim=3584, vec_dim=0, guidance_embed=False, txt_rmsnorm=True)


@register_model("qwen_image")
def build_qwen_image(dtype=torch.bfloat16, device=None, **overrides):
    """Qwen-Image-architecture MMDiT: 60 dual-stream blocks, hidden 3072, 24 x 128 heads, MLP 12288,
    text width 3584, 16-channel latents patchified 2x2 (the reference's entry is a placeholder:
    src/inference/qwen_image.rs:9-21, 85-90; crates/models/qwen_image/src/lib.rs:7-12)."""
    cfg = MMDiTConfig(**{**QWEN_IMAGE.__dict__, **overrides})
    return MMDiT(cfg, dtype=dtype, device=device)


@register_model("chroma")
def build_chroma(dtype=torch.bfloat16, device=None, **overrides):
    """Chroma is FLUX-derived (crates/training/src/chroma/registry.rs:36, 147-221): same blocks,
    no guidance / pooled-vector embedders."""
    cfg = MMDiTConfig(**{**FLUX_DEV.__dict__, "guidance_embed": False, "vec_dim": 0, **overrides})
    return MMDiT(cfg, dtype=dtype, device=device)


@register_model("tiny_mmdit")
def build_tiny(dtype=torch.float32, device=None, **overrides):
    cfg = MMDiTConfig(**{**TINY.__dict__, **overrides})
    return MMDiT(cfg, dtype=dtype, device=device)

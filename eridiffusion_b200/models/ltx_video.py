"""LTX-style video DiT: adaLN-single blocks (self-attention with RMS QK-norm across heads and 3-D
rotary embedding, text cross-attention, GELU-tanh feed-forward), 1x1x1 patches of a 128-channel
video latent.

Architecture facts follow the reference's inference model (src/models/ltx2_model.rs:53-151):
48 blocks, 32 heads x 128, FFN 4x, cross-attention width 4096, caption projection, timestep x1000,
``scale_shift_table[6, dim] + temb`` giving shift/scale/gate for attention and feed-forward
(:646-668), un-modulated text cross-attention, RMSNorm over the whole inner dimension for q and k
(:549-551), rotary angles from fractional 3-D patch coordinates: ``freqs = theta^linspace(0,1) *
pi/2``, angle ``(2*grid - 1) * freq``, interleaved pairs, cos-pad 1 / sin-pad 0 for the
remainder dims (:284-381, 404-436).

With a ``UlyssesContext`` the sequence is sharded over ranks: the QKV projection scatters head
groups to their owners in its epilogue, the out-projection gathers its input inside its launch.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from ..ops import functional as F
from ..ops import reference as R
from .layers import Linear, MLPEmbedder, SmallLinear, timestep_embedding
from .registry import register_model


@dataclass
class LTXConfig:
    in_channels: int = 128
    hidden: int = 4096
    num_heads: int = 32
    depth: int = 48
    mlp_ratio: float = 4.0
    context_dim: int = 4096
    caption_dim: int = 4096
    theta: float = 10000.0
    max_pos: tuple = (20, 2048, 2048)
    time_embed_dim: int = 256

    @property
    def head_dim(self):
        return self.hidden // self.num_heads


def rope_3d_table(coords, dim, theta=10000.0, max_pos=(20, 2048, 2048)):
    """coords [L, 3] (frame, row, col) -> cos/sin [L, dim/2] over the whole inner dimension."""
    n_axis = 3
    per = dim // (2 * n_axis)                      # frequencies per axis
    freqs = (theta ** torch.linspace(0, 1, per, device=coords.device, dtype=torch.float64)) * (math.pi / 2)
    frac = coords.double() / torch.tensor(max_pos, device=coords.device, dtype=torch.float64)
    ang = ((2 * frac - 1).unsqueeze(-1) * freqs).transpose(-1, -2).reshape(coords.shape[0], -1)  # [L, per*3]
    cos, sin = torch.cos(ang), torch.sin(ang)
    pad = dim // 2 - cos.shape[1]
    if pad > 0:
        cos = torch.cat([torch.ones(cos.shape[0], pad, device=cos.device, dtype=cos.dtype), cos], 1)
        sin = torch.cat([torch.zeros(sin.shape[0], pad, device=sin.device, dtype=sin.dtype), sin], 1)
    return cos.float(), sin.float()


def video_coords(frames, h, w, device=None):
    f, y, x = torch.meshgrid(torch.arange(frames, device=device), torch.arange(h, device=device),
                             torch.arange(w, device=device), indexing="ij")
    return torch.stack([f, y, x], -1).reshape(-1, 3).float()


def _rope_full(x, cos, sin):
    """x [B, L, C] rotated over interleaved pairs of the whole channel dim (cos/sin [L, C/2])."""
    return R.rope_rotate(x.unsqueeze(2), cos, sin).squeeze(2).to(x.dtype)


class LTXBlock(nn.Module):
    def __init__(self, cfg: LTXConfig, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.heads, self.dim = cfg.num_heads, D
        self.scale_shift_table = nn.Parameter(torch.randn(6, D, device=device).mul_(D ** -0.5).to(dtype))
        self.attn1_qkv = Linear(D, 3 * D, dtype=dtype, device=device)
        self.attn1_qnorm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
        self.attn1_knorm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
        self.attn1_out = Linear(D, D, dtype=dtype, device=device)
        self.attn2_q = Linear(D, D, dtype=dtype, device=device)
        self.attn2_kv = Linear(cfg.context_dim, 2 * D, dtype=dtype, device=device)
        self.attn2_qnorm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
        self.attn2_knorm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
        self.attn2_out = Linear(D, D, dtype=dtype, device=device)
        self.ff_in = Linear(D, int(D * cfg.mlp_ratio), dtype=dtype, device=device)
        self.ff_out = Linear(int(D * cfg.mlp_ratio), D, dtype=dtype, device=device)

    def _self_attention_local(self, h, cos, sin):
        B, L, D = h.shape
        qkv = self.attn1_qkv(h)
        q, k, v = qkv.split(D, dim=-1)
        q = F.norm_modulate(q.contiguous(), weight=self.attn1_qnorm, rms=True)
        k = F.norm_modulate(k.contiguous(), weight=self.attn1_knorm, rms=True)
        q, k = _rope_full(q, cos, sin), _rope_full(k, cos, sin)
        sh = (B, L, self.heads, D // self.heads)
        cp = getattr(self, "context_parallel", None)
        if cp is not None:
            # tokens are sharded over the group; keys / values travel around the ring
            from ..parallel.ring_attention import ring_attention
            return ring_attention(q.view(sh).contiguous(), k.view(sh).contiguous(), v.contiguous().view(sh),
                                  group=cp.group).view(B, L, D)
        return F.attention(q.view(sh), k.view(sh), v.contiguous().view(sh)).view(B, L, D)

    def _self_attention_ulysses(self, h, cos, sin, u, eps=1e-6):
        from ..parallel.ulysses import dist_rmsnorm, ulysses_qkv
        import torch.distributed as dist
        B, Ll, D = h.shape
        W, G, r = u.world, u.G, u.rank
        recv, rowsq = ulysses_qkv(h, self.attn1_qkv, u, want_rowsq=True)
        rstd_local = torch.rsqrt(rowsq.view(2, B, Ll) / D + eps)
        if W > 1:
            allr = torch.empty(W, 2, B, Ll, dtype=rstd_local.dtype, device=h.device)
            dist.all_gather_into_tensor(allr, rstd_local.contiguous(), group=u.pg.group)
            rstd = allr.permute(1, 2, 0, 3).reshape(2, B, W * Ll)
        else:
            rstd = rstd_local
        sl = slice(r * G, (r + 1) * G)
        q = dist_rmsnorm(recv[:, :, 0], rstd[0], self.attn1_qnorm[sl], D, u.pg)
        k = dist_rmsnorm(recv[:, :, 1], rstd[1], self.attn1_knorm[sl], D, u.pg)
        c, s = cos[:, r * G // 2:(r + 1) * G // 2], sin[:, r * G // 2:(r + 1) * G // 2]
        q, k = _rope_full(q, c, s), _rope_full(k, c, s)
        hl = self.heads // W
        sh = (B, u.Lt, hl, G // hl)
        # with one slot per layer the attention output is written where the peers' out-projection
        # launches fetch it
        out = u.attn_buffer(getattr(self, "layer_idx", 0), hl)
        return F.attention(q.view(sh), k.view(sh), recv[:, :, 2].contiguous().view(sh), out=out).view(B, u.Lt, G)

    def forward(self, x, ctx, temb6, cos, sin, u=None):
        x, ff_mod = self.forward_attn(x, ctx, temb6, cos, sin, u)
        return self.forward_ff(x, ff_mod)

    def forward_attn(self, x, ctx, temb6, cos, sin, u=None):
        """Self-attention and text cross-attention; returns the stream and the feed-forward's
        (shift, scale, gate), so that a caller can put work between the two halves of the block."""
        B, L, D = x.shape
        mod = self.scale_shift_table.unsqueeze(0) + temb6                    # [B, 6, D]
        sh_a, sc_a, g_a, sh_m, sc_m, g_m = (mod[:, i] for i in range(6))
        h = F.norm_modulate(x, sc_a, sh_a, rms=True)
        if u is None:
            attn = self._self_attention_local(h, cos, sin)
            x = self.attn1_out(attn, residual=x, gate=g_a)
        else:
            from ..parallel.ulysses import ulysses_out_proj
            attn = self._self_attention_ulysses(h, cos, sin, u)
            x = ulysses_out_proj(attn, self.attn1_out, u, residual=x, gate=g_a)
        # text cross-attention (keys/values from the replicated text tokens: no communication)
        q = F.norm_modulate(self.attn2_q(x), weight=self.attn2_qnorm, rms=True)
        kv = self.attn2_kv(ctx)
        k, v = kv.split(D, dim=-1)
        k = F.norm_modulate(k.contiguous(), weight=self.attn2_knorm, rms=True)
        hd = D // self.heads
        ca = F.attention(q.view(B, L, self.heads, hd), k.view(B, -1, self.heads, hd),
                         v.contiguous().view(B, -1, self.heads, hd)).view(B, L, D)
        x = self.attn2_out(ca, residual=x)
        return x, (sh_m, sc_m, g_m)

    def forward_ff(self, x, ff_mod):
        sh_m, sc_m, g_m = ff_mod
        h = F.norm_modulate(x, sc_m, sh_m, rms=True)
        return self.ff_out(self.ff_in(h, act="gelu"), residual=x, gate=g_m)


class LTXVideo(nn.Module):
    def __init__(self, cfg: LTXConfig = LTXConfig(), dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        self.patchify_proj = Linear(cfg.in_channels, D, dtype=dtype, device=device)
        self.time_embed = MLPEmbedder(cfg.time_embed_dim, D, dtype=dtype, device=device)
        self.adaln_single = SmallLinear(D, 6 * D, dtype=dtype, device=device)
        self.caption_in = Linear(cfg.caption_dim, D, dtype=dtype, device=device)
        self.caption_out = Linear(D, cfg.context_dim, dtype=dtype, device=device)
        self.blocks = nn.ModuleList(LTXBlock(cfg, dtype, device) for _ in range(cfg.depth))
        for i, blk in enumerate(self.blocks):
            blk.layer_idx = i            # selects the block's attention-output slot under Ulysses
        self.scale_shift_table = nn.Parameter(torch.randn(2, D, device=device).mul_(D ** -0.5).to(dtype))
        self.proj_out = Linear(D, cfg.in_channels, dtype=dtype, device=device)
        self.ulysses = None
        self._rope = {}

    def set_sequence_parallel(self, u):
        self.ulysses = u

    def set_context_parallel(self, group=None, enabled=True):
        """Ring-attention context parallelism: every rank of ``group`` (default: all ranks) feeds
        its contiguous token slice; only the self-attention communicates (key / value slices around
        the ring), every other layer is per token. Unlike Ulysses the degree is not bounded by the
        head count. Mutually exclusive with ``set_sequence_parallel``."""
        from types import SimpleNamespace
        import torch.distributed as dist
        cp = SimpleNamespace(group=group, world=dist.get_world_size(group), rank=dist.get_rank(group)) if enabled else None
        self.context = cp
        for blk in self.blocks:
            blk.context_parallel = cp

    def rope(self, frames, h, w, device):
        key = (frames, h, w, str(device))
        if key not in self._rope:
            self._rope[key] = rope_3d_table(video_coords(frames, h, w, device), self.cfg.hidden,
                                            self.cfg.theta, self.cfg.max_pos)
        return self._rope[key]

    def forward(self, x, ctx, t, grid_fhw, y=None, guidance=None):
        """x [B, L_local, C] tokens of this rank (all tokens without sequence parallelism);
        ctx [B, Lt, caption_dim]; t [B] in [0, 1]; grid_fhw = (frames, h, w) of the full clip."""
        cfg = self.cfg
        dt = self.patchify_proj.weight.dtype
        u = self.ulysses
        cos, sin = self.rope(*grid_fhw, x.device)
        cp = getattr(self, "context", None)
        if cp is not None:
            if u is not None:
                raise ValueError("context parallelism and Ulysses sequence parallelism are mutually exclusive")
            Ll = x.shape[1]
            if Ll * cp.world != cos.shape[0]:
                raise ValueError("local token count times the group size does not match the grid")
            cos, sin = cos[cp.rank * Ll:(cp.rank + 1) * Ll], sin[cp.rank * Ll:(cp.rank + 1) * Ll]
        elif u is None and cos.shape[0] != x.shape[1]:
            raise ValueError("token count does not match the grid")
        temb = self.time_embed(timestep_embedding(t, cfg.time_embed_dim).to(dt))       # [B, D]
        temb6 = self.adaln_single(temb, silu_in=True).view(-1, 6, cfg.hidden)
        ctx = self.caption_out(self.caption_in(ctx, act="gelu"))
        h = self.patchify_proj(x)
        if u is not None:
            lo = u.rank * u.Ll
            cos_l, sin_l = cos, sin                     # self-attention sees the whole sequence
        for blk in self.blocks:
            h = blk(h, ctx, temb6, cos, sin, u)
        mod = self.scale_shift_table.unsqueeze(0) + temb.unsqueeze(1)
        h = F.norm_modulate(h, mod[:, 1], mod[:, 0], rms=False)
        return self.proj_out(h)

    def lora_targets(self):
        return [r"blocks\.\d+\.(attn1_qkv|attn1_out|attn2_q|attn2_kv|attn2_out|ff_in|ff_out)$"]

    def block_list(self):
        return list(self.blocks)


@register_model("ltx_video")
def build_ltx(dtype=torch.bfloat16, device=None, **overrides):
    cfg = LTXConfig(**{**LTXConfig().__dict__, **overrides})
    return LTXVideo(cfg, dtype=dtype, device=device)

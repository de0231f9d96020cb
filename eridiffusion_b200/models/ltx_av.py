"""LTX-2 audio + video transformer: two token streams with cross-modal attention in every block.

Follows the reference's dual-stream model (src/models/ltx2_model.rs:6-40, 588-871, 878-1100):

* video stream as in ``ltx_video.py`` (inner 32 x 128 = 4096, 3-D rotary embedding);
* audio stream with its own width (32 heads x 64 = 2048), 128-channel audio latent, 1-D (time)
  rotary embedding, own adaLN-single time embedding, own caption projection;
* per block, in this order: self-attention of each stream; text cross-attention of each stream;
  **audio-to-video** attention (queries = video, keys / values = audio) and **video-to-audio**
  attention (queries = audio, keys / values = video), both reading RMS-normalised streams that
  are modulated by ``table[0:4] + temb`` (scale, shift for a2v; scale, shift for v2a) and gated by
  ``table[4] + temb_gate`` (:802-871); feed-forward of each stream;
* the cross-modal time embedding uses the timestep scaled by
  ``cross_attn_timestep_scale_multiplier`` (1000) for the gates (:1014).

Cross-modal attention runs at the audio width (heads x 64) for both directions; rotary phases on
the time axis only, so that a video token and an audio token of the same instant line up.

The blocks reuse ``LTXBlock`` for each stream's own sub-layers, so every GEMM, norm and attention
goes through the same fused ops (and the video stream can still run under Ulysses; the audio stream
and the cross-modal attention see whole sequences and are replicated).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn

from ..ops import functional as F
from .layers import Linear, MLPEmbedder, SmallLinear, timestep_embedding
from .ltx_video import LTXBlock, LTXConfig, _rope_full, rope_3d_table, video_coords
from .registry import register_model


@dataclass
class LTXAVConfig:
    video: LTXConfig = field(default_factory=LTXConfig)
    audio_in_channels: int = 128
    audio_heads: int = 32
    audio_head_dim: int = 64
    audio_context_dim: int = 2048
    audio_max_pos: float = 20.0               # seconds spanned by the rotary table's unit interval
    audio_latents_per_second: float = 25.0    # sampling_rate / hop_length / scale_factor = 16000/160/4
    video_fps: float = 25.0
    cross_attn_timestep_scale: float = 1000.0

    @property
    def audio_dim(self):
        return self.audio_heads * self.audio_head_dim

    def audio_stream_config(self) -> LTXConfig:
        v = self.video
        return LTXConfig(in_channels=self.audio_in_channels, hidden=self.audio_dim, num_heads=self.audio_heads,
                         depth=v.depth, mlp_ratio=v.mlp_ratio, context_dim=self.audio_context_dim,
                         caption_dim=v.caption_dim, theta=v.theta, max_pos=v.max_pos,
                         time_embed_dim=v.time_embed_dim)


def rope_1d_table(seconds, dim, theta=10000.0, max_pos=20.0):
    """Time-axis rotary table: ``seconds`` [L] -> cos/sin [L, dim/2], same frequency law as the
    video table (``theta^linspace(0,1) * pi/2``, angle ``(2 * t/max_pos - 1) * freq``)."""
    per = dim // 2
    freqs = (theta ** torch.linspace(0, 1, per, device=seconds.device, dtype=torch.float64)) * (math.pi / 2)
    ang = (2 * seconds.double() / max_pos - 1).unsqueeze(-1) * freqs
    return torch.cos(ang).float(), torch.sin(ang).float()


class CrossModalAttention(nn.Module):
    """Queries from one stream, keys / values from the other, at ``inner`` = heads x head_dim."""

    def __init__(self, q_dim, kv_dim, inner, heads, dtype, device):
        super().__init__()
        self.heads, self.inner = heads, inner
        self.to_q = Linear(q_dim, inner, dtype=dtype, device=device)
        self.to_kv = Linear(kv_dim, 2 * inner, dtype=dtype, device=device)
        self.q_norm = nn.Parameter(torch.ones(inner, dtype=dtype, device=device))
        self.k_norm = nn.Parameter(torch.ones(inner, dtype=dtype, device=device))
        self.to_out = Linear(inner, q_dim, dtype=dtype, device=device)

    def forward(self, xq, xkv, rope_q, rope_k, residual, gate):
        B, Lq, _ = xq.shape
        q = F.norm_modulate(self.to_q(xq), weight=self.q_norm, rms=True)
        k, v = self.to_kv(xkv).split(self.inner, dim=-1)
        k = F.norm_modulate(k.contiguous(), weight=self.k_norm, rms=True)
        q, k = _rope_full(q, *rope_q), _rope_full(k, *rope_k)
        hd = self.inner // self.heads
        o = F.attention(q.view(B, Lq, self.heads, hd), k.view(B, -1, self.heads, hd),
                        v.contiguous().view(B, -1, self.heads, hd)).view(B, Lq, self.inner)
        return self.to_out(o, residual=residual, gate=gate)


class LTXAVBlock(nn.Module):
    def __init__(self, cfg: LTXAVConfig, dtype, device):
        super().__init__()
        Dv, Da = cfg.video.hidden, cfg.audio_dim
        self.video = LTXBlock(cfg.video, dtype, device)
        self.audio = LTXBlock(cfg.audio_stream_config(), dtype, device)
        self.a2v = CrossModalAttention(Dv, Da, Da, cfg.audio_heads, dtype, device)
        self.v2a = CrossModalAttention(Da, Dv, Da, cfg.audio_heads, dtype, device)
        # rows: a2v scale, a2v shift, v2a scale, v2a shift, gate
        self.video_ca_table = nn.Parameter(torch.randn(5, Dv, device=device).mul_(Dv ** -0.5).to(dtype))
        self.audio_ca_table = nn.Parameter(torch.randn(5, Da, device=device).mul_(Da ** -0.5).to(dtype))

    def forward(self, xv, xa, ctx_v, ctx_a, temb_v, temb_a, ca_v, ca_a, rope_v, rope_a, rope_vt, rope_at, u=None):
        """ca_v / ca_a: ([B, 4, D] scale-shift, [B, D] gate) of the cross-modal time embedding;
        rope_vt / rope_at: time-axis tables at the cross-modal width."""
        xv, ff_v = self.video.forward_attn(xv, ctx_v, temb_v, *rope_v, u)
        xa, ff_a = self.audio.forward_attn(xa, ctx_a, temb_a, *rope_a)
        mv = self.video_ca_table[:4].unsqueeze(0) + ca_v[0]                      # [B, 4, Dv]
        ma = self.audio_ca_table[:4].unsqueeze(0) + ca_a[0]
        gv = self.video_ca_table[4].unsqueeze(0) + ca_v[1]                       # a2v gate [B, Dv]
        ga = self.audio_ca_table[4].unsqueeze(0) + ca_a[1]                       # v2a gate [B, Da]
        # both directions read the streams as they are BEFORE either cross-modal update
        v_a2v = F.norm_modulate(xv, mv[:, 0], mv[:, 1], rms=True)
        a_a2v = F.norm_modulate(xa, ma[:, 0], ma[:, 1], rms=True)
        v_v2a = F.norm_modulate(xv, mv[:, 2], mv[:, 3], rms=True)
        a_v2a = F.norm_modulate(xa, ma[:, 2], ma[:, 3], rms=True)
        xv = self.a2v(v_a2v, a_a2v, rope_vt, rope_at, residual=xv, gate=gv)
        xa = self.v2a(a_v2a, v_v2a, rope_at, rope_vt, residual=xa, gate=ga)
        return self.video.forward_ff(xv, ff_v), self.audio.forward_ff(xa, ff_a)


class _StreamIO(nn.Module):
    """Per-stream input / output layers (patch projection, adaLN-single, caption projection,
    output modulation table and projection)."""

    def __init__(self, cfg: LTXConfig, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.cfg = cfg
        self.patchify_proj = Linear(cfg.in_channels, D, dtype=dtype, device=device)
        self.time_embed = MLPEmbedder(cfg.time_embed_dim, D, dtype=dtype, device=device)
        self.adaln_single = SmallLinear(D, 6 * D, dtype=dtype, device=device)
        self.ca_time_embed = MLPEmbedder(cfg.time_embed_dim, D, dtype=dtype, device=device)
        self.ca_scale_shift = SmallLinear(D, 4 * D, dtype=dtype, device=device)
        self.ca_gate = SmallLinear(D, D, dtype=dtype, device=device)
        self.caption_in = Linear(cfg.caption_dim, D, dtype=dtype, device=device)
        self.caption_out = Linear(D, cfg.context_dim, dtype=dtype, device=device)
        self.scale_shift_table = nn.Parameter(torch.randn(2, D, device=device).mul_(D ** -0.5).to(dtype))
        self.proj_out = Linear(D, cfg.in_channels, dtype=dtype, device=device)

    def embed(self, x, ctx, t, gate_scale):
        cfg, dt = self.cfg, self.patchify_proj.weight.dtype
        temb = self.time_embed(timestep_embedding(t, cfg.time_embed_dim).to(dt))
        temb6 = self.adaln_single(temb, silu_in=True).view(-1, 6, cfg.hidden)
        ct = self.ca_time_embed(timestep_embedding(t, cfg.time_embed_dim).to(dt))
        cg = self.ca_time_embed(timestep_embedding(t * (gate_scale / 1000.0), cfg.time_embed_dim).to(dt))
        ca = (self.ca_scale_shift(ct, silu_in=True).view(-1, 4, cfg.hidden), self.ca_gate(cg, silu_in=True))
        return self.patchify_proj(x), self.caption_out(self.caption_in(ctx, act="gelu")), temb, temb6, ca

    def head(self, h, temb):
        mod = self.scale_shift_table.unsqueeze(0) + temb.unsqueeze(1)
        return self.proj_out(F.norm_modulate(h, mod[:, 1], mod[:, 0], rms=False))


class LTXAudioVideo(nn.Module):
    def __init__(self, cfg: LTXAVConfig | None = None, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg = cfg or LTXAVConfig()
        self.video_io = _StreamIO(cfg.video, dtype, device)
        self.audio_io = _StreamIO(cfg.audio_stream_config(), dtype, device)
        self.blocks = nn.ModuleList(LTXAVBlock(cfg, dtype, device) for _ in range(cfg.video.depth))
        self._rope = {}

    def tables(self, grid_fhw, n_audio, device):
        key = (tuple(grid_fhw), n_audio, str(device))
        if key not in self._rope:
            c = self.cfg
            coords = video_coords(*grid_fhw, device)
            rope_v = rope_3d_table(coords, c.video.hidden, c.video.theta, c.video.max_pos)
            a_sec = torch.arange(n_audio, device=device, dtype=torch.float64) / c.audio_latents_per_second
            v_sec = coords[:, 0].double() / c.video_fps
            rope_a = rope_1d_table(a_sec, c.audio_dim, c.video.theta, c.audio_max_pos)
            rope_vt = rope_1d_table(v_sec, c.audio_dim, c.video.theta, c.audio_max_pos)
            self._rope[key] = (rope_v, rope_a, rope_vt, rope_a)
        return self._rope[key]

    def forward(self, xv, xa, ctx, t, grid_fhw, t_audio=None, ctx_audio=None):
        """xv [B, Lv, 128] video tokens, xa [B, La, 128] audio tokens, ctx [B, Lt, caption_dim]
        (``ctx_audio`` defaults to the same text), t [B] in [0, 1] (``t_audio``: separate audio
        timestep, as the reference allows). Returns (video prediction, audio prediction)."""
        c = self.cfg
        t_audio = t if t_audio is None else t_audio
        rope_v, rope_a, rope_vt, rope_at = self.tables(grid_fhw, xa.shape[1], xv.device)
        if rope_v[0].shape[0] != xv.shape[1]:
            raise ValueError("video token count does not match the grid")
        hv, cv, tv, tv6, cav = self.video_io.embed(xv, ctx, t, c.cross_attn_timestep_scale)
        ha, ca_txt, ta, ta6, caa = self.audio_io.embed(xa, ctx if ctx_audio is None else ctx_audio, t_audio,
                                                       c.cross_attn_timestep_scale)
        for blk in self.blocks:
            hv, ha = blk(hv, ha, cv, ca_txt, tv6, ta6, cav, caa, rope_v, rope_a, rope_vt, rope_at)
        return self.video_io.head(hv, tv), self.audio_io.head(ha, ta)

    def forward_video_only(self, xv, ctx, t, grid_fhw):
        """Video path without the audio stream and the cross-modal layers (the reference's
        ``forward_video_only``, ltx2_model.rs:634)."""
        c = self.cfg
        rope_v = rope_3d_table(video_coords(*grid_fhw, xv.device), c.video.hidden, c.video.theta, c.video.max_pos)
        hv, cv, tv, tv6, _ = self.video_io.embed(xv, ctx, t, c.cross_attn_timestep_scale)
        for blk in self.blocks:
            hv = blk.video(hv, cv, tv6, *rope_v)
        return self.video_io.head(hv, tv)

    def lora_targets(self):
        return [r"blocks\.\d+\.(video|audio)\.(attn1_qkv|attn1_out|attn2_q|attn2_kv|attn2_out|ff_in|ff_out)$",
                r"blocks\.\d+\.(a2v|v2a)\.(to_q|to_kv|to_out)$"]

    def block_list(self):
        return list(self.blocks)


@register_model("ltx_av")
def build_ltx_av(dtype=torch.bfloat16, device=None, audio=None, **video_overrides):
    video = LTXConfig(**{**LTXConfig().__dict__, **video_overrides})
    return LTXAudioVideo(LTXAVConfig(video=video, **(audio or {})), dtype=dtype, device=device)

"""Text encoders used to pre-compute conditioning: CLIP text towers (CLIP-L, OpenCLIP bigG), the T5
encoder, and a Qwen3 / Gemma-3 style decoder stack read at a hidden layer.

Reference: crates/common/text (``ClipL``, ``OpenClipG``: ``forward`` -> hidden states, ``pooled``;
``attn_mask_from_lengths``), src/models/text_encoder_complete.rs (CLIP + T5), qwen3_encoder.rs and
gemma3_encoder.rs. Training runs on cached embeddings, so these models sit on the pre-processing
path (``cli/cache_embeddings.py``); they use the same fused ops as the diffusion models.
Tokenisation is out of scope here: the encoders take token ids (the cache CLI accepts any
``transformers`` tokenizer directory).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as TF

from ..ops import functional as F
from .layers import Linear, rope_table
from .registry import register_model


def attn_mask_from_lengths(lengths, max_len, device=None):
    """[B] lengths -> boolean key mask [B, 1, 1, T] (True = attend)."""
    ar = torch.arange(max_len, device=device)
    return (ar[None, :] < torch.as_tensor(lengths, device=device)[:, None])[:, None, None, :]


# ------------------------------------------------------------------------------------ CLIP
@dataclass
class ClipTextConfig:
    vocab_size: int = 49408
    hidden: int = 768
    layers: int = 12
    heads: int = 12
    max_len: int = 77
    mlp_ratio: float = 4.0
    act: str = "quick_gelu"          # CLIP-L: quick_gelu; OpenCLIP bigG: gelu
    proj_dim: int | None = 768       # text projection for the pooled output (None = no projection)
    eos_token_id: int = 49407

    @staticmethod
    def clip_l():
        return ClipTextConfig()

    @staticmethod
    def open_clip_g():
        return ClipTextConfig(hidden=1280, layers=32, heads=20, act="gelu", proj_dim=1280)


class _ClipLayer(nn.Module):
    def __init__(self, cfg, kw):
        super().__init__()
        d = cfg.hidden
        self.heads = cfg.heads
        self.ln1 = nn.LayerNorm(d, **kw)
        self.qkv = Linear(d, 3 * d, **kw)
        self.out = Linear(d, d, **kw)
        self.ln2 = nn.LayerNorm(d, **kw)
        self.fc1 = Linear(d, int(d * cfg.mlp_ratio), **kw)
        self.fc2 = Linear(int(d * cfg.mlp_ratio), d, **kw)
        self.act = cfg.act

    def forward(self, x, mask):
        B, T, D = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.heads, D // self.heads).unbind(2)
        x = x + self.out(F.attention(q.contiguous(), k.contiguous(), v.contiguous(), mask=mask).reshape(B, T, D))
        h = self.fc1(self.ln2(x))
        h = h * torch.sigmoid(1.702 * h) if self.act == "quick_gelu" else TF.gelu(h)
        return x + self.fc2(h)


class ClipTextEncoder(nn.Module):
    def __init__(self, cfg: ClipTextConfig = ClipTextConfig(), dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        kw = dict(dtype=dtype, device=device)
        self.token_embedding = nn.Embedding(cfg.vocab_size, cfg.hidden, **kw)
        self.position_embedding = nn.Parameter(torch.zeros(cfg.max_len, cfg.hidden, **kw))
        self.layers = nn.ModuleList(_ClipLayer(cfg, kw) for _ in range(cfg.layers))
        self.final_ln = nn.LayerNorm(cfg.hidden, **kw)
        self.text_projection = Linear(cfg.hidden, cfg.proj_dim, bias=False, **kw) if cfg.proj_dim else None

    def forward(self, ids, output_layer: int = -1):
        """ids [B, T] -> (hidden states [B, T, D] of layer ``output_layer`` (-1 = last, -2 =
        penultimate, as SDXL uses), pooled [B, proj] taken at the EOS token of the final layer)."""
        B, T = ids.shape
        x = self.token_embedding(ids) + self.position_embedding[:T]
        causal = torch.ones(T, T, dtype=torch.bool, device=ids.device).tril()[None, None]
        hidden = []
        for ly in self.layers:
            x = ly(x, causal)
            hidden.append(x)
        last = self.final_ln(x)
        eos = (ids == self.cfg.eos_token_id).int().argmax(dim=-1)
        pooled = last[torch.arange(B, device=ids.device), eos]
        if self.text_projection is not None:
            pooled = self.text_projection(pooled)
        out = last if output_layer == -1 else hidden[output_layer]
        return out, pooled


# ------------------------------------------------------------------------------------ T5
@dataclass
class T5Config:
    vocab_size: int = 32128
    hidden: int = 4096
    layers: int = 24
    heads: int = 64
    head_dim: int = 64
    ff: int = 10240
    rel_buckets: int = 32
    rel_max_distance: int = 128

    @staticmethod
    def xxl():
        return T5Config()


class _T5Norm(nn.Module):
    def __init__(self, d, kw):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d, **kw))

    def forward(self, x):
        return F.norm_modulate(x, weight=self.weight, rms=True, eps=1e-6)


class _T5Layer(nn.Module):
    def __init__(self, cfg, kw):
        super().__init__()
        inner = cfg.heads * cfg.head_dim
        self.heads, self.head_dim = cfg.heads, cfg.head_dim
        self.ln1 = _T5Norm(cfg.hidden, kw)
        self.qkv = Linear(cfg.hidden, 3 * inner, bias=False, **kw)
        self.o = Linear(inner, cfg.hidden, bias=False, **kw)
        self.ln2 = _T5Norm(cfg.hidden, kw)
        self.wi = Linear(cfg.hidden, 2 * cfg.ff, bias=False, **kw)       # [gelu gate | value]
        self.wo = Linear(cfg.ff, cfg.hidden, bias=False, **kw)

    def forward(self, x, bias):
        B, T, _ = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.heads, self.head_dim).unbind(2)
        # T5 attention is unscaled and carries an additive relative-position bias
        o = F.attention(q.contiguous(), k.contiguous(), v.contiguous(), scale=1.0, mask=bias)
        x = x + self.o(o.reshape(B, T, -1))
        return x + self.wo(F.glu(self.wi(self.ln2(x)), "gelu", act_first=True))


class T5Encoder(nn.Module):
    def __init__(self, cfg: T5Config = T5Config(), dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        kw = dict(dtype=dtype, device=device)
        self.shared = nn.Embedding(cfg.vocab_size, cfg.hidden, **kw)
        self.rel_bias = nn.Embedding(cfg.rel_buckets, cfg.heads, **kw)
        self.layers = nn.ModuleList(_T5Layer(cfg, kw) for _ in range(cfg.layers))
        self.final_ln = _T5Norm(cfg.hidden, kw)

    def _buckets(self, T, device):
        cfg = self.cfg
        rel = torch.arange(T, device=device)[None, :] - torch.arange(T, device=device)[:, None]
        nb = cfg.rel_buckets // 2                                         # bidirectional
        ret = (rel > 0).long() * nb
        n = rel.abs()
        max_exact = nb // 2
        large = max_exact + (torch.log(n.float().clamp(min=1) / max_exact) /
                             math.log(cfg.rel_max_distance / max_exact) * (nb - max_exact)).long()
        return ret + torch.where(n < max_exact, n, large.clamp(max=nb - 1))

    def forward(self, ids, key_mask=None):
        """ids [B, T]; key_mask [B, T] bool (True = real token) -> hidden states [B, T, D]."""
        B, T = ids.shape
        x = self.shared(ids)
        bias = self.rel_bias(self._buckets(T, ids.device)).permute(2, 0, 1)[None].to(x.dtype)   # [1, H, T, T]
        if key_mask is not None:
            bias = bias + (~key_mask)[:, None, None, :].to(x.dtype) * -1e4
        bias = bias.expand(B, -1, -1, -1)
        for ly in self.layers:
            x = ly(x, bias)
        return self.final_ln(x)


# ------------------------------------------------------------------- Qwen3 / Gemma-3 style stack
@dataclass
class DecoderTextConfig:
    vocab_size: int = 151936
    hidden: int = 2560
    layers: int = 36
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    ff: int = 9728
    rope_theta: float = 1e6
    qk_norm: bool = True            # Qwen3 normalises q and k per head
    output_layer: int = -2          # hidden state handed to the diffusion model

    @staticmethod
    def qwen3_4b():
        return DecoderTextConfig()

    @staticmethod
    def gemma3_like():
        return DecoderTextConfig(vocab_size=262144, hidden=2560, layers=34, heads=8, kv_heads=4, head_dim=256,
                                 ff=10240, rope_theta=1e6)


class _DecoderLayer(nn.Module):
    def __init__(self, cfg, kw):
        super().__init__()
        self.cfg = cfg
        self.ln1 = _T5Norm(cfg.hidden, kw)
        self.q = Linear(cfg.hidden, cfg.heads * cfg.head_dim, bias=False, **kw)
        self.kv = Linear(cfg.hidden, 2 * cfg.kv_heads * cfg.head_dim, bias=False, **kw)
        self.o = Linear(cfg.heads * cfg.head_dim, cfg.hidden, bias=False, **kw)
        self.q_norm = nn.Parameter(torch.ones(cfg.head_dim, **kw)) if cfg.qk_norm else None
        self.k_norm = nn.Parameter(torch.ones(cfg.head_dim, **kw)) if cfg.qk_norm else None
        self.ln2 = _T5Norm(cfg.hidden, kw)
        self.gate_up = Linear(cfg.hidden, 2 * cfg.ff, bias=False, **kw)   # [silu gate | value]
        self.down = Linear(cfg.ff, cfg.hidden, bias=False, **kw)

    def forward(self, x, cos, sin, mask):
        cfg = self.cfg
        B, T, _ = x.shape
        h = self.ln1(x)
        q = self.q(h).view(B, T, cfg.heads, cfg.head_dim)
        k, v = self.kv(h).view(B, T, 2, cfg.kv_heads, cfg.head_dim).unbind(2)
        if self.q_norm is not None:
            q = F.norm_modulate(q.reshape(B, T * cfg.heads, cfg.head_dim), weight=self.q_norm, rms=True).view_as(q)
            k = F.norm_modulate(k.reshape(B, T * cfg.kv_heads, cfg.head_dim), weight=self.k_norm, rms=True).view_as(k)
        from ..ops.reference import rope_rotate
        q, k = rope_rotate(q, cos, sin).to(x.dtype), rope_rotate(k, cos, sin).to(x.dtype)
        rep = cfg.heads // cfg.kv_heads
        k = k.repeat_interleave(rep, dim=2)
        v = v.repeat_interleave(rep, dim=2)
        x = x + self.o(F.attention(q.contiguous(), k.contiguous(), v.contiguous(), mask=mask).reshape(B, T, -1))
        return x + self.down(F.glu(self.gate_up(self.ln2(x)), "silu", act_first=True))


class DecoderTextEncoder(nn.Module):
    """Causal decoder used as a text encoder: returns the hidden state of ``cfg.output_layer``."""

    def __init__(self, cfg: DecoderTextConfig = DecoderTextConfig(), dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        kw = dict(dtype=dtype, device=device)
        self.embed = nn.Embedding(cfg.vocab_size, cfg.hidden, **kw)
        self.layers = nn.ModuleList(_DecoderLayer(cfg, kw) for _ in range(cfg.layers))
        self.final_ln = _T5Norm(cfg.hidden, kw)

    def forward(self, ids, key_mask=None):
        B, T = ids.shape
        x = self.embed(ids)
        pos = torch.arange(T, device=ids.device, dtype=torch.float32)[:, None]
        cos, sin = rope_table(pos, (self.cfg.head_dim,), self.cfg.rope_theta)
        mask = torch.ones(T, T, dtype=torch.bool, device=ids.device).tril()[None, None]
        if key_mask is not None:
            mask = mask & key_mask[:, None, None, :]
        hidden = []
        for ly in self.layers:
            x = ly(x, cos, sin, mask)
            hidden.append(x)
        if self.cfg.output_layer == -1:
            return self.final_ln(x)
        return hidden[self.cfg.output_layer]


@register_model("clip_l")
def build_clip_l(dtype=torch.bfloat16, device=None, **ov):
    return ClipTextEncoder(ClipTextConfig(**{**ClipTextConfig.clip_l().__dict__, **ov}), dtype, device)


@register_model("open_clip_g")
def build_clip_g(dtype=torch.bfloat16, device=None, **ov):
    return ClipTextEncoder(ClipTextConfig(**{**ClipTextConfig.open_clip_g().__dict__, **ov}), dtype, device)


@register_model("t5_encoder")
def build_t5(dtype=torch.bfloat16, device=None, **ov):
    return T5Encoder(T5Config(**{**T5Config().__dict__, **ov}), dtype, device)


@register_model("qwen3_encoder")
def build_qwen3(dtype=torch.bfloat16, device=None, **ov):
    return DecoderTextEncoder(DecoderTextConfig(**{**DecoderTextConfig.qwen3_4b().__dict__, **ov}), dtype, device)


@register_model("gemma3_encoder")
def build_gemma3(dtype=torch.bfloat16, device=None, **ov):
    return DecoderTextEncoder(DecoderTextConfig(**{**DecoderTextConfig.gemma3_like().__dict__, **ov}), dtype, device)

"""Trainable SD3.5 adapter projections used when the backbone is frozen.

The reference's SD3.5 trainer puts three small trainable maps around the frozen MMDiT
(crates/training/src/sd35/projections.rs:16-214):

* ``Latent1x1Conv``  -- 16-channel latent ``[B, 16, H, W]`` -> ``[B, hidden, H, W]`` (a 1x1
  convolution, i.e. one GEMM over the pixels), weight ``N(0, 1/sqrt(16))``, zero bias;
* ``TextLinearPad``  -- concatenated text features ``[B, S, 6144]`` cut or zero-padded to 77
  tokens, then projected to ``hidden``;
* ``VelocityHead``   -- ``[B, hidden, H, W]`` -> 16-channel velocity ``[B, 16, H, W]``.

The reference computes them as fp32 matmuls on permuted copies. Here the latent is read
channels-last so the pixel GEMM needs no transposed copy, and the GEMM runs through the
framework's ``Linear`` (tcgen05 kernel on the GPU, fp32 accumulate), which also makes the three
maps adapter-injectable like any other projection.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from .layers import Linear

TARGET_TOKENS = 77
TEXT_INPUT_DIM = 6144
LATENT_CHANNELS = 16


def _init(lin: Linear, fan_in: int, seed=None):
    g = torch.Generator().manual_seed(seed) if seed is not None else None
    with torch.no_grad():
        w = torch.randn(lin.weight.shape, generator=g) * (1.0 / max(1, fan_in)) ** 0.5
        lin.weight.copy_(w.to(lin.weight.dtype))
        if lin.bias is not None:
            lin.bias.zero_()


class Latent1x1Conv(nn.Module):
    def __init__(self, hidden: int, dtype=torch.bfloat16, device=None, seed=None):
        super().__init__()
        self.hidden = hidden
        self.proj = Linear(LATENT_CHANNELS, hidden, dtype=dtype, device=device)
        _init(self.proj, LATENT_CHANNELS, seed)

    def forward(self, latents: torch.Tensor) -> torch.Tensor:
        if latents.dim() != 4:
            raise ValueError(f"Latent1x1Conv expects a 4-D tensor, got {tuple(latents.shape)}")
        B, C, H, W = latents.shape
        if C != LATENT_CHANNELS:
            raise ValueError(f"latent channels mismatch: expected {LATENT_CHANNELS}, got {C}")
        x = latents.permute(0, 2, 3, 1).reshape(B, H * W, C).to(self.proj.weight.dtype)
        return self.proj(x).view(B, H, W, self.hidden).permute(0, 3, 1, 2)


class TextLinearPad(nn.Module):
    def __init__(self, hidden: int, dtype=torch.bfloat16, device=None, seed=None,
                 in_dim: int = TEXT_INPUT_DIM, tokens: int = TARGET_TOKENS):
        super().__init__()
        self.hidden, self.in_dim, self.tokens = hidden, in_dim, tokens
        self.proj = Linear(in_dim, hidden, dtype=dtype, device=device)
        _init(self.proj, in_dim, seed)

    def forward(self, text: torch.Tensor) -> torch.Tensor:
        if text.dim() != 3 or text.shape[-1] != self.in_dim:
            raise ValueError(f"TextLinearPad expects [B, S, {self.in_dim}], got {tuple(text.shape)}")
        B, S, _ = text.shape
        if S > self.tokens:
            text = text[:, : self.tokens]
        elif S < self.tokens:
            text = torch.nn.functional.pad(text, (0, 0, 0, self.tokens - S))
        return self.proj(text.to(self.proj.weight.dtype).contiguous())


class VelocityHead(nn.Module):
    def __init__(self, hidden: int, dtype=torch.bfloat16, device=None, seed=None):
        super().__init__()
        self.proj = Linear(hidden, LATENT_CHANNELS, dtype=dtype, device=device)
        _init(self.proj, hidden, seed)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if hidden_states.dim() != 4:
            raise ValueError(f"VelocityHead expects a 4-D tensor, got {tuple(hidden_states.shape)}")
        B, C, H, W = hidden_states.shape
        x = hidden_states.permute(0, 2, 3, 1).reshape(B, H * W, C).to(self.proj.weight.dtype)
        return self.proj(x).view(B, H, W, LATENT_CHANNELS).permute(0, 3, 1, 2)


def trainable_projections(hidden: int, dtype=torch.bfloat16, device=None, seed=0):
    """The three maps as one ``ModuleDict`` (keys ``latent_in``, ``text_in``, ``velocity_out``)."""
    return nn.ModuleDict({
        "latent_in": Latent1x1Conv(hidden, dtype, device, seed),
        "text_in": TextLinearPad(hidden, dtype, device, seed + 1),
        "velocity_out": VelocityHead(hidden, dtype, device, seed + 2),
    })

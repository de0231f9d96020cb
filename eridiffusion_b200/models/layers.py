"""Building blocks shared by the transformer model families.

``Linear`` owns a bf16 weight and routes through the fused linear op; an adapter (LoRA family)
can be attached to it, and a frozen weight can keep a transposed copy so that the input-gradient
GEMM reads a K-major operand (a deliberate HBM-for-speed trade on a 180 GB part).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import functional as F

import os as _os

_KEEP_TRANSPOSE = _os.environ.get("ERI_B200_FROZEN_TRANSPOSE") == "1"


class Linear(nn.Module):
    def __init__(self, in_features, out_features, bias=True, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.empty(out_features, dtype=dtype, device=device)) if bias else None
        self.adapter = None          # set by adapters.inject()
        self._wt = None              # cached transpose of a frozen weight
        self.reset_parameters()

    def reset_parameters(self, gen: torch.Generator | None = None):
        std = 1.0 / math.sqrt(self.in_features)
        with torch.no_grad():
            w = torch.empty(self.weight.shape, dtype=torch.float32, device=self.weight.device)
            w.normal_(0.0, std, generator=gen)
            self.weight.copy_(w)
            if self.bias is not None:
                self.bias.zero_()

    def frozen_transpose(self):
        """[in, out] copy of a weight that does not require grad (built once, on demand).

        Off unless ``ERI_B200_FROZEN_TRANSPOSE=1``: the GEMM reads W as an MN-major operand for
        dX = dY W at the same speed as a K-major transposed copy (measured), so the copy only
        costs memory."""
        if not _KEEP_TRANSPOSE or self.weight.requires_grad or not self.weight.is_cuda:
            return None
        if self._wt is None or self._wt.device != self.weight.device:
            self._wt = self.weight.detach().t().contiguous()
        return self._wt

    def drop_transpose(self):
        self._wt = None

    def forward(self, x, act=None, residual=None, gate=None):
        if self.adapter is not None:
            return self.adapter(self, x, act=act, residual=residual, gate=gate)
        return F.linear(x, self.weight, self.bias, act=act, residual=residual, gate=gate,
                        wt=self.frozen_transpose() if torch.is_grad_enabled() else None)

    def extra_repr(self):
        return f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}"


def _pair_spec(lin):
    """(weight, bias, lora triple or None) of a layer whose forward is exactly one fused linear: a plain
    ``Linear`` without hooks, bare or with a plain LoRA adapter that applies no dropout. None otherwise."""
    if type(lin) is not Linear or lin._forward_hooks or lin._forward_pre_hooks or _KEEP_TRANSPOSE:
        return None
    ad = lin.adapter
    if ad is None:
        return lin.weight, lin.bias, None
    if getattr(ad, "kind", None) != "lora" or type(ad).__name__ != "LoRA" or ad._forward_hooks:
        return None
    if ad.dropout > 0 and ad.training:
        return None
    return lin.weight, lin.bias, (ad.lora_A, ad.lora_B, ad.scale)


def linear_pair(lin0, x0, lin1, x1, act=None, residual=(None, None), gate=(None, None)):
    """``(lin0(x0), lin1(x1))`` for two layers of equal shape (the image and the text projection of a
    dual-stream block). When both are plain or plain-LoRA layers their main GEMMs run as one grouped launch
    (``F.linear_pair``), so the small text-stream product fills the last, partly empty round of the image
    one instead of leaving most SMs idle in a launch of its own."""
    s0, s1 = _pair_spec(lin0), _pair_spec(lin1)
    if s0 is None or s1 is None or not F._GEMM_GROUP:
        return (lin0(x0, act=act, residual=residual[0], gate=gate[0]),
                lin1(x1, act=act, residual=residual[1], gate=gate[1]))
    return F.linear_pair(x0, (*s0, residual[0], gate[0]), x1, (*s1, residual[1], gate[1]), act=act)


def mlp_pair(up0, down0, x0, up1, down1, x1, act="gelu", residual=(None, None), gate=(None, None)):
    """``(down0(act(up0(x0))), down1(act(up1(x1))))`` with residual and gate on the down-projections: the MLPs
    of the image and the text stream of a dual-stream block. When all four layers qualify for grouped
    launches, the gates are not trainable and ``ERI_B200_MLP_FUSE=1``, the activation's derivative is applied in
    the epilogue of the down-projections' input-gradient GEMM instead of in a pass of its own. Off by default:
    the epilogue's reads of the pre-activation cost the GEMM more than the separate 25 us pass (FLUX LoRA step
    202.4-203.2 ms fused against 199.6-199.8 ms, alternating runs on one GPU)."""
    su0, sd0, su1, sd1 = _pair_spec(up0), _pair_spec(down0), _pair_spec(up1), _pair_spec(down1)
    fuse = (_MLP_FUSE and F._GEMM_GROUP and act in ("gelu", "silu") and None not in (su0, sd0, su1, sd1)
            and not any(g is not None and g.requires_grad for g in gate) and torch.is_grad_enabled())
    if fuse:
        lu0, lu1 = (*su0, None, None), (*su1, None, None)
        ld0, ld1 = (*sd0, residual[0], gate[0]), (*sd1, residual[1], gate[1])
        h_shape0 = (*x0.shape[:-1], up0.out_features)
        h_shape1 = (*x1.shape[:-1], up1.out_features)
        # stand-ins with the hidden activations' shape, device and dtype (no storage) for the second check
        fuse = (F.linear_pair_ok(x0, lu0, x1, lu1)
                and F.linear_pair_ok(x0.new_empty(1).expand(h_shape0), ld0, x1.new_empty(1).expand(h_shape1), ld1))
    if not fuse:
        h0, h1 = linear_pair(up0, x0, up1, x1, act=act)
        return linear_pair(down0, h0, down1, h1, residual=residual, gate=gate)
    p0, p1, h0, h1 = F.linear_pair(x0, lu0, x1, lu1, act=act, emit_pre=True)
    return F.linear_pair(h0, ld0, h1, ld1, act_in=act, x_pre=(p0, p1))


_MLP_FUSE = _os.environ.get("ERI_B200_MLP_FUSE", "0") == "1"


class SmallLinear(Linear):
    """Linear applied to a few conditioning rows (adaLN modulation, embedders)."""

    def forward(self, x, silu_in=False):
        return F.small_linear(x, self.weight, self.bias, silu_in=silu_in)


def timestep_embedding(t, dim, max_period=10000.0, time_factor=1000.0):
    """Sinusoidal embedding [B, dim] of t in [0, 1] scaled by ``time_factor``."""
    t = t.float() * time_factor
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t[:, None] * freqs[None]
    emb = torch.cat([torch.cos(args), torch.sin(args)], dim=-1)
    if dim % 2:
        emb = torch.cat([emb, torch.zeros_like(emb[:, :1])], dim=-1)
    return emb


class MLPEmbedder(nn.Module):
    def __init__(self, in_dim, hidden, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.in_layer = SmallLinear(in_dim, hidden, dtype=dtype, device=device)
        self.out_layer = SmallLinear(hidden, hidden, dtype=dtype, device=device)

    def forward(self, x):
        return self.out_layer(self.in_layer(x), silu_in=True)


class Modulation(nn.Module):
    """adaLN modulation: Linear(SiLU(vec)) split into ``n`` chunks of width ``dim``."""

    def __init__(self, dim, n, dtype=torch.bfloat16, device=None, cond_dim=None):
        super().__init__()
        self.n, self.dim = n, dim
        self.lin = SmallLinear(cond_dim or dim, n * dim, dtype=dtype, device=device)

    def forward(self, vec):
        out = self.lin(vec, silu_in=True)          # [B, n*dim]
        return out.split(self.dim, dim=-1)          # strided views, consumed without copies


def rope_table(ids, axes_dim, theta=10000.0):
    """cos/sin tables [L, sum(axes_dim)/2] (fp32) for N-axis rotary embedding of interleaved
    pairs; ``ids`` is [L, n_axes] (FLUX: (type, row, col) with axes_dim (16, 56, 56);
    reference layout: src/kernels/rope.cu:49-57)."""
    cos, sin = [], []
    for i, d in enumerate(axes_dim):
        scale = torch.arange(0, d, 2, dtype=torch.float64, device=ids.device) / d
        omega = 1.0 / (theta ** scale)
        ang = ids[:, i].double()[:, None] * omega[None]
        cos.append(torch.cos(ang))
        sin.append(torch.sin(ang))
    return torch.cat(cos, -1).float(), torch.cat(sin, -1).float()


def image_ids(h, w, device=None, t=0):
    ids = torch.zeros(h, w, 3, device=device)
    ids[..., 0] = t
    ids[..., 1] = torch.arange(h, device=device)[:, None]
    ids[..., 2] = torch.arange(w, device=device)[None, :]
    return ids.view(h * w, 3)


class RMSNormScale(nn.Module):
    """Learned per-head scale used by RMS QK-norm (the normalisation itself is fused downstream)."""

    def __init__(self, dim, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.scale = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

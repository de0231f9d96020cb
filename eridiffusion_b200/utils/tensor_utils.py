"""Broadcast, stable-softmax and safe-math helpers.

Reference: crates/training/src/tensor_utils.rs (broadcast helpers, numerically stable softmax /
log-softmax, safe division / log / sqrt, NaN scrubbing, fp32-semantics reductions) and
crates/core/src/safe_ops.rs. These are the host-framework versions used by losses, metrics and
samplers; the hot path has its own fused kernels.
"""
from __future__ import annotations

import torch


def broadcast_to_rank(v: torch.Tensor, like: torch.Tensor) -> torch.Tensor:
    """[B] or [B, 1...] -> [B, 1, ..., 1] with the rank of ``like``."""
    return v.reshape(v.shape[0], *([1] * (like.dim() - 1)))


def broadcast_over_tokens(v: torch.Tensor, tokens: int) -> torch.Tensor:
    """[B, D] -> a [B, tokens, D] view (no copy)."""
    return v.unsqueeze(1).expand(-1, tokens, -1)


def stable_softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """Softmax in fp32 with the row maximum subtracted; rows that are entirely ``-inf`` give zeros
    instead of NaN (a fully masked query). Returns ``x.dtype``."""
    xf = x.float()
    m = xf.amax(dim=dim, keepdim=True)
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    e = torch.exp(xf - m)
    s = e.sum(dim=dim, keepdim=True)
    return (e / s.clamp_min(torch.finfo(torch.float32).tiny)).to(x.dtype)


def stable_log_softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    xf = x.float()
    m = xf.amax(dim=dim, keepdim=True)
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
    z = xf - m
    return (z - torch.log(torch.exp(z).sum(dim=dim, keepdim=True).clamp_min(torch.finfo(torch.float32).tiny))).to(x.dtype)


def safe_div(a, b, eps: float = 1e-8):
    """a / b with |b| kept at least ``eps`` (sign preserved; b == 0 counts as +eps)."""
    b = torch.as_tensor(b, dtype=a.dtype if torch.is_tensor(a) else None)
    sign = torch.where(b < 0, -torch.ones_like(b), torch.ones_like(b))
    return a / (sign * b.abs().clamp_min(eps))


def safe_log(x, eps: float = 1e-12):
    return torch.log(x.clamp_min(eps))


def safe_sqrt(x, eps: float = 0.0):
    return torch.sqrt(x.clamp_min(eps))


def safe_rsqrt(x, eps: float = 1e-12):
    return torch.rsqrt(x.clamp_min(eps))


def nan_to_zero(x):
    return torch.nan_to_num(x, nan=0.0, posinf=0.0, neginf=0.0)


def has_nonfinite(x) -> bool:
    return not bool(torch.isfinite(x).all())


def mean_fp32(x, dim=None, keepdim=False):
    """Reduction with fp32 accumulation whatever the storage dtype; result in fp32."""
    return x.float().mean() if dim is None else x.float().mean(dim=dim, keepdim=keepdim)


def sum_as(x, dim, dtype, keepdim=True):
    """``sum_dim_keepdim_as``: reduce in fp32, store as ``dtype``."""
    return x.float().sum(dim=dim, keepdim=keepdim).to(dtype)


def clamp_finite(x, lo, hi):
    """Clamp and replace NaN with the interval's midpoint (the reference clamps predictions and
    targets to +-10 before the loss)."""
    return torch.nan_to_num(x, nan=0.5 * (lo + hi)).clamp(lo, hi)

"""Numerical-stability switches (crates/common/stability: ``allow_tf32``, ``sanitize_attn_mask``
clamping additive masks to [-1e4, 0], ``compute_loss_fp32``)."""
from __future__ import annotations

import torch


def allow_tf32(enabled: bool = True) -> None:
    """fp32 matmuls/convolutions may use TF32 tensor cores (bf16 paths are unaffected)."""
    torch.backends.cuda.matmul.allow_tf32 = enabled
    torch.backends.cudnn.allow_tf32 = enabled


def sanitize_attn_mask(mask: torch.Tensor | None, dtype=torch.bfloat16):
    """Boolean masks become additive (0 keep / -1e4 drop); additive masks are clamped to
    [-1e4, 0] so that a fully masked row yields a uniform, finite softmax instead of NaN."""
    if mask is None:
        return None
    if mask.dtype == torch.bool:
        out = torch.zeros(mask.shape, dtype=dtype, device=mask.device)
        return out.masked_fill(~mask, -1e4)
    return mask.clamp(min=-1e4, max=0.0).to(dtype)


def compute_loss_fp32(pred: torch.Tensor, target: torch.Tensor, reduction="mean"):
    """MSE with fp32 accumulation whatever the input dtype."""
    d = pred.float() - target.float()
    sq = d * d
    return sq.mean() if reduction == "mean" else (sq.sum() if reduction == "sum" else sq)

"""Loss objects by name, the multi-scale "LPIPS proxy", and the masked epsilon loss with an
annealed residual clamp.

* ``create_loss(kind, weight, ...)``: ``mse | mae | l1 | huber | lpips | perceptual | flow_matching
  | v`` as callables ``(pred, target) -> scalar`` with a validated non-negative finite weight
  (crates/training/src/loss.rs:22-43, 386-445). ``perceptual``, ``flow_matching`` and ``v`` are
  weighted mean squared errors in the reference too.
* ``LpipsProxyLoss``: not the learned metric. The reference compares hand-set filter responses:
  a 3x3 Laplacian-like edge filter at full resolution, a 4-neighbour Laplacian at 1/2 and a
  second-difference texture filter at 1/4 (mean-pooled grey images), plus per-channel mean and
  standard deviation for RGB inputs, and averages the mean squared differences
  (crates/training/src/loss.rs:190-330).
* ``masked_eps_loss_safe``: mean squared error over [B, T, D] with an optional [B, T] mask, where the
  residual is clamped symmetrically during the first ``clamp_warmup_steps`` steps; the limit moves
  from ``clamp_start`` to ``clamp_end`` on half a cosine (crates/training/src/policy.rs:169-214).
  With a mask the mean is over kept elements (the reference divides by all elements, which
  shrinks the loss with the masked fraction).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as tf


def _check_weight(w: float) -> float:
    w = float(w)
    if not math.isfinite(w) or w < 0.0:
        raise ValueError(f"invalid loss weight: {w}")
    return w


class _WeightedLoss:
    name = "loss"

    def __init__(self, weight: float = 1.0):
        self.weight = _check_weight(weight)

    def _check(self, pred, target):
        if pred.shape != target.shape:
            raise ValueError(f"{self.name}: pred {tuple(pred.shape)} and target {tuple(target.shape)} must match")

    def __call__(self, pred, target):
        self._check(pred, target)
        return self.compute(pred.float(), target.float()) * self.weight


class MseLoss(_WeightedLoss):
    name = "MSE"

    def compute(self, p, t):
        return (p - t).pow(2).mean()


class MaeLoss(_WeightedLoss):
    name = "MAE"

    def compute(self, p, t):
        return (p - t).abs().mean()


class HuberLoss(_WeightedLoss):
    name = "Huber"

    def __init__(self, weight=1.0, delta=1.0):
        super().__init__(weight)
        self.delta = float(delta)

    def compute(self, p, t):
        d = p - t
        a = d.abs()
        return torch.where(a <= self.delta, 0.5 * d.pow(2), self.delta * (a - 0.5 * self.delta)).mean()


class PerceptualLoss(MseLoss):
    name = "Perceptual"


class FlowMatchingLoss(MseLoss):
    name = "FlowMatching"


class VLoss(MseLoss):
    name = "V"


class LpipsProxyLoss(_WeightedLoss):
    name = "LPIPS"
    _K1 = (-1.0, -1.0, -1.0, -1.0, 8.0, -1.0, -1.0, -1.0, -1.0)
    _K2 = (0.0, -1.0, 0.0, -1.0, 4.0, -1.0, 0.0, -1.0, 0.0)
    _K3 = (1.0, -2.0, 1.0, -2.0, 4.0, -2.0, 1.0, -2.0, 1.0)

    @staticmethod
    def _down(x, f):
        return tf.avg_pool2d(x, f)

    def features(self, x):
        """[B, C, H, W] -> list of feature tensors (H and W multiples of 4)."""
        k = lambda v: torch.tensor(v, dtype=x.dtype, device=x.device).view(1, 1, 3, 3)
        grey = x.mean(1, keepdim=True) if x.shape[1] == 3 else x
        if grey.shape[1] != 1:
            grey = grey.reshape(-1, 1, *grey.shape[-2:])            # other channel counts: filter each plane
        out = [tf.conv2d(grey, k(self._K1), padding=1).abs(),
               tf.conv2d(self._down(grey, 2), k(self._K2), padding=1).abs(),
               tf.conv2d(self._down(grey, 4), k(self._K3), padding=1).abs()]
        if x.shape[1] == 3:
            out.append(x.mean((2, 3), keepdim=True))
            out.append(x.var((2, 3), unbiased=False, keepdim=True).sqrt())
        return out

    def compute(self, p, t):
        if p.dim() != 4:
            raise ValueError("LPIPS: expects [B, C, H, W]")
        fp, ft = self.features(p), self.features(t)
        return sum((a - b).pow(2).mean() for a, b in zip(fp, ft)) / len(fp)


_KINDS = {"mse": MseLoss, "mae": MaeLoss, "l1": MaeLoss, "huber": HuberLoss, "lpips": LpipsProxyLoss,
          "perceptual": PerceptualLoss, "flow_matching": FlowMatchingLoss, "flowmatching": FlowMatchingLoss, "v": VLoss}


def create_loss(kind: str, weight: float = 1.0, **kw):
    k = kind.lower()
    if k not in _KINDS:
        raise ValueError(f"unknown loss {kind!r}; known: {sorted(set(_KINDS))}")
    return _KINDS[k](weight, **kw)


def clamp_limit(global_step: int, warmup_steps: int, clamp_start: float, clamp_end: float):
    """Residual clamp in effect at ``global_step`` (``None`` once the warm-up is over)."""
    if warmup_steps <= 0 or global_step >= warmup_steps:
        return None
    k = 0.5 * (1.0 + math.cos(math.pi * global_step / max(1, warmup_steps)))
    return clamp_end + (clamp_start - clamp_end) * k


def masked_eps_loss_safe(pred_eps, true_eps, mask_bt=None, global_step: int = 0, clamp_warmup_steps: int = 0,
                         clamp_start: float = 1.0, clamp_end: float = 10.0):
    """pred / true [B, T, D]; mask [B, T] (1 = keep) or None. The prediction keeps its dtype and its
    autograd history; the target is cast to it."""
    diff = pred_eps - true_eps.to(pred_eps.dtype)
    lim = clamp_limit(global_step, clamp_warmup_steps, clamp_start, clamp_end)
    if lim is not None:
        diff = diff.clamp(-lim, lim)
    sq = diff.float().pow(2)
    if mask_bt is None:
        return sq.mean()
    m = mask_bt.to(sq.dtype).unsqueeze(-1)
    return (sq * m).sum() / (m.sum() * sq.shape[-1]).clamp_min(1.0)

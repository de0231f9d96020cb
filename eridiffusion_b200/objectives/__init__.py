"""Training objectives: timestep samplers, forward-noising coefficients, regression targets and
loss weights for flow matching and DDPM-style (eps / v / x0) training.

Every objective reduces to four per-sample coefficients (a, s, ca, cb):
``x_t = a * x0 + s * eps`` and ``target = ca * eps + cb * x0`` — the form the fused
``noise_mix`` kernel consumes.

Reference behaviour reproduced here:
* flow matching ``x_t = (1-t) x0 + t eps``, target ``eps - x0``
  (crates/training/src/pipelines/flux_pipeline.rs:185-216, sd3_pipeline.rs:160-182);
* sigmoid-shift schedule ``sigma(t) = sigmoid(shift (2t-1))`` (src/trainers/pipeline_flux_lora.rs:288-363);
* dynamic shifting ``shift = lerp(0.5, 1.15; seq 256 -> 4096)``, ``t' = t + shift t (1-t)``
  (flux_pipeline.rs:248-265);
* SD3.5 ``t = 0.5 tanh(shift (2u-1)) + 0.5`` and weight ``sqrt(snr/(1+snr))``
  (crates/training/src/sd35_trainer_impl.rs:146-169, 234-290);
* DDPM: 1000 steps, scaled-linear betas 0.00085 -> 0.012, eps / v / x0 targets, zero-terminal-SNR,
  alpha-bar clamped to [1e-8, 0.999] (crates/training/src/pipelines/sdxl_pipeline.rs:52-194);
* min-SNR-gamma weight ``min(snr, gamma) / snr`` (src/trainers/snr_weighting.rs:23-74);
* the phase-4 FLUX trainer's additive-noise eps objective ``x_t = x0 + sigma eps``, target ``eps``,
  ``sigma = sigma_min r^{-t}`` with ``r = max(sigma_max / sigma_min, 1 + 1e-6)``, t uniform in
  [0, 1), sigma clamped to [1e-3, 1] (crates/training/src/flux_trainer.rs:312-325, 410-414;
  crates/training/src/policy.rs:90-95).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


# ------------------------------------------------------------------------- timestep samplers
def sample_uniform(n, gen=None, device="cpu"):
    return torch.rand(n, generator=gen, device=device)


def sample_logit_normal(n, mean=0.0, std=1.0, gen=None, device="cpu"):
    return torch.sigmoid(torch.randn(n, generator=gen, device=device) * std + mean)


def shift_time(t, shift):
    """Resolution shift used by flow models: t' = s t / (1 + (s - 1) t)."""
    return shift * t / (1.0 + (shift - 1.0) * t)


def sigmoid_shift(t, shift=3.0):
    return torch.sigmoid(shift * (2.0 * t - 1.0))


def tanh_shift(u, shift=3.0, eps=1e-5):
    return (0.5 * torch.tanh(shift * (2.0 * u - 1.0)) + 0.5).clamp(eps, 1.0 - eps)


def dynamic_shift(t, seq_len, base_len=256, max_len=4096, base_shift=0.5, max_shift=1.15):
    m = (max_shift - base_shift) / (max_len - base_len)
    shift = base_shift + m * (min(max(seq_len, base_len), max_len) - base_len)
    return t + shift * t * (1.0 - t)


def sample_timesteps(kind, n, gen=None, device="cpu", **kw):
    """kind: uniform | logit_normal | shifted_logit_normal | sigmoid_shift | tanh_shift |
    dynamic_shift. Returns t in (0, 1)."""
    if kind == "uniform":
        return sample_uniform(n, gen, device)
    if kind == "logit_normal":
        return sample_logit_normal(n, kw.get("mean", 0.0), kw.get("std", 1.0), gen, device)
    if kind == "shifted_logit_normal":
        t = sample_logit_normal(n, kw.get("mean", 0.0), kw.get("std", 1.0), gen, device)
        return shift_time(t, kw.get("shift", 3.0))
    if kind == "sigmoid_shift":
        return sigmoid_shift(sample_uniform(n, gen, device), kw.get("shift", 3.0))
    if kind == "tanh_shift":
        return tanh_shift(sample_uniform(n, gen, device), kw.get("shift", 3.0))
    if kind == "dynamic_shift":
        return dynamic_shift(sample_uniform(n, gen, device), kw.get("seq_len", 4096))
    raise ValueError(f"unknown timestep sampler {kind!r}")


# ------------------------------------------------------------------------- flow matching
@dataclass
class FlowMatching:
    sampler: str = "logit_normal"
    sampler_kw: dict | None = None
    weighting: str = "none"          # none | snr_sqrt (SD3.5) | over_t (target / max(t, 1e-5))

    def sample_t(self, n, gen=None, device="cpu"):
        return sample_timesteps(self.sampler, n, gen, device, **(self.sampler_kw or {}))

    def coefficients(self, t):
        """[4, B] rows (a, s, ca, cb) for x_t = (1-t) x0 + t eps, target = eps - x0."""
        one = torch.ones_like(t)
        return torch.stack([1.0 - t, t, one, -one]).float()

    def loss_weight(self, t):
        if self.weighting == "snr_sqrt":
            snr = t / (1.0 - t).clamp_min(1e-8)
            return torch.sqrt(snr / (1.0 + snr))
        return None

    def model_time(self, t):
        return t


# ------------------------------------------------------------------------- phase-4 eps objective
@dataclass
class SigmaEps:
    """Additive-noise epsilon prediction of the reference's phase-4 FLUX LoRA trainer: the clean
    latent is NOT scaled down, ``x_t = x0 + sigma(t) eps`` and the network regresses ``eps`` under a
    plain MSE. ``sigma(t) = sigma_min * r^{-t}`` (t uniform in [0, 1)) falls from ``sigma_min`` at
    t = 0 towards ``sigma_min / r`` — the formula is kept exactly as the reference computes it,
    including that ``sigma_max`` only enters through the ratio — and is then bounded to
    [``floor``, ``ceil``] = [1e-3, 1]."""
    sigma_min: float = 0.02
    sigma_max: float = 1.0
    floor: float = 1e-3
    ceil: float = 1.0

    def sample_t(self, n, gen=None, device="cpu"):
        return sample_uniform(n, gen, device)

    def sigma(self, t):
        ratio = max(self.sigma_max / self.sigma_min, 1.0 + 1e-6)
        return (self.sigma_min * torch.exp(-t.float() * math.log(ratio))).clamp(self.floor, self.ceil)

    def coefficients(self, t):
        """[4, B] rows (a, s, ca, cb): x_t = x0 + sigma eps, target = eps."""
        sg = self.sigma(t)
        one, zero = torch.ones_like(sg), torch.zeros_like(sg)
        return torch.stack([one, sg, one, zero]).float()

    def loss_weight(self, t):
        return None

    def model_time(self, t):
        return self.sigma(t)


# ------------------------------------------------------------------------- DDPM family
def make_betas(schedule="scaled_linear", n=1000, beta_start=0.00085, beta_end=0.012):
    if schedule == "linear":
        return torch.linspace(beta_start, beta_end, n, dtype=torch.float64)
    if schedule == "scaled_linear":
        return torch.linspace(beta_start ** 0.5, beta_end ** 0.5, n, dtype=torch.float64) ** 2
    if schedule == "cosine":
        s = 0.008
        x = torch.linspace(0, n, n + 1, dtype=torch.float64)
        ac = torch.cos(((x / n) + s) / (1 + s) * math.pi * 0.5) ** 2
        ac = ac / ac[0]
        return (1 - ac[1:] / ac[:-1]).clamp(max=0.999)
    raise ValueError(schedule)


def rescale_zero_terminal_snr(betas):
    alphas_bar_sqrt = torch.cumprod(1.0 - betas, 0).sqrt()
    a0, aT = alphas_bar_sqrt[0].clone(), alphas_bar_sqrt[-1].clone()
    alphas_bar_sqrt = (alphas_bar_sqrt - aT) * a0 / (a0 - aT)
    ab = alphas_bar_sqrt ** 2
    alphas = torch.cat([ab[:1], ab[1:] / ab[:-1]])
    return 1.0 - alphas


@dataclass
class DDPM:
    num_steps: int = 1000
    schedule: str = "scaled_linear"
    beta_start: float = 0.00085
    beta_end: float = 0.012
    prediction: str = "epsilon"      # epsilon | v | sample
    zero_terminal_snr: bool = False
    min_snr_gamma: float | None = None

    def __post_init__(self):
        betas = make_betas(self.schedule, self.num_steps, self.beta_start, self.beta_end)
        if self.zero_terminal_snr:
            betas = rescale_zero_terminal_snr(betas)
        self.betas = betas
        self.alphas_cumprod = torch.cumprod(1.0 - betas, 0).clamp(1e-8, 0.999).float()

    def sample_t(self, n, gen=None, device="cpu"):
        return torch.randint(0, self.num_steps, (n,), generator=gen, device=device)

    def _ab(self, t):
        idx = t.round().long().clamp(0, self.num_steps - 1)
        return self.alphas_cumprod.to(t.device)[idx]

    def coefficients(self, t):
        ab = self._ab(t)
        sa, sn = ab.sqrt(), (1.0 - ab).sqrt()
        zero, one = torch.zeros_like(sa), torch.ones_like(sa)
        if self.prediction == "epsilon":
            ca, cb = one, zero
        elif self.prediction == "v":
            ca, cb = sa, -sn
        elif self.prediction == "sample":
            ca, cb = zero, one
        else:
            raise ValueError(self.prediction)
        return torch.stack([sa, sn, ca, cb]).float()

    def snr(self, t):
        ab = self._ab(t)
        return ab / (1.0 - ab)

    def loss_weight(self, t):
        if self.min_snr_gamma is None:
            return None
        snr = self.snr(t)
        w = torch.minimum(snr, torch.full_like(snr, self.min_snr_gamma)) / snr
        if self.prediction == "v":
            w = torch.minimum(snr, torch.full_like(snr, self.min_snr_gamma)) / (snr + 1.0)
        return w

    def model_time(self, t):
        return t.float()


def min_snr_weight(snr, gamma=5.0):
    return torch.minimum(snr, torch.full_like(snr, gamma)) / snr


# ------------------------------------------------------------------------- losses
def loss_fn(kind, pred, target, weight=None, mask=None, huber_delta=1.0):
    """kind: mse | l1 | huber. ``weight`` is per sample, ``mask`` per element (1 = keep).
    (crates/training/src/loss.rs:22-43, sdxl_pipeline.rs:497-521.)"""
    from ..ops import functional as F
    if kind == "mse" and mask is None:
        return F.mse_loss(pred, target, weight)
    d = pred.float() - target.float()
    if kind == "mse":
        e = d.pow(2)
    elif kind == "l1":
        e = d.abs()
    elif kind == "huber":
        a = d.abs()
        e = torch.where(a <= huber_delta, 0.5 * d.pow(2), huber_delta * (a - 0.5 * huber_delta))
    else:
        # named objects (lpips / perceptual / mae / flow_matching / v): whole-tensor reductions
        from .losses import create_loss
        if weight is not None or mask is not None:
            raise ValueError(f"loss {kind!r} takes no per-sample weight or mask")
        return create_loss(kind)(pred, target)
    if weight is not None:
        e = e * weight.float().view(-1, *([1] * (e.dim() - 1)))
    if mask is not None:
        m = mask.float().expand_as(e)
        return (e * m).sum() / m.sum().clamp_min(1.0)
    return e.mean()


def mean_flow_target(eps, x0, t, r):
    """Mean-flow regression target ``(eps - x0) / max(r - t, 1e-4)`` for two times t < r
    (crates/training/src/pipelines/sd3_pipeline.rs:272-343)."""
    dt = (r - t).clamp_min(1e-4).view(-1, *([1] * (x0.dim() - 1)))
    return (eps - x0) / dt

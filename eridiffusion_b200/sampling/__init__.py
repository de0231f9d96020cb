"""Inference samplers used for validation images during training and by the generate CLIs.

* flow-matching Euler with the resolution shift ``t' = s t / (1 + (s-1) t)``
  (debug_full_loop.py:46-52; src/inference/flux_sampling.rs:64-71 shifted-sigmoid schedule);
* Karras sigmas (rho 7) and a log-linear schedule over [0.029, 14]
  (crates/training/src/sdxl/scheduler.rs:45-78);
* Euler, Euler-ancestral (crates/common/sampler/src/euler_a.rs:5-50), Heun
  (crates/training/src/sdxl/infer.rs:218-219, 520-523);
* DDIM and DPM-Solver++(2M) (src/schedulers/mod.rs:79-305, 309-410);
* classifier-free guidance mix (crates/training/src/sdxl/infer.rs:726).

Every sampler takes ``denoise(x, sigma_or_t) -> prediction`` so that it is model agnostic.
"""
from __future__ import annotations

import math

import torch

from ..objectives import make_betas


def cfg_mix(cond, uncond, scale):
    return uncond + scale * (cond - uncond)


# ------------------------------------------------------------------------- schedules
def flow_timesteps(steps, shift=1.0, device="cpu"):
    t = torch.linspace(1.0, 0.0, steps + 1, device=device)
    if shift != 1.0:
        t = shift * t / (1.0 + (shift - 1.0) * t)
    return t


def flux_shift_for_seq(seq_len, base_len=256, max_len=4096, base_shift=0.5, max_shift=1.15):
    m = (max_shift - base_shift) / (max_len - base_len)
    return math.exp(base_shift + m * (seq_len - base_len))


def karras_sigmas(steps, sigma_min=0.029, sigma_max=14.0, rho=7.0, device="cpu"):
    ramp = torch.linspace(0, 1, steps, device=device)
    mn, mx = sigma_min ** (1 / rho), sigma_max ** (1 / rho)
    s = (mx + ramp * (mn - mx)) ** rho
    return torch.cat([s, s.new_zeros(1)])


def loglinear_sigmas(steps, sigma_min=0.029, sigma_max=14.0, device="cpu"):
    s = torch.exp(torch.linspace(math.log(sigma_max), math.log(sigma_min), steps, device=device))
    return torch.cat([s, s.new_zeros(1)])


def ddpm_sigmas(num_train=1000, schedule="scaled_linear", beta_start=0.00085, beta_end=0.012):
    ac = torch.cumprod(1 - make_betas(schedule, num_train, beta_start, beta_end), 0)
    return ((1 - ac) / ac).sqrt().float()


def sigma_to_timestep(sigma, train_sigmas):
    """Nearest-neighbour inverse of the training sigma table (log space)."""
    ls = train_sigmas.log()
    d = (sigma.log().view(-1, 1) - ls.view(1, -1)).abs()
    return d.argmin(1)


# ------------------------------------------------------------------------- flow matching
@torch.no_grad()
def sample_flow_euler(velocity, x, steps=20, shift=1.0):
    """x: noise at t=1; ``velocity(x, t[B]) -> v`` with dx/dt = v. Returns the sample at t=0."""
    ts = flow_timesteps(steps, shift, x.device)
    for i in range(steps):
        t, tn = ts[i], ts[i + 1]
        v = velocity(x, t.expand(x.shape[0]))
        x = x + (tn - t) * v
    return x


# ------------------------------------------------------------------------- k-diffusion style (eps models)
def _to_d(x, sigma, denoised):
    return (x - denoised) / sigma


@torch.no_grad()
def sample_euler(denoise, x, sigmas):
    """``denoise(x, sigma) -> x0 estimate``; x starts as noise * sigmas[0]."""
    for i in range(len(sigmas) - 1):
        d = _to_d(x, sigmas[i], denoise(x, sigmas[i]))
        x = x + d * (sigmas[i + 1] - sigmas[i])
    return x


@torch.no_grad()
def sample_euler_ancestral(denoise, x, sigmas, eta=1.0, gen=None):
    for i in range(len(sigmas) - 1):
        s, sn = sigmas[i], sigmas[i + 1]
        den = denoise(x, s)
        su = min(sn, eta * (sn ** 2 * (s ** 2 - sn ** 2) / s ** 2) ** 0.5) if sn > 0 else sn * 0
        sd = (sn ** 2 - su ** 2) ** 0.5
        x = x + _to_d(x, s, den) * (sd - s)
        if sn > 0:
            x = x + torch.randn(x.shape, generator=gen, device=x.device, dtype=x.dtype) * su
    return x


@torch.no_grad()
def sample_heun(denoise, x, sigmas):
    for i in range(len(sigmas) - 1):
        s, sn = sigmas[i], sigmas[i + 1]
        d = _to_d(x, s, denoise(x, s))
        x2 = x + d * (sn - s)
        if sn == 0:
            x = x2
        else:
            d2 = _to_d(x2, sn, denoise(x2, sn))
            x = x + 0.5 * (d + d2) * (sn - s)
    return x


@torch.no_grad()
def sample_dpmpp_2m(denoise, x, sigmas):
    old = None
    t_fn = lambda s: -torch.log(s)
    for i in range(len(sigmas) - 1):
        s, sn = sigmas[i], sigmas[i + 1]
        den = denoise(x, s)
        if sn == 0:
            x = den
            break
        t, tn = t_fn(s), t_fn(sn)
        h = tn - t
        if old is None:
            x = (sn / s) * x - (-h).expm1() * den
        else:
            h_last = t - t_fn(sigmas[i - 1])
            r = h_last / h
            dd = (1 + 1 / (2 * r)) * den - (1 / (2 * r)) * old
            x = (sn / s) * x - (-h).expm1() * dd
        old = den
    return x


# ------------------------------------------------------------------------- DDIM on the discrete chain
@torch.no_grad()
def sample_ddim(eps_model, x, steps=50, num_train=1000, schedule="scaled_linear", eta=0.0, gen=None,
                prediction="epsilon"):
    ac = torch.cumprod(1 - make_betas(schedule, num_train), 0).float().to(x.device)
    ts = torch.linspace(num_train - 1, 0, steps).round().long()
    for i, t in enumerate(ts):
        a_t = ac[t]
        a_p = ac[ts[i + 1]] if i + 1 < len(ts) else torch.tensor(1.0, device=x.device)
        out = eps_model(x, t.expand(x.shape[0]).to(x.device))
        if prediction == "v":
            eps = a_t.sqrt() * out + (1 - a_t).sqrt() * x
        elif prediction == "sample":
            eps = (x - a_t.sqrt() * out) / (1 - a_t).sqrt()
        else:
            eps = out
        x0 = (x - (1 - a_t).sqrt() * eps) / a_t.sqrt()
        sig = eta * ((1 - a_p) / (1 - a_t) * (1 - a_t / a_p)).clamp_min(0).sqrt()
        x = a_p.sqrt() * x0 + (1 - a_p - sig ** 2).clamp_min(0).sqrt() * eps
        if eta > 0 and i + 1 < len(ts):
            x = x + sig * torch.randn(x.shape, generator=gen, device=x.device, dtype=x.dtype)
    return x


def eps_denoiser(eps_model, train_sigmas, prediction="epsilon"):
    """Wrap an eps / v model trained on the discrete chain as ``denoise(x, sigma) -> x0``."""
    def denoise(x, sigma):
        s = sigma if torch.is_tensor(sigma) else torch.tensor(sigma, device=x.device)
        t = sigma_to_timestep(s.view(1), train_sigmas.to(x.device)).expand(x.shape[0])
        c_in = 1.0 / (s ** 2 + 1).sqrt()
        out = eps_model(x * c_in, t)
        if prediction == "v":
            return x / (s ** 2 + 1) - out * s / (s ** 2 + 1).sqrt()
        return x - s * out
    return denoise


SAMPLERS = {"euler": sample_euler, "euler_a": sample_euler_ancestral, "heun": sample_heun,
            "dpmpp_2m": sample_dpmpp_2m}


# ------------------------------------------------------------------------- model-level helpers
@torch.no_grad()
def generate_flow(model, txt, pooled, height=1024, width=1024, steps=20, guidance=3.5, shift=None, seed=0,
                  channels=16, patch=2, dtype=torch.bfloat16, neg_txt=None, neg_pooled=None, cfg_scale=1.0):
    """Sample latents [B, C, H/8, W/8] from an MMDiT-style flow model (FLUX / Qwen / SD3 family)."""
    from ..ops import reference as R
    dev = txt.device
    B = txt.shape[0]
    h, w = height // 8, width // 8
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(B, channels, h, w, device=dev, generator=g, dtype=torch.float32).to(dtype)
    tok = R.patchify(x, patch)
    if shift is None:
        shift = flux_shift_for_seq(tok.shape[1])
    gv = torch.full((B,), float(guidance), device=dev)

    def velocity(z, t):
        v = model(z, txt, t, pooled, gv, grid_hw=(h // patch, w // patch))
        if cfg_scale != 1.0 and neg_txt is not None:
            vu = model(z, neg_txt, t, neg_pooled, gv, grid_hw=(h // patch, w // patch))
            v = cfg_mix(v, vu, cfg_scale)
        return v

    tok = sample_flow_euler(velocity, tok, steps, shift)
    return R.unpatchify(tok, channels, h, w, patch)


def latents_to_uint8(img):
    """[B, 3, H, W] in [-1, 1] -> uint8 HWC on the host (clamp((x+1)/2) * 255, the reference's
    post-decode kernel: crates/common/vae/src/sdxl.rs:36-50)."""
    from ..ops import _native as N
    from ..ops import functional as F
    if img.is_cuda and img.dtype == torch.bfloat16 and F.get_backend() == "fused":
        x = img.contiguous()
        out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
        N.check(N.require().eri_post_clamp_u8(x.data_ptr(), out.data_ptr(), x.numel(), N.stream_ptr()), "post_clamp")
    else:
        out = ((img.float() + 1) * 0.5).clamp(0, 1).mul(255).round().to(torch.uint8)
    return out.permute(0, 2, 3, 1).cpu()


def save_png(img_uint8_hwc, path):
    from PIL import Image
    Image.fromarray(img_uint8_hwc.numpy()).save(path)

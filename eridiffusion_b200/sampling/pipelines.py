"""Per-family inference schedules and one pipeline object over every registered model family.

Covers the reference's per-model samplers and its unified front end:

* ``flux_timesteps``: shifted-sigmoid time grid, ``t' = sigmoid(shift * t) / sigmoid(shift)``
  (src/inference/flux_sampling.rs:64-71).
* ``FlowMatchScheduler``: the SD3.5 scheduler, ``sigma(t) = sigmoid(shift * (2 t - 1))`` with an
  Euler velocity step (src/inference/sd35_sampling.rs:43-92).
* ``ltx_sigma_schedule`` / ``LTX_DISTILLED_SIGMAS`` / ``euler_denoise_flow``: token-count dependent
  shift with an optional terminal value, the fixed distilled grid, and the Euler loop whose last
  step returns the denoised sample ``x - sigma * v`` (src/inference/ltx2_sampling.rs:5-90).
* ``ModelType`` / ``MemoryConfig`` / ``UnifiedInferencePipeline``: model type from a checkpoint
  path, per-type memory policy, ``generate`` / ``generate_image``
  (src/inference/unified_inference.rs:10-215, 940). The reference sizes its policy for 16-20 GB
  cards (CPU offload, sequential offload, 256-512 pixel VAE tiles); here the defaults keep every
  model resident in 180 GB and offloading is something the caller switches on.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass

import torch

from . import (cfg_mix, ddpm_sigmas, eps_denoiser, generate_flow, karras_sigmas, latents_to_uint8, sample_ddim,
               sample_dpmpp_2m, sample_euler, sample_euler_ancestral, sample_heun)


# ------------------------------------------------------------------------------------ schedules
def flux_timesteps(steps: int, shift: float = 3.0, device="cpu"):
    """``steps + 1`` times from 1 to 0 on the shifted-sigmoid grid."""
    t = torch.linspace(1.0, 0.0, steps + 1, device=device)
    sig = lambda v: 1.0 / (1.0 + torch.exp(-v))
    return sig(shift * t) / sig(torch.tensor(float(shift), device=device))


class FlowMatchScheduler:
    """Linear time grid 1 -> 0 mapped through ``sigmoid(shift * (2 t - 1))``; ``step`` moves the
    sample along the predicted velocity by the difference of two mapped times."""

    def __init__(self, num_inference_steps: int, shift: float = 3.0):
        if num_inference_steps < 2:
            raise ValueError("FlowMatchScheduler needs at least 2 steps")
        self.num_inference_steps, self.shift = num_inference_steps, float(shift)
        self.timesteps = [1.0 - i / (num_inference_steps - 1) for i in range(num_inference_steps)]

    def apply_shift(self, t: float) -> float:
        return 1.0 / (1.0 + math.exp(-self.shift * (2.0 * t - 1.0)))

    def sigmas(self, device="cpu"):
        """Mapped times followed by a final 0, usable with ``euler_denoise_flow``."""
        return torch.tensor([self.apply_shift(t) for t in self.timesteps] + [0.0], device=device)

    def step(self, model_output, timestep: float, sample):
        t = self.apply_shift(timestep)
        t_prev = self.apply_shift(timestep - 1.0 / self.num_inference_steps) if timestep > 0.0 else 0.0
        if t > 0.999:
            return sample
        return sample + model_output * (t_prev - t)

    def add_noise(self, x0, noise, timestep: float):
        s = self.apply_shift(timestep)
        return (1.0 - s) * x0 + s * noise


LTX_DISTILLED_SIGMAS = (1.0, 0.99375, 0.9875, 0.98125, 0.975, 0.909375, 0.725, 0.421875, 0.0)


def ltx_sigma_schedule(num_steps: int, num_latent_tokens: int, base_shift: float = 0.95, max_shift: float = 2.05,
                       terminal: float = 0.1):
    """``num_steps + 1`` sigmas from 1 to 0: the shift grows linearly with the token count between
    1024 and 4096 tokens, ``sigma = e^s / (e^s + 1/t - 1)``, then non-zero values are stretched so
    that the smallest one is ``terminal``."""
    m = (max_shift - base_shift) / (4096.0 - 1024.0)
    b = base_shift - m * 1024.0
    shift = min(max(num_latent_tokens * m + b, base_shift), max_shift)
    es = math.exp(shift)
    out = []
    for i in range(num_steps + 1):
        t = 1.0 - i / num_steps
        out.append(0.0 if t <= 0.0 else 1.0 if t >= 1.0 else es / (es + (1.0 / t - 1.0)))
    if 0.0 < terminal < 1.0:
        out = [s * (1.0 - terminal) + terminal if s > 0.0 else s for s in out]
        out[-1] = 0.0
    return out


def euler_denoise_flow(model_fn, noise, sigmas):
    """Euler integration of a velocity model over ``sigmas``; the step that lands on sigma 0
    returns the denoised sample ``x - sigma * v`` exactly."""
    x = noise
    sig = [float(s) for s in sigmas]
    for i in range(len(sig) - 1):
        s, s_next = sig[i], sig[i + 1]
        v = model_fn(x, s)
        x = x - v * s if s_next == 0.0 else x + v * (s_next - s)
    return x


# ------------------------------------------------------------------------------------ model types
@dataclass
class MemoryConfig:
    max_gpu_memory_gb: float = 160.0
    cpu_offload: bool = False
    sequential_offload: bool = False
    vae_tiling: bool = True
    vae_tile_size: int = 64            # latent pixels per tile (512 image pixels)
    attention_slicing: bool = False


class ModelType(enum.Enum):
    SDXL = "sdxl"
    SD35_MEDIUM = "sd35_medium"
    SD35_LARGE = "sd35_large"
    FLUX_SCHNELL = "flux_schnell"
    FLUX_DEV = "flux_dev"
    CHROMA = "chroma"
    QWEN_IMAGE = "qwen_image"
    KLEIN = "klein"
    ZIMAGE = "zimage"
    LTX = "ltx_video"
    WAN22 = "wan22"

    @classmethod
    def from_path(cls, path) -> "ModelType":
        s = str(path).lower()
        if "sdxl" in s:
            return cls.SDXL
        if "sd3.5" in s or "sd35" in s or "sd3_5" in s:
            return cls.SD35_MEDIUM if "medium" in s else cls.SD35_LARGE
        if "flux" in s:
            if "klein" in s:
                return cls.KLEIN
            return cls.FLUX_SCHNELL if "schnell" in s else cls.FLUX_DEV
        for key, mt in (("chroma", cls.CHROMA), ("qwen", cls.QWEN_IMAGE), ("klein", cls.KLEIN), ("zimage", cls.ZIMAGE),
                        ("z-image", cls.ZIMAGE), ("z_image", cls.ZIMAGE), ("ltx", cls.LTX), ("wan2", cls.WAN22)):
            if key in s:
                return mt
        raise ValueError(f"could not determine the model type from the path {path!r}")

    @property
    def family(self) -> str:
        """Registry name of the architecture (``models.build_model``)."""
        return {"sd35_medium": "sd35", "sd35_large": "sd35", "flux_schnell": "flux", "flux_dev": "flux"}.get(
            self.value, self.value)

    @property
    def is_video(self) -> bool:
        return self in (ModelType.LTX, ModelType.WAN22)

    def default_steps(self) -> int:
        return {ModelType.FLUX_SCHNELL: 4, ModelType.SDXL: 30, ModelType.LTX: 8}.get(self, 20)

    def default_guidance(self) -> float:
        return {ModelType.FLUX_SCHNELL: 0.0, ModelType.SDXL: 7.0, ModelType.SD35_MEDIUM: 4.5,
                ModelType.SD35_LARGE: 4.5}.get(self, 3.5)

    def memory_config(self, gpu_memory_gb: float = 180.0) -> MemoryConfig:
        """Everything resident when the card has room (180 GB holds every family in bf16); below
        48 GB the reference's policy applies: offload, sequential offload for the large flow
        models, smaller VAE tiles."""
        if gpu_memory_gb >= 48.0:
            return MemoryConfig(max_gpu_memory_gb=gpu_memory_gb * 0.9)
        big = self not in (ModelType.SDXL,)
        return MemoryConfig(max_gpu_memory_gb=gpu_memory_gb * 0.8, cpu_offload=True, sequential_offload=big,
                            vae_tile_size=32 if self in (ModelType.FLUX_DEV, ModelType.FLUX_SCHNELL) else 64,
                            attention_slicing=self in (ModelType.FLUX_DEV, ModelType.FLUX_SCHNELL))


# ------------------------------------------------------------------------------------ video sampling
def generate_video_flow(model, txt, frames: int, height: int, width: int, channels: int, steps: int = 8, seed: int = 0,
                        sigmas=None, dtype=torch.bfloat16, neg_txt=None, cfg_scale: float = 1.0):
    """Sample video latents [B, C, frames, height, width] (latent units) from a token-major video
    flow model called as ``model(tokens [B, L, C], txt, t [B], (frames, h, w))``."""
    dev = txt.device
    B = txt.shape[0]
    L = frames * height * width
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(B, L, channels, device=dev, generator=g, dtype=torch.float32).to(dtype)
    if sigmas is None:
        sigmas = LTX_DISTILLED_SIGMAS if steps == len(LTX_DISTILLED_SIGMAS) - 1 else ltx_sigma_schedule(steps, L)

    def velocity(z, s):
        t = torch.full((B,), float(s), device=dev)
        v = model(z, txt, t, (frames, height, width))
        if cfg_scale != 1.0 and neg_txt is not None:
            v = cfg_mix(v, model(z, neg_txt, t, (frames, height, width)), cfg_scale)
        return v.to(z.dtype)

    tok = euler_denoise_flow(velocity, x, sigmas)
    return tok.transpose(1, 2).reshape(B, channels, frames, height, width)


# ------------------------------------------------------------------------------------ pipeline
_K_SAMPLERS = {"euler": sample_euler, "heun": sample_heun, "dpmpp_2m": sample_dpmpp_2m}


class UnifiedInferencePipeline:
    """One ``generate`` for every family. ``model`` is the denoiser (already on its device),
    ``vae`` an optional ``AutoencoderKL`` for decoding, ``text_encode`` an optional callable
    ``prompt -> (txt [1, T, D], pooled [1, P] or None)``; without it the caller passes embeddings.
    With ``memory.cpu_offload`` the model sits in host memory between calls and is moved to
    ``device`` for the duration of ``generate``."""

    def __init__(self, model, model_type: ModelType, vae=None, text_encode=None, memory: MemoryConfig | None = None,
                 device=None, dtype=None):
        self.model, self.model_type, self.vae, self.text_encode = model, model_type, vae, text_encode
        p = next(model.parameters())
        self.device = torch.device(device) if device is not None else p.device
        self.dtype = dtype or p.dtype
        self.memory = memory or model_type.memory_config(
            torch.cuda.get_device_properties(self.device).total_memory / 2 ** 30 if self.device.type == "cuda" else 180.0)
        if self.memory.cpu_offload:
            self.model.to("cpu")

    def model_info(self) -> str:
        n = sum(p.numel() for p in self.model.parameters())
        return f"{self.model_type.value}: {n / 1e9:.2f} B parameters, {self.dtype}, device {self.device}, " \
               f"offload={'on' if self.memory.cpu_offload else 'off'}"

    def _embed(self, prompt, txt, pooled):
        if txt is None:
            if self.text_encode is None:
                raise ValueError("pass txt= (and pooled=) embeddings or construct the pipeline with text_encode")
            txt, pooled = self.text_encode(prompt)
        return txt.to(self.device, self.dtype), None if pooled is None else pooled.to(self.device, self.dtype)

    @torch.no_grad()
    def generate(self, prompt: str = "", negative_prompt: str = "", width: int = 1024, height: int = 1024,
                 steps: int | None = None, guidance_scale: float | None = None, seed: int = 0, txt=None, pooled=None,
                 neg_txt=None, neg_pooled=None, sampler: str = "euler", frames: int = 1, cfg_scale: float = 1.0):
        """Latents: [B, C, H/8, W/8] for image families, [B, C, frames, H/32, W/32] for LTX-style
        video models. ``guidance_scale`` is the distilled-guidance input of FLUX-style models and
        the classifier-free scale of SDXL; ``cfg_scale`` adds true classifier-free guidance to a
        flow model (needs the negative embeddings)."""
        mt = self.model_type
        steps = steps or mt.default_steps()
        guidance_scale = mt.default_guidance() if guidance_scale is None else guidance_scale
        txt, pooled = self._embed(prompt, txt, pooled)
        if neg_txt is None and self.text_encode is not None and (cfg_scale != 1.0 or mt is ModelType.SDXL):
            neg_txt, neg_pooled = self.text_encode(negative_prompt)
        if neg_txt is not None:
            neg_txt = neg_txt.to(self.device, self.dtype)
            neg_pooled = None if neg_pooled is None else neg_pooled.to(self.device, self.dtype)
        if self.memory.cpu_offload:
            self.model.to(self.device)
        try:
            if mt is ModelType.SDXL:
                return self._generate_sdxl(txt, pooled, neg_txt, neg_pooled, width, height, steps, guidance_scale,
                                           seed, sampler)
            if mt.is_video:
                ch = getattr(self.model.cfg, "in_channels", 128)
                return generate_video_flow(self.model, txt, frames, height // 32, width // 32, ch, steps, seed,
                                           dtype=self.dtype, neg_txt=neg_txt, cfg_scale=cfg_scale)
            ch = getattr(self.model.cfg, "in_channels", 64) // 4
            return generate_flow(self.model, txt, pooled, height, width, steps, guidance_scale, seed=seed,
                                 channels=ch, dtype=self.dtype, neg_txt=neg_txt, neg_pooled=neg_pooled,
                                 cfg_scale=cfg_scale)
        finally:
            if self.memory.cpu_offload:
                self.model.to("cpu")

    def _generate_sdxl(self, ctx, pooled, neg_ctx, neg_pooled, width, height, steps, scale, seed, sampler):
        m, dev, dt = self.model, self.device, self.dtype
        B = ctx.shape[0]
        tid = torch.tensor([[height, width, 0, 0, height, width]] * B, dtype=torch.float32, device=dev)
        train_sigmas = ddpm_sigmas().to(dev)
        eps = lambda x, t: m(x, t, ctx, pooled, tid)
        den = eps_denoiser(eps, train_sigmas)
        if scale != 1.0:
            zc = torch.zeros_like(ctx) if neg_ctx is None else neg_ctx
            zp = torch.zeros_like(pooled) if neg_pooled is None else neg_pooled
            den_u, cond = eps_denoiser(lambda x, t: m(x, t, zc, zp, tid), train_sigmas), den
            den = lambda x, s: cfg_mix(cond(x, s), den_u(x, s), scale)
        sig = karras_sigmas(steps, device=dev)
        gen = torch.Generator(device=dev).manual_seed(seed)
        x = torch.randn(B, 4, height // 8, width // 8, device=dev, generator=gen).to(dt) * sig[0]
        if sampler == "euler_a":
            return sample_euler_ancestral(den, x, sig, gen=gen)
        if sampler == "ddim":
            return sample_ddim(eps, x / sig[0], steps=steps, gen=gen)
        if sampler not in _K_SAMPLERS:
            raise ValueError(f"unknown sampler {sampler!r}")
        return _K_SAMPLERS[sampler](den, x, sig)

    @torch.no_grad()
    def decode(self, latents):
        """uint8 images [B, H, W, 3] (tiled decode when the memory policy asks for it)."""
        if self.vae is None:
            raise ValueError("the pipeline was built without a VAE")
        lat = latents.to(self.dtype)
        img = self.vae.tiled_decode(lat, tile=self.memory.vae_tile_size) if self.memory.vae_tiling and \
            max(lat.shape[-2:]) > self.memory.vae_tile_size else self.vae.decode(lat)
        return latents_to_uint8(img)

    def generate_image(self, prompt: str = "", **kw):
        """``generate`` followed by ``decode``: uint8 [B, H, W, 3]."""
        return self.decode(self.generate(prompt, **kw))

"""Augmentations for images, latents and captions
(crates/training/src/augmentation.rs:9-332: colour jitter, cutout, mixup, caption dropout /
shuffle / synonyms, latent noise / flip; noise offset and input perturbation:
crates/training/src/pipelines/base_pipeline.rs:201-222)."""
from __future__ import annotations

import random

import torch


class ColorJitter:
    def __init__(self, brightness=0.1, contrast=0.1, saturation=0.1, seed=0):
        self.b, self.c, self.s = brightness, contrast, saturation
        self.g = torch.Generator().manual_seed(seed)

    def _u(self, a):
        return 1.0 + (torch.rand((), generator=self.g).item() * 2 - 1) * a

    def __call__(self, img):                      # [3, H, W] in [0, 1]
        img = img * self._u(self.b)
        mean = img.mean()
        img = (img - mean) * self._u(self.c) + mean
        gray = img.mean(0, keepdim=True)
        img = (img - gray) * self._u(self.s) + gray
        return img.clamp(0, 1)


class Cutout:
    def __init__(self, size=32, p=0.5, seed=0):
        self.size, self.p, self.g = size, p, torch.Generator().manual_seed(seed)

    def __call__(self, img):
        if torch.rand((), generator=self.g).item() > self.p:
            return img
        _, h, w = img.shape
        y = int(torch.randint(0, max(1, h - self.size), (1,), generator=self.g))
        x = int(torch.randint(0, max(1, w - self.size), (1,), generator=self.g))
        img = img.clone()
        img[:, y:y + self.size, x:x + self.size] = 0
        return img


def mixup(x, alpha=0.2, gen=None):
    lam = torch.distributions.Beta(alpha, alpha).sample().item() if alpha > 0 else 1.0
    perm = torch.randperm(x.shape[0], generator=gen)
    return lam * x + (1 - lam) * x[perm], perm, lam


def latent_flip(latents, p=0.5, gen=None):
    mask = torch.rand(latents.shape[0], generator=gen) < p
    out = latents.clone()
    out[mask] = out[mask].flip(-1)
    return out


def latent_noise(latents, std=0.01, gen=None):
    return latents + torch.randn(latents.shape, generator=gen).to(latents) * std


def noise_offset(noise, strength=0.05, gen=None):
    """Per-channel constant offset added to the sampled noise."""
    off = torch.randn(noise.shape[0], noise.shape[1], *([1] * (noise.dim() - 2)), generator=gen)
    return noise + strength * off.to(noise)


def input_perturbation(noise, gamma=0.1, gen=None):
    return noise + gamma * torch.randn(noise.shape, generator=gen).to(noise)


class CaptionAugment:
    def __init__(self, dropout=0.0, shuffle_tokens=False, keep_tokens=1, synonyms=None, trigger_word=None, seed=0):
        self.dropout, self.shuffle, self.keep = dropout, shuffle_tokens, keep_tokens
        self.syn, self.trigger = synonyms or {}, trigger_word
        self.r = random.Random(seed)

    def __call__(self, caption: str) -> str:
        if self.dropout > 0 and self.r.random() < self.dropout:
            return ""
        toks = [t.strip() for t in caption.split(",") if t.strip()]
        if self.shuffle and len(toks) > self.keep:
            head, tail = toks[: self.keep], toks[self.keep:]
            self.r.shuffle(tail)
            toks = head + tail
        toks = [self.r.choice(self.syn[t]) if t in self.syn and self.r.random() < 0.5 else t for t in toks]
        out = ", ".join(toks)
        if self.trigger and self.trigger not in out:
            out = f"{self.trigger}, {out}" if out else self.trigger
        return out

"""Aspect-ratio bucketed image and still-image "video" datasets.

``BucketedImageDataset`` covers the reference's ``Wan22ImageDataset``
(crates/data/src/wan22_image_dataset.rs:30-131) and ``BucketedVideoDataset`` its
``Wan22VideoDataset`` (crates/data/src/wan22_video_dataset.rs:39-170): files are found recursively
(six levels) with a ``.txt`` caption beside them, every file goes to the bucket whose width/height
ratio is nearest its own, captions get ``[trigger]`` replaced and an empty caption a default.
Where the reference returns zero latents as a bootstrap placeholder, these datasets return the
resized pixels (and latents when a ``VaePreprocessor`` is attached), batch more than one sample per
bucket, and walk the buckets in a seeded order.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from pathlib import Path

import torch

from . import xorshift_permutation
from .vae_preprocess import IMAGE_EXT


@dataclass
class BucketDataConfig:
    dataset_dir: str
    buckets: list = field(default_factory=lambda: [(1024, 1024)])     # (height, width)
    min_size: int = 0
    max_size: int = 0
    caption_trigger_word: str | None = None
    cache_latents: bool = False
    batch_size: int = 1
    seed: int = 0


@dataclass
class VideoDataConfig:
    dataset_dir: str
    buckets: list = field(default_factory=lambda: [(480, 832)])
    time_buckets: list = field(default_factory=list)                   # allowed frame counts
    frames: int = 1
    downscale_only: bool = False
    caption_trigger_word: str | None = None


def walk_images(root, max_depth=6):
    root = Path(root)
    if not root.exists():
        raise FileNotFoundError(f"dataset_dir not found: {root}")
    out = []
    base = len(root.parts)
    for d, _, names in os.walk(root):
        if len(Path(d).parts) - base >= max_depth:
            continue
        for n in sorted(names):
            p = Path(d) / n
            if p.suffix.lower() in IMAGE_EXT:
                cap = p.with_suffix(".txt")
                out.append((p, cap if cap.exists() else None))
    out.sort(key=lambda t: str(t[0]))
    return out


def nearest_bucket(width, height, buckets):
    """Index of the (height, width) bucket whose aspect ratio is nearest ``width / height``."""
    ar = width / height
    best, best_d = 0, float("inf")
    for i, (bh, bw) in enumerate(buckets):
        d = abs(ar - bw / bh)
        if d < best_d:
            best, best_d = i, d
    return best


def _caption(cap_path, trigger, default):
    text = ""
    if cap_path is not None:
        try:
            text = Path(cap_path).read_text()
        except OSError:
            text = ""
    if trigger:
        text = text.replace("[trigger]", trigger)
    return text.strip() or default


def _load_resized(path, bh, bw):
    from PIL import Image
    import numpy as np
    img = Image.open(path).convert("RGB").resize((bw, bh), Image.LANCZOS)
    x = torch.from_numpy(np.asarray(img).copy()).float()
    return x / 127.5 - 1.0                                            # [H, W, 3] in [-1, 1]


def _image_size(path):
    from PIL import Image
    with Image.open(path) as im:
        return im.size                                                # (width, height)


class BucketedImageDataset:
    def __init__(self, cfg: BucketDataConfig, device="cpu", preprocessor=None):
        if not cfg.buckets:
            raise ValueError("bucketed dataset: at least one bucket required")
        self.cfg, self.device, self.pre = cfg, torch.device(device), preprocessor
        self.files = walk_images(cfg.dataset_dir)
        if not self.files:
            raise FileNotFoundError("no images found")
        self.by_bucket = [[] for _ in cfg.buckets]
        for i, (p, _) in enumerate(self.files):
            try:
                w, h = _image_size(p)
            except Exception:
                continue
            if cfg.min_size and min(w, h) < cfg.min_size:
                continue
            if cfg.max_size and max(w, h) > cfg.max_size:
                continue
            self.by_bucket[nearest_bucket(w, h, cfg.buckets)].append(i)
        self.epoch = 0

    def num_files(self):
        return len(self.files)

    def buckets_summary(self):
        return [(tuple(hw), len(v)) for hw, v in zip(self.cfg.buckets, self.by_bucket)]

    def batches_per_epoch(self):
        bs = self.cfg.batch_size
        return sum((len(v) + bs - 1) // bs for v in self.by_bucket)

    def __iter__(self):
        """One epoch: every bucket's files in a seeded order, batches never mix buckets."""
        bs = self.cfg.batch_size
        plan = []
        for bi, v in enumerate(self.by_bucket):
            order = [v[j] for j in xorshift_permutation(len(v), self.cfg.seed + self.epoch * 7919 + bi)]
            plan += [(bi, order[k:k + bs]) for k in range(0, len(order), bs)]
        plan = [plan[j] for j in xorshift_permutation(len(plan), self.cfg.seed + self.epoch)]
        self.epoch += 1
        for bi, idx in plan:
            yield self.load_batch(bi, idx)

    def load_batch(self, bi, idx):
        bh, bw = self.cfg.buckets[bi]
        imgs = torch.stack([_load_resized(self.files[i][0], bh, bw) for i in idx])      # [B, H, W, 3]
        prompts = [_caption(self.files[i][1], self.cfg.caption_trigger_word, "a photo") for i in idx]
        if self.device.type == "cuda":
            imgs = imgs.pin_memory().to(self.device, non_blocking=True)
        batch = {"images": imgs.to(torch.bfloat16), "prompts": prompts, "h": bh, "w": bw,
                 "paths": [str(self.files[i][0]) for i in idx]}
        if self.pre is not None:
            with torch.no_grad():
                batch["latents"] = self.pre.vae.encode(imgs.permute(0, 3, 1, 2), sample=False)
        return batch


class BucketedVideoDataset:
    """Still images presented as clips: each sample is resized to its spatial bucket and paired with
    a frame count (the first time bucket, or ``frames``)."""

    def __init__(self, cfg: VideoDataConfig, device="cpu"):
        if not cfg.buckets:
            raise ValueError("video dataset: buckets required")
        self.cfg, self.device = cfg, torch.device(device)
        self.files = walk_images(cfg.dataset_dir)
        if not self.files:
            raise FileNotFoundError("no images found for video dataset")

    def num_files(self):
        return len(self.files)

    def pick_bucket(self, width, height):
        bh, bw = self.cfg.buckets[nearest_bucket(width, height, self.cfg.buckets)]
        t = self.cfg.time_buckets[0] if self.cfg.time_buckets else max(1, self.cfg.frames)
        return bh, bw, t

    def buckets_summary(self):
        counts = {}
        for p, _ in self.files:
            try:
                w, h = _image_size(p)
            except Exception:
                continue
            bh, bw, _ = self.pick_bucket(w, h)
            counts[(bh, bw)] = counts.get((bh, bw), 0) + 1
        return sorted((h, w, c) for (h, w), c in counts.items())

    def next_batch(self, index):
        p, cap = self.files[index % len(self.files)]
        w0, h0 = _image_size(p)
        bh, bw, t = self.pick_bucket(w0, h0)
        if self.cfg.downscale_only and (w0 < bw or h0 < bh):
            raise ValueError(f"upscaling forbidden: {p} ({w0}x{h0}) -> bucket {bw}x{bh}")
        img = _load_resized(p, bh, bw).unsqueeze(0)
        if self.device.type == "cuda":
            img = img.pin_memory().to(self.device, non_blocking=True)
        return {"images": img.to(torch.bfloat16), "prompts": [_caption(cap, self.cfg.caption_trigger_word,
                                                                        "a short video")],
                "h": bh, "w": bw, "t": t, "latent_shape": (1, t, max(1, bh // 8), max(1, bw // 8))}

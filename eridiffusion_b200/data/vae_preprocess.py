"""Image folder -> VAE latents: decode, centre-crop, resize, normalise, encode in micro-batches, and
(as a command) write sharded safetensors files plus a ``manifest.jsonl``.

    python -m eridiffusion_b200.data.vae_preprocess --input imgs/ --out latents/ --vae-kind flux \
        [--vae-path vae.safetensors | --model-paths modelPaths.yaml --model-id flux_dev] \
        [--size 1024] [--microbatch 4] [--shard-size 512] [--tile 512]

Covers the reference's ``VaePreprocessor::encode_paths`` (crates/data/src/vae_preprocessor.rs:77-126),
``load_vae_spec_from_model_paths`` (:205-245) and the ``vae_preprocess`` binary
(crates/data/src/bin/vae_preprocess.rs:92-246). The pixels go to the GPU as one pinned uint8
batch per micro-batch and are normalised there; latents come back channel-first ``[B, C, H/8, W/8]``.
"""
from __future__ import annotations

import argparse
import json
import sys
from dataclasses import dataclass
from pathlib import Path

import torch
from safetensors.torch import save_file

IMAGE_EXT = (".jpg", ".jpeg", ".png", ".webp", ".bmp", ".tiff")


@dataclass
class PreprocessConfig:
    target_size: tuple = (1024, 1024)        # (height, width)
    center_crop: bool = True
    normalize_to_neg1_1: bool = True
    microbatch: int = 4


@dataclass
class SampleInfo:
    path: str
    orig_hw: tuple
    crop_xy: tuple
    out_hw: tuple


@dataclass
class VaeSpec:
    kind: str = "sdxl"                       # sdxl | sd35 | flux
    path: str = ""
    latent_div: int = 8
    latent_channels: int = 4
    latent_scale: float = 0.18215
    latent_shift: float = 0.0


_KIND_DEFAULTS = {"sdxl": (4, 0.13025, 0.0), "sd35": (16, 1.5305, 0.0609), "flux": (16, 0.3611, 0.1159)}


def load_vae_spec_from_model_paths(yaml_path, model_id) -> VaeSpec:
    import yaml
    mp = yaml.safe_load(Path(yaml_path).read_text()) or {}
    models = mp.get("models") or {}
    if model_id not in models:
        raise KeyError(f"model_id '{model_id}' not found in modelPaths")
    v = (models[model_id] or {}).get("vae")
    if not v:
        raise KeyError(f"models.{model_id}.vae missing in modelPaths")
    kind = v.get("kind", "")
    if kind not in _KIND_DEFAULTS:
        raise ValueError(f"unsupported vae.kind '{kind}'")
    spec = VaeSpec(kind=kind, path=str(v.get("path", "")), latent_div=int(v.get("latent_div", 0)),
                   latent_channels=int(v.get("latent_channels", 0)), latent_scale=float(v.get("latent_scale", 0.0)),
                   latent_shift=float(v.get("latent_shift", _KIND_DEFAULTS[kind][2])))
    if not spec.path.strip():
        raise ValueError(f"vae.path is empty for model_id '{model_id}'")
    if spec.latent_div <= 0 or spec.latent_channels <= 0:
        raise ValueError("vae.latent_div and vae.latent_channels must be > 0")
    if not (spec.latent_scale > 0.0 and spec.latent_scale == spec.latent_scale and spec.latent_scale != float("inf")):
        raise ValueError("vae.latent_scale must be > 0")
    return spec


def load_preprocess_rgb(path, cfg: PreprocessConfig):
    """uint8 tensor [H, W, 3] after the optional centre crop and the Lanczos resize, plus the
    original (h, w) and the crop origin."""
    from PIL import Image
    import numpy as np
    img = Image.open(path).convert("RGB")
    ow, oh = img.size
    cx = cy = 0
    if cfg.center_crop:
        side = min(ow, oh)
        cx, cy = (ow - side) // 2, (oh - side) // 2
        img = img.crop((cx, cy, cx + side, cy + side))
    th, tw = cfg.target_size
    img = img.resize((tw, th), Image.LANCZOS)
    return torch.from_numpy(np.asarray(img).copy()), (oh, ow), (cx, cy)


class VaePreprocessor:
    def __init__(self, vae, device=None, tile=None):
        """``vae``: an ``AutoencoderKL`` (already on its device). ``tile``: encode in overlapping
        tiles of this many pixels (for images too large for one pass)."""
        self.vae = vae
        self.device = torch.device(device) if device is not None else next(vae.parameters()).device
        self.tile = tile

    @classmethod
    def from_spec(cls, spec: VaeSpec, device="cuda", dtype=torch.bfloat16, tile=None):
        from ..models.vae import AutoencoderKL, VaeConfig
        cfg = VaeConfig(latent_channels=spec.latent_channels, scaling_factor=spec.latent_scale,
                        shift_factor=spec.latent_shift, latent_div=spec.latent_div)
        vae = AutoencoderKL(cfg, dtype=dtype, device=device)
        if spec.path:
            from ..io.safetensors import load_file
            vae.load_state_dict(load_file(spec.path), strict=False)
        return cls(vae.eval(), device, tile)

    @torch.no_grad()
    def encode_paths(self, paths, cfg: PreprocessConfig = PreprocessConfig(), sample=False):
        if not paths:
            raise ValueError("encode_paths: empty input list")
        infos, imgs = [], []
        for p in paths:
            rgb, orig_hw, crop_xy = load_preprocess_rgb(p, cfg)
            imgs.append(rgb)
            infos.append(SampleInfo(str(p), orig_hw, crop_xy, (rgb.shape[0], rgb.shape[1])))
        chunks = []
        mb = max(1, cfg.microbatch)
        for i in range(0, len(imgs), mb):
            u8 = torch.stack(imgs[i:i + mb])                       # [b, H, W, 3] uint8
            if self.device.type == "cuda":
                u8 = u8.pin_memory().to(self.device, non_blocking=True)
            x = u8.permute(0, 3, 1, 2).float() / 255.0
            if cfg.normalize_to_neg1_1:
                x = x * 2.0 - 1.0
            if self.tile:
                lat = self.vae.tiled_encode(x, tile=self.tile, overlap=self.tile // 4)
            else:
                lat = self.vae.encode(x, sample=sample)
            chunks.append(lat)
        return torch.cat(chunks, 0), infos


def find_images(root):
    return sorted(p for p in Path(root).rglob("*") if p.is_file() and p.suffix.lower() in IMAGE_EXT)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--input", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--cuda", type=int, default=0)
    ap.add_argument("--cpu", action="store_true", help="run the encoder on the CPU (tests)")
    ap.add_argument("--vae-kind", choices=sorted(_KIND_DEFAULTS))
    ap.add_argument("--vae-path")
    ap.add_argument("--model-paths")
    ap.add_argument("--model-id")
    ap.add_argument("--latent-div", type=int)
    ap.add_argument("--latent-channels", type=int)
    ap.add_argument("--latent-scale", type=float)
    ap.add_argument("--size", type=int, default=1024)
    ap.add_argument("--no-center-crop", action="store_true")
    ap.add_argument("--no-normalize", action="store_true")
    ap.add_argument("--microbatch", type=int, default=4)
    ap.add_argument("--shard-size", type=int, default=512)
    ap.add_argument("--tile", type=int)
    ap.add_argument("--base-channels", type=int, default=128, help="encoder width (smaller for tests)")
    a = ap.parse_args(argv)
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    paths = find_images(a.input)
    if not paths:
        raise SystemExit(f"no images found under {a.input}")
    if a.model_paths and a.model_id:
        spec = load_vae_spec_from_model_paths(a.model_paths, a.model_id)
    else:
        if not a.vae_kind:
            raise SystemExit("--vae-kind required (or provide --model-paths and --model-id)")
        ch, sc, sh = _KIND_DEFAULTS[a.vae_kind]
        spec = VaeSpec(kind=a.vae_kind, path=a.vae_path or "", latent_channels=ch, latent_scale=sc, latent_shift=sh)
    if a.vae_kind:
        spec.kind = a.vae_kind
    if a.vae_path:
        spec.path = a.vae_path
    for k in ("latent_div", "latent_channels", "latent_scale"):
        if getattr(a, k) is not None:
            setattr(spec, k, getattr(a, k))
    dev = "cpu" if a.cpu else f"cuda:{a.cuda}"
    dt = torch.float32 if a.cpu else torch.bfloat16
    from ..models.vae import AutoencoderKL, VaeConfig
    vcfg = VaeConfig(latent_channels=spec.latent_channels, scaling_factor=spec.latent_scale,
                     shift_factor=spec.latent_shift, latent_div=spec.latent_div, base=a.base_channels)
    vae = AutoencoderKL(vcfg, dtype=dt, device=dev).eval()
    if spec.path:
        from ..io.safetensors import load_file
        vae.load_state_dict(load_file(spec.path), strict=False)
    pre = VaePreprocessor(vae, dev, a.tile)
    cfg = PreprocessConfig((a.size, a.size), not a.no_center_crop, not a.no_normalize, max(1, a.microbatch))

    shard, rows, shard_idx, n = {}, [], 0, 0

    def flush():
        nonlocal shard, rows, shard_idx
        if not shard:
            return
        name = f"latents_{shard_idx:05d}.safetensors"
        save_file(shard, str(out / name))
        with open(out / "manifest.jsonl", "a") as mf:
            for key, info in rows:
                mf.write(json.dumps({"key": key, "shard": name, "path": info.path, "orig_hw": list(info.orig_hw),
                                     "crop_xy": list(info.crop_xy), "out_hw": list(info.out_hw)}) + "\n")
        shard, rows = {}, []
        shard_idx += 1

    (out / "manifest.jsonl").write_text("")
    step = max(1, a.microbatch)
    for i in range(0, len(paths), step):
        lat, infos = pre.encode_paths(paths[i:i + step], cfg)
        for j, info in enumerate(infos):
            key = f"sample_{n:08d}"
            shard[key] = lat[j].to("cpu").contiguous()
            rows.append((key, info))
            n += 1
            if len(shard) >= a.shard_size:
                flush()
    flush()
    print(json.dumps({"samples": n, "shards": shard_idx, "out": str(out), "latent_shape": list(lat.shape[1:])}))
    return 0


if __name__ == "__main__":
    sys.exit(main())

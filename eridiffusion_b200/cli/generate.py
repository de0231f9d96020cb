"""Image generation from cached text embeddings (or random ones), for every registered family.

    python -m eridiffusion_b200.cli.generate --family flux --out img.png \
        [--model weights.safetensors] [--lora lora.safetensors] [--vae vae.safetensors] \
        [--txt t5.safetensors --pooled clip.safetensors] [--steps 20] [--guidance 3.5] \
        [--height 1024 --width 1024] [--seed 0] [--sampler euler|euler_a|heun|dpmpp_2m|ddim]

One entry point for what the reference splits into ``klein_generate``, ``zimage_generate``,
``ltx2_generate`` (src/bin), ``sdxl_cli`` (inference/bin/sdxl_cli.rs) and ``sample_sdxl``
(crates/apps/sample_sdxl): flow-matching families run the shifted Euler sampler
(src/inference/flux_sampling.rs:64-71), SDXL runs a Karras-sigma k-diffusion sampler with
classifier-free guidance (crates/training/src/sdxl/scheduler.rs:45-78, sdxl/infer.rs:726). Without
``--vae`` the latents are written as a safetensors file instead of a PNG.
"""
from __future__ import annotations

import argparse
import sys

import torch

from .. import sampling as S
from ..data import load_cached_tensor
from ..io import safetensors as st
from ..models import build_model

FLOW_FAMILIES = {"flux": (16, 4096, 768), "chroma": (16, 4096, 0), "krea": (16, 4096, 768),
                 "qwen_image": (16, 3584, 0), "sd35": (16, 4096, 2048), "klein": (32, 7680, 0),
                 "zimage": (16, 2560, 0), "lumina": (16, 2304, 0), "hunyuan": (16, 4096, 768),
                 "hidream": (16, 4096, 2048), "tiny_mmdit": (16, 128, 64)}


def _embeds(a, dev, dt, ctx_dim, vec_dim, tokens):
    g = torch.Generator().manual_seed(a.seed + 1)
    txt = load_cached_tensor(a.txt, dt).to(dev)[None] if a.txt else torch.randn(1, tokens, ctx_dim, generator=g).to(dt).to(dev)
    if txt.dim() == 4:
        txt = txt[0]
    pooled = None
    if vec_dim:
        pooled = load_cached_tensor(a.pooled, dt).to(dev).view(1, -1) if a.pooled else \
            torch.randn(1, vec_dim, generator=g).to(dt).to(dev)
    return txt, pooled


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--family", default="flux")
    ap.add_argument("--model"); ap.add_argument("--lora"); ap.add_argument("--vae")
    ap.add_argument("--txt"); ap.add_argument("--pooled"); ap.add_argument("--out", default="out.png")
    ap.add_argument("--steps", type=int, default=20); ap.add_argument("--guidance", type=float, default=3.5)
    ap.add_argument("--cfg-scale", type=float, default=1.0)
    ap.add_argument("--height", type=int, default=1024); ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--seed", type=int, default=0); ap.add_argument("--sampler", default="euler")
    ap.add_argument("--frames", type=int, default=9, help="latent frames (video families)")
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--override", action="append", default=[], help="model config override key=value")
    a = ap.parse_args(argv)
    dev = torch.device(a.device)
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    ov = {}
    for kv in a.override:
        k, v = kv.split("=", 1)
        ov[k] = eval(v, {"__builtins__": {}})            # numbers / tuples only
    model = build_model(a.family, device=dev, dtype=dt, **ov).eval()
    if a.model:
        from ..io.weights import load_model_weights
        load_model_weights(model, a.model, a.family)
    if a.lora:
        from ..adapters.lora import load_adapters_into
        load_adapters_into(model, a.lora)
    with torch.no_grad():
        if a.family == "sdxl":
            g = torch.Generator().manual_seed(a.seed + 1)
            ctx = load_cached_tensor(a.txt, dt).to(dev)[None] if a.txt else torch.randn(1, 77, model.cfg.context_dim, generator=g).to(dt).to(dev)
            pooled = load_cached_tensor(a.pooled, dt).to(dev).view(1, -1) if a.pooled else torch.randn(1, model.cfg.pooled_dim, generator=g).to(dt).to(dev)
            tid = torch.tensor([[a.height, a.width, 0, 0, a.height, a.width]], dtype=torch.float32, device=dev)
            train_sigmas = S.ddpm_sigmas().to(dev)
            den = S.eps_denoiser(lambda x, t: model(x, t, ctx, pooled, tid), train_sigmas)
            if a.cfg_scale != 1.0:
                zc, zp = torch.zeros_like(ctx), torch.zeros_like(pooled)
                den_u = S.eps_denoiser(lambda x, t: model(x, t, zc, zp, tid), train_sigmas)
                cond = den
                den = lambda x, s: S.cfg_mix(cond(x, s), den_u(x, s), a.cfg_scale)
            sig = S.karras_sigmas(a.steps, device=dev)
            gen = torch.Generator(device=dev).manual_seed(a.seed)
            x = torch.randn(1, 4, a.height // 8, a.width // 8, device=dev, generator=gen).to(dt) * sig[0]
            fn = {"euler": S.sample_euler, "heun": S.sample_heun, "dpmpp_2m": S.sample_dpmpp_2m}.get(a.sampler)
            if a.sampler == "euler_a":
                lat = S.sample_euler_ancestral(den, x, sig, gen=gen)
            elif a.sampler == "ddim":
                lat = S.sample_ddim(lambda x, t: model(x, t, ctx, pooled, tid), x / sig[0], steps=a.steps, gen=gen)
            else:
                lat = fn(den, x, sig)
            vae_kind = "vae_sdxl"
        elif a.family in FLOW_FAMILIES:
            ch, ctx_dim, vec_dim = FLOW_FAMILIES[a.family]
            ctx_dim = getattr(model.cfg, "context_dim", getattr(model.cfg, "caption_dim", ctx_dim))
            vec_dim = getattr(model.cfg, "vec_dim", vec_dim)
            ch = getattr(model.cfg, "in_channels", ch * 4) // 4
            txt, pooled = _embeds(a, dev, dt, ctx_dim, vec_dim, 64 if a.family == "tiny_mmdit" else 512)
            lat = S.generate_flow(model, txt, pooled, a.height, a.width, a.steps, a.guidance, seed=a.seed,
                                  channels=ch, dtype=dt, cfg_scale=a.cfg_scale)
            vae_kind = "vae_flux"
        elif a.family in ("ltx_video", "wan22"):
            # video families: token-major flow model, Euler over the token-count dependent sigma grid
            from ..sampling.pipelines import generate_video_flow
            ctx_dim = getattr(model.cfg, "caption_dim", getattr(model.cfg, "context_dim", 4096))
            txt, _ = _embeds(a, dev, dt, ctx_dim, 0, 256)
            ch = getattr(model.cfg, "in_channels", 128)
            lat = generate_video_flow(model, txt, a.frames, a.height // 32, a.width // 32, ch, a.steps, a.seed,
                                      dtype=dt, cfg_scale=1.0)
            a.vae = None                                   # video latents are written as they are
        else:
            raise SystemExit(f"family {a.family!r} has no sampler")
        if a.vae:
            vae = build_model(vae_kind, device=dev, dtype=dt).eval()
            from ..io.weights import load_model_weights
            load_model_weights(vae, a.vae, vae_kind, strict=False)
            img = vae.tiled_decode(lat.to(dt))
            S.save_png(S.latents_to_uint8(img)[0], a.out)
            print(f"wrote {a.out}")
        else:
            out = a.out if a.out.endswith(".safetensors") else a.out + ".latents.safetensors"
            st.save_file({"latent": lat.float().cpu()}, out, metadata={"family": a.family, "seed": str(a.seed)})
            print(f"wrote {out} (latents {tuple(lat.shape)}; pass --vae to decode)")
    return 0


if __name__ == "__main__":
    sys.exit(main())

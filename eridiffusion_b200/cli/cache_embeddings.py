"""Pre-compute the training cache: VAE latents and text-encoder hidden states, one safetensors file
per tensor, plus the manifest that ``CachedEmbeddingLoader`` reads.

    python -m eridiffusion_b200.cli.cache_embeddings --family flux --images DIR --out CACHE \
        [--vae vae.safetensors] [--t5 t5.safetensors --t5-tokenizer DIR] \
        [--clip clip.safetensors --clip-tokenizer DIR] [--size 1024] [--manifest manifest.tsv]

Counterpart of the reference's ``vae_preprocess`` (crates/data/src/bin/vae_preprocess.rs), the
``cache_*`` / ``encode_*`` binaries (src/bin) and the ``cache_*_embeddings*.py`` helpers, with the
same on-disk contract (crates/training/src/flux_preprocessor.rs:82-129: one tensor per file under
key ``latent`` / ``text_embed``; manifest columns ``latents_path, t5_path, clip_path, caption`` for
FLUX-family models and ``latents_path, clip_l_path, clip_g_path, pooled_path`` for SDXL). Captions
come from ``<image>.txt`` files next to the images. Encoders whose weights are not given are
skipped with a note; their manifest columns are left empty. Images are read with PIL when it is
installed, else only ``.npy`` arrays ([H, W, 3] uint8) are accepted.
"""
from __future__ import annotations

import argparse
import sys
from pathlib import Path

import torch

from ..data import save_cached_tensor
from ..models import build_model

IMG_EXT = (".png", ".jpg", ".jpeg", ".webp", ".bmp", ".npy")


def load_image(path: Path, size: int) -> torch.Tensor:
    """-> float [3, size, size] in [-1, 1] (centre crop to a square, bilinear resize)."""
    if path.suffix == ".npy":
        import numpy as np
        arr = torch.from_numpy(np.load(path))
    else:
        try:
            from PIL import Image
        except ImportError as e:                       # pragma: no cover - depends on the image
            raise RuntimeError("PIL is not installed: convert images to .npy ([H, W, 3] uint8)") from e
        import numpy as np
        arr = torch.from_numpy(np.asarray(Image.open(path).convert("RGB")))
    x = arr.permute(2, 0, 1).float() / 127.5 - 1.0
    _, h, w = x.shape
    s = min(h, w)
    x = x[:, (h - s) // 2:(h - s) // 2 + s, (w - s) // 2:(w - s) // 2 + s]
    if s != size:
        x = torch.nn.functional.interpolate(x[None], size=(size, size), mode="bilinear", align_corners=False)[0]
    return x


def _tokenize(tok_dir, text, max_len):
    from ..data.tokenizers import HfTokenizer
    return HfTokenizer(tok_dir, max_len)(text)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--family", default="flux", help="flux | sdxl (decides VAE kind and manifest columns)")
    ap.add_argument("--images", required=True); ap.add_argument("--out", required=True)
    ap.add_argument("--vae"); ap.add_argument("--t5"); ap.add_argument("--t5-tokenizer")
    ap.add_argument("--clip"); ap.add_argument("--clip-tokenizer"); ap.add_argument("--clip-g"); ap.add_argument("--clip-g-tokenizer")
    ap.add_argument("--size", type=int, default=1024); ap.add_argument("--t5-tokens", type=int, default=512)
    ap.add_argument("--manifest"); ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--random-init", action="store_true", help="run encoders with random weights (smoke tests)")
    ap.add_argument("--override", action="append", default=[], help="encoder config override kind:key=value")
    a = ap.parse_args(argv)
    dev = torch.device(a.device)
    dt = torch.bfloat16 if dev.type == "cuda" else torch.float32
    out = Path(a.out)
    out.mkdir(parents=True, exist_ok=True)
    ov = {}
    for item in a.override:
        kind, kv = item.split(":", 1)
        k, v = kv.split("=", 1)
        ov.setdefault(kind, {})[k] = eval(v, {"__builtins__": {}})

    def make(kind, weights):
        if not weights and not a.random_init:
            print(f"note: no weights for {kind}; skipping")
            return None
        m = build_model(kind, device=dev, dtype=dt, **ov.get(kind, {})).eval()
        if weights:
            from ..io.weights import load_model_weights
            load_model_weights(m, weights, kind, strict=False)
        return m

    sdxl = a.family == "sdxl"
    vae = make("vae_sdxl" if sdxl else "vae_flux", a.vae)
    t5 = None if sdxl else make("t5_encoder", a.t5)
    clip = make("clip_l", a.clip)
    clip_g = make("open_clip_g", a.clip_g) if sdxl else None
    images = sorted(p for p in Path(a.images).iterdir() if p.suffix.lower() in IMG_EXT)
    cols = ("latents_path", "clip_l_path", "clip_g_path", "pooled_path", "caption") if sdxl else \
        ("latents_path", "t5_path", "clip_path", "caption")
    rows = []
    with torch.no_grad():
        for p in images:
            cap_file = p.with_suffix(".txt")
            caption = cap_file.read_text().strip() if cap_file.exists() else ""
            rec = {c: "" for c in cols}
            rec["caption"] = caption.replace("\t", " ").replace("\n", " ")
            if vae is not None:
                z = vae.tiled_encode(load_image(p, a.size)[None].to(dev).to(dt))
                save_cached_tensor(out / f"{p.stem}.latent.safetensors", z[0].float().cpu().to(torch.bfloat16), "latent")
                rec["latents_path"] = f"{p.stem}.latent.safetensors"

            def ids_for(tok_dir, model, n):
                if tok_dir:
                    return _tokenize(tok_dir, caption, n)
                vocab = model.cfg.vocab_size                # no tokenizer: deterministic hash ids (smoke)
                g = torch.Generator().manual_seed(abs(hash(caption)) % (2 ** 31))
                return torch.randint(0, vocab - 1, (1, n), generator=g), torch.ones(1, n, dtype=torch.bool)

            if t5 is not None:
                ids, mask = ids_for(a.t5_tokenizer, t5, a.t5_tokens)
                h = t5(ids.to(dev), mask.to(dev))
                save_cached_tensor(out / f"{p.stem}.t5.safetensors", h[0].float().cpu().to(torch.bfloat16), "text_embed")
                rec["t5_path"] = f"{p.stem}.t5.safetensors"
            if clip is not None:
                ids, _ = ids_for(a.clip_tokenizer, clip, 77)
                h, pooled = clip(ids.to(dev), output_layer=-2 if sdxl else -1)
                if sdxl:
                    save_cached_tensor(out / f"{p.stem}.clip_l.safetensors", h[0].float().cpu().to(torch.bfloat16), "text_embed")
                    rec["clip_l_path"] = f"{p.stem}.clip_l.safetensors"
                else:
                    save_cached_tensor(out / f"{p.stem}.clip.safetensors", pooled[0].float().cpu().to(torch.bfloat16), "text_embed")
                    rec["clip_path"] = f"{p.stem}.clip.safetensors"
            if clip_g is not None:
                ids, _ = ids_for(a.clip_g_tokenizer, clip_g, 77)
                h, pooled = clip_g(ids.to(dev), output_layer=-2)
                save_cached_tensor(out / f"{p.stem}.clip_g.safetensors", h[0].float().cpu().to(torch.bfloat16), "text_embed")
                save_cached_tensor(out / f"{p.stem}.pooled.safetensors", pooled[0].float().cpu().to(torch.bfloat16), "text_embed")
                rec["clip_g_path"], rec["pooled_path"] = f"{p.stem}.clip_g.safetensors", f"{p.stem}.pooled.safetensors"
            rows.append(rec)
            print(f"cached {p.name}")
    man = Path(a.manifest) if a.manifest else out / "manifest.tsv"
    man.write_text("\t".join(cols) + "\n" + "".join("\t".join(r[c] for c in cols) + "\n" for r in rows))
    print(f"wrote {man} ({len(rows)} rows)")
    return 0


if __name__ == "__main__":
    sys.exit(main())

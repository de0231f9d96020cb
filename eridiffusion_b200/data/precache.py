"""Folder dataset with on-the-fly caching, in the encode-everything-then-free order.

* ``TextEmbeddingCache``: persistent cache of text-encoder outputs keyed by the SHA-256 of
  (encoder tag, prompt); one safetensors file per prompt with ``text_hidden`` (and ``pooled`` when
  the encoder has one), the key names of the reference's helper scripts
  (src/trainers/text_embedding_cache.rs; cache_zimage_embeddings_v2.py:45-49 strips padding by the
  attention mask before saving, as ``put`` does when a mask is given).
* ``DatasetCache``: ``{root}/cache/vae/{dataset}/`` and ``{root}/cache/text/{dataset}/`` with one
  safetensors file per sample (src/trainers/flux_cache_manager.rs:1-60).
* ``precache_folder``: the sequential pipeline of the reference's SimpleTuner-style trainer
  (src/trainers/pipeline_flux_lora_sequential.rs:98-557): encode all latents, release the VAE,
  encode all captions, release the text encoders, then write the manifest the cached-embedding
  loader reads. Samples already in the cache are skipped, so a second run costs nothing.
"""
from __future__ import annotations

import gc
import hashlib
import json
from pathlib import Path

import torch
from safetensors.torch import load_file, save_file

from .buckets import walk_images


def _free(obj_holder: list):
    """Drop the only reference to a model and return its memory to the allocator."""
    obj_holder.clear()
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


class TextEmbeddingCache:
    def __init__(self, root, encoder_tag: str = "default"):
        self.root = Path(root)
        self.root.mkdir(parents=True, exist_ok=True)
        self.tag = encoder_tag
        self.hits = self.misses = 0

    def key(self, prompt: str) -> str:
        return hashlib.sha256(f"{self.tag}\0{prompt}".encode()).hexdigest()

    def path(self, prompt: str) -> Path:
        return self.root / f"{self.key(prompt)}.safetensors"

    def has(self, prompt: str) -> bool:
        return self.path(prompt).exists()

    def get(self, prompt: str, device="cpu", dtype=None):
        """(text_hidden [T, D], pooled [P] or None), or ``None`` when the prompt is not cached."""
        p = self.path(prompt)
        if not p.exists():
            self.misses += 1
            return None
        self.hits += 1
        d = load_file(str(p))
        cv = lambda t: t.to(device=device, dtype=dtype or t.dtype)
        return cv(d["text_hidden"]), cv(d["pooled"]) if "pooled" in d else None

    def put(self, prompt: str, hidden, pooled=None, mask=None):
        """hidden [T, D] (or [1, T, D]); with ``mask`` [T] only the kept positions are stored."""
        h = hidden.detach()
        if h.dim() == 3:
            h = h[0]
        if mask is not None:
            h = h[mask.reshape(-1).bool().to(h.device)]
        d = {"text_hidden": h.to("cpu").contiguous()}
        if pooled is not None:
            d["pooled"] = pooled.detach().reshape(-1).to("cpu").contiguous()
        save_file(d, str(self.path(prompt)))

    def get_or_encode(self, prompt: str, encode, **kw):
        """``encode(prompt) -> (hidden, pooled or None[, mask])`` runs only on a miss."""
        r = self.get(prompt, **kw)
        if r is None:
            out = encode(prompt)
            self.put(prompt, out[0], out[1] if len(out) > 1 else None, out[2] if len(out) > 2 else None)
            r = self.get(prompt, **kw)
            self.hits -= 1                                  # the read-back is not a cache hit
        return r


class DatasetCache:
    def __init__(self, root, dataset: str):
        self.vae_dir = Path(root) / "cache" / "vae" / dataset
        self.text_dir = Path(root) / "cache" / "text" / dataset
        self.vae_dir.mkdir(parents=True, exist_ok=True)
        self.text_dir.mkdir(parents=True, exist_ok=True)

    @staticmethod
    def _stem(image_path) -> str:
        p = Path(image_path)
        return f"{p.stem}_{hashlib.sha256(str(p).encode()).hexdigest()[:10]}"

    def latent_path(self, image_path) -> Path:
        return self.vae_dir / f"{self._stem(image_path)}.safetensors"

    def text_path(self, image_path) -> Path:
        return self.text_dir / f"{self._stem(image_path)}.safetensors"


def precache_folder(dataset_dir, cache_root, dataset_name, make_vae, make_text_encoder, size=1024, microbatch=4,
                    trigger_word=None, manifest_name="manifest.jsonl"):
    """``make_vae() -> AutoencoderKL`` and ``make_text_encoder() -> callable(prompt) -> (hidden,
    pooled or None[, mask])`` are factories so that each model exists only during its own phase.
    Returns the manifest path and a report of what was encoded and what was already cached."""
    from .vae_preprocess import PreprocessConfig, VaePreprocessor
    files = walk_images(dataset_dir)
    if not files:
        raise FileNotFoundError(f"no images under {dataset_dir}")
    cache = DatasetCache(cache_root, dataset_name)
    report = {"samples": len(files), "latents_encoded": 0, "texts_encoded": 0}

    # phase 1: latents
    todo = [p for p, _ in files if not cache.latent_path(p).exists()]
    if todo:
        holder = [make_vae()]
        pre = VaePreprocessor(holder[0])
        cfg = PreprocessConfig((size, size), True, True, microbatch)
        for i in range(0, len(todo), microbatch):
            chunk = todo[i:i + microbatch]
            lat, _ = pre.encode_paths(chunk, cfg)
            for p, z in zip(chunk, lat):
                save_file({"latent": z.to("cpu").contiguous()}, str(cache.latent_path(p)))
            report["latents_encoded"] += len(chunk)
        del pre
        _free(holder)

    # phase 2: captions
    def caption_of(cap):
        text = Path(cap).read_text().strip() if cap is not None else ""
        return text.replace("[trigger]", trigger_word) if trigger_word else text

    todo_t = [(p, cap) for p, cap in files if not cache.text_path(p).exists()]
    if todo_t:
        holder = [make_text_encoder()]
        with torch.no_grad():
            for p, cap in todo_t:
                out = holder[0](caption_of(cap))
                hidden, pooled = out[0], out[1] if len(out) > 1 else None
                mask = out[2] if len(out) > 2 else None
                h = hidden[0] if hidden.dim() == 3 else hidden
                if mask is not None:
                    h = h[mask.reshape(-1).bool().to(h.device)]
                d = {"text_hidden": h.detach().to("cpu").contiguous()}
                if pooled is not None:
                    d["pooled"] = pooled.detach().reshape(-1).to("cpu").contiguous()
                save_file(d, str(cache.text_path(p)))
                report["texts_encoded"] += 1
        _free(holder)

    # manifest (paths relative to the cache root)
    root = Path(cache_root)
    mpath = root / manifest_name
    with open(mpath, "w") as f:
        for p, cap in files:
            f.write(json.dumps({"latents_path": str(cache.latent_path(p).relative_to(root)),
                                "t5_path": str(cache.text_path(p).relative_to(root)), "clip_path": "",
                                "caption": caption_of(cap), "metadata": {"source": str(p)}}) + "\n")
    return mpath, report

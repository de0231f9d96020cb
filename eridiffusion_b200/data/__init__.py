"""Cached-embedding data pipeline.

* manifest loaders for FLUX-style (``latents_path, t5_path, clip_path, caption`` + typed extra
  columns) and SDXL-style (``latents_path, clip_l_path, clip_g_path, pooled_path``) datasets in
  ``.tsv`` or ``.jsonl`` form, paths resolved against ``root_dir``
  (crates/training/src/flux/data_loader.rs:358-463, crates/training/src/sdxl/data_loader.rs:28-140);
* cache files: one safetensors file per tensor, key tried in order ``data``, ``latent``,
  ``text_embed``, else the first tensor; F32/F16/BF16 -> bf16; a leading batch dim of 1 is
  squeezed (crates/training/src/flux_preprocessor.rs:82-129);
* deterministic xorshift shuffle seeded by the epoch (flux/data_loader.rs:725-734);
* text padded to the batch maximum with a ``[B, 1, 1, T]`` mask (:254-264);
* a SHA-256 keyed JSON index cache of the parsed manifest (:488-617);
* per-batch host-to-device byte telemetry (:641-656);
* batches are assembled in pinned host memory by a prefetch thread and copied on a side stream;
* synthetic N(0,1) batch generators for every model family (flux/data.rs:78-97,
  bin/sdxl_10steps.rs:149-219).
"""
from __future__ import annotations

import csv
import hashlib
import json
import os
import queue
import threading
from dataclasses import dataclass, field
from pathlib import Path

import torch

from ..io import safetensors as st


# ------------------------------------------------------------------------- deterministic shuffle
def xorshift_permutation(n: int, seed: int) -> list[int]:
    """Fisher-Yates driven by xorshift64*, identical on every platform."""
    s = (seed * 0x9E3779B97F4A7C15 + 0xD1B54A32D192ED03) & 0xFFFFFFFFFFFFFFFF or 0x2545F4914F6CDD1D
    idx = list(range(n))
    for i in range(n - 1, 0, -1):
        s ^= (s >> 12)
        s ^= (s << 25) & 0xFFFFFFFFFFFFFFFF
        s ^= (s >> 27)
        r = (s * 0x2545F4914F6CDD1D) & 0xFFFFFFFFFFFFFFFF
        j = r % (i + 1)
        idx[i], idx[j] = idx[j], idx[i]
    return idx


# ------------------------------------------------------------------------- cache files
_KEY_ORDER = ("data", "latent", "text_embed", "text_hidden")


def load_cached_tensor(path, dtype=torch.bfloat16):
    with st.SafeFile(path) as f:
        keys = f.keys()
        key = next((k for k in _KEY_ORDER if k in keys), keys[0])
        t = f.get(key)
    if t.dim() >= 3 and t.shape[0] == 1:
        t = t.squeeze(0)
    return t.to(dtype)


def load_cached_key(path, key, dtype=torch.bfloat16):
    """One named tensor of a cache file, or ``None`` when the file has no such key."""
    with st.SafeFile(path) as f:
        if key not in f.keys():
            return None
        return f.get(key).to(dtype)


def load_cached_tensors(paths, dtype=torch.bfloat16, prefetcher=None):
    """``load_cached_tensor`` for many files at once. With a native ``Prefetcher`` every payload is
    queued first, so the reads of a batch overlap on the worker threads."""
    if prefetcher is None:
        return [load_cached_tensor(p, dtype) for p in paths]
    win = getattr(prefetcher, "max_inflight", 1)
    if len(paths) > win:                      # never queue more than the prefetcher holds at once
        out = []
        for i in range(0, len(paths), win):
            out += load_cached_tensors(paths[i:i + win], dtype, prefetcher)
        return out
    pending = []
    for p in paths:
        f = st.SafeFile(p)
        keys = f.keys()
        key = next((k for k in _KEY_ORDER if k in keys), keys[0])
        pending.append((f, key, prefetcher.submit_tensor(f, key)))
    out = []
    for f, key, ticket in pending:
        try:
            raw = prefetcher.wait(ticket)
            dt, shape = f.info(key)
            t = raw.view(dt).view(shape).clone() if raw.numel() else torch.empty(shape, dtype=dt)
        finally:
            prefetcher.release(ticket)
            f.close()
        if t.dim() >= 3 and t.shape[0] == 1:
            t = t.squeeze(0)
        out.append(t.to(dtype))
    return out


def save_cached_tensor(path, t, key="data"):
    st.save_file({key: t}, path)


# ------------------------------------------------------------------------- manifests
@dataclass
class ManifestEntry:
    paths: dict
    caption: str = ""
    metadata: dict = field(default_factory=dict)


FLUX_COLUMNS = ("latents_path", "t5_path", "clip_path")
SDXL_COLUMNS = ("latents_path", "clip_l_path", "clip_g_path", "pooled_path")


def _typed(v: str):
    for cast in (int, float):
        try:
            return cast(v)
        except (TypeError, ValueError):
            pass
    if isinstance(v, str) and v.lower() in ("true", "false"):
        return v.lower() == "true"
    return v


def parse_manifest(path, columns=FLUX_COLUMNS, root_dir=None, validate=False) -> list[ManifestEntry]:
    path = Path(path)
    root = Path(root_dir) if root_dir else path.parent
    entries = []
    if path.suffix == ".jsonl":
        rows = [json.loads(l) for l in path.read_text().splitlines() if l.strip()]
    else:
        with open(path, newline="") as f:
            rows = list(csv.DictReader(f, delimiter="\t"))
    for i, row in enumerate(rows):
        missing = [c for c in columns if c not in row]
        if missing:
            raise KeyError(f"{path}:{i + 1}: missing columns {missing}")
        paths = {c: str((root / row[c]).resolve()) if not os.path.isabs(row[c]) else row[c] for c in columns}
        meta = dict(row.get("metadata") or {}) if isinstance(row.get("metadata"), dict) else {}
        for k, v in row.items():
            if k not in columns and k not in ("caption", "metadata"):
                meta[k] = _typed(v)
        if validate:
            for p in paths.values():
                if not os.path.exists(p):
                    raise FileNotFoundError(f"{path}:{i + 1}: {p}")
        entries.append(ManifestEntry(paths, row.get("caption", "") or "", meta))
    return entries


def manifest_index(path, columns=FLUX_COLUMNS, root_dir=None, index_path=None, validate=False):
    """Parsed manifest cached as JSON next to it, keyed by the SHA-256 of the manifest bytes."""
    path = Path(path)
    digest = hashlib.sha256(path.read_bytes() + str(root_dir).encode()).hexdigest()
    index_path = Path(index_path) if index_path else path.with_suffix(path.suffix + ".index.json")
    if index_path.exists():
        try:
            doc = json.loads(index_path.read_text())
            if doc.get("sha256") == digest and doc.get("columns") == list(columns):
                return [ManifestEntry(**e) for e in doc["entries"]]
        except (json.JSONDecodeError, TypeError, KeyError):
            pass
    entries = parse_manifest(path, columns, root_dir, validate)
    try:
        index_path.write_text(json.dumps({"sha256": digest, "columns": list(columns),
                                          "entries": [e.__dict__ for e in entries]}))
    except OSError:
        pass
    return entries


# ------------------------------------------------------------------------- loaders
class CachedEmbeddingLoader:
    """Iterates batches of cached latents + text embeddings.

    ``next()`` returns a dict of device tensors: FLUX kind -> ``latents [B,C,H,W]``, ``txt
    [B,T,ctx]`` (padded to the batch maximum), ``txt_mask [B,1,1,T]``, ``pooled [B,vec]``,
    ``captions``; SDXL kind -> ``latents``, ``clip_l``, ``clip_g``, ``pooled``, ``time_ids
    [B,6]``. A background thread assembles the next batches in pinned memory.
    """

    def __init__(self, manifest, kind="flux", batch_size=1, root_dir=None, index_path=None,
                 shuffle=True, repeat=1, seed=0, device="cpu", rank=0, world=1, prefetch=2,
                 validate=False, drop_last=True):
        self.kind = kind
        cols = FLUX_COLUMNS if kind == "flux" else SDXL_COLUMNS
        self.entries = manifest_index(manifest, cols, root_dir, index_path, validate) * max(1, repeat)
        if not self.entries:
            raise ValueError("empty manifest")
        self.batch_size, self.shuffle, self.seed = batch_size, shuffle, seed
        self.device = torch.device(device)
        self.rank, self.world = rank, world
        self.drop_last = drop_last
        self.epoch = 0
        self.h2d_bytes = 0
        self.h2d_batches = 0
        self._order = self._make_order()
        self._pos = 0
        self._q = queue.Queue(maxsize=max(1, prefetch))
        self._stop = threading.Event()
        self._stream = torch.cuda.Stream() if self.device.type == "cuda" else None
        # native read-ahead threads for the per-sample files (csrc/host/prefetch.cpp) when built
        self._pf = None
        if os.environ.get("ERI_B200_NATIVE_PREFETCH", "1") == "1":
            try:
                from ..io.native_host import Prefetcher
                self._pf = Prefetcher(threads=4, max_inflight=max(8, 4 * batch_size))
            except Exception:
                self._pf = None
        self._thread = threading.Thread(target=self._worker, daemon=True)
        self._thread.start()

    def __len__(self):
        per_rank = len(self.entries) // self.world
        return per_rank // self.batch_size if self.drop_last else -(-per_rank // self.batch_size)

    def _make_order(self):
        n = len(self.entries)
        order = xorshift_permutation(n, self.seed + self.epoch) if self.shuffle else list(range(n))
        return order[self.rank::self.world]

    def _load_host(self, idxs):
        es = [self.entries[i] for i in idxs]
        pin = self.device.type == "cuda"
        out = {"captions": [e.caption for e in es], "metadata": [e.metadata for e in es]}
        many = lambda col: load_cached_tensors([e.paths[col] for e in es], prefetcher=self._pf)
        lat = torch.stack(many("latents_path"))
        out["latents"] = lat
        if self.kind == "flux":
            txts = many("t5_path")
            T = max(t.shape[0] for t in txts)
            txt = torch.zeros(len(es), T, txts[0].shape[-1], dtype=torch.bfloat16)
            mask = torch.zeros(len(es), 1, 1, T, dtype=torch.bool)
            for i, t in enumerate(txts):
                txt[i, : t.shape[0]] = t
                mask[i, ..., : t.shape[0]] = True
            out["txt"], out["txt_mask"] = txt, mask
            if all(str(e.paths.get("clip_path") or "") not in ("", ".") and Path(e.paths["clip_path"]).is_file() for e in es):
                out["pooled"] = torch.stack([t.reshape(-1) for t in many("clip_path")])
            else:
                # folder caches written by ``data.precache`` keep the pooled vector inside the text file
                pooled = [load_cached_key(e.paths["t5_path"], "pooled") for e in es]
                if all(p is not None for p in pooled):
                    out["pooled"] = torch.stack([p.reshape(-1) for p in pooled])
        else:
            out["clip_l"] = torch.stack(many("clip_l_path"))
            out["clip_g"] = torch.stack(many("clip_g_path"))
            out["pooled"] = torch.stack([t.reshape(-1) for t in many("pooled_path")])
            h, w = lat.shape[-2] * 8, lat.shape[-1] * 8
            ids = [[e.metadata.get("orig_h", h), e.metadata.get("orig_w", w), e.metadata.get("crop_y", 0),
                    e.metadata.get("crop_x", 0), e.metadata.get("tgt_h", h), e.metadata.get("tgt_w", w)] for e in es]
            out["time_ids"] = torch.tensor(ids, dtype=torch.float32)
        if pin:
            out = {k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in out.items()}
        return out

    def _worker(self):
        while not self._stop.is_set():
            if self._pos + self.batch_size > len(self._order):
                if self._pos < len(self._order) and not self.drop_last:
                    idxs = self._order[self._pos:]
                else:
                    self.epoch += 1
                    self._order, self._pos = self._make_order(), 0
                    idxs = self._order[: self.batch_size]
            else:
                idxs = self._order[self._pos:self._pos + self.batch_size]
            self._pos += len(idxs)
            try:
                item = self._load_host(idxs)
            except Exception as e:          # surfaced to the consumer
                item = e
            while not self._stop.is_set():
                try:
                    self._q.put(item, timeout=0.1)
                    break
                except queue.Full:
                    continue

    def next(self):
        item = self._q.get()
        if isinstance(item, Exception):
            raise item
        if self.device.type != "cuda":
            return item
        out = {}
        with torch.cuda.stream(self._stream):
            for k, v in item.items():
                if torch.is_tensor(v):
                    out[k] = v.to(self.device, non_blocking=True)
                    self.h2d_bytes += v.numel() * v.element_size()
                else:
                    out[k] = v
        torch.cuda.current_stream().wait_stream(self._stream)
        self.h2d_batches += 1
        return out

    __next__ = next

    def __iter__(self):
        return self

    def telemetry(self):
        return {"h2d_mb": self.h2d_bytes / 2 ** 20, "batches": self.h2d_batches, "epoch": self.epoch}

    def close(self):
        self._stop.set()
        if self._pf is not None:
            self._thread.join(timeout=5)
            self._pf.close()
            self._pf = None


# ------------------------------------------------------------------------- synthetic batches
def synthetic_batch(kind="flux", batch=1, device="cpu", dtype=torch.bfloat16, seed=0, height=1024, width=1024,
                    text_tokens=None, frames=33):
    """N(0,1) latents / embeddings of the shapes each model family trains on."""
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).to(dtype).to(device)
    if kind in ("flux", "chroma"):
        return {"latents": mk(batch, 16, height // 8, width // 8), "txt": mk(batch, text_tokens or 512, 4096),
                "pooled": mk(batch, 768)}
    if kind == "tiny_mmdit":
        return {"latents": mk(batch, 16, 32, 32), "txt": mk(batch, 64, 128), "pooled": mk(batch, 64)}
    if kind == "qwen_image":
        return {"latents": mk(batch, 16, height // 8, width // 8), "txt": mk(batch, text_tokens or 256, 3584)}
    if kind == "sdxl":
        return {"latents": mk(batch, 4, height // 8, width // 8), "txt": mk(batch, 77, 2048), "pooled": mk(batch, 1280),
                "time_ids": torch.tensor([[height, width, 0, 0, height, width]] * batch, dtype=torch.float32, device=device)}
    if kind == "sd15":
        return {"latents": mk(batch, 4, height // 8, width // 8), "txt": mk(batch, 77, 768)}
    if kind in ("sd3", "sd35"):
        return {"latents": mk(batch, 16, height // 8, width // 8), "txt": mk(batch, text_tokens or 333, 4096),
                "pooled": mk(batch, 2048)}
    if kind in ("ltx", "ltx_video"):
        h, w = height // 32, width // 32
        return {"latents": mk(batch, 128, frames * h * w, 1), "txt": mk(batch, text_tokens or 256, 4096),
                "grid_fhw": (frames, h, w)}
    if kind == "wan22":
        return {"latents": mk(batch, 16, frames, height // 8, width // 8), "txt": mk(batch, 512, 4096)}
    raise ValueError(kind)


# ------------------------------------------------------------------------- generic dataset API
class Dataset:
    def __len__(self):
        raise NotImplementedError

    def __getitem__(self, i):
        raise NotImplementedError


class Compose:
    def __init__(self, transforms):
        self.transforms = list(transforms)

    def __call__(self, x):
        for t in self.transforms:
            x = t(x)
        return x


class Normalize:
    def __init__(self, mean=0.5, std=0.5):
        self.mean, self.std = mean, std

    def __call__(self, img):
        return (img - self.mean) / self.std


class RandomCrop:
    def __init__(self, size, seed=0):
        self.size, self.g = size, torch.Generator().manual_seed(seed)

    def __call__(self, img):
        _, h, w = img.shape
        th, tw = (self.size, self.size) if isinstance(self.size, int) else self.size
        y = int(torch.randint(0, max(1, h - th + 1), (1,), generator=self.g))
        x = int(torch.randint(0, max(1, w - tw + 1), (1,), generator=self.g))
        return img[:, y:y + th, x:x + tw]


class ImageFolderDataset(Dataset):
    """Images with side-car caption files (``folder_path`` + ``caption_ext`` of the YAML)."""

    EXT = (".png", ".jpg", ".jpeg", ".webp", ".bmp")

    def __init__(self, folder, caption_ext="txt", transform=None, resolution=None):
        self.items = sorted(p for p in Path(folder).rglob("*") if p.suffix.lower() in self.EXT)
        self.caption_ext, self.transform, self.resolution = caption_ext, transform, resolution

    def __len__(self):
        return len(self.items)

    def __getitem__(self, i):
        from PIL import Image
        import numpy as np
        p = self.items[i]
        img = Image.open(p).convert("RGB")
        if self.resolution:
            img = img.resize((self.resolution, self.resolution), Image.BICUBIC)
        x = torch.from_numpy(np.asarray(img).copy()).permute(2, 0, 1).float() / 255.0
        if self.transform:
            x = self.transform(x)
        cap = p.with_suffix("." + self.caption_ext)
        return {"image": x, "caption": cap.read_text().strip() if cap.exists() else "", "path": str(p)}


class DataLoader:
    """Minimal batching iterator over a ``Dataset`` with deterministic shuffling."""

    def __init__(self, dataset, batch_size=1, shuffle=True, seed=0, drop_last=True, collate=None):
        self.ds, self.bs, self.shuffle, self.seed, self.drop_last = dataset, batch_size, shuffle, seed, drop_last
        self.collate = collate or self._default_collate
        self.epoch = 0

    @staticmethod
    def _default_collate(items):
        out = {}
        for k in items[0]:
            v = [it[k] for it in items]
            out[k] = torch.stack(v) if torch.is_tensor(v[0]) else v
        return out

    def __iter__(self):
        n = len(self.ds)
        order = xorshift_permutation(n, self.seed + self.epoch) if self.shuffle else list(range(n))
        self.epoch += 1
        for i in range(0, n, self.bs):
            idx = order[i:i + self.bs]
            if len(idx) < self.bs and self.drop_last:
                return
            yield self.collate([self.ds[j] for j in idx])


def bucket_key(width, height, step=64):
    """Aspect bucket of an image (crates/training/src/io.rs: bucket_key)."""
    return (max(step, round(width / step) * step), max(step, round(height / step) * step))

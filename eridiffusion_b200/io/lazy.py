"""Lazy, prefix-scoped access to one or several safetensors files.

``LazyLoader`` indexes the headers of every file once and reads a tensor only when it is asked
for (memory-mapped: nothing else of the file is touched); ``prefixed`` / ``pp`` return a view that
prepends a key prefix, the way model constructors walk a checkpoint. Covers the reference's
``LazySafetensorsLoader`` / ``LazyPrefixedLoader`` (src/loaders/lazy_safetensors.rs:12-237) and
``PrefixedWeightLoader`` / ``MemoryEfficientFluxLoader::from_safetensors_multi``
(src/loaders/memory_efficient_loader.rs:11-90). Tensors go to the requested device through a
pinned staging copy when the device is a GPU.
"""
from __future__ import annotations

from pathlib import Path

import torch

from .safetensors import SafeFile


class LazyLoader:
    def __init__(self, paths, device="cpu", dtype=None):
        if isinstance(paths, (str, Path)):
            p = Path(paths)
            paths = sorted(p.glob("*.safetensors")) if p.is_dir() else [p]
        self.files = [SafeFile(p) for p in paths]
        if not self.files:
            raise FileNotFoundError("no safetensors files given")
        self.device, self.dtype = torch.device(device), dtype
        self._where = {}
        for f in self.files:
            for k in f.keys():
                if k in self._where:
                    raise KeyError(f"{k} appears in both {self._where[k].path} and {f.path}")
                self._where[k] = f
        self.bytes_read = 0

    # ------------------------------------------------------------------ lookup
    def keys(self):
        return list(self._where)

    def has_key(self, name) -> bool:
        return name in self._where

    def tensor_meta(self, name):
        """(shape, dtype) without reading the data, or ``None``."""
        f = self._where.get(name)
        if f is None:
            return None
        dt, shape = f.info(name)
        return shape, dt

    def load_tensor(self, name, device=None, dtype=None, shape=None):
        f = self._where.get(name)
        if f is None:
            raise KeyError(f"tensor {name!r} not found in {[x.path for x in self.files]}")
        t = f.get(name)
        if shape is not None and tuple(t.shape) != tuple(shape):
            raise ValueError(f"{name}: shape {tuple(t.shape)} != expected {tuple(shape)}")
        self.bytes_read += t.numel() * t.element_size()
        dtype = dtype or self.dtype
        if dtype is not None:
            t = t.to(dtype)
        dev = torch.device(device) if device is not None else self.device
        if dev.type == "cuda":
            return t.pin_memory().to(dev, non_blocking=True)
        return t

    tensor = load_tensor

    def load_prefix(self, prefix, strip=True, **kw):
        """Every tensor under ``prefix`` as a dict (keys without the prefix when ``strip``)."""
        n = len(prefix)
        return {(k[n:] if strip else k): self.load_tensor(k, **kw) for k in self._where if k.startswith(prefix)}

    def prefixed(self, prefix):
        return PrefixedLoader(self, prefix)

    pp = prefixed

    def close(self):
        for f in self.files:
            f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


class PrefixedLoader:
    """View of a ``LazyLoader`` under a key prefix; prefixes nest with ``pp``."""

    def __init__(self, base: LazyLoader, prefix: str):
        self.base = base
        self.prefix = prefix if not prefix or prefix.endswith(".") else prefix + "."

    def _k(self, name):
        return self.prefix + name

    def keys(self):
        n = len(self.prefix)
        return [k[n:] for k in self.base.keys() if k.startswith(self.prefix)]

    def has_key(self, name) -> bool:
        return self.base.has_key(self._k(name))

    def tensor_meta(self, name):
        return self.base.tensor_meta(self._k(name))

    def load_tensor(self, name, **kw):
        return self.base.load_tensor(self._k(name), **kw)

    tensor = load_tensor

    def prefixed(self, prefix):
        return PrefixedLoader(self.base, self._k(prefix))

    pp = prefixed

    def load_into(self, module: torch.nn.Module, strict: bool = True):
        """Copy the tensors under this prefix into ``module``'s parameters and buffers by name."""
        own = dict(module.named_parameters())
        own.update(dict(module.named_buffers()))
        missing = [n for n in own if not self.has_key(n)]
        extra = [k for k in self.keys() if k not in own]
        if strict and (missing or extra):
            raise KeyError(f"{self.prefix}: missing={missing[:5]} unexpected={extra[:5]}")
        with torch.no_grad():
            for n, p in own.items():
                if self.has_key(n):
                    p.copy_(self.load_tensor(n, device=p.device, dtype=p.dtype, shape=p.shape))
        return missing, extra

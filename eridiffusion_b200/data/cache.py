"""Two-level tensor cache keyed by the source file path: L1 in host (pinned) memory with a byte
budget, L2 on disk as one safetensors file plus a JSON side-car per entry.

Same behaviour as the reference's ``CacheManager`` (crates/data/src/cache_manager.rs:40-137): the
key is the SHA-256 of the path, a miss in memory falls through to disk and promotes the entry,
``put`` writes both levels, entries are evicted from memory until the new one fits, and hit / miss
counters are kept per level. Differences: the memory level counts bytes instead of whole megabytes
(the reference's integer-megabyte estimate makes every tensor under 1 MiB free), eviction is least-
recently-used instead of hash-map order, and L1 entries are pinned so that the copy to the GPU can be
asynchronous.
"""
from __future__ import annotations

import hashlib
import json
import threading
import time
from collections import OrderedDict
from dataclasses import asdict, dataclass, field
from pathlib import Path

import torch
from safetensors.torch import load_file, save_file

CACHE_VERSION = 1
_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32,
           "BOOL": torch.bool}
_NAMES = {v: k for k, v in _DTYPES.items()}


@dataclass
class CacheMetadata:
    original_path: str
    cache_version: int = CACHE_VERSION
    dtype: str = "BF16"
    shape: list = field(default_factory=list)
    timestamp: int = 0


@dataclass
class CacheEntry:
    tensor: torch.Tensor
    metadata: CacheMetadata


@dataclass
class CacheStats:
    memory_hits: int = 0
    memory_misses: int = 0
    disk_hits: int = 0
    disk_misses: int = 0
    total_requests: int = 0
    evictions: int = 0


class CacheManager:
    def __init__(self, disk_cache_dir, memory_limit_mb=1024, device="cpu", pin=None):
        self.dir = Path(disk_cache_dir)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.limit = int(memory_limit_mb) << 20
        self.device = torch.device(device)
        self.pin = torch.cuda.is_available() if pin is None else pin
        self._mem: OrderedDict[str, CacheEntry] = OrderedDict()
        self._bytes = 0
        self._lock = threading.Lock()
        self.stats = CacheStats()

    @staticmethod
    def cache_key(path) -> str:
        return hashlib.sha256(str(path).encode()).hexdigest()

    @staticmethod
    def _nbytes(t):
        return t.numel() * t.element_size()

    def memory_bytes(self):
        return self._bytes

    def __len__(self):
        return len(self._mem)

    # ------------------------------------------------------------------ lookups
    def get(self, path):
        """The entry for ``path`` (tensor on ``self.device``), or ``None``."""
        key = self.cache_key(path)
        with self._lock:
            self.stats.total_requests += 1
            e = self._mem.get(key)
            if e is not None:
                self._mem.move_to_end(key)
                self.stats.memory_hits += 1
                return self._materialise(e)
            self.stats.memory_misses += 1
        stem = self.dir / key
        if stem.with_suffix(".tensor").exists() and stem.with_suffix(".meta").exists():
            try:
                e = self._load(stem)
            except Exception:
                e = None
            if e is not None:
                with self._lock:
                    self.stats.disk_hits += 1
                    self._insert(key, e)
                return self._materialise(e)
        with self._lock:
            self.stats.disk_misses += 1
        return None

    def put(self, path, tensor, metadata=None):
        if tensor.dtype not in _NAMES:
            raise ValueError(f"unsupported dtype for the cache: {tensor.dtype}")
        host = tensor.detach().to("cpu").contiguous()
        if self.pin:
            host = host.pin_memory()
        md = metadata or CacheMetadata(original_path=str(path))
        md.dtype, md.shape = _NAMES[host.dtype], list(host.shape)
        md.timestamp = md.timestamp or int(time.time())
        e = CacheEntry(host, md)
        key = self.cache_key(path)
        with self._lock:
            self._insert(key, e)
        stem = self.dir / key
        save_file({"data": host}, str(stem.with_suffix(".tensor")))
        stem.with_suffix(".meta").write_text(json.dumps(asdict(md)))

    def get_or_compute(self, path, fn):
        """``get(path)``, computing and storing ``fn(path)`` on a miss."""
        e = self.get(path)
        if e is None:
            self.put(path, fn(path))
            e = self.get(path)
        return e

    def clear_memory(self):
        with self._lock:
            self._mem.clear()
            self._bytes = 0

    # ------------------------------------------------------------------ internals
    def _materialise(self, e):
        if self.device.type == "cpu":
            return e
        return CacheEntry(e.tensor.to(self.device, non_blocking=True), e.metadata)

    def _insert(self, key, e):
        size = self._nbytes(e.tensor)
        old = self._mem.pop(key, None)
        if old is not None:
            self._bytes -= self._nbytes(old.tensor)
        while self._mem and self._bytes + size > self.limit:
            _, ev = self._mem.popitem(last=False)
            self._bytes -= self._nbytes(ev.tensor)
            self.stats.evictions += 1
        self._mem[key] = e
        self._bytes += size

    def _load(self, stem):
        md = CacheMetadata(**json.loads(stem.with_suffix(".meta").read_text()))
        t = load_file(str(stem.with_suffix(".tensor")))["data"]
        if list(t.shape) != list(md.shape):
            raise ValueError(f"shape mismatch: stored={list(t.shape)} meta={md.shape}")
        want = _DTYPES.get(md.dtype.upper())
        if want is None:
            raise ValueError(f"unknown dtype: {md.dtype}")
        if t.dtype != want:
            t = t.to(want)
        if self.pin:
            t = t.pin_memory()
        return CacheEntry(t, md)

"""safetensors reader / writer.

File layout: 8-byte little-endian header length, JSON header
``{name: {dtype, shape, data_offsets}, "__metadata__": {...}}``, then the raw tensor bytes.
The writer emits tensors sorted by name, which makes files byte-reproducible
(the reference sorts before serialising: crates/training/src/checkpoint_safetensors.rs:102-112).
The reader memory-maps the file; ``StrictLoader`` enforces that exactly the expected key set was
consumed (crates/common/weights/src/strict_loader.rs:21-92, strict_checkpoint.rs:111-118).

When the native host library is built, large reads go mmap -> pinned staging -> async H2D on a
side stream (``csrc/host/safetensors_io.cpp``); the pure-Python path below is always available.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from pathlib import Path

import numpy as np
import torch

_DT = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_DT_INV = {v: k for k, v in _DT.items()}
_NP = {
    "F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I64": np.int64,
    "I32": np.int32, "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_,
}


def save_file(tensors: dict, path, metadata: dict | None = None):
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    header, off = {}, 0
    names = sorted(tensors)
    blobs = []
    for n in names:
        t = tensors[n].detach().contiguous().cpu()
        if t.dtype not in _DT_INV:
            raise TypeError(f"{n}: unsupported dtype {t.dtype}")
        nb = t.numel() * t.element_size()
        header[n] = {"dtype": _DT_INV[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nb]}
        off += nb
        blobs.append(t)
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    tmp = path.with_suffix(path.suffix + ".tmp")
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for t in blobs:
            if t.numel() == 0:
                continue
            t = t.reshape(-1)
            raw = t.view(torch.uint8) if t.dtype != torch.bool else t.to(torch.uint8)
            f.write(raw.reshape(-1).numpy().tobytes())
    os.replace(tmp, path)


class SafeFile:
    """Memory-mapped safetensors file."""

    def __init__(self, path):
        self.path = str(path)
        self._f = open(self.path, "rb")
        (hl,) = struct.unpack("<Q", self._f.read(8))
        if hl > 100 * 1024 * 1024:
            raise ValueError(f"{path}: header length {hl} is not plausible")
        self.header = json.loads(self._f.read(hl))
        self.metadata = self.header.pop("__metadata__", {})
        self._base = 8 + hl
        size = os.path.getsize(self.path)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        for n, e in self.header.items():
            b, e_ = e["data_offsets"]
            if e_ < b or self._base + e_ > size:
                raise ValueError(f"{path}: tensor {n} runs past the end of the file")

    def keys(self):
        return list(self.header)

    def info(self, name):
        e = self.header[name]
        return _DT[e["dtype"]], tuple(e["shape"])

    def get(self, name, device="cpu", dtype=None):
        e = self.header[name]
        b, e_ = e["data_offsets"]
        npdt = _NP[e["dtype"]]
        arr = np.frombuffer(self._mm, dtype=npdt, count=(e_ - b) // np.dtype(npdt).itemsize,
                            offset=self._base + b)
        t = torch.from_numpy(arr.copy()) if arr.size else torch.empty(0)
        if e["dtype"] == "BF16":
            t = t.view(torch.bfloat16)
        elif e["dtype"] == "BOOL":
            t = t.to(torch.bool)
        t = t.view(e["shape"])
        if dtype is not None:
            t = t.to(dtype)
        return t.to(device) if str(device) != "cpu" else t

    def close(self):
        if self._mm is not None:
            self._mm.close()
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def load_file(path, device="cpu", dtype=None, prefix_filter=None):
    with SafeFile(path) as f:
        return {k: f.get(k, device, dtype) for k in f.keys()
                if prefix_filter is None or any(k.startswith(p) for p in prefix_filter)}


def read_metadata(path):
    with SafeFile(path) as f:
        return dict(f.metadata)


class StrictLoader:
    """Tracks which keys were read; ``finish()`` raises unless used == available (or the expected
    set when given)."""

    def __init__(self, path, expected=None):
        self.file = SafeFile(path)
        self.used = set()
        self.expected = set(expected) if expected is not None else None

    def get(self, name, device="cpu", dtype=None, shape=None):
        if name not in self.file.header:
            raise KeyError(f"{self.file.path}: missing tensor {name!r}")
        t = self.file.get(name, device, dtype)
        if shape is not None and tuple(t.shape) != tuple(shape):
            raise ValueError(f"{name}: shape {tuple(t.shape)} != expected {tuple(shape)}")
        self.used.add(name)
        return t

    def finish(self):
        avail = set(self.file.keys())
        target = self.expected if self.expected is not None else avail
        missing, unused = target - self.used, avail - self.used
        self.file.close()
        if missing or unused:
            raise KeyError(f"strict load failed: missing={sorted(missing)[:5]} unused={sorted(unused)[:5]}")


def assert_not_text_encoder(keys):
    """Guard against pointing the trainer at a text-encoder file
    (crates/common/weights: assert_not_text_encoder)."""
    bad = [k for k in keys if k.startswith(("text_model.", "encoder.block.", "shared.weight"))]
    if bad:
        raise ValueError(f"file looks like a text encoder (e.g. {bad[0]})")

"""Device selection and per-device bookkeeping (crates/core/src/device.rs ``Device::{Cpu,Cuda(i)}``,
``DeviceManager``; crates/common/telemetry ``memory_mb`` / ``now_millis``). One process drives one
GPU: ``DeviceManager.bind_local_rank`` picks it from LOCAL_RANK and never touches another."""
from __future__ import annotations

import os
import time
from dataclasses import dataclass

import torch

from .errors import DeviceError


@dataclass(frozen=True)
class Device:
    kind: str = "cpu"          # "cpu" | "cuda"
    index: int = 0

    @staticmethod
    def parse(spec) -> "Device":
        if isinstance(spec, Device):
            return spec
        if isinstance(spec, torch.device):
            return Device(spec.type, spec.index or 0)
        s = str(spec).lower()
        if s in ("cpu", "host"):
            return Device("cpu", 0)
        if s.startswith("cuda") or s.startswith("gpu") or s.isdigit():
            idx = s.split(":")[1] if ":" in s else (s if s.isdigit() else "0")
            return Device("cuda", int(idx))
        raise DeviceError(f"unknown device spec {spec!r}")

    @property
    def torch(self) -> torch.device:
        return torch.device(self.kind, self.index) if self.kind == "cuda" else torch.device("cpu")

    def __str__(self):
        return f"cuda:{self.index}" if self.kind == "cuda" else "cpu"


class DeviceManager:
    """Tracks the process's device and its memory high-water marks."""

    def __init__(self):
        self.device = Device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else Device()

    def bind_local_rank(self) -> Device:
        if torch.cuda.is_available():
            idx = int(os.environ.get("LOCAL_RANK", "0")) % max(1, torch.cuda.device_count())
            torch.cuda.set_device(idx)
            self.device = Device("cuda", idx)
        return self.device

    def set(self, spec) -> Device:
        d = Device.parse(spec)
        if d.kind == "cuda":
            if not torch.cuda.is_available():
                raise DeviceError("CUDA device requested but none is visible")
            if d.index >= torch.cuda.device_count():
                raise DeviceError(f"cuda:{d.index} requested, {torch.cuda.device_count()} visible")
            torch.cuda.set_device(d.index)
        self.device = d
        return d

    def properties(self) -> dict:
        if self.device.kind != "cuda":
            return {"name": "cpu"}
        p = torch.cuda.get_device_properties(self.device.index)
        return {"name": p.name, "sms": p.multi_processor_count, "total_memory": p.total_memory,
                "capability": (p.major, p.minor)}

    def memory(self) -> dict:
        if self.device.kind != "cuda":
            return {"allocated_mb": 0.0, "reserved_mb": 0.0, "peak_mb": 0.0, "free_mb": 0.0}
        free, total = torch.cuda.mem_get_info(self.device.index)
        mb = 1.0 / (1 << 20)
        return {"allocated_mb": torch.cuda.memory_allocated(self.device.index) * mb,
                "reserved_mb": torch.cuda.memory_reserved(self.device.index) * mb,
                "peak_mb": torch.cuda.max_memory_allocated(self.device.index) * mb,
                "free_mb": free * mb, "total_mb": total * mb}

    def synchronize(self):
        if self.device.kind == "cuda":
            torch.cuda.synchronize(self.device.index)


_MANAGER = None


def current_device() -> Device:
    global _MANAGER
    if _MANAGER is None:
        _MANAGER = DeviceManager()
    return _MANAGER.device


def memory_mb(device=None) -> float:
    """Bytes currently allocated by tensors on the device, in MiB."""
    if not torch.cuda.is_available():
        return 0.0
    d = Device.parse(device) if device is not None else current_device()
    return torch.cuda.memory_allocated(d.index) / (1 << 20) if d.kind == "cuda" else 0.0


def now_millis() -> int:
    return int(time.time() * 1000)


def set_seed(seed: int) -> None:
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)

"""Name -> (id, tensor) parameter registry and device-memory guards.

Counterpart of the reference's ``ParamRegistry`` / ``ParamId`` (crates/common/weights/src/
registry.rs:7-94: ``insert, get, id_of, iter, set_requires_grad, get_by_id, assign, remove,
emit_json_summary``) and of ``vram_used_gb`` / ``assert_vram_below`` (registry.rs:96-114, NVML
behind a feature flag). Ids are stable for the life of the registry, so optimizer state and
block-swap plans can refer to a parameter after its tensor has been replaced or released.

Two indexes (by name and by id) make every operation O(1); the reference scans the map for the
by-id operations.
"""
from __future__ import annotations

import json
from collections import Counter
from dataclasses import dataclass

import torch


@dataclass(frozen=True, order=True)
class ParamId:
    value: int


class ParamRegistry:
    def __init__(self):
        self._by_name: dict[str, tuple[ParamId, torch.Tensor]] = {}
        self._name_of: dict[ParamId, str] = {}
        self._next = 1

    def insert(self, name: str, t: torch.Tensor) -> ParamId:
        """Register (or re-register under a fresh id) ``name``."""
        old = self._by_name.get(name)
        if old is not None:
            del self._name_of[old[0]]
        pid = ParamId(self._next)
        self._next += 1
        self._by_name[name] = (pid, t)
        self._name_of[pid] = name
        return pid

    @classmethod
    def from_module(cls, module: torch.nn.Module, prefix: str = ""):
        reg = cls()
        for n, p in module.named_parameters():
            reg.insert(prefix + n, p)
        return reg

    def get(self, name: str):
        e = self._by_name.get(name)
        return None if e is None else e[1]

    def id_of(self, name: str):
        e = self._by_name.get(name)
        return None if e is None else e[0]

    def name_of(self, pid: ParamId):
        return self._name_of.get(pid)

    def get_by_id(self, pid: ParamId):
        n = self._name_of.get(pid)
        return None if n is None else self._by_name[n][1]

    def __iter__(self):
        for name, (pid, t) in self._by_name.items():
            yield name, pid, t

    def __len__(self):
        return len(self._by_name)

    def __contains__(self, name):
        return name in self._by_name

    def set_requires_grad(self, ids, on: bool = True):
        """Gradient policy: off for everything, ``on`` for the given ids only."""
        want = set(ids)
        for name, (pid, t) in self._by_name.items():
            flag = on and pid in want
            if t.is_leaf:
                t.requires_grad_(flag and t.is_floating_point())
            else:
                self._by_name[name] = (pid, t.detach().requires_grad_(flag and t.is_floating_point()))

    def assign(self, pid: ParamId, new_t: torch.Tensor):
        n = self._name_of.get(pid)
        if n is None:
            raise KeyError(f"{pid} not found for assign()")
        self._by_name[n] = (pid, new_t)

    def remove(self, name: str) -> bool:
        """Drop a parameter (releases a block-swapped layer's tensors)."""
        e = self._by_name.pop(name, None)
        if e is None:
            return False
        del self._name_of[e[0]]
        return True

    def total_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for _, _, t in self)

    def emit_json_summary(self) -> str:
        dt = Counter(str(t.dtype).replace("torch.", "") for _, _, t in self)
        dev = Counter(str(t.device) for _, _, t in self)
        return json.dumps({"count": len(self), "bytes": self.total_bytes(),
                           "trainable": sum(1 for _, _, t in self if t.requires_grad),
                           "dtypes": dict(dt), "devices": dict(dev)}, sort_keys=True)


def vram_used_gb(device: int = 0, nvml=None) -> float:
    """Memory in use on ``device`` as the driver sees it (all processes), in GiB. Reads NVML
    (``pynvml``; pass a stand-in through ``nvml`` in tests); without NVML falls back to
    ``torch.cuda.mem_get_info``."""
    if nvml is None:
        try:
            import pynvml as nvml
        except ImportError:
            nvml = None
    if nvml is not None:
        try:
            nvml.nvmlInit()
            h = nvml.nvmlDeviceGetHandleByIndex(device)
            return nvml.nvmlDeviceGetMemoryInfo(h).used / 2 ** 30
        except Exception:
            if not torch.cuda.is_available():
                raise
    if not torch.cuda.is_available():
        raise RuntimeError("vram_used_gb: neither NVML nor a CUDA device is available")
    free, total = torch.cuda.mem_get_info(device)
    return (total - free) / 2 ** 30


def assert_vram_below(limit_gb: float, device: int = 0, nvml=None):
    used = vram_used_gb(device, nvml)
    if used > limit_gb:
        raise MemoryError(f"VRAM used {used:.2f} GB exceeds limit {limit_gb:.2f} GB")
    return used

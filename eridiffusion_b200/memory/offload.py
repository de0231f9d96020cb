"""Whole-model offloading and the memory-strategy controller.

Reference: ``ModelOffloader{offload_model, load_model, is_loaded, is_offloaded, get_stats,
clear_offloaded, register_model, cleanup_memory}`` (src/trainers/model_offloader.rs:16-202): the
sequential pipeline keeps VAE, text encoders and the diffusion model on the GPU one at a time; and
``MemoryOptimizer`` with ``MemoryStrategy``, ``MemoryPressure``, batch-size auto-adjust,
``MemoryStats{usage_percent, remaining_mb}`` and ``get_optimization_tips``
(src/trainers/memory_optimizer.rs:13-369).

Offloaded weights live in PINNED host memory, so that bringing a model back is one asynchronous
copy per tensor on a side stream at link speed, and the copy of model i + 1 can run under the
compute of model i (``prefetch``). The reference keeps pageable host copies and loads
synchronously.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass

import torch


class ModelOffloader:
    def __init__(self, device=None, pin: bool | None = None):
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        self.pin = torch.cuda.is_available() if pin is None else pin
        self._host: dict[str, dict[str, torch.Tensor]] = {}
        self._loaded: dict[str, int] = {}
        self._pending: dict[str, tuple] = {}
        self._stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    # -- registration / state
    def register_model(self, name: str, size_bytes: int):
        self._loaded[name] = int(size_bytes)

    def is_loaded(self, name: str) -> bool:
        return name in self._loaded

    def is_offloaded(self, name: str) -> bool:
        return name in self._host

    def get_stats(self):
        """(number of models on the device, number offloaded to the host)."""
        return len(self._loaded), len(self._host)

    def offloaded_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for w in self._host.values() for t in w.values())

    # -- movement
    def offload_model(self, name: str, weights):
        """``weights``: {key: tensor} or an ``nn.Module`` (its parameters and buffers are moved in
        place and keep their identity, so optimizers and adapters stay valid)."""
        module = weights if isinstance(weights, torch.nn.Module) else None
        tensors = dict(module.state_dict(keep_vars=True)) if module is not None else dict(weights)
        host = {}
        for k, t in tensors.items():
            h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=self.pin and t.numel() > 0)
            h.copy_(t.detach(), non_blocking=False)
            host[k] = h
            if module is not None:
                t.data = h
        self._host[name] = host
        self._loaded.pop(name, None)
        self.cleanup_memory()
        return host

    def prefetch(self, name: str):
        """Start the host-to-device copies of ``name`` on the side stream; ``load_model`` then only
        waits for them."""
        if name in self._pending or name not in self._host:
            return
        if self._stream is None:
            self._pending[name] = ({k: h for k, h in self._host[name].items()}, None)
            return
        with torch.cuda.stream(self._stream):
            dev = {k: h.to(self.device, non_blocking=True) for k, h in self._host[name].items()}
            ev = torch.cuda.Event()
            ev.record(self._stream)
        self._pending[name] = (dev, ev)

    def load_model(self, name: str, module: torch.nn.Module | None = None):
        """Back to the device. With ``module`` the tensors are re-bound in place; the dict of
        device tensors is returned either way."""
        if name not in self._host:
            raise KeyError(f"model {name!r} is not offloaded")
        self.prefetch(name)
        dev, ev = self._pending.pop(name)
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
            for t in dev.values():
                t.record_stream(torch.cuda.current_stream(self.device))
        if module is not None:
            for k, t in module.state_dict(keep_vars=True).items():
                t.data = dev[k]
        self._loaded[name] = sum(t.numel() * t.element_size() for t in dev.values())
        del self._host[name]
        return dev

    def clear_offloaded(self):
        self._host.clear()
        self._pending.clear()

    def cleanup_memory(self):
        if torch.cuda.is_available():
            torch.cuda.empty_cache()


# ---------------------------------------------------------------------------- strategy controller
class MemoryStrategy(str, enum.Enum):
    NONE = "none"                           # everything resident (the default on a 180 GB part)
    CONSERVATIVE = "conservative"           # activation checkpointing
    AGGRESSIVE = "aggressive"               # + quantised base weights, 8-bit optimizer state
    EXTREME = "extreme"                     # + block swap / sequential model offload


class MemoryPressure(str, enum.Enum):
    LOW = "low"
    MEDIUM = "medium"
    HIGH = "high"
    CRITICAL = "critical"


@dataclass
class MemoryStats:
    current_mb: float
    peak_mb: float
    limit_mb: float
    pressure: MemoryPressure
    batch_size: int
    oom_count: int

    def usage_percent(self) -> float:
        return 100.0 * self.current_mb / max(self.limit_mb, 1e-9)

    def remaining_mb(self) -> float:
        return max(0.0, self.limit_mb - self.current_mb)


class MemoryOptimizer:
    def __init__(self, strategy: MemoryStrategy | str = MemoryStrategy.NONE, memory_limit_gb: float = 180.0,
                 batch_size: int = 1):
        self.strategy = MemoryStrategy(strategy)
        self.limit_mb = memory_limit_gb * 1024.0
        self.current_mb = self.peak_mb = 0.0
        self.batch_size, self.min_bs, self.max_bs = batch_size, 1, max(1, batch_size)
        self.oom_count = 0
        self._calm = 0

    def set_batch_size_limits(self, lo: int, hi: int):
        self.min_bs, self.max_bs = max(1, lo), max(lo, hi)
        self.batch_size = min(max(self.batch_size, self.min_bs), self.max_bs)

    def apply_strategy(self) -> dict:
        """Settings for the job factory / trainer config that realise the strategy."""
        s = self.strategy
        order = [MemoryStrategy.NONE, MemoryStrategy.CONSERVATIVE, MemoryStrategy.AGGRESSIVE, MemoryStrategy.EXTREME]
        lvl = order.index(s)
        return {"activation_checkpointing": lvl >= 1, "quantize_base": lvl >= 2,
                "optimizer": "adamw8bit" if lvl >= 2 else None, "block_swap": lvl >= 3,
                "sequential_model_offload": lvl >= 3, "vae_tiling": lvl >= 2}

    def update_memory_usage(self, current_mb: float):
        self.current_mb = current_mb
        self.peak_mb = max(self.peak_mb, current_mb)

    def record_oom(self):
        self.oom_count += 1
        self._calm = 0

    def get_memory_pressure(self) -> MemoryPressure:
        u = self.current_mb / max(self.limit_mb, 1e-9)
        return (MemoryPressure.CRITICAL if u > 0.95 else MemoryPressure.HIGH if u > 0.85 else
                MemoryPressure.MEDIUM if u > 0.6 else MemoryPressure.LOW)

    def adjust_batch_size(self) -> int:
        """Halve under critical pressure or after an OOM, step down under high pressure, step up
        after ten consecutive calm readings."""
        p = self.get_memory_pressure()
        if p == MemoryPressure.CRITICAL:
            self.batch_size, self._calm = max(self.min_bs, self.batch_size // 2), 0
        elif p == MemoryPressure.HIGH:
            self.batch_size, self._calm = max(self.min_bs, self.batch_size - 1), 0
        elif p == MemoryPressure.LOW:
            self._calm += 1
            if self._calm >= 10:
                self.batch_size, self._calm = min(self.max_bs, self.batch_size + 1), 0
        else:
            self._calm = 0
        return self.batch_size

    def optimize_tensor(self, tensor: torch.Tensor, name: str = "") -> torch.Tensor:
        """Under the aggressive strategies, fp32 tensors that are not normalisation or embedding
        parameters are stored as bf16."""
        if self.strategy in (MemoryStrategy.AGGRESSIVE, MemoryStrategy.EXTREME) and tensor.dtype == torch.float32 \
                and not any(k in name for k in ("norm", "embed", "scale_shift")):
            return tensor.to(torch.bfloat16)
        return tensor

    def get_stats(self) -> MemoryStats:
        return MemoryStats(self.current_mb, self.peak_mb, self.limit_mb, self.get_memory_pressure(), self.batch_size,
                           self.oom_count)


def get_optimization_tips(stats: MemoryStats) -> list[str]:
    tips = []
    if stats.usage_percent() > 85:
        tips.append("enable activation checkpointing (gradient_checkpointing: true)")
        tips.append("store the frozen base weights quantised (model.quantize: true) for LoRA runs")
    if stats.usage_percent() > 95 or stats.oom_count:
        tips.append("reduce the batch size and raise grad_accum_steps to keep the effective batch")
        tips.append("shard parameters and optimizer state over more GPUs (parallel.zero_stage: 3)")
        tips.append("turn on block swap (use_layer_streaming) as the last resort: it trades step time for memory")
    if stats.usage_percent() < 40 and not stats.oom_count:
        tips.append("memory is mostly free: a larger batch per GPU amortises weight reads")
    return tips

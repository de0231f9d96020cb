"""Gradient accumulation: configuration, a named-gradient accumulator, dynamic step adjustment.

Covers the reference's accumulation service (crates/training/src/accumulation.rs:11-321:
``AccumulationConfig{steps, normalize, dtype, sync_mode, reduction}``, ``GradientAccumulator``,
``DynamicAccumulator``, ``GradientCheckpointing`` layer selection and the ``utils`` helpers) and the
loss-driven accumulator (crates/training/src/gradient_accumulator.rs:68-230, ``GradientStats``).

The ``Trainer`` accumulates straight into the flat gradient arena and reduces across ranks once per
optimizer step, which is ``SyncMode.DEFERRED``. ``SyncMode.IMMEDIATE`` reduces every micro-batch
(gradients leave the rank as soon as they exist; more traffic, less skew at the boundary) and
``SyncMode.ADAPTIVE`` picks between the two from the measured step time, as the reference's
``get_optimal_config`` does. In the reference the field is never read by a communication layer
(its collectives are no-ops); here ``GradientAccumulator`` takes the reduction as a callable, so
the same object works over gloo, NCCL or the symmetric-heap collectives.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, replace

import torch


class SyncMode(str, enum.Enum):
    IMMEDIATE = "immediate"
    DEFERRED = "deferred"
    ADAPTIVE = "adaptive"


class ReductionMode(str, enum.Enum):
    MEAN = "mean"
    SUM = "sum"
    WEIGHTED_MEAN = "weighted_mean"


_DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


@dataclass
class AccumulationConfig:
    steps: int = 1
    normalize: bool = True
    dtype: str = "float32"
    sync_mode: SyncMode = SyncMode.IMMEDIATE
    reduction: ReductionMode = ReductionMode.MEAN
    weight: float = 1.0                     # factor of ``ReductionMode.WEIGHTED_MEAN``

    def __post_init__(self):
        self.sync_mode = SyncMode(self.sync_mode)
        self.reduction = ReductionMode(self.reduction)
        if self.dtype not in _DTYPES:
            raise ValueError(f"accumulation dtype {self.dtype!r}: expected one of {sorted(_DTYPES)}")
        if self.steps < 1:
            raise ValueError("accumulation steps must be >= 1")


@dataclass
class GradientStats:
    """Norm statistics of the accumulated gradients (gradient_accumulator.rs:230)."""
    total_norm: float = 0.0
    max_norm: float = 0.0
    min_norm: float = 0.0
    num_tensors: int = 0
    num_nonfinite: int = 0


class GradientAccumulator:
    """Sums named gradients over ``config.steps`` micro-batches in ``config.dtype``.

    ``reduce_fn(tensor)`` (optional) performs the cross-rank reduction in place. With
    ``SyncMode.IMMEDIATE`` it runs on every incoming gradient, with ``DEFERRED`` once per name in
    ``get_gradients``. ``ADAPTIVE`` behaves as ``DEFERRED`` until ``set_sync_mode`` says otherwise.
    """

    def __init__(self, config: AccumulationConfig | None = None, reduce_fn=None):
        self.config = config or AccumulationConfig()
        self.reduce_fn = reduce_fn
        self._sums: dict[str, torch.Tensor] = {}
        self._counts: dict[str, int] = {}
        self._pending: set[str] = set()
        self.current_step = 0
        self.syncs = 0                       # number of reductions issued (telemetry, tests)
        self._mode = SyncMode.DEFERRED if self.config.sync_mode == SyncMode.ADAPTIVE else self.config.sync_mode

    def set_sync_mode(self, mode):
        self._mode = SyncMode(mode)

    @property
    def sync_mode(self):
        return self._mode

    @torch.no_grad()
    def accumulate(self, name: str, gradient: torch.Tensor, scale: float | None = None):
        g = gradient.detach().to(_DTYPES[self.config.dtype])
        if scale is not None:
            g = g * scale
        elif g.data_ptr() == gradient.data_ptr():
            g = g.clone()
        if self._mode == SyncMode.IMMEDIATE and self.reduce_fn is not None:
            self.reduce_fn(g)
            self.syncs += 1
        elif self.reduce_fn is not None:
            self._pending.add(name)
        if name in self._sums:
            self._sums[name].add_(g)
            self._counts[name] += 1
        else:
            self._sums[name], self._counts[name] = g, 1

    def step(self):
        """Mark the end of one micro-batch."""
        self.current_step += 1

    def should_sync(self) -> bool:
        return self.current_step > 0 and self.current_step % self.config.steps == 0

    should_step = should_sync
    is_ready = should_sync

    @torch.no_grad()
    def get_gradients(self) -> dict[str, torch.Tensor]:
        """Reduced, normalised gradients; the accumulator is reset."""
        out = {}
        cfg = self.config
        for name, s in self._sums.items():
            if name in self._pending and self.reduce_fn is not None:
                self.reduce_fn(s)
                self.syncs += 1
            n = self._counts[name]
            if cfg.reduction == ReductionMode.SUM or not cfg.normalize:
                out[name] = s
            elif cfg.reduction == ReductionMode.WEIGHTED_MEAN:
                out[name] = s * (cfg.weight / n)
            else:
                out[name] = s / n
        self.reset()
        return out

    def reset(self):
        self._sums, self._counts, self._pending = {}, {}, set()
        self.current_step = 0

    def memory_usage(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._sums.values())

    def stats(self) -> GradientStats:
        norms, bad = [], 0
        for t in self._sums.values():
            n = float(t.float().norm())
            if n != n or n == float("inf"):
                bad += 1
            else:
                norms.append(n)
        if not norms:
            return GradientStats(num_tensors=len(self._sums), num_nonfinite=bad)
        return GradientStats(total_norm=sum(n * n for n in norms) ** 0.5, max_norm=max(norms),
                             min_norm=min(norms), num_tensors=len(self._sums), num_nonfinite=bad)

    def apply_to(self, named_params):
        """Write the reduced gradients into ``p.grad`` of ``{name: parameter}``."""
        grads = self.get_gradients()
        for name, p in dict(named_params).items():
            if name in grads:
                p.grad = grads[name].to(p.dtype).view_as(p)
        return grads


class DynamicAccumulator:
    """Doubles the accumulation steps (cap 64) while memory is over the threshold, halves them
    under half of it; proposes a sync mode from the recent step times
    (accumulation.rs:152-221)."""

    MAX_STEPS = 64

    def __init__(self, base_config: AccumulationConfig, memory_threshold: int):
        self.config = replace(base_config)
        self.memory_threshold = memory_threshold
        self.step_times: list[float] = []
        self.memory_usage: list[int] = []

    def adjust_steps(self, current_memory: int, step_time: float) -> int:
        self.memory_usage.append(current_memory)
        self.step_times.append(step_time)
        if current_memory > self.memory_threshold:
            self.config.steps = min(self.config.steps * 2, self.MAX_STEPS)
        elif current_memory < self.memory_threshold // 2:
            self.config.steps = max(self.config.steps // 2, 1)
        return self.config.steps

    def get_optimal_config(self) -> AccumulationConfig:
        if len(self.step_times) < 10:
            return replace(self.config)
        avg_t = sum(self.step_times[-10:]) / 10.0
        avg_m = sum(self.memory_usage[-10:]) // 10
        cfg = replace(self.config)
        cfg.sync_mode = SyncMode.DEFERRED if avg_t > 1.0 else SyncMode.IMMEDIATE
        if avg_t < 0.75 and avg_m < self.memory_threshold // 2:
            cfg.steps = min(cfg.steps + 1, self.MAX_STEPS)
        return cfg


class CheckpointSelection:
    """Which layers recompute their activations (accumulation.rs:224-260). The recomputation itself
    lives in ``train/act_checkpoint.py``; this is the book-keeping the reference keeps beside the
    accumulator."""

    def __init__(self, enabled: bool, segment_size: int = 1):
        self.enabled, self.segment_size = enabled, max(1, segment_size)
        self.layers: list[str] = []

    def checkpoint_layer(self, name: str):
        if self.enabled and name not in self.layers:
            self.layers.append(name)

    def select_every(self, names):
        """Mark every ``segment_size``-th layer of ``names``."""
        for i, n in enumerate(names):
            if i % self.segment_size == 0:
                self.checkpoint_layer(n)
        return self.layers

    def should_checkpoint(self, name: str) -> bool:
        return self.enabled and name in self.layers

    def estimate_memory_savings(self, total_layers: int) -> float:
        if not self.enabled or total_layers <= 0:
            return 0.0
        return len(self.layers) / total_layers * 0.33


def effective_batch_size(batch_size: int, accumulation_steps: int, world_size: int | None = None) -> int:
    local = batch_size * accumulation_steps
    return local * world_size if world_size else local


def estimate_memory_requirement(model_params: int, batch_size: int, accumulation_steps: int,
                                dtype_bytes: int) -> int:
    """Parameters + gradients + one accumulated copy + a 4x-parameters activation estimate per
    sample (accumulation.rs:279-298)."""
    p = model_params * dtype_bytes
    return 3 * p + model_params * 4 * batch_size * accumulation_steps * dtype_bytes


def create_accumulation_schedule(total_steps: int, warmup_steps: int, max_accumulation: int) -> list[int]:
    """Linear ramp from 1 to ``max_accumulation`` over the warm-up, constant afterwards."""
    out = []
    for s in range(total_steps):
        if s < warmup_steps:
            out.append(1 + (s * (max_accumulation - 1)) // warmup_steps)
        else:
            out.append(max_accumulation)
    return out

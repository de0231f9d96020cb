"""Learning-rate schedules, dynamic loss scaling and EMA.

Schedules mirror the reference's set (crates/training/src/scheduler.rs:71-399: constant, linear,
cosine, cosine-with-restarts, polynomial, exponential, step; schedulers.rs:63-399: one-cycle,
reduce-on-plateau, warm restarts, chaining; chroma/train.rs:298-336: warm-up + decay with
``backoff``). Each is a pure function of the step so that resume needs only the step counter.
"""
from __future__ import annotations

import math

import torch

from ..ops import _native as N
from ..ops import functional as F


class LRSchedule:
    def __init__(self, base_lr, kind="constant", warmup_steps=0, total_steps=0, min_lr=0.0,
                 cycles=1, power=1.0, gamma=0.999, step_size=1000, max_lr=None, pct_start=0.3):
        self.base_lr, self.kind = base_lr, kind
        self.warmup, self.total, self.min_lr = warmup_steps, total_steps, min_lr
        self.cycles, self.power, self.gamma, self.step_size = cycles, power, gamma, step_size
        self.max_lr, self.pct_start = max_lr or base_lr, pct_start
        self.scale = 1.0            # multiplied in by back-off events

    def backoff(self, factor=0.5):
        self.scale *= factor

    def __call__(self, step: int) -> float:
        lr = self._lr(step) * self.scale
        return max(lr, 0.0)

    def _lr(self, step):
        b = self.base_lr
        if self.kind != "one_cycle" and self.warmup > 0 and step < self.warmup:
            return b * (step + 1) / self.warmup
        s = step - self.warmup
        n = max(1, self.total - self.warmup)
        p = min(1.0, s / n)
        k = self.kind
        if k == "constant":
            return b
        if k == "linear":
            return self.min_lr + (b - self.min_lr) * (1 - p)
        if k == "cosine":
            return self.min_lr + (b - self.min_lr) * 0.5 * (1 + math.cos(math.pi * p))
        if k in ("cosine_with_restarts", "warm_restarts"):
            q = (p * self.cycles) % 1.0 if p < 1.0 else 1.0
            return self.min_lr + (b - self.min_lr) * 0.5 * (1 + math.cos(math.pi * q))
        if k == "polynomial":
            return self.min_lr + (b - self.min_lr) * (1 - p) ** self.power
        if k == "exponential":
            return b * self.gamma ** s
        if k == "step":
            return b * self.gamma ** (s // self.step_size)
        if k == "one_cycle":
            up = int(self.pct_start * self.total)
            if step < up:
                return b + (self.max_lr - b) * step / max(1, up)
            q = (step - up) / max(1, self.total - up)
            return self.min_lr + (self.max_lr - self.min_lr) * 0.5 * (1 + math.cos(math.pi * min(q, 1.0)))
        raise ValueError(f"unknown schedule {k!r}")

    def apply(self, optimizer, step):
        lr = self(step)
        for g in optimizer.param_groups:
            g["lr"] = lr * g.get("lr_mult", 1.0)
        return lr


class ChainedSchedule:
    """Sequence of (schedule, num_steps) segments."""

    def __init__(self, segments):
        self.segments = segments

    def __call__(self, step):
        for sch, n in self.segments:
            if step < n:
                return sch(step)
            step -= n
        return self.segments[-1][0](self.segments[-1][1] - 1)


class ReduceLROnPlateau:
    def __init__(self, base_lr, factor=0.5, patience=10, min_lr=0.0, threshold=1e-4):
        self.lr, self.factor, self.patience, self.min_lr, self.th = base_lr, factor, patience, min_lr, threshold
        self.best, self.bad = float("inf"), 0

    def observe(self, metric):
        if metric < self.best - self.th:
            self.best, self.bad = metric, 0
        else:
            self.bad += 1
            if self.bad > self.patience:
                self.lr, self.bad = max(self.min_lr, self.lr * self.factor), 0
        return self.lr


class GradScaler:
    """Dynamic loss scale with growth / back-off and inf detection
    (crates/training/src/mixed_precision.rs:58-222). bf16 training runs with scale 1 and only the
    finite check; fp16 parameters use the full mechanism."""

    def __init__(self, init_scale=1.0, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000,
                 enabled=True, max_scale=2.0 ** 24):
        self.scale, self.growth, self.backoff = init_scale, growth_factor, backoff_factor
        self.interval, self.enabled, self.max_scale = growth_interval, enabled, max_scale
        self._good = 0
        self.found_inf = False

    def scale_loss(self, loss):
        return loss * self.scale if self.enabled and self.scale != 1.0 else loss

    def check(self, grad_sumsq) -> bool:
        """True when the gradients are finite (reads one scalar from the device)."""
        v = float(grad_sumsq)
        self.found_inf = not math.isfinite(v)
        return not self.found_inf

    def update(self):
        if not self.enabled:
            return
        if self.found_inf:
            self.scale = max(self.scale * self.backoff, 1.0)
            self._good = 0
        else:
            self._good += 1
            if self._good >= self.interval:
                self.scale = min(self.scale * self.growth, self.max_scale)
                self._good = 0

    def state_dict(self):
        return {"scale": self.scale, "growth": self._good}

    def load_state_dict(self, sd):
        self.scale, self._good = float(sd["scale"]), int(sd.get("growth", 0))


class EMA:
    """fp32 shadow of the trainable parameters with warm-up decay and swap-in/out
    (crates/common/ema/src/ema.rs:7-175; src/trainers/ema.rs:21-363 adds ``current_decay``
    warm-up and the half-life / window helpers). Over a ``ParamArena`` the update is one launch."""

    def __init__(self, params_or_arena, decay=0.999, warmup=True, update_every=1):
        self.arena = params_or_arena if hasattr(params_or_arena, "data") and hasattr(params_or_arena, "offsets") else None
        self.params = self.arena.params if self.arena else [p for p in params_or_arena]
        self.decay, self.warmup, self.update_every = decay, warmup, update_every
        self.num_updates = 0
        if self.arena:
            self.shadow = self.arena.data.detach().float().clone()
        else:
            self.shadow = [p.detach().float().clone() for p in self.params]
        self._backup = None

    @staticmethod
    def decay_from_half_life(steps):
        return 0.5 ** (1.0 / max(1, steps))

    @staticmethod
    def decay_from_window(steps):
        return 1.0 - 2.0 / (steps + 1.0)

    def current_decay(self):
        if not self.warmup:
            return self.decay
        n = self.num_updates
        return min(self.decay, (1.0 + n) / (10.0 + n))

    @torch.no_grad()
    def update(self):
        self.num_updates += 1
        if self.num_updates % self.update_every:
            return
        d = self.current_decay()
        if self.arena:
            data = self.arena.data
            if data.is_cuda and data.dtype == torch.bfloat16 and F.get_backend() == "fused":
                N.check(N.require().eri_ema_update(self.shadow.data_ptr(), data.data_ptr(),
                                                   data.numel(), d, N.stream_ptr()), "ema")
            else:
                self.shadow.mul_(d).add_(data.float(), alpha=1 - d)
        else:
            for s, p in zip(self.shadow, self.params):
                s.mul_(d).add_(p.detach().float(), alpha=1 - d)

    def shadow_of(self, i):
        if self.arena:
            o, p = self.arena.offsets[i], self.params[i]
            return self.shadow[o:o + p.numel()].view(p.shape)
        return self.shadow[i]

    @torch.no_grad()
    def swap_in(self):
        """Replace live parameters with the averaged ones (for validation); ``swap_out`` restores."""
        self._backup = [p.detach().clone() for p in self.params]
        for i, p in enumerate(self.params):
            p.copy_(self.shadow_of(i).to(p.dtype))

    @torch.no_grad()
    def swap_out(self):
        for p, b in zip(self.params, self._backup):
            p.copy_(b)
        self._backup = None

    def applied(self):
        """``with ema.applied(): ...`` runs the body on the averaged weights and restores the live
        ones afterwards, also when the body raises (crates/common/ema/src/ema.rs: ``EMAContext``)."""
        return EMAContext(self)

    def state_dict(self, names=None, dtype=torch.float32):
        names = names or [str(i) for i in range(len(self.params))]
        return {f"ema.{n}": self.shadow_of(i).to(dtype).contiguous() for i, n in enumerate(names)}

    def load_state_dict(self, sd, names=None):
        names = names or [str(i) for i in range(len(self.params))]
        with torch.no_grad():
            for i, n in enumerate(names):
                self.shadow_of(i).copy_(sd[f"ema.{n}"].float())


class EMAContext:
    """Swap-in / swap-out guard around evaluation or sampling with the averaged weights."""

    def __init__(self, ema: EMA):
        self.ema = ema

    def __enter__(self):
        self.ema.swap_in()
        return self.ema

    def __exit__(self, *exc):
        self.ema.swap_out()
        return False

"""Progress tracking, device-memory tracking and metric loggers for long runs.

Reference: ``ProgressTracker{start_phase, update, update_step, update_memory, log_error,
print_summary}``, ``MemoryTracker::get_memory_usage_mb`` and ``ErrorRecovery::retry``
(src/trainers/pipeline_progress_tracker.rs:8-315; the retry lives in ``train/services.py: retry``);
``ConsoleLogger`` with ``ConsoleFormat``, buffered ``CSVLogger``, ``MultiLogger`` and the step
``ProgressTracker`` with ETA (crates/training/src/metrics_extended.rs:10-435).

Everything here is host-side and prints through an injectable ``print_fn`` so it can be tested and
redirected; nothing synchronises the device (the caller passes already-read floats).
"""
from __future__ import annotations

import json
import time
from collections import deque

import torch


def _fmt_time(sec: float) -> str:
    sec = int(max(0, sec))
    h, r = divmod(sec, 3600)
    m, s = divmod(r, 60)
    return f"{h:d}:{m:02d}:{s:02d}" if h else f"{m:d}:{s:02d}"


class MemoryTracker:
    """Device memory in MiB: allocator view (``allocated`` / ``reserved`` / peak) and the driver's
    view (used by all processes). On a machine without CUDA every figure is 0."""

    def __init__(self, device_id: int = 0):
        self.device_id = device_id
        self.peak_mb = 0.0

    def get_memory_usage_mb(self) -> float:
        if not torch.cuda.is_available():
            return 0.0
        mb = torch.cuda.memory_allocated(self.device_id) / 2 ** 20
        self.peak_mb = max(self.peak_mb, mb)
        return mb

    def snapshot(self) -> dict:
        if not torch.cuda.is_available():
            return {"allocated_mb": 0.0, "reserved_mb": 0.0, "peak_mb": 0.0, "device_used_mb": 0.0}
        free, total = torch.cuda.mem_get_info(self.device_id)
        return {"allocated_mb": torch.cuda.memory_allocated(self.device_id) / 2 ** 20,
                "reserved_mb": torch.cuda.memory_reserved(self.device_id) / 2 ** 20,
                "peak_mb": torch.cuda.max_memory_allocated(self.device_id) / 2 ** 20,
                "device_used_mb": (total - free) / 2 ** 20}


class ProgressTracker:
    """Phases (pre-encoding, loading, training ...) with item counts, then per-step loss /
    gradient-norm / learning-rate statistics, a moving-average step time and an ETA."""

    def __init__(self, total_steps: int, print_fn=print, window: int = 50, clock=time.time, bar_width: int = 30):
        self.total_steps, self.print_fn, self.clock, self.bar_width = total_steps, print_fn, clock, bar_width
        self.start = clock()
        self.phase, self.phase_start = None, self.start
        self.phases: list[tuple[str, float]] = []
        self.step = 0
        self.losses, self.grad_norms = deque(maxlen=window), deque(maxlen=window)
        self.step_times = deque(maxlen=window)
        self._last_step_t = None
        self.best_loss = float("inf")
        self.peak_memory_mb = 0.0
        self.errors: list[str] = []

    # -- phases
    def start_phase(self, name: str):
        now = self.clock()
        if self.phase is not None:
            self.phases.append((self.phase, now - self.phase_start))
        self.phase, self.phase_start = name, now
        self.print_fn(f"== {name} ==")

    def bar(self, done: int, total: int) -> str:
        frac = 0.0 if total <= 0 else min(1.0, done / total)
        n = int(round(frac * self.bar_width))
        return "[" + "=" * n + " " * (self.bar_width - n) + f"] {100 * frac:5.1f}%"

    def update(self, items_done: int, total_items: int, message: str = ""):
        el = self.clock() - self.phase_start
        eta = el / items_done * (total_items - items_done) if items_done else 0.0
        self.print_fn(f"{self.bar(items_done, total_items)} {items_done}/{total_items} "
                      f"elapsed {_fmt_time(el)} eta {_fmt_time(eta)} {message}".rstrip())

    # -- steps
    def update_step(self, step: int, loss: float, grad_norm: float | None = None, lr: float | None = None,
                    quiet: bool = False):
        now = self.clock()
        if self._last_step_t is not None and step > self.step:
            self.step_times.append((now - self._last_step_t) / (step - self.step))
        self._last_step_t, self.step = now, step
        if loss == loss:
            self.losses.append(loss)
            self.best_loss = min(self.best_loss, loss)
        if grad_norm is not None and grad_norm == grad_norm:
            self.grad_norms.append(grad_norm)
        if quiet:
            return None
        line = (f"{self.bar(step, self.total_steps)} step {step}/{self.total_steps} loss {loss:.4f} "
                f"(avg {self.avg_loss():.4f})")
        if grad_norm is not None:
            line += f" grad {grad_norm:.3f}"
        if lr is not None:
            line += f" lr {lr:.2e}"
        if self.step_times:
            line += f" {self.sec_per_step():.3f}s/it eta {_fmt_time(self.eta_seconds())}"
        self.print_fn(line)
        return line

    def avg_loss(self) -> float:
        return sum(self.losses) / len(self.losses) if self.losses else float("nan")

    def sec_per_step(self) -> float:
        return sum(self.step_times) / len(self.step_times) if self.step_times else 0.0

    def eta_seconds(self) -> float:
        return self.sec_per_step() * max(0, self.total_steps - self.step)

    def update_memory(self, current_mb: float):
        self.peak_memory_mb = max(self.peak_memory_mb, current_mb)

    def log_error(self, error: str):
        self.errors.append(error)
        self.print_fn(f"error: {error}")

    def summary(self) -> dict:
        now = self.clock()
        phases = list(self.phases)
        if self.phase is not None:
            phases.append((self.phase, now - self.phase_start))
        return {"steps": self.step, "total_steps": self.total_steps, "elapsed_s": now - self.start,
                "avg_loss": self.avg_loss(), "best_loss": self.best_loss,
                "avg_grad_norm": sum(self.grad_norms) / len(self.grad_norms) if self.grad_norms else None,
                "sec_per_step": self.sec_per_step(), "peak_memory_mb": self.peak_memory_mb,
                "errors": len(self.errors), "phases": phases}

    def print_summary(self):
        s = self.summary()
        self.print_fn(f"finished {s['steps']}/{s['total_steps']} steps in {_fmt_time(s['elapsed_s'])}; "
                      f"avg loss {s['avg_loss']:.4f}, best {s['best_loss']:.4f}, "
                      f"{s['sec_per_step']:.3f}s/it, peak memory {s['peak_memory_mb']:.0f} MiB, "
                      f"{s['errors']} error(s)")
        for name, sec in s["phases"]:
            self.print_fn(f"  phase {name}: {_fmt_time(sec)}")

    finish = print_summary


# ---------------------------------------------------------------------------- loggers
class MetricLogger:
    def log(self, step: int, metrics: dict): ...
    def flush(self): ...
    def close(self):
        self.flush()


class ConsoleLogger(MetricLogger):
    """``format``: ``simple`` (``step 10 | loss=0.1 lr=1e-4``), ``detailed`` (one metric per
    line) or ``json``; prints every ``interval`` steps."""

    def __init__(self, interval: int = 1, format: str = "simple", print_fn=print):
        if format not in ("simple", "detailed", "json"):
            raise ValueError(f"console format {format!r}")
        self.interval, self.format, self.print_fn = max(1, interval), format, print_fn

    def log(self, step, metrics):
        if step % self.interval:
            return
        if self.format == "json":
            self.print_fn(json.dumps({"step": step, **metrics}, sort_keys=True))
        elif self.format == "detailed":
            self.print_fn(f"step {step}")
            for k in sorted(metrics):
                self.print_fn(f"  {k:<20s} {_num(metrics[k])}")
        else:
            self.print_fn(f"step {step} | " + " ".join(f"{k}={_num(metrics[k])}" for k in sorted(metrics)))


def _num(v):
    if isinstance(v, float):
        return f"{v:.6g}"
    return str(v)


class BufferedCSVLogger(MetricLogger):
    """Rows are kept in memory and written every ``buffer_size`` rows (and on ``flush``). The column
    set is fixed by the first row; later unknown keys are ignored, missing ones left empty."""

    def __init__(self, path: str, buffer_size: int = 100):
        self.path, self.buffer_size = path, max(1, buffer_size)
        self.fields = None
        self.rows: list[list[str]] = []

    def log(self, step, metrics):
        if self.fields is None:
            self.fields = sorted(metrics)
            with open(self.path, "w") as f:
                f.write(",".join(["step", *self.fields]) + "\n")
        self.rows.append([str(step), *[_num(metrics[k]) if k in metrics else "" for k in self.fields]])
        if len(self.rows) >= self.buffer_size:
            self.flush()

    def flush(self):
        if self.rows:
            with open(self.path, "a") as f:
                f.writelines(",".join(r) + "\n" for r in self.rows)
            self.rows = []


class MultiLogger(MetricLogger):
    def __init__(self, loggers):
        self.loggers = list(loggers)

    def log(self, step, metrics):
        for lg in self.loggers:
            lg.log(step, metrics)

    def flush(self):
        for lg in self.loggers:
            lg.flush()

    def close(self):
        for lg in self.loggers:
            lg.close()


class LoggerCallback:
    """Adapter from ``run_training``'s callback protocol to a ``MetricLogger`` / ``ProgressTracker``."""
    stop_training = False

    def __init__(self, logger: MetricLogger | None = None, tracker: ProgressTracker | None = None):
        self.logger, self.tracker = logger, tracker

    def on_train_begin(self, trainer):
        if self.tracker:
            self.tracker.start_phase("training")

    def on_step_end(self, trainer, step, logs):
        numeric = {k: v for k, v in logs.items() if isinstance(v, (int, float)) and k != "step"}
        if self.logger:
            self.logger.log(step, numeric)
        if self.tracker:
            self.tracker.update_step(step, logs.get("loss", float("nan")), logs.get("grad_norm"), logs.get("lr"),
                                     quiet=True)
            self.tracker.update_memory(logs.get("alloc_mb", 0.0))

    def on_checkpoint(self, trainer, path):
        pass

    def on_train_end(self, trainer):
        if self.logger:
            self.logger.close()
        if self.tracker:
            self.tracker.print_summary()

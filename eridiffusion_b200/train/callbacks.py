"""Event-based callbacks and their manager.

Reference: ``CallbackEvent`` / ``CallbackContext`` / ``Callback::on_event``, ``ModelCheckpoint``
(monitor, mode, save_best_only, save_weights_only, period), ``LRSchedulerCallback``,
``GradientClipping``, ``LambdaCallback`` and ``CallbackManager`` (crates/training/src/callbacks.rs:
5-579). The step-oriented callbacks used by ``run_training`` (early stopping, CSV / JSONL /
TensorBoard loggers, sampling) live in ``train/services.py``; ``CallbackManager`` implements that
protocol too, so one manager can be handed to ``run_training`` and fan events out to event-based
callbacks.
"""
from __future__ import annotations

import enum
import math
import os
from dataclasses import dataclass, field


class CallbackEvent(str, enum.Enum):
    TRAINING_START = "training_start"
    TRAINING_END = "training_end"
    EPOCH_START = "epoch_start"
    EPOCH_END = "epoch_end"
    BATCH_START = "batch_start"
    BATCH_END = "batch_end"
    VALIDATION_START = "validation_start"
    VALIDATION_END = "validation_end"
    CHECKPOINT_SAVED = "checkpoint_saved"
    METRIC_LOGGED = "metric_logged"


@dataclass
class CallbackContext:
    global_step: int = 0
    epoch: int = 0
    batch: int = 0
    loss: float | None = None
    metrics: dict = field(default_factory=dict)
    trainer: object = None
    payload: object = None                  # event argument (checkpoint path, (metric, value) ...)


class EventCallback:
    name = "callback"
    enabled = True
    stop_training = False

    def on_event(self, event: CallbackEvent, ctx: CallbackContext):
        raise NotImplementedError


class ModelCheckpoint(EventCallback):
    """Saves through ``trainer.save_checkpoint`` every ``period`` batch-end events, or only when the
    monitored metric improves (``save_best_only``). ``save_fn(trainer, directory)`` overrides the
    writer (e.g. adapter-only export)."""
    name = "model_checkpoint"

    def __init__(self, save_dir: str, monitor: str | None = None, mode: str = "min", save_best_only: bool = False,
                 save_weights_only: bool = False, period: int = 1, save_fn=None):
        if mode not in ("min", "max"):
            raise ValueError("mode must be min or max")
        self.save_dir, self.monitor_name, self.mode = save_dir, monitor, mode
        self.save_best_only, self.save_weights_only, self.period = save_best_only, save_weights_only, max(1, period)
        self.best_value, self.best_path, self.saved = None, None, []
        self.save_fn = save_fn

    def monitor(self, metric: str, mode: str = "min"):
        self.monitor_name, self.mode = metric, mode
        return self

    def _improved(self, v):
        return self.best_value is None or (v < self.best_value if self.mode == "min" else v > self.best_value)

    def on_event(self, event, ctx):
        if event != CallbackEvent.BATCH_END or ctx.global_step % self.period:
            return
        value = None
        if self.monitor_name is not None:
            value = ctx.loss if self.monitor_name == "loss" else ctx.metrics.get(self.monitor_name)
            if value is None or not math.isfinite(value):
                return
        if self.save_best_only:
            if value is None:
                raise ValueError("save_best_only needs a monitored metric")
            if not self._improved(value):
                return
        if value is not None and self._improved(value):
            self.best_value = value
        os.makedirs(self.save_dir, exist_ok=True)
        path = (self.save_fn or (lambda tr, d: tr.save_checkpoint(d)))(ctx.trainer, self.save_dir)
        self.saved.append(path)
        if value is not None and value == self.best_value:
            self.best_path = path
        return path


class LRSchedulerCallback(EventCallback):
    """Applies ``schedule(step)`` to the optimizer's groups at batch start; ``plateau``
    (``ReduceLROnPlateau``) is fed the monitored metric at validation end instead."""
    name = "lr_scheduler"

    def __init__(self, optimizer, schedule=None, plateau=None, monitor: str = "val_loss"):
        self.optimizer, self.schedule, self.plateau, self.monitor = optimizer, schedule, plateau, monitor
        self.last_lr = None

    def _set(self, lr):
        self.last_lr = lr
        for g in self.optimizer.param_groups:
            g["lr"] = lr * g.get("lr_mult", 1.0)

    def on_event(self, event, ctx):
        if event == CallbackEvent.BATCH_START and self.schedule is not None:
            self._set(self.schedule(ctx.global_step))
        elif event == CallbackEvent.VALIDATION_END and self.plateau is not None and self.monitor in ctx.metrics:
            self._set(self.plateau.observe(ctx.metrics[self.monitor]))


class GradientClipping(EventCallback):
    """Clips the global norm of ``params`` when asked (call ``clip()`` between backward and the
    optimizer step, or let the manager do it on ``BATCH_END`` for loops that step afterwards)."""
    name = "gradient_clipping"

    def __init__(self, params, max_norm: float = 1.0, norm_type: float = 2.0):
        self.params, self.max_norm, self.norm_type = list(params), max_norm, norm_type
        self.last_norm = None
        self.num_clipped = 0

    def clip(self):
        import torch
        n = float(torch.nn.utils.clip_grad_norm_(self.params, self.max_norm, self.norm_type))
        self.last_norm = n
        self.num_clipped += n > self.max_norm
        return n

    def on_event(self, event, ctx):
        if event == CallbackEvent.BATCH_END:
            return self.clip()


class LambdaCallback(EventCallback):
    def __init__(self, fn, name: str = "lambda", events=None):
        self.fn, self.name = fn, name
        self.events = None if events is None else {CallbackEvent(e) for e in events}

    def on_event(self, event, ctx):
        if self.events is None or event in self.events:
            return self.fn(event, ctx)


class CallbackManager:
    """Ordered fan-out of events. Also speaks ``run_training``'s callback protocol."""

    def __init__(self, callbacks=()):
        self.callbacks = list(callbacks)
        self.context = CallbackContext()
        self.errors: list[tuple[str, str]] = []

    def add(self, cb):
        self.callbacks.append(cb)
        return self

    def get(self, name):
        return next((c for c in self.callbacks if c.name == name), None)

    def remove(self, name) -> bool:
        n = len(self.callbacks)
        self.callbacks = [c for c in self.callbacks if c.name != name]
        return len(self.callbacks) < n

    def trigger(self, event, payload=None, strict=True):
        """Calls every enabled callback; with ``strict=False`` a failing callback is recorded in
        ``errors`` and the others still run."""
        event = CallbackEvent(event)
        self.context.payload = payload
        out = []
        for cb in self.callbacks:
            if not cb.enabled:
                continue
            try:
                out.append(cb.on_event(event, self.context))
            except Exception as e:
                if strict:
                    raise
                self.errors.append((cb.name, repr(e)))
        return out

    @property
    def stop_training(self):
        return any(getattr(c, "stop_training", False) for c in self.callbacks)

    # -- run_training protocol
    def on_train_begin(self, trainer):
        self.context.trainer = trainer
        self.trigger(CallbackEvent.TRAINING_START)

    def on_step_end(self, trainer, step, logs):
        c = self.context
        c.trainer, c.global_step, c.batch, c.loss = trainer, step, step, logs.get("loss")
        c.metrics = {k: v for k, v in logs.items() if isinstance(v, (int, float))}
        self.trigger(CallbackEvent.BATCH_END)
        for k, v in c.metrics.items():
            if k.startswith("val_"):
                self.trigger(CallbackEvent.METRIC_LOGGED, (k, v))

    def on_checkpoint(self, trainer, path):
        self.trigger(CallbackEvent.CHECKPOINT_SAVED, path)

    def on_train_end(self, trainer):
        self.trigger(CallbackEvent.TRAINING_END)

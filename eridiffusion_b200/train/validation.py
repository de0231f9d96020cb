"""Held-out validation: fixed-timestep losses, history, best step, early stopping, reports.

Counterpart of the reference's validation stack (src/trainers/validation.rs:11-275:
``ValidationConfig``, ``ValidationDataset``, ``ValidationMetrics{add_batch_loss, add_timestep_loss,
avg_loss, summary}``, ``ValidationRunner{validate, metrics_history, best_checkpoint_step,
save_metrics}``; src/trainers/validation_advanced.rs:16-630: early stopping with monitor /
min_delta / patience / mode, custom metrics, CSV export; src/trainers/validation_formatter.rs:
9-358: textual report, per-timestep table, progress bar).

The loss is evaluated at FIXED timesteps with FIXED noise (seeded per sample and timestep), so that
two validation runs differ only by the weights. That is what makes the curve usable for choosing a
checkpoint; random timesteps, as in the training loss, would add more variance than a few hundred
steps of training remove. Evaluation runs under ``torch.no_grad`` with the trainer's own forward
function, objective and loss, optionally on the EMA weights.
"""
from __future__ import annotations

import csv
import json
import sys
import time
from dataclasses import asdict, dataclass, field

import torch

from ..objectives import loss_fn
from ..ops import functional as F


@dataclass
class EarlyStoppingConfig:
    monitor: str = "val_loss"
    min_delta: float = 0.0
    patience: int = 5
    mode: str = "min"                       # min | max


@dataclass
class ValidationConfig:
    batch_size: int = 1
    every_n_steps: int = 500
    num_samples: int | None = None
    eval_timesteps: tuple = (0.1, 0.3, 0.5, 0.7, 0.9)      # fractions of the schedule
    use_ema: bool = False
    seed: int = 1234
    early_stopping: EarlyStoppingConfig | None = None


@dataclass
class ValidationMetrics:
    step: int = 0
    timestamp: float = 0.0
    loss: float = 0.0
    loss_per_timestep: list = field(default_factory=list)   # [(timestep, loss)]
    num_samples: int = 0
    custom_metrics: dict = field(default_factory=dict)
    elapsed_s: float = 0.0
    _sum: float = 0.0
    _by_t: dict = field(default_factory=dict)

    def add_batch_loss(self, loss: float, batch_size: int):
        self._sum += loss * batch_size
        self.num_samples += batch_size
        self.loss = self._sum / max(1, self.num_samples)

    def add_timestep_loss(self, timestep, loss: float, n: int = 1):
        s, c = self._by_t.get(timestep, (0.0, 0))
        self._by_t[timestep] = (s + loss * n, c + n)
        self.loss_per_timestep = sorted((t, s / c) for t, (s, c) in self._by_t.items())

    def avg_loss(self) -> float:
        return self.loss

    def value(self, name: str) -> float:
        return self.loss if name in ("val_loss", "loss") else self.custom_metrics[name]

    def summary(self) -> str:
        return format_validation_summary(self)

    def to_dict(self):
        d = asdict(self)
        d.pop("_sum"), d.pop("_by_t")
        return d


class ValidationDataset:
    """A fixed list of batches (dicts with ``latents`` and the conditioning the forward function
    reads). ``from_loader`` takes the first ``num_samples`` samples of any batch iterator."""

    def __init__(self, batches):
        self.batches = list(batches)

    @classmethod
    def from_loader(cls, loader, num_samples=None):
        out, n = [], 0
        for b in loader:
            out.append(b)
            n += b["latents"].shape[0]
            if num_samples is not None and n >= num_samples:
                break
        return cls(out)

    def __len__(self):
        return sum(b["latents"].shape[0] for b in self.batches)

    def is_empty(self):
        return not self.batches


class EarlyStopper:
    def __init__(self, cfg: EarlyStoppingConfig):
        self.cfg, self.best, self.bad = cfg, None, 0

    def observe(self, value: float) -> bool:
        """Returns True when training should stop."""
        c = self.cfg
        better = self.best is None or (value < self.best - c.min_delta if c.mode == "min"
                                       else value > self.best + c.min_delta)
        if better:
            self.best, self.bad = value, 0
        else:
            self.bad += 1
        return self.bad >= c.patience


class ValidationRunner:
    def __init__(self, dataset: ValidationDataset, config: ValidationConfig | None = None, output_dir=None,
                 formatter=None):
        self.dataset, self.config = dataset, config or ValidationConfig()
        self.output_dir = output_dir
        self.history: list[ValidationMetrics] = []
        self.stopper = EarlyStopper(self.config.early_stopping) if self.config.early_stopping else None
        self.should_stop = False
        self.formatter = formatter
        self.custom: dict = {}                 # name -> fn(pred, target, batch) -> float

    def should_validate(self, step: int) -> bool:
        n = self.config.every_n_steps
        return n > 0 and step > 0 and step % n == 0 and not self.dataset.is_empty()

    def add_metric(self, name, fn):
        self.custom[name] = fn

    @torch.no_grad()
    def validate(self, trainer, step: int | None = None) -> ValidationMetrics:
        cfg = self.config
        step = trainer.step if step is None else step
        m = ValidationMetrics(step=step, timestamp=time.time())
        t0 = time.time()
        ema = trainer.ema if cfg.use_ema and getattr(trainer, "ema", None) is not None else None
        was_training = trainer.model.training
        trainer.model.eval()
        if ema is not None:
            ema.swap_in()
        custom_sum = {k: 0.0 for k in self.custom}
        try:
            if self.formatter:
                self.formatter.print_header(step)
            seen = 0
            for bi, batch in enumerate(self.dataset.batches):
                x0 = batch["latents"]
                B = x0.shape[0]
                for ti, frac in enumerate(cfg.eval_timesteps):
                    t = self._timestep(trainer, frac, B, x0.device)
                    coef = trainer.objective.coefficients(t)
                    xt, target = F.noise_mix(x0, coef, seed=cfg.seed, offset=(bi * 64 + ti) << 24,
                                             eps=batch.get("noise"), patch=trainer.cfg.patch)
                    pred = trainer.forward_fn(trainer.model, xt, trainer.objective.model_time(t), batch,
                                              trainer.cfg)
                    loss = float(loss_fn(trainer.cfg.loss, pred, target, trainer.objective.loss_weight(t)))
                    m.add_timestep_loss(frac, loss, B)
                    m.add_batch_loss(loss, B)
                    for k, fn in self.custom.items():
                        custom_sum[k] += float(fn(pred, target, batch)) * B
                seen += B
                if self.formatter:
                    self.formatter.print_batch_progress(bi + 1, len(self.dataset.batches))
                if cfg.num_samples is not None and seen >= cfg.num_samples:
                    break
        finally:
            if ema is not None:
                ema.swap_out()
            trainer.model.train(was_training)
        # every sample is counted once per timestep in the running mean
        n_eval = max(1, m.num_samples)
        m.custom_metrics = {k: v / n_eval for k, v in custom_sum.items()}
        m.num_samples = m.num_samples // max(1, len(cfg.eval_timesteps))
        m.elapsed_s = time.time() - t0
        self.history.append(m)
        if self.stopper is not None:
            self.should_stop = self.stopper.observe(m.value(self.config.early_stopping.monitor))
        if self.formatter:
            self.formatter.print_results(m, self.best_metrics())
        if self.output_dir:
            self.save_metrics(self.output_dir)
        return m

    @staticmethod
    def _timestep(trainer, frac, B, device):
        obj = trainer.objective
        n = getattr(obj, "num_steps", None)
        if n:                                    # discrete schedule: an index
            return torch.full((B,), int(round(frac * (n - 1))), device=device, dtype=torch.long)
        return torch.full((B,), float(frac), device=device)

    def metrics_history(self):
        return self.history

    def best_metrics(self):
        if not self.history:
            return None
        es = self.config.early_stopping
        name, mode = (es.monitor, es.mode) if es else ("val_loss", "min")
        pick = min if mode == "min" else max
        return pick(self.history, key=lambda h: h.value(name))

    def best_step(self):
        b = self.best_metrics()
        return None if b is None else b.step

    best_checkpoint_step = best_step

    def save_metrics(self, output_dir):
        import os
        os.makedirs(output_dir, exist_ok=True)
        path = os.path.join(output_dir, "validation_metrics.json")
        with open(path, "w") as f:
            json.dump({"best_step": self.best_step(), "history": [h.to_dict() for h in self.history]}, f, indent=1)
        return path

    def export_metrics_csv(self, path):
        ts = sorted({t for h in self.history for t, _ in h.loss_per_timestep})
        names = sorted({k for h in self.history for k in h.custom_metrics})
        with open(path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["step", "timestamp", "loss", "num_samples", *[f"loss_t{t}" for t in ts], *names])
            for h in self.history:
                by_t = dict(h.loss_per_timestep)
                w.writerow([h.step, f"{h.timestamp:.3f}", f"{h.loss:.6f}", h.num_samples,
                            *[f"{by_t[t]:.6f}" if t in by_t else "" for t in ts],
                            *[f"{h.custom_metrics.get(k, float('nan')):.6f}" for k in names]])
        return path


# ---------------------------------------------------------------------------- text reports
def format_timestep_losses(loss_per_timestep) -> str:
    if not loss_per_timestep:
        return "  (no per-timestep losses)"
    hi = max(v for _, v in loss_per_timestep) or 1.0
    rows = []
    for t, v in loss_per_timestep:
        bar = "#" * max(1, int(round(24 * v / hi)))
        rows.append(f"  t={t:<8g} {v:10.6f}  {bar}")
    return "\n".join(rows)


def format_validation_summary(m: ValidationMetrics) -> str:
    head = f"validation @ step {m.step}: loss {m.loss:.6f} over {m.num_samples} samples ({m.elapsed_s:.1f}s)"
    extra = "".join(f"\n  {k}: {v:.6f}" for k, v in sorted(m.custom_metrics.items()))
    return f"{head}\n{format_timestep_losses(m.loss_per_timestep)}{extra}"


class ValidationFormatter:
    """Console output of a validation pass (validation_formatter.rs:9-233)."""

    def __init__(self, color_output=False, show_progress=True, stream=None):
        self.color, self.show_progress, self.stream = color_output, show_progress, stream or sys.stdout

    def _c(self, code, s):
        return f"\033[{code}m{s}\033[0m" if self.color else s

    def _p(self, s):
        print(s, file=self.stream)

    def print_header(self, step):
        self._p(self._c("1;36", f"=== validation at step {step} ==="))

    def print_batch_progress(self, current, total):
        if self.show_progress:
            self._p(f"  batch {current}/{total}")

    def print_results(self, m: ValidationMetrics, best: ValidationMetrics | None = None):
        self._p(format_validation_summary(m))
        if best is not None:
            tag = "new best" if best is m else f"best so far {best.loss:.6f} at step {best.step}"
            self._p(self._c("32" if best is m else "33", f"  {tag}"))

    def print_early_stopping_warning(self, checks_without_improvement, patience):
        self._p(self._c("33", f"  no improvement for {checks_without_improvement}/{patience} validations"))

    def print_complete(self, elapsed_secs):
        self._p(f"validation complete in {elapsed_secs:.1f}s")

    def print_error(self, error):
        self._p(self._c("31", f"validation error: {error}"))


class ValidationCallback:
    """``run_training`` callback: validates every ``every_n_steps`` optimizer steps and sets
    ``stop_training`` when the early-stopping rule fires."""
    stop_training = False

    def __init__(self, runner: ValidationRunner):
        self.runner = runner

    def on_train_begin(self, trainer):
        pass

    def on_step_end(self, trainer, step, logs):
        if self.runner.should_validate(step):
            m = self.runner.validate(trainer, step)
            logs["val_loss"] = m.loss
        self.stop_training = self.runner.should_stop

    def on_checkpoint(self, trainer, path):
        pass

    def on_train_end(self, trainer):
        pass

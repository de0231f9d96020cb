"""Training services around the step: callbacks, metrics, telemetry CSV, NaN-safety policy,
step watchdog, retry helper, graceful interrupt, run driver.

Reference parts: ``Callback`` + ``EarlyStopping`` / ``CSVLogger`` / ``TensorBoardCallback``
(crates/training/src/callbacks.rs:31-158), ``MetricsTracker`` with moving averages
(crates/training/src/metrics.rs:12-196), ``MetricsLogger`` JSONL (metrics_logger.rs),
``TelemetryCsv`` columns and ``EXPECT_STEP_SEC`` (telemetry.rs:15-62), ``NanSafetyCfg`` skip /
scale back-off / LR back-off (crates/training/src/chroma/train.rs:268-290, 1262-1378), SIGINT ->
graceful checkpoint (:669-681), ``ErrorRecovery::retry`` with exponential back-off
(src/trainers/pipeline_progress_tracker.rs:280-315), ``TrainingVerifier`` / ``TrainingHealth``
(src/training_verifier.rs:40-307), per-step console line (crates/training/src/run.rs:278).
"""
from __future__ import annotations

import json
import math
import os
import signal
import threading
import time
from pathlib import Path
from collections import deque
from dataclasses import dataclass, field

import torch


# ------------------------------------------------------------------------- callbacks
class Callback:
    def on_train_begin(self, trainer): ...
    def on_step_end(self, trainer, step, logs): ...
    def on_checkpoint(self, trainer, path): ...
    def on_train_end(self, trainer): ...
    stop_training = False


class EarlyStopping(Callback):
    def __init__(self, monitor="loss", patience=100, min_delta=0.0, mode="min"):
        self.monitor, self.patience, self.min_delta, self.mode = monitor, patience, min_delta, mode
        self.best, self.bad = None, 0

    def on_step_end(self, trainer, step, logs):
        v = logs.get(self.monitor)
        if v is None or not math.isfinite(v):
            return
        better = self.best is None or (v < self.best - self.min_delta if self.mode == "min"
                                       else v > self.best + self.min_delta)
        if better:
            self.best, self.bad = v, 0
        else:
            self.bad += 1
            if self.bad >= self.patience:
                self.stop_training = True


class CSVLogger(Callback):
    def __init__(self, path, fields=("step", "loss", "grad_norm", "lr", "sec_per_it", "samples_per_s")):
        self.path, self.fields = path, fields
        self._wrote_header = os.path.exists(path)

    def on_step_end(self, trainer, step, logs):
        with open(self.path, "a") as f:
            if not self._wrote_header:
                f.write(",".join(self.fields) + "\n")
                self._wrote_header = True
            f.write(",".join(str(logs.get(k, "")) for k in self.fields) + "\n")


class JSONLLogger(Callback):
    def __init__(self, path):
        self.path = path

    def on_step_end(self, trainer, step, logs):
        with open(self.path, "a") as f:
            f.write(json.dumps({"step": step, **{k: v for k, v in logs.items() if isinstance(v, (int, float, str))}}) + "\n")


class TensorBoardCallback(Callback):
    """Writes scalars through ``torch.utils.tensorboard`` when it is importable; otherwise keeps
    the scalars in ``.history`` (the reference's writer is a stub too)."""

    def __init__(self, logdir):
        self.history = []
        try:
            from torch.utils.tensorboard import SummaryWriter
            self.writer = SummaryWriter(logdir)
        except Exception:
            self.writer = None

    def on_step_end(self, trainer, step, logs):
        for k, v in logs.items():
            if isinstance(v, (int, float)):
                if self.writer:
                    self.writer.add_scalar(k, v, step)
                else:
                    self.history.append((step, k, v))


class SampleCallback(Callback):
    """Validation sampling during training: every ``sample_every`` optimizer steps the model is
    put in eval mode, the unified inference pipeline draws one sample per prompt embedding with the
    configured sampler settings, and the latents (PNG files when a VAE is attached) are written to
    ``out_dir/samples`` (``sample.sample_every`` of the YAML; crates/training/src/trainer.rs:379-382).
    ``embeddings``: list of (txt [1, T, D], pooled [1, P] or None), e.g. from the embedding cache;
    with none given, seeded random embeddings of the right shape stand in so that the hook still
    exercises the sampler."""

    def __init__(self, sample_cfg, family: str, out_dir, embeddings=None, vae=None, rank: int = 0, frames: int = 1):
        self.cfg, self.family, self.out = sample_cfg, family, Path(out_dir) / "samples"
        self.embeddings, self.vae, self.rank, self.frames = embeddings, vae, rank, frames
        self.written = []

    def _model_type(self):
        from ..sampling.pipelines import ModelType
        for mt in ModelType:
            if mt.family == self.family:
                return mt
        return ModelType.FLUX_DEV               # MMDiT-style call signature

    def _embeds(self, model, n):
        if self.embeddings:
            return self.embeddings
        c = model.cfg
        dim = getattr(c, "context_dim", getattr(c, "caption_dim", 4096))
        vec = getattr(c, "vec_dim", getattr(c, "pooled_dim", 0))
        p = next(model.parameters())
        out = []
        for i in range(max(1, n)):
            g = torch.Generator().manual_seed(1000 + i)
            out.append((torch.randn(1, 64, dim, generator=g).to(p.device, p.dtype),
                        torch.randn(1, vec, generator=g).to(p.device, p.dtype) if vec else None))
        return out

    def on_step_end(self, trainer, step, logs):
        every = self.cfg.sample_every
        if not every or step % every or self.rank != 0:
            return
        from ..io import safetensors as st
        from ..sampling import save_png
        from ..sampling.pipelines import UnifiedInferencePipeline
        model = trainer.model
        was_training = model.training
        model.eval()
        try:
            pipe = UnifiedInferencePipeline(model, self._model_type(), vae=self.vae)
            self.out.mkdir(parents=True, exist_ok=True)
            for i, (txt, pooled) in enumerate(self._embeds(model, len(self.cfg.prompts))):
                seed = self.cfg.seed + (i if self.cfg.walk_seed else 0)
                lat = pipe.generate(txt=txt, pooled=pooled, width=self.cfg.width, height=self.cfg.height,
                                    steps=self.cfg.sample_steps, guidance_scale=self.cfg.guidance_scale, seed=seed,
                                    frames=self.frames)
                stem = self.out / f"step{step:07d}_{i}"
                if self.vae is not None and lat.dim() == 4:
                    save_png(pipe.decode(lat)[0], str(stem) + ".png")
                    self.written.append(str(stem) + ".png")
                else:
                    st.save_file({"latent": lat.float().cpu()}, str(stem) + ".safetensors",
                                 metadata={"step": str(step), "seed": str(seed)})
                    self.written.append(str(stem) + ".safetensors")
        finally:
            model.train(was_training)


# ------------------------------------------------------------------------- metrics
class MetricsTracker:
    def __init__(self, window=100):
        self.window = window
        self.series: dict[str, deque] = {}
        self.totals: dict[str, float] = {}
        self.counts: dict[str, int] = {}

    def update(self, **kv):
        for k, v in kv.items():
            if v is None:
                continue
            self.series.setdefault(k, deque(maxlen=self.window)).append(float(v))
            self.totals[k] = self.totals.get(k, 0.0) + float(v)
            self.counts[k] = self.counts.get(k, 0) + 1

    def moving_average(self, k):
        s = self.series.get(k)
        return sum(s) / len(s) if s else float("nan")

    def mean(self, k):
        return self.totals.get(k, 0.0) / max(1, self.counts.get(k, 0))

    def summary(self):
        return {k: {"ma": self.moving_average(k), "mean": self.mean(k), "n": self.counts[k]} for k in self.series}


TELEMETRY_COLUMNS = ("step", "fw_sec", "bw_sec", "h2d_mb_s", "d2h_mb_s", "gpu_mem_peak", "tokens_per_s",
                     "grad_norm", "loss", "fused", "samples_per_s_box", "step_ms_device_max")


class TelemetryCsv:
    def __init__(self, path):
        self.path = path
        if not os.path.exists(path):
            with open(path, "w") as f:
                f.write(",".join(TELEMETRY_COLUMNS) + "\n")

    def row(self, **kv):
        with open(self.path, "a") as f:
            f.write(",".join(str(kv.get(c, "")) for c in TELEMETRY_COLUMNS) + "\n")


class StepTimeoutError(RuntimeError):
    pass


class StepWatchdog:
    """Host-side watchdog around each step: ``EXPECT_STEP_SEC`` (or ``limit_s``) bounds the wall
    time; a step that exceeds it raises ``StepTimeoutError`` at its end, and a background thread
    calls ``on_stall`` if a step never ends (so a rank waiting on a dead peer is noticed on the
    host, not by hanging a GPU)."""

    def __init__(self, limit_s=None, on_stall=None, hard_factor=10.0):
        env = os.environ.get("EXPECT_STEP_SEC")
        self.limit = limit_s if limit_s is not None else (float(env) if env else None)
        self.on_stall, self.hard = on_stall, hard_factor
        self._t0 = None
        self._stop = threading.Event()
        self.stalled = False
        if self.limit and on_stall:
            threading.Thread(target=self._watch, daemon=True).start()

    def _watch(self):
        while not self._stop.wait(min(1.0, self.limit)):
            t0 = self._t0
            if t0 is not None and time.time() - t0 > self.limit * self.hard:
                self.stalled = True
                self.on_stall()
                self._t0 = None

    def begin(self):
        self._t0 = time.time()

    def end(self):
        dt = time.time() - self._t0 if self._t0 else 0.0
        self._t0 = None
        if self.limit and dt > self.limit:
            raise StepTimeoutError(f"step took {dt:.2f}s, expected <= {self.limit}s")
        return dt

    def close(self):
        self._stop.set()


# ------------------------------------------------------------------------- NaN safety
@dataclass
class NanSafetyConfig:
    max_skips: int = 50
    lr_backoff: float = 0.5
    scale_backoff: float = 0.5
    reset_optimizer_after: int = 0          # consecutive skips before the optimizer state is reset
    group_grad_norm_budget: float | None = None
    zero_bad_grads: bool = True


class NanGuard:
    """Decides what to do with a non-finite loss / gradient norm: skip the step (the optimizer
    kernels already leave parameters and state untouched when the squared norm is not finite),
    back the learning rate off, count, and give up after ``max_skips``."""

    def __init__(self, cfg: NanSafetyConfig | None = None):
        self.cfg = cfg or NanSafetyConfig()
        self.skips = 0
        self.consecutive = 0

    def check(self, trainer, loss_value: float, grad_norm: float | None = None) -> bool:
        ok = math.isfinite(loss_value) and (grad_norm is None or math.isfinite(grad_norm))
        if ok:
            self.consecutive = 0
            return True
        self.skips += 1
        self.consecutive += 1
        trainer.nan_skips = self.skips
        trainer.schedule.backoff(self.cfg.lr_backoff)
        trainer.scaler.found_inf = True
        trainer.scaler.update()
        if self.cfg.zero_bad_grads:
            trainer.arena.zero_grad()
        if self.cfg.reset_optimizer_after and self.consecutive >= self.cfg.reset_optimizer_after:
            opt = trainer.optimizer
            for name in ("m_q", "v_q", "m_absmax", "v_absmax", "m", "v"):
                t = getattr(opt, name, None)
                if torch.is_tensor(t):
                    t.zero_()
        if self.skips > self.cfg.max_skips:
            raise FloatingPointError(f"{self.skips} non-finite steps: giving up")
        return False


def retry(fn, attempts=3, base_delay=0.5, exceptions=(Exception,), sleep=time.sleep):
    """Exponential back-off retry (3 attempts by default, like ``ErrorRecovery::retry``)."""
    for i in range(attempts):
        try:
            return fn()
        except exceptions:
            if i == attempts - 1:
                raise
            sleep(base_delay * (2 ** i))


class ResilientBatches:
    """Iterator wrapper for the data path: a batch whose production raises (an unreadable file, a
    decode error) is skipped and counted instead of ending the run; ``max_consecutive`` failures in
    a row re-raise the last error, since then the source itself is broken. ``StopIteration`` passes
    through."""

    def __init__(self, batches, max_consecutive: int = 8, on_error=None, exceptions=(Exception,)):
        self._it = iter(batches)
        self.max_consecutive, self.on_error, self.exceptions = max_consecutive, on_error, exceptions
        self.skipped = 0

    def __iter__(self):
        return self

    def __next__(self):
        bad = 0
        while True:
            try:
                return next(self._it)
            except StopIteration:
                raise
            except self.exceptions as e:
                bad += 1
                self.skipped += 1
                if self.on_error is not None:
                    self.on_error(e)
                if bad >= self.max_consecutive:
                    raise


class GracefulInterrupt:
    """SIGINT / SIGTERM set a flag; the loop checkpoints and leaves at the next step boundary."""

    def __init__(self):
        self.flag = False
        self._old = {}

    def __enter__(self):
        for s in (signal.SIGINT, signal.SIGTERM):
            try:
                self._old[s] = signal.signal(s, self._handler)
            except ValueError:      # not the main thread
                pass
        return self

    def _handler(self, *_):
        self.flag = True

    def __exit__(self, *a):
        for s, h in self._old.items():
            signal.signal(s, h)


# ------------------------------------------------------------------------- verifier
class TrainingVerifier:
    """Checks that gradients are non-zero / finite and that parameters move
    (``GradientInspector`` / ``ParameterTracker``, src/training_verifier.rs:80-307)."""

    def __init__(self, arena):
        self.arena = arena
        self._snap = arena.data.detach().float().clone()

    def gradients(self):
        g = self.arena.grad.float()
        return {"finite": bool(torch.isfinite(g).all()), "nonzero_frac": float((g != 0).float().mean()),
                "norm": float(g.norm())}

    def parameters_changed(self):
        d = (self.arena.data.float() - self._snap).abs().max().item()
        self._snap.copy_(self.arena.data.float())
        return d

    def health(self):
        g = self.gradients()
        if not g["finite"]:
            return "diverged"
        if g["nonzero_frac"] == 0:
            return "dead_gradients"
        return "healthy"

    def verify_training_step(self, loss, step, grad_norm=None, grad_range=(1e-8, 1e3), loss_range=(0.0, 100.0)):
        """One report per step in the shape of the reference's ``verify_training_step``
        (src/training_verifier.rs:326-400): gradient, parameter, loss-trend and memory checks, and
        an overall health of ``healthy`` / ``warning`` (at most two soft issues) / ``failed``.
        ``grad_norm``: the step's global gradient norm when the gradients themselves were already
        cleared by the optimizer step (``Trainer.grad_norm()``); otherwise the arena's are read."""
        if not hasattr(self, "analyzer"):
            self.analyzer, self.memory, self.log = TrainingAnalyzer(loss_range), MemoryMonitor(), []
        issues = []
        if grad_norm is not None:
            n = float(grad_norm)
            g = {"finite": n == n and abs(n) != float("inf"), "nonzero_frac": 1.0 if n != 0 else 0.0, "norm": n}
        else:
            g = self.gradients()
        if g["nonzero_frac"] == 0:
            issues.append("No gradients detected")
        if not g["finite"]:
            issues.append("Non-finite gradients")
        elif g["nonzero_frac"] and not (grad_range[0] <= g["norm"] <= grad_range[1]):
            issues.append(f"Gradient magnitude out of range: {g['norm']:.2e}")
        moved = self.parameters_changed()
        if step > 0 and moved == 0:
            issues.append("Parameters not updating")
        ls = self.analyzer.analyze_loss(float(loss))
        if not ls["is_finite"]:
            issues.append("Loss is not finite")
        elif not ls["in_expected_range"]:
            issues.append(f"Loss out of range: {float(loss)}")
        ms = self.memory.check_memory()
        if not ms["within_bounds"]:
            issues.append(f"Memory usage too high: {ms['current_usage_gb']:.1f}GB")
        if not ms["stable"]:
            issues.append("Memory usage unstable")
        hard = any("not updating" in i or "No gradients" in i for i in issues)
        health = "healthy" if not issues else ("warning" if len(issues) <= 2 and not hard else "failed")
        rep = {"step": step, "health": health, "issues": issues, "gradients": g, "param_max_delta": moved,
               "loss": ls, "memory": ms}
        self.log.append(rep)
        return rep


class TrainingAnalyzer:
    """Loss bookkeeping: finiteness, range, and the trend of the last five values against the five
    before them (2 % band), as ``TrainingAnalyzer::analyze_loss`` (src/training_verifier.rs:225-262)."""

    def __init__(self, loss_range=(0.0, 100.0)):
        self.loss_history, self.loss_range = [], loss_range

    def analyze_loss(self, loss):
        self.loss_history.append(loss)
        finite = loss == loss and abs(loss) != float("inf")
        h = self.loss_history
        trend = "warming_up"
        if len(h) >= 10:
            recent, older = sum(h[-5:]) / 5.0, sum(h[-10:-5]) / 5.0
            trend = "decreasing" if recent < older * 0.98 else "increasing" if recent > older * 1.02 else "stable"
        return {"is_finite": finite, "in_expected_range": finite and self.loss_range[0] < loss < self.loss_range[1],
                "trend": trend, "current_loss": loss}


class MemoryMonitor:
    """Device memory in use per step, its peak, whether it stays under ``limit_frac`` of the device
    and whether the five-step average moved by less than ``drift_gb`` (the reference's
    ``MemoryMonitor`` reports a constant, src/training_verifier.rs:266-305; this one reads the
    allocator)."""

    def __init__(self, limit_frac=0.95, drift_gb=0.5, reader=None):
        self.peak_usage, self.usage_history = 0.0, []
        self.limit_frac, self.drift_gb, self._reader = limit_frac, drift_gb, reader

    def _read(self):
        if self._reader is not None:
            return self._reader()
        if torch.cuda.is_available():
            free, total = torch.cuda.mem_get_info()
            return torch.cuda.memory_allocated() / 2 ** 30, total / 2 ** 30
        return 0.0, float("inf")

    def check_memory(self):
        cur, total = self._read()
        self.usage_history.append(cur)
        self.peak_usage = max(self.peak_usage, cur)
        h, stable = self.usage_history, True
        if len(h) >= 10:
            stable = abs(sum(h[-5:]) / 5.0 - sum(h[-10:-5]) / 5.0) < self.drift_gb
        return {"current_usage_gb": cur, "peak_usage_gb": self.peak_usage,
                "within_bounds": cur < self.limit_frac * total, "stable": stable}


# ------------------------------------------------------------------------- run driver
def run_training(trainer, batches, steps, callbacks=(), log_every=10, world=1, batch_size=1, nan_guard=None,
                 watchdog=None, print_fn=print, heartbeat=None):
    """Drive ``trainer`` for ``steps`` optimizer steps over the iterator ``batches``.
    Prints the reference's per-step line (loss, grad_norm, sec/it, alloc_MB, samples/s) every
    ``log_every`` steps; reading the loss is the only host synchronisation. ``heartbeat``
    (``parallel.health.Heartbeat``) is checked between steps: when a peer is gone this rank writes
    its checkpoint and leaves with ``RankFailure`` before it launches anything that would wait
    for the missing rank."""
    cbs = list(callbacks)
    guard = nan_guard or NanGuard()
    for cb in cbs:
        cb.on_train_begin(trainer)
    it = iter(batches)
    t_last = time.time()
    with GracefulInterrupt() as intr:
        while trainer.step < steps:
            if heartbeat is not None:
                try:
                    heartbeat.check()
                except Exception:
                    if getattr(trainer.cfg, "out_dir", None):
                        trainer.save_checkpoint()
                    raise
            if watchdog:
                watchdog.begin()
            step_before = trainer.step
            loss = trainer.train_step(next(it))
            if watchdog:
                watchdog.end()
            if trainer.step == step_before:
                continue                                   # still accumulating
            s = trainer.step
            if s % log_every == 0 or s == steps or cbs:
                lv = float(loss)
                gn = trainer.grad_norm()
                gnv = float(gn) if gn is not None else None
                now = time.time()
                sec_it = (now - t_last) / (log_every if s % log_every == 0 else 1)
                t_last = now
                guard.check(trainer, lv, gnv)
                logs = {"step": s, "loss": lv, "grad_norm": gnv, "lr": trainer.optimizer.param_groups[0]["lr"],
                        "sec_per_it": sec_it, "samples_per_s": batch_size * world / max(sec_it, 1e-9),
                        "alloc_mb": torch.cuda.memory_allocated() / 2 ** 20 if torch.cuda.is_available() else 0.0,
                        "nan_skips": guard.skips}
                if s % log_every == 0 or s == steps:
                    print_fn(f"step {s}/{steps} loss {lv:.4f} grad_norm {gnv if gnv is None else round(gnv, 4)} "
                             f"sec/it {sec_it:.3f} alloc_MB {logs['alloc_mb']:.0f} samples/s {logs['samples_per_s']:.2f}")
                    trainer.log_row(lv, sec_it)
                for cb in cbs:
                    cb.on_step_end(trainer, s, logs)
                if any(cb.stop_training for cb in cbs):
                    break
            if intr.flag:
                if trainer.cfg.out_dir:
                    trainer.save_checkpoint()
                break
    for cb in cbs:
        cb.on_train_end(trainer)
    return trainer

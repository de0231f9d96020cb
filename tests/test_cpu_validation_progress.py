"""Validation runner, sanity checks, progress tracking and metric loggers (CPU)."""
import csv
import io
import json

import pytest
import torch

from tests.test_cpu_training import batch, make_trainer


def test_validation_is_repeatable_and_tracks_best(tmp_path):
    from eridiffusion_b200.train.services import run_training
    from eridiffusion_b200.train.validation import (EarlyStoppingConfig, ValidationCallback, ValidationConfig,
                                                    ValidationDataset, ValidationFormatter, ValidationRunner)
    tr = make_trainer()
    ds = ValidationDataset([batch(11), batch(12)])
    assert len(ds) == 4
    out = io.StringIO()
    cfg = ValidationConfig(every_n_steps=2, eval_timesteps=(0.25, 0.75),
                           early_stopping=EarlyStoppingConfig(patience=2, min_delta=10.0))
    runner = ValidationRunner(ds, cfg, output_dir=str(tmp_path), formatter=ValidationFormatter(stream=out))
    runner.add_metric("mae", lambda pred, target, b: (pred.float() - target.float()).abs().mean())
    m0 = runner.validate(tr, 0)
    m0b = runner.validate(tr, 0)
    assert m0.loss == m0b.loss and m0.loss_per_timestep == m0b.loss_per_timestep     # fixed t, fixed noise
    assert [t for t, _ in m0.loss_per_timestep] == [0.25, 0.75] and m0.num_samples == 4
    assert abs(m0.loss - sum(v for _, v in m0.loss_per_timestep) / 2) < 1e-6
    assert m0.custom_metrics["mae"] > 0
    assert not any(p.grad is not None and p.grad.abs().sum() > 0 for p in tr.arena.params)
    runner.history.clear(); runner.stopper.best = None; runner.stopper.bad = 0
    b = batch()
    cb = ValidationCallback(runner)
    run_training(tr, iter([b] * 50), steps=20, callbacks=[cb], log_every=100, print_fn=lambda *_: None)
    # min_delta=10 means nothing ever counts as an improvement after the first: stop after 1 + 2 validations
    assert cb.stop_training and tr.step == 6 and [h.step for h in runner.history] == [2, 4, 6]
    assert runner.best_step() in (2, 4, 6)
    saved = json.load(open(tmp_path / "validation_metrics.json"))
    assert len(saved["history"]) == 3 and saved["best_step"] == runner.best_step()
    rows = list(csv.reader(open(runner.export_metrics_csv(tmp_path / "v.csv"))))
    assert rows[0][:4] == ["step", "timestamp", "loss", "num_samples"] and "loss_t0.25" in rows[0] and "mae" in rows[0]
    assert len(rows) == 4
    text = out.getvalue()
    assert "validation at step 0" in text and "t=0.25" in text and "new best" in text


def test_validation_on_ema_weights_restores_live_weights():
    from eridiffusion_b200.train.validation import ValidationConfig, ValidationDataset, ValidationRunner
    tr = make_trainer(ema_decay=0.5)
    b = batch()
    for _ in range(3):
        tr.train_step(b)
    live = tr.arena.data.clone()
    ds = ValidationDataset([batch(11)])
    m_live = ValidationRunner(ds, ValidationConfig(use_ema=False)).validate(tr)
    m_ema = ValidationRunner(ds, ValidationConfig(use_ema=True)).validate(tr)
    assert torch.equal(tr.arena.data, live)
    assert m_live.loss != m_ema.loss


def test_discrete_schedule_timestep_mapping():
    from eridiffusion_b200.objectives import DDPM
    from eridiffusion_b200.train.validation import ValidationRunner

    class T:
        objective = DDPM()
    t = ValidationRunner._timestep(T, 0.5, 3, "cpu")
    assert t.dtype == torch.long and t.tolist() == [500, 500, 500]


def test_sanity_checks():
    from eridiffusion_b200.train.sanity import (ModelSanityChecker, SanityError, assert_optimizer_only_touches_lora,
                                                run_training_sanity_checks)
    tr = make_trainer()
    loss = tr.train_step(batch())
    chk = ModelSanityChecker.from_module(tr.model)
    run_training_sanity_checks(chk, loss, step=0)
    assert_optimizer_only_touches_lora(tr.param_names)
    with pytest.raises(SanityError, match="non-adapter"):
        assert_optimizer_only_touches_lora(["img_in.weight"])
    with pytest.raises(SanityError, match="loss is"):
        chk.assert_loss_is_valid(float("nan"))
    base = next(p for n, p in tr.model.named_parameters() if "lora" not in n)
    base.requires_grad_(True)
    with pytest.raises(SanityError, match="not frozen"):
        chk.assert_trainable_is_only_lora()
    base.requires_grad_(False)
    with torch.no_grad():
        keep = base.flatten()[0].clone()
        base.flatten()[0] = float("inf")
        with pytest.raises(SanityError, match="NaN or Inf"):
            chk.assert_all_weights_finite()
        base.flatten()[0] = 1e6
        with pytest.raises(SanityError, match="extreme"):
            chk.assert_all_weights_finite()
        base.flatten()[0] = keep
    a, b = torch.zeros(2, 4, requires_grad=True), torch.zeros(4, 2, requires_grad=True)
    with pytest.raises(SanityError, match="both matrices"):
        ModelSanityChecker([("blk.q.lora_A", a), ("blk.q.lora_B", b)]).assert_no_zero_lora()
    ModelSanityChecker([("blk.q.lora_A", torch.ones(2, 4)), ("blk.q.lora_B", b)]).assert_no_zero_lora()
    w = torch.ones(3)
    with pytest.raises(SanityError, match="received a gradient"):
        ModelSanityChecker([("proj.weight", w)]).assert_only_lora_has_gradients({"proj.weight": torch.ones(3)})


def test_progress_tracker_eta_and_summary():
    from eridiffusion_b200.train.progress import ProgressTracker
    now = [100.0]
    lines = []
    pt = ProgressTracker(10, print_fn=lines.append, clock=lambda: now[0], bar_width=10)
    pt.start_phase("caching")
    now[0] += 4
    pt.update(2, 4, "latents")
    assert "2/4" in lines[-1] and "eta 0:04" in lines[-1] and "[=====     ]" in lines[-1]
    pt.start_phase("training")
    for s in range(1, 5):
        now[0] += 2
        pt.update_step(s, 1.0 / s, grad_norm=0.5, lr=1e-4)
    assert abs(pt.sec_per_step() - 2.0) < 1e-9 and abs(pt.eta_seconds() - 12.0) < 1e-9
    assert "eta 0:12" in lines[-1] and "step 4/10" in lines[-1]
    pt.update_step(5, float("nan"), quiet=True)
    pt.update_memory(123.0); pt.update_memory(50.0)
    pt.log_error("disk full")
    s = pt.summary()
    assert s["best_loss"] == 0.25 and s["peak_memory_mb"] == 123.0 and s["errors"] == 1
    assert s["phases"][0] == ("caching", 4.0) and s["phases"][1][0] == "training"
    pt.print_summary()
    assert any("peak memory 123" in l for l in lines)


def test_loggers(tmp_path):
    from eridiffusion_b200.train.progress import (BufferedCSVLogger, ConsoleLogger, LoggerCallback, MemoryTracker,
                                                  MultiLogger, ProgressTracker)
    lines = []
    path = tmp_path / "m.csv"
    csvl = BufferedCSVLogger(str(path), buffer_size=2)
    ml = MultiLogger([ConsoleLogger(2, "simple", lines.append), ConsoleLogger(1, "json", lines.append), csvl])
    ml.log(1, {"loss": 0.5, "lr": 1e-4})
    assert len(open(path).read().splitlines()) == 1                       # header only, row buffered
    ml.log(2, {"loss": 0.25, "lr": 1e-4, "extra": 3})
    assert len(open(path).read().splitlines()) == 3
    ml.log(3, {"loss": 0.125})
    ml.close()
    rows = list(csv.reader(open(path)))
    assert rows[0] == ["step", "loss", "lr"] and rows[3] == ["3", "0.125", ""]
    assert json.loads(lines[0]) == {"step": 1, "loss": 0.5, "lr": 1e-4}
    assert "step 2 | extra=3 loss=0.25" in lines[1]
    with pytest.raises(ValueError):
        ConsoleLogger(format="xml")
    d = []
    ConsoleLogger(1, "detailed", d.append).log(7, {"loss": 1.0})
    assert d[0] == "step 7" and d[1].split() == ["loss", "1"]
    assert MemoryTracker().get_memory_usage_mb() >= 0.0 and "peak_mb" in MemoryTracker().snapshot()
    out = []
    cb = LoggerCallback(ConsoleLogger(1, "simple", out.append), ProgressTracker(3, print_fn=out.append))
    cb.on_train_begin(None)
    cb.on_step_end(None, 1, {"step": 1, "loss": 0.3, "grad_norm": None, "lr": 1e-3, "alloc_mb": 9.0})
    cb.on_train_end(None)
    assert any("loss=0.3" in l for l in out) and any("finished 1/3" in l for l in out)

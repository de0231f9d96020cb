"""Event callbacks with their manager, mixed-precision policy objects (CPU)."""
import pytest
import torch

from eridiffusion_b200.train.callbacks import (CallbackEvent, CallbackManager, EventCallback, GradientClipping,
                                               LambdaCallback, LRSchedulerCallback, ModelCheckpoint)
from eridiffusion_b200.train.mixed_precision import (AMPContext, LossScaleConfig, MixedPrecisionConfig,
                                                     MixedPrecisionOptimizer, estimate_memory)


class _FakeTrainer:
    def __init__(self):
        self.saves = []

    def save_checkpoint(self, d):
        self.saves.append(d)
        return f"{d}/ckpt{len(self.saves)}"


def test_model_checkpoint_best_only_and_period(tmp_path):
    tr = _FakeTrainer()
    best = ModelCheckpoint(str(tmp_path / "best"), save_best_only=True).monitor("val_loss", "min")
    every2 = ModelCheckpoint(str(tmp_path / "all"), period=2)
    every2.name = "periodic"
    events = []
    mgr = CallbackManager([best, every2, LambdaCallback(lambda e, c: events.append((e, c.payload)), events=[
        "training_start", "metric_logged", "checkpoint_saved", "training_end"])])
    mgr.on_train_begin(tr)
    for step, v in enumerate([0.9, 0.7, 0.8, float("nan"), 0.6], start=1):
        mgr.on_step_end(tr, step, {"loss": 1.0, "val_loss": v, "note": "x"})
    mgr.on_checkpoint(tr, "p")
    mgr.on_train_end(tr)
    assert len(best.saved) == 3 and best.best_value == 0.6 and best.best_path == best.saved[-1]
    assert len(every2.saved) == 2 and (tmp_path / "all").is_dir()
    kinds = [e for e, _ in events]
    assert kinds[0] == CallbackEvent.TRAINING_START and kinds[-1] == CallbackEvent.TRAINING_END
    assert (CallbackEvent.CHECKPOINT_SAVED, "p") in events
    assert sum(k == CallbackEvent.METRIC_LOGGED for k in kinds) == 5
    assert mgr.get("periodic") is every2 and mgr.remove("periodic") and not mgr.remove("periodic")
    with pytest.raises(ValueError):
        ModelCheckpoint("x", save_best_only=True).on_event(CallbackEvent.BATCH_END, mgr.context)


def test_manager_error_isolation_and_stop_flag():
    class Boom(EventCallback):
        name = "boom"

        def on_event(self, event, ctx):
            raise RuntimeError("nope")

    class Stop(EventCallback):
        name = "stop"

        def on_event(self, event, ctx):
            self.stop_training = ctx.global_step >= 2
    off = LambdaCallback(lambda e, c: 1 / 0, name="off")
    off.enabled = False
    mgr = CallbackManager([Boom(), Stop(), off])
    with pytest.raises(RuntimeError):
        mgr.trigger("batch_end")
    mgr.context.global_step = 2
    mgr.trigger("batch_end", strict=False)
    assert mgr.errors == [("boom", "RuntimeError('nope')")] and mgr.stop_training


def test_lr_and_clipping_callbacks():
    from eridiffusion_b200.optim import LRSchedule, ReduceLROnPlateau
    p = torch.nn.Parameter(torch.ones(4))
    opt = torch.optim.SGD([{"params": [p], "lr_mult": 0.5}], lr=1.0)
    mgr = CallbackManager([LRSchedulerCallback(opt, LRSchedule(1e-2, "linear", total_steps=10),
                                               ReduceLROnPlateau(1e-2, factor=0.1, patience=0))])
    mgr.context.global_step = 5
    mgr.trigger("batch_start")
    assert abs(opt.param_groups[0]["lr"] - 0.5 * 5e-3) < 1e-12
    mgr.context.metrics = {"val_loss": 1.0}
    mgr.trigger("validation_end")
    mgr.trigger("validation_end")                              # no improvement -> reduced
    assert abs(mgr.get("lr_scheduler").last_lr - 1e-3) < 1e-12
    p.grad = torch.full((4,), 3.0)
    gc = GradientClipping([p], max_norm=1.0)
    assert abs(gc.clip() - 6.0) < 1e-6 and abs(float(p.grad.norm()) - 1.0) < 1e-5 and gc.num_clipped == 1


def test_mixed_precision_optimizer_fp16_with_inf_skip():
    cfg = MixedPrecisionConfig(enabled=True, dtype="float16", loss_scale=LossScaleConfig(init_scale=1024.0,
                                                                                          growth_interval=2))
    w = torch.nn.Parameter(torch.ones(8, dtype=torch.float16))
    mp = MixedPrecisionOptimizer(lambda ps: torch.optim.SGD(ps, lr=2.0 ** -12), [w], cfg.make_scaler(),
                                 gradient_clipping=None)
    for _ in range(3):
        loss = mp.scale_loss((w.float() * 1.0).sum())
        loss.backward()
        assert mp.step()
        mp.zero_grad()
    # three updates of 2^-12 each: invisible in fp16 one at a time (ulp at 1.0 is 2^-10), kept by the master
    assert abs(float(mp.master_params[0].detach()[0]) - (1 - 3 * 2.0 ** -12)) < 1e-7
    assert mp.scaler.scale == 2048.0                           # grew after two good steps
    w.grad = torch.full((8,), float("inf"), dtype=torch.float16)
    before = mp.master_params[0].clone()
    assert not mp.step() and mp.skipped_steps == 1 and mp.scaler.scale == 1024.0
    assert torch.equal(mp.master_params[0], before) and w.grad is None
    sd = mp.state_dict()
    mp.load_state_dict(sd)
    st = MixedPrecisionConfig(enabled=True, loss_scale=LossScaleConfig.static(128.0)).make_scaler()
    st.found_inf = True; st.update()
    assert st.scale == 128.0
    assert not MixedPrecisionConfig(enabled=True, dtype="bfloat16").make_scaler().enabled
    with pytest.raises(ValueError):
        MixedPrecisionConfig(opt_level="O9")


def test_amp_context_and_memory_estimate():
    amp = AMPContext(MixedPrecisionConfig(enabled=True, dtype="bfloat16", opt_level="O1"), device="cpu")
    assert amp.should_cast("linear") and not amp.should_cast("softmax") and not amp.should_cast("layer_norm")
    assert AMPContext(MixedPrecisionConfig(enabled=True, opt_level="O2"), "cpu").should_cast("layer_norm")
    x = torch.ones(2)
    assert amp.cast("matmul", x).dtype == torch.bfloat16 and amp.cast("loss", x.bfloat16()).dtype == torch.float32
    with amp.autocast():
        assert (torch.ones(2, 2) @ torch.ones(2, 2)).dtype == torch.bfloat16
    off = AMPContext(MixedPrecisionConfig(enabled=False), "cpu")
    with off.autocast():
        assert (torch.ones(2, 2) @ torch.ones(2, 2)).dtype == torch.float32
    e = estimate_memory(1000, 10_000, MixedPrecisionConfig(enabled=True))
    assert e.fp32_total == 1000 * 16 + 40_000 and e.mp_total == 1000 * 16 + 20_000 and 0 < e.savings_percent < 50
    assert estimate_memory(1000, 10_000, MixedPrecisionConfig(enabled=False)).savings_percent == 0.0

"""Phase timer, NVTX no-op ranges, loss analyzer, memory monitor and the per-step verification report."""
import torch

from eridiffusion_b200.models import build_model
from eridiffusion_b200.data import synthetic_batch
from eridiffusion_b200.adapters import AdapterConfig
from eridiffusion_b200.train.services import MemoryMonitor, TrainingAnalyzer, TrainingVerifier
from eridiffusion_b200.train.trainer import Trainer, TrainerConfig
from eridiffusion_b200.utils import trace


def test_phase_timer_and_ranges():
    t = trace.PhaseTimer()
    for _ in range(3):
        with t.phase("a"):
            torch.randn(64, 64) @ torch.randn(64, 64)
        with t.phase("b"):
            pass
    s = t.summary()
    assert list(s) == ["a", "b"] and s["a"]["calls"] == 3 and abs(sum(v["share"] for v in s.values()) - 1) < 1e-6
    assert "a " in t.format()
    off = trace.PhaseTimer(enabled=False)
    with off.phase("x"):
        pass
    assert off.summary() == {}
    with trace.range("no gpu: does nothing"):
        pass
    m = build_model("tiny_mmdit", device="cpu", dtype=torch.float32)
    hs = trace.annotate_blocks(m)
    assert len(hs) == 2 * (len(m.double_blocks) + len(m.single_blocks))
    for h in hs:
        h.remove()


def test_analyzer_trend_and_memory_monitor():
    a = TrainingAnalyzer()
    for i in range(9):
        assert a.analyze_loss(1.0)["trend"] == "warming_up"
    assert a.analyze_loss(1.0)["trend"] == "stable"
    for _ in range(5):
        r = a.analyze_loss(0.5)
    assert r["trend"] == "decreasing" and r["in_expected_range"]
    for _ in range(5):
        r = a.analyze_loss(2.0)
    assert r["trend"] == "increasing"
    assert not a.analyze_loss(float("nan"))["is_finite"]
    usage = iter([1.0] * 5 + [3.0] * 5 + [100.0])
    mm = MemoryMonitor(reader=lambda: (next(usage), 80.0))
    for _ in range(9):
        assert mm.check_memory()["stable"]
    assert not mm.check_memory()["stable"]
    r = mm.check_memory()
    assert not r["within_bounds"] and r["peak_usage_gb"] == 100.0


def test_verify_training_step_and_trainer_phases(monkeypatch):
    monkeypatch.setenv("ERI_B200_PHASE_TIMING", "1")
    torch.manual_seed(0)
    m = build_model("tiny_mmdit", device="cpu", dtype=torch.float32)
    cfg = TrainerConfig(mode="lora", adapter=AdapterConfig(rank=4, alpha=4, dtype=torch.float32), optimizer="adamw",
                        lr=1e-2, seed=1)
    tr = Trainer(m, cfg)
    ver = TrainingVerifier(tr.arena)
    rep = None
    for i in range(3):
        loss = tr.train_step(synthetic_batch("tiny_mmdit", 2, "cpu", torch.float32, i))
        rep = ver.verify_training_step(float(loss), i, grad_norm=tr.grad_norm())
    assert rep["health"] in ("healthy", "warning") and rep["param_max_delta"] > 0
    assert rep["loss"]["trend"] == "warming_up" and len(ver.log) == 3
    tr.arena.grad.zero_()
    rep = ver.verify_training_step(float("nan"), 4)
    assert rep["health"] == "failed" and "No gradients detected" in rep["issues"] and "Loss is not finite" in rep["issues"]
    s = tr.phases.summary()
    assert list(s) == ["noise", "forward", "backward", "optimizer"] and s["forward"]["calls"] == 3


def test_sample_callback_writes_latents(tmp_path):
    from eridiffusion_b200.config import SampleCfg
    from eridiffusion_b200.io import safetensors as st
    from eridiffusion_b200.train.services import SampleCallback, run_training
    torch.manual_seed(0)
    m = build_model("tiny_mmdit", device="cpu", dtype=torch.float32)
    cfg = TrainerConfig(mode="lora", adapter=AdapterConfig(rank=4, alpha=4, dtype=torch.float32), optimizer="adamw",
                        lr=1e-3, seed=1, total_steps=4)
    tr = Trainer(m, cfg)
    cb = SampleCallback(SampleCfg(sample_every=2, width=64, height=64, sample_steps=2, prompts=["a", "b"], walk_seed=True),
                        "tiny_mmdit", tmp_path)
    batches = (synthetic_batch("tiny_mmdit", 1, "cpu", torch.float32, i) for i in range(100))
    run_training(tr, batches, 4, callbacks=[cb], log_every=1, print_fn=lambda *_: None)
    assert len(cb.written) == 4 and m.training                       # steps 2 and 4, two prompts each
    f = tmp_path / "samples" / "step0000002_1.safetensors"
    assert f.exists() and st.load_file(f)["latent"].shape == (1, 16, 8, 8)
    assert st.read_metadata(f)["seed"] == "43"
